"""Host-side mirror of the reference's code predictor frame (`code_predictor::...::capture_step`,
devices/rtx4090-24g/qwen3_tts_1_7b.cu:13616-13905), for a batch of streams, on this library's entry points.

Per audio frame the reference runs 15 steps of a 5-layer decoder (hidden 1024, 16 query / 8 KV heads of 128,
SwiGLU 3072, vocabulary 2048, at most 16 cached positions): step 0 feeds two rows (the talker's last hidden state
and the embedding of the first code), every later step one row (the embedding of the code just drawn); each step
ends with the final norm, that step's own head, a draw (greedy or top-k) and that step's own embedding table.  The
layer has exactly the talker layer's structure and its attention the same GQA shape, so a frame here is 16 token
steps through the same seven launches per layer that the talker step uses (`qm_rmsnorm`, `qm_qkv_linear`,
`qm_decode_step`, `qm_linear`, `qm_add_postnorm`, `qm_gate_up_swiglu`, `qm_linear`), with `qm_final_head_sample`
and `qm_embedding_gather` closing each step.  The two rows of step 0 go through as two consecutive positions,
which is the same causal attention.  Nothing synchronises with the host, so a frame can be captured as one CUDA
graph, as the reference does (:13907-13935).

Weights are whatever the caller supplies; `random_weights` draws the shapes of the reference's checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass, field

OUTER_HIDDEN = 2048      # kOuterHidden
HIDDEN = 1024            # kHidden
INTERMEDIATE = 3072      # kIntermediate
LAYERS = 5               # kLayers
Q_HEADS, KV_HEADS, HEAD_DIM = 16, 8, 128
VOCAB = 2048             # kVocab
STEPS = 15               # kSteps
MAX_CACHE = 16           # kMaxCache


@dataclass
class PredictorDims:
    outer_hidden: int = OUTER_HIDDEN
    hidden: int = HIDDEN
    intermediate: int = INTERMEDIATE
    layers: int = LAYERS
    vocab: int = VOCAB
    steps: int = STEPS


@dataclass
class PredictorWeights:
    projection: object = None          # [hidden][outer_hidden], bias [hidden]  (small_to_mtp projection, :13623-13630)
    projection_bias: object = None
    layers: list = field(default_factory=list)   # dicts: in_norm, post_norm, q, k, v, o, q_norm, k_norm, gate, up, down
    final_norm: object = None
    heads: list = field(default_factory=list)        # per step [vocab][hidden]
    embeddings: list = field(default_factory=list)   # per step [vocab][outer_hidden]


def random_weights(dims: PredictorDims, generator, scale=0.02):
    """Random bf16 weights in the reference checkpoint's shapes (torch CUDA tensors)."""
    import torch

    def w(*shape, s=scale):
        return (torch.randn(*shape, generator=generator, device="cuda") * s).to(torch.bfloat16)

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device="cuda")

    nq, nk = Q_HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM
    out = PredictorWeights(projection=w(dims.hidden, dims.outer_hidden), projection_bias=w(dims.hidden), final_norm=ones(dims.hidden))
    for _ in range(dims.layers):
        out.layers.append({
            "in_norm": ones(dims.hidden), "post_norm": ones(dims.hidden), "q_norm": ones(HEAD_DIM), "k_norm": ones(HEAD_DIM),
            "q": w(nq, dims.hidden), "k": w(nk, dims.hidden), "v": w(nk, dims.hidden), "o": w(dims.hidden, nq),
            "gate": w(dims.intermediate, dims.hidden), "up": w(dims.intermediate, dims.hidden),
            "down": w(dims.hidden, dims.intermediate),
        })
    for _ in range(dims.steps):
        out.heads.append(w(dims.vocab, dims.hidden))
        out.embeddings.append(w(dims.vocab, dims.outer_hidden, s=1.0))
    return out


class CodePredictor:
    """One frame of the code predictor for `streams` streams at once."""

    def __init__(self, package, streams: int, weights: PredictorWeights, dims: PredictorDims | None = None):
        import torch

        self.dims = dims or PredictorDims()
        self.streams, self.weights = streams, weights
        # 16 positions fit one 64-token page per stream
        self.engine = package.TalkerAttention(layers=self.dims.layers, num_pages=streams, q_heads=Q_HEADS, kv_heads=KV_HEADS,
                                              max_positions=64)
        self.engine.workspace(streams)
        self.page_table = torch.arange(streams, dtype=torch.int32, device="cuda").view(streams, 1)
        self.positions = torch.zeros((streams,), dtype=torch.int32, device="cuda")
        d = self.dims

        def buf(cols):
            return torch.empty((streams, cols), dtype=torch.bfloat16, device="cuda")

        nq, nk = Q_HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM
        self.hidden_a, self.hidden_b = buf(d.hidden), buf(d.hidden)
        self.norm, self.attn_out, self.residual, self.post, self.act = buf(d.hidden), buf(d.hidden), buf(d.hidden), buf(d.hidden), buf(d.intermediate)
        self.q, self.k, self.v = buf(nq), buf(nk), buf(nk)
        self.context = torch.empty((streams, Q_HEADS, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
        self.logits = buf(d.vocab)
        self.next_input = buf(d.outer_hidden)
        self.codes = torch.zeros((d.steps, streams), dtype=torch.int32, device="cuda")
        self.step_logits = None        # set to a list to keep every step's logits (tests)

    def close(self):
        self.engine.close()

    def _token_step(self, row_input):
        """One row per stream through the projection and the layers (capture_step's body, :13623-13842)."""
        eng, w = self.engine, self.weights
        b = self.streams
        cur, nxt = self.hidden_a, self.hidden_b
        eng.launch_linear_m1(row_input, w.projection, bias=w.projection_bias, out=cur)
        for index, layer in enumerate(w.layers):
            eng.launch_rmsnorm(cur, layer["in_norm"], out=self.norm)
            eng.launch_qkv_m1(self.norm, layer["q"], layer["k"], layer["v"], out=(self.q, self.k, self.v))
            eng.decode_step(index, self.q.view(b, Q_HEADS, HEAD_DIM), self.k.view(b, KV_HEADS, HEAD_DIM),
                            self.v.view(b, KV_HEADS, HEAD_DIM), layer["q_norm"], layer["k_norm"], self.positions,
                            self.page_table, out=self.context)
            eng.launch_linear_m1(self.context.view(b, Q_HEADS * HEAD_DIM), layer["o"], out=self.attn_out)
            eng.launch_add_postnorm_m1(cur, self.attn_out, layer["post_norm"], residual=self.residual, normalized=self.post)
            eng.launch_gate_up_swiglu_m1(self.post, layer["gate"], layer["up"], out=self.act)
            eng.launch_linear_m1(self.act, layer["down"], residual=self.residual, out=nxt)
            cur, nxt = nxt, cur
        self.positions.add_(1)
        return cur

    def frame(self, talker_hidden, first_code_embedding, rng_state=None, top_k=0, temperature=0.9):
        """Runs the 15 steps; returns codes [steps][streams] (int32, on the device).  Greedy when top_k is 0,
        otherwise top-k sampling from each stream's SplitMix64 state (gpu_sample_topk_bf16_kernel, :7602-7660)."""
        eng, w, d = self.engine, self.weights, self.dims
        self.positions.zero_()
        self._token_step(talker_hidden)                      # first row of step 0: only fills the cache
        row_input = first_code_embedding
        for step in range(d.steps):
            last = self._token_step(row_input)
            eng.launch_rmsnorm(last, w.final_norm, out=self.norm)
            eng.launch_linear_m1(self.norm, w.heads[step], out=self.logits)
            if self.step_logits is not None:
                self.step_logits.append(self.logits.clone())
            eng.final_head_sample(self.logits, flags=0, top_k=top_k, temperature=temperature, rng_state=rng_state,
                                  codes=self.codes[step])
            eng.embedding_gather(w.embeddings[step], self.codes[step], out=self.next_input)
            row_input = self.next_input
        return self.codes
