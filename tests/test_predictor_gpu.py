"""A code-predictor frame (reference capture_step, 17.cu:13616-13905) on the library's entry points against the same
chain built from the oracle's operators: reduced widths (hidden 256, SwiGLU 512, 2 layers, 4 steps), real head shape
(16 / 8 heads of 128, vocabulary 2048).  Each step's logits are compared under the path's tolerance (the oracle's
operators are pinned to the reference's predictor kernels by tests/test_predictor_golden_cpu.py); the oracle
chain is fed the library's own codes, so a near-tie cannot send the two chains down different paths, and each code
is checked to be exactly what the restated sampler draws from the library's logits."""
import importlib

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu

HQ, HKV, D = 16, 8, 128


def bits_of_weights(w):
    b = scenario._bits
    return {
        "projection": b(w.projection), "projection_bias": b(w.projection_bias), "final_norm": b(w.final_norm),
        "layers": [{k: b(v) for k, v in layer.items()} for layer in w.layers],
        "heads": [b(h) for h in w.heads], "embeddings": [b(e) for e in w.embeddings],
    }


def oracle_token_step(w, row_input, position, key_caches, value_caches, cos, sin):
    """One row per stream through the projection and the layers, with the oracle's operators."""
    streams = row_input.shape[0]
    cur = oracle.linear(row_input, w["projection"], bias=w["projection_bias"])
    for li, layer in enumerate(w["layers"]):
        normed = oracle.rmsnorm(cur, layer["in_norm"])
        q = oracle.linear(normed, layer["q"]).reshape(streams, HQ, D)
        k = oracle.linear(normed, layer["k"]).reshape(streams, HKV, D)
        v = oracle.linear(normed, layer["v"]).reshape(streams, HKV, D)
        ctx = np.empty((streams, HQ, D), dtype=np.uint16)
        for s in range(streams):
            kc, vc = key_caches[li][s], value_caches[li][s]
            qr = oracle.append(q[s:s + 1], k[s:s + 1], v[s:s + 1], layer["q_norm"], layer["k_norm"], cos[position:position + 1],
                               sin[position:position + 1], position, kc, vc)
            ctx[s] = oracle.decode_attention(qr, [kc], [vc], [position + 1], mode="ref")[0]
        attn = oracle.linear(ctx.reshape(streams, HQ * D), layer["o"])
        residual, post = oracle.add_postnorm(cur, attn, layer["post_norm"])
        act = oracle.gate_up_swiglu(post, layer["gate"], layer["up"])
        cur = oracle.linear(act, layer["down"], residual=residual)
    return cur


@pytest.mark.parametrize("top_k", [0, 50])
def test_predictor_frame_matches_oracle_chain(qm, top_k):
    import torch

    predictor = importlib.import_module("qingming_qwen3_tts_b200.predictor")
    dims = predictor.PredictorDims(outer_hidden=512, hidden=256, intermediate=512, layers=2, vocab=2048, steps=4)
    streams = 3
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)
    weights = predictor.random_weights(dims, gen, scale=0.06)
    for layer in weights.layers:       # norm weights that are not all ones
        for name in ("in_norm", "post_norm", "q_norm", "k_norm"):
            layer[name] = (1.0 + 0.1 * torch.randn(layer[name].shape, generator=gen, device="cuda")).to(torch.bfloat16)
    talker_hidden = torch.randn(streams, dims.outer_hidden, generator=gen, device="cuda").to(torch.bfloat16)
    first_embedding = torch.randn(streams, dims.outer_hidden, generator=gen, device="cuda").to(torch.bfloat16)
    states = torch.tensor([11, 22, 33], dtype=torch.int64, device="cuda")
    states_before = states.cpu().numpy().astype(np.uint64)

    runner = predictor.CodePredictor(qm, streams, weights, dims)
    try:
        runner.step_logits = []
        codes = runner.frame(talker_hidden, first_embedding, rng_state=states, top_k=top_k).cpu().numpy()
        torch.cuda.synchronize()
        assert runner.engine.status() == 0
        got_logits = [scenario._bits(x) for x in runner.step_logits]
    finally:
        runner.close()

    w = bits_of_weights(weights)
    cos, sin = oracle.make_rope(64)
    key_caches = [[np.zeros((HKV, 64, D), dtype=np.uint16) for _ in range(streams)] for _ in range(dims.layers)]
    value_caches = [[np.zeros((HKV, 64, D), dtype=np.uint16) for _ in range(streams)] for _ in range(dims.layers)]
    oracle_token_step(w, scenario._bits(talker_hidden), 0, key_caches, value_caches, cos, sin)
    row_input = scenario._bits(first_embedding)
    state = [int(x) for x in states_before]
    worst = {"max_abs": 0.0, "mean_rel": 0.0}
    for step in range(dims.steps):
        last = oracle_token_step(w, row_input, step + 1, key_caches, value_caches, cos, sin)
        want_logits = oracle.linear(oracle.rmsnorm(last, w["final_norm"]), w["heads"][step])
        m = oracle.error_metrics(oracle.bf16_to_f32(got_logits[step]), oracle.bf16_to_f32(want_logits))
        worst = {k: max(worst[k], m[k]) for k in worst}
        scale = float(np.abs(oracle.bf16_to_f32(want_logits)).max())
        print(f"predictor step {step}: max_abs {m['max_abs']:.4f} mean_rel {m['mean_rel']:.5f} logits up to {scale:.2f}")
        # Per-step budget: the path's mean-relative tolerance (1e-2), and at most 5e-2 absolute on logits that reach
        # 4 (a bf16 ulp is 0.016 at 2 and 0.031 at 4; two layers of one-ulp differences add up to two or three).
        # Every step is teacher-forced with the library's own codes and so starts from the oracle's inputs.
        assert m["max_abs"] <= 5e-2 and m["mean_rel"] <= 1e-2, (step, m, scale)
        for s in range(streams):
            # the library's code is what the restated sampler draws from the library's own logits
            code, _, state[s], _ = oracle.final_head_sample(got_logits[step][s], flags=0, top_k=top_k, temperature=0.9,
                                                            rng_state=state[s])
            assert code == codes[step][s], (step, s)
        row_input = w["embeddings"][step][codes[step]]            # teacher forcing with the library's codes
    print("predictor frame", worst)
    assert worst["max_abs"] <= 5e-2 and worst["mean_rel"] <= 1e-2, worst
    if top_k:
        assert [int(x) for x in states.cpu().numpy().astype(np.uint64)] == state
