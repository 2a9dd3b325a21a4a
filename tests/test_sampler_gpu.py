"""qm_final_head_sample and qm_embedding_gather on the GPU against the oracle and against what the reference's own
final-head kernels returned (tests/golden/reference_sampler_golden.npz).  Codes, processed scores and SplitMix64
states are integers / exact floats: everything is compared bit for bit."""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import sampler_cases as sc

GOLDEN_PATH = Path(__file__).resolve().parent / "golden" / "reference_sampler_golden.npz"
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine(qm):
    eng = qm.TalkerAttention(layers=1, num_pages=8, q_heads=16, kv_heads=8, max_positions=64)
    yield eng
    eng.close()


def run_batch(engine, cases, top_k, flags):
    """All `cases` as one batch (they share top_k and flags, as one launch does)."""
    import torch

    logits = torch.from_numpy(np.stack([c.logits for c in cases]).view(np.int16)).cuda().view(torch.bfloat16)
    history = torch.from_numpy(np.stack([c.history for c in cases])).cuda()
    generation = torch.tensor([c.generation_index for c in cases], dtype=torch.int32, device="cuda")
    state = torch.tensor([c.rng_state for c in cases], dtype=torch.int64, device="cuda")
    processed = torch.empty((len(cases), sc.VOCAB), dtype=torch.float32, device="cuda")
    codes = engine.final_head_sample(logits, generation, history, flags=flags, eos_token=sc.EOS, top_k=top_k,
                                     temperature=cases[0].temperature, rng_state=state, processed=processed)
    torch.cuda.synchronize()
    assert engine.status() == 0
    return codes.cpu().numpy(), processed.cpu().numpy(), state.cpu().numpy().astype(np.uint64), history.cpu().numpy()


@pytest.mark.parametrize("name", sorted(sc.CASES))
def test_single_stream_matches_oracle_and_reference_kernels(engine, name):
    c = sc.SamplerCase(name)
    codes, processed, state, history = run_batch(engine, [c], c.top_k, c.flags)
    want = oracle.final_head_sample(c.logits, c.history, c.generation_index, c.flags, eos_token=sc.EOS, top_k=c.top_k,
                                    temperature=c.temperature, rng_state=c.rng_state)
    assert codes[0] == want[0]
    assert np.array_equal(processed[0].view(np.uint32), want[1].view(np.uint32))
    assert int(state[0]) == want[2]
    assert np.array_equal(history[0], want[3])
    golden = np.load(GOLDEN_PATH)
    assert codes[0] == int(golden[f"{name}_code"])
    assert np.array_equal(processed[0].view(np.uint32), golden[f"{name}_processed"].view(np.uint32))
    assert int(state[0]) == int(golden[f"{name}_state"])
    assert history[0][c.generation_index] == int(golden[f"{name}_recorded"])


def test_batch_of_streams_each_with_its_own_history_and_state(engine):
    rng = np.random.default_rng(5)
    cases = []
    for i in range(48):
        c = sc.SamplerCase("topk_processed")
        c.logits = oracle.f32_to_bf16((rng.standard_normal(sc.VOCAB) * 3.0).astype(np.float32))
        c.generation_index = int(rng.integers(0, 300))
        c.history[: c.generation_index] = rng.integers(0, 2048, size=c.generation_index)
        c.rng_state = int(rng.integers(1, 2**62))
        cases.append(c)
    flags = sc.REPETITION | sc.SUPPRESS | sc.RECORD
    for top_k in (0, 50):
        codes, processed, state, history = run_batch(engine, cases, top_k, flags)
        for i, c in enumerate(cases):
            want = oracle.final_head_sample(c.logits, c.history, c.generation_index, flags, eos_token=sc.EOS, top_k=top_k,
                                            temperature=c.temperature, rng_state=c.rng_state)
            assert codes[i] == want[0], (top_k, i)
            assert int(state[i]) == want[2]
            assert history[i][c.generation_index] == want[0]


@pytest.mark.parametrize("vocab,top_k", [(2048, 50), (3072, 64), (3072, 65), (3072, 200), (4096, 50), (50, 50), (70, 8),
                                         (64, 64), (65, 3), (1, 5), (2048, 5000)])
def test_top_k_selection_paths_against_the_oracle(engine, vocab, top_k):
    """Up to 64 candidates the kernel selects the best 64 keys with per-warp bitonic networks, beyond that it sorts
    everything; small vocabularies leave most of the first block as padding.  Eight draws per shape, some with
    ties between equal scores, each against the oracle: code and SplitMix64 state."""
    import torch

    rng = np.random.default_rng(1000 * vocab + top_k)
    streams = 8
    values = (rng.standard_normal((streams, vocab)) * 3.0).astype(np.float32)
    values[1] = np.round(values[1] * 4) / 4               # many exactly equal scores
    values[2] = 0.0                                       # all equal
    bits = oracle.f32_to_bf16(values)
    states = rng.integers(1, 2**62, size=streams)
    logits = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    state = torch.tensor(states, dtype=torch.int64, device="cuda")
    codes = engine.final_head_sample(logits, flags=0, eos_token=0, reserved_begin=vocab, top_k=top_k, temperature=0.9,
                                     rng_state=state)
    torch.cuda.synchronize()
    assert engine.status() == 0
    codes, state = codes.cpu().numpy(), state.cpu().numpy().astype(np.uint64)
    for i in range(streams):
        want = oracle.final_head_sample(bits[i], np.zeros(8, dtype=np.int32), 0, 0, eos_token=0, top_k=top_k, temperature=0.9,
                                        rng_state=int(states[i]), reserved_begin=vocab)
        assert codes[i] == want[0], (i, codes[i], want[0])
        assert int(state[i]) == want[2]


def test_consecutive_steps_draw_from_the_state_in_order(engine):
    import torch

    golden = np.load(GOLDEN_PATH)
    c = sc.SamplerCase("topk_processed")
    logits = torch.from_numpy(c.logits.view(np.int16)[None]).cuda().view(torch.bfloat16)
    history = torch.from_numpy(c.history[None].copy()).cuda()
    generation = torch.tensor([c.generation_index], dtype=torch.int32, device="cuda")
    state = torch.tensor([c.rng_state], dtype=torch.int64, device="cuda")
    flags = sc.REPETITION | sc.SUPPRESS | sc.RECORD
    codes = []
    for _ in range(16):
        out = engine.final_head_sample(logits, generation, history, flags=flags, eos_token=sc.EOS, top_k=50,
                                       temperature=c.temperature, rng_state=state)
        codes.append(int(out.cpu()[0]))
        generation += 1
    assert codes == golden["chain_codes"].tolist()
    assert int(state.cpu().numpy().astype(np.uint64)[0]) == int(golden["chain_state"])


def test_embedding_gather_copies_rows_and_reports_bad_ids(engine):
    import torch

    table = torch.randn(3072, 2048, device="cuda").to(torch.bfloat16)
    ids = torch.randint(0, 3072, (64,), device="cuda", dtype=torch.int32)
    out = engine.embedding_gather(table, ids)
    assert torch.equal(out, table[ids.long()])
    assert engine.status() == 0
    ids[3] = 5000
    out = engine.embedding_gather(table, ids)
    torch.cuda.synchronize()
    assert engine.status() == 2           # QM_DEVSTAT_BAD_POS
    assert torch.equal(out[3], table[3071])


def test_argument_checks(engine, qm):
    import torch

    logits = torch.zeros((2, 5000), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(qm.QmError):
        engine.final_head_sample(logits)                      # vocabulary beyond 4096
    logits = torch.zeros((2, 3072), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(qm.QmError):
        engine.final_head_sample(logits, top_k=50)            # sampling without a state
    with pytest.raises(qm.QmError):
        engine.final_head_sample(logits, flags=sc.REPETITION)  # penalty without a history


def test_degenerate_rows(engine):
    """Rows where nothing is finite, where everything is equal, a vocabulary smaller than the sort size, and a top_k
    beyond the vocabulary: same answers as the restated reference chain, and no draw is consumed when the weights do
    not add up to something positive (the reference returns before drawing)."""
    import torch

    vocab = 2048
    rows = {
        "all_minus_inf": np.full(vocab, -np.inf, dtype=np.float32),
        "all_equal": np.full(vocab, 1.25, dtype=np.float32),
        "one_finite": np.where(np.arange(vocab) == 777, 3.0, -np.inf).astype(np.float32),
        "ramp": np.linspace(-4, 4, vocab, dtype=np.float32),
    }
    for top_k in (0, 50, 5000):
        for name, values in rows.items():
            bits = oracle.f32_to_bf16(values)
            logits = torch.from_numpy(bits.view(np.int16)[None]).cuda().view(torch.bfloat16)
            state = torch.tensor([12345], dtype=torch.int64, device="cuda")
            code = engine.final_head_sample(logits, flags=0, top_k=top_k, temperature=0.9, rng_state=state)
            torch.cuda.synchronize()
            want = oracle.final_head_sample(bits, flags=0, top_k=top_k, temperature=0.9, rng_state=12345)
            assert int(code.cpu()[0]) == want[0], (name, top_k)
            assert int(state.cpu().numpy().astype(np.uint64)[0]) == want[2], (name, top_k)
    assert engine.status() == 0
