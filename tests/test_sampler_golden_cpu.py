"""Pins the oracle's final-head chain (logits -> code) to the reference's own kernels: codes, processed scores and
SplitMix64 states in tests/golden/reference_sampler_golden.npz came from those kernels on a B200
(tests/golden/make_reference_sampler_golden.py).  Bit for bit."""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import sampler_cases as sc

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_sampler_golden.npz")


@pytest.mark.parametrize("name", sorted(sc.CASES))
def test_oracle_final_head_matches_reference_kernels(name):
    c = sc.SamplerCase(name)
    code, processed, state, history = oracle.final_head_sample(c.logits, c.history, c.generation_index, c.flags,
                                                               eos_token=sc.EOS, top_k=c.top_k, temperature=c.temperature,
                                                               rng_state=c.rng_state)
    assert code == int(GOLDEN[f"{name}_code"])
    assert np.array_equal(processed.view(np.uint32), GOLDEN[f"{name}_processed"].view(np.uint32))
    assert state == int(GOLDEN[f"{name}_state"])
    assert history[c.generation_index] == int(GOLDEN[f"{name}_recorded"])


def test_oracle_chain_of_draws_matches_reference_kernels():
    c = sc.SamplerCase("topk_processed")
    state, history, codes = c.rng_state, c.history.copy(), []
    flags = sc.REPETITION | sc.SUPPRESS | sc.RECORD
    for step in range(16):
        code, _, state, history = oracle.final_head_sample(c.logits, history, c.generation_index + step, flags,
                                                           eos_token=sc.EOS, top_k=c.top_k, temperature=c.temperature,
                                                           rng_state=state)
        codes.append(code)
    assert codes == GOLDEN["chain_codes"].tolist()
    assert state == int(GOLDEN["chain_state"])


def test_suppression_and_penalty_semantics():
    c = sc.SamplerCase("greedy_processed_first_step")
    _, processed, _, _ = oracle.final_head_sample(c.logits, c.history, 0, sc.SUPPRESS, eos_token=sc.EOS)
    assert processed[sc.EOS] == -np.inf and np.all(processed[2048:] == -np.inf)
    _, processed, _, _ = oracle.final_head_sample(c.logits, c.history, 2, sc.SUPPRESS, eos_token=sc.EOS)
    assert np.isfinite(processed[sc.EOS]) and np.all(np.delete(processed[2048:], sc.EOS - 2048) == -np.inf)
    c = sc.SamplerCase("greedy_processed_late")
    raw = oracle.bf16_to_f32(c.logits)
    _, processed, _, _ = oracle.final_head_sample(c.logits, c.history, c.generation_index, sc.REPETITION, eos_token=sc.EOS)
    seen = np.zeros(sc.VOCAB, dtype=bool)
    seen[c.history[: c.generation_index]] = True
    assert np.array_equal(processed[~seen], raw[~seen])
    pos = seen & (raw >= 0)
    assert np.all(processed[pos] < raw[pos] + 1e-12) and np.all(processed[seen & (raw < 0)] < raw[seen & (raw < 0)])
