"""Pins the CPU oracle to the reference's own kernels.

tests/golden/reference_kernels_golden.npz holds the outputs of the reference's CUDA kernels (compiled unmodified
from its source tree, launched on a B200 by tests/golden/make_reference_golden.py) on the seeded scenarios below.
The oracle's bf16-faithful mode must reproduce them: the only permitted differences come from libm expf / sqrtf
versus the device expf / rsqrtf, which flip the last bf16 bit of a few elements.
"""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario
from golden.make_reference_golden import DECODE_CASES, PREFILL_CASES

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_kernels_golden.npz")


def ulp_distance(a, b):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + (x & 0x7FFF))
    return np.abs(key(a) - key(b))


def assert_nearly_identical(got, want, max_fraction):
    dist = ulp_distance(got, want)
    # one flipped rounding early in the five-rounding chain can move the final value by two ulps
    assert dist.max() <= 2, f"max ulp distance {dist.max()}"
    assert (dist != 0).mean() <= max_fraction, f"{(dist != 0).mean():.5f} of elements differ"


def assert_context_close(got, want, max_fraction=5e-3):
    # attention outputs are sums near zero, where ulp distance is meaningless: bound the absolute difference
    # (one bf16 ulp of a value below 1 is at most 2^-8) and the share of elements that differ at all
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -8, diff.max()
    assert (got != want).mean() <= max_fraction, (got != want).mean()


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_decode_append_and_attention_match_reference_kernels(name):
    seed, lengths, rw = DECODE_CASES[name]
    exp = scenario.DecodeScenario(seed=seed, lengths=lengths, random_weights=rw).expected()
    assert_nearly_identical(exp["q_rot"], GOLDEN[f"{name}_q_rot"], 1e-3)
    assert_nearly_identical(exp["key_rows"], GOLDEN[f"{name}_key_rows"], 1e-3)
    assert_context_close(exp["out_ref"], GOLDEN[f"{name}_context"])


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_append_and_attention_match_reference_kernels(name):
    seed, lengths, rw = PREFILL_CASES[name]
    ps = scenario.PrefillScenario(seed=seed, lengths=lengths, random_weights=rw)
    q_rot, kcs, _ = ps.expected_append()
    assert_nearly_identical(q_rot, GOLDEN[f"{name}_q_rot"], 1e-3)
    for s in range(ps.batch):
        n = int(ps.lengths[s])
        assert_nearly_identical(kcs[s][:, :n], GOLDEN[f"{name}_key_cache_{s}"], 1e-3)
    out, mask = ps.expected_attention(mode="ref")
    assert mask.all()
    assert_context_close(out, GOLDEN[f"{name}_context"])


def test_reference_itself_is_within_the_stated_tolerance_of_fp32():
    # how far the reference's bf16 materialisation sits from exact arithmetic on the same inputs
    seed, lengths, rw = DECODE_CASES["dec_b"]
    exp = scenario.DecodeScenario(seed=seed, lengths=lengths, random_weights=rw).expected()
    m = oracle.error_metrics(oracle.bf16_to_f32(GOLDEN["dec_b_context"]), exp["out_fp32"])
    assert m["max_abs"] <= 2e-2 and m["mean_rel"] <= 1e-2, m
