"""Pins the oracle's layer operators to the reference's own kernels (tests/golden/reference_layer_golden.npz,
produced on a B200 by tests/golden/make_reference_layer_golden.py).  RMSNorm, linear, residual add and SwiGLU agree
bit for bit on these cases; a differing last bit from libm vs device expf / rsqrtf would still be tolerated."""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import layer_cases

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_layer_golden.npz")


def nearly_identical(got, want, max_fraction=1e-3):
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -5 and (got != want).mean() <= max_fraction


@pytest.mark.parametrize("name", sorted(layer_cases.CASES))
def test_oracle_layer_operators_match_reference_kernels(name):
    seed, rows = layer_cases.CASES[name]
    c = layer_cases.LayerCase(seed, rows)
    nearly_identical(oracle.rmsnorm(c.x, c.norm_w), GOLDEN[f"{name}_rmsnorm"])
    assert np.array_equal(oracle.linear(c.x, c.w), GOLDEN[f"{name}_linear"])
    assert np.array_equal(oracle.linear(c.x, c.w, c.bias, c.residual), GOLDEN[f"{name}_linear_bias_residual"])
    res, nrm = oracle.add_postnorm(c.x, c.attn, c.norm_w)
    assert np.array_equal(res, GOLDEN[f"{name}_residual"])
    nearly_identical(nrm, GOLDEN[f"{name}_postnorm"])
    nearly_identical(oracle.gate_up_swiglu(c.x, c.gate_w, c.up_w), GOLDEN[f"{name}_swiglu"])


def test_double_precision_mode_is_close_to_reference_mode():
    c = layer_cases.LayerCase(303, 4)
    m = oracle.error_metrics(oracle.bf16_to_f32(oracle.linear(c.x, c.w, mode="f64")), oracle.bf16_to_f32(oracle.linear(c.x, c.w)))
    assert m["max_abs"] <= 2e-2 and m["mean_rel"] <= 1e-2, m
