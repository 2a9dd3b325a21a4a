"""Pins the oracle's double-precision projections to the reference's own prefill-loop kernels
(tests/golden/reference_prefill_projection_golden.npz: native_ops::linear_bf16, code_predictor::launch_add and
launch_swiglu run on a B200 by tests/golden/make_reference_prefill_projection_golden.py).  The reference sums each
dot product over 32 lanes in fp32, the oracle in double precision: a last bf16 bit may differ in a few outputs per
ten thousand, nothing more."""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import prefill_projection_cases as cases

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_prefill_projection_golden.npz")


def last_bit_only(got, want, max_fraction=1e-3):
    g, w = oracle.bf16_to_f32(got), oracle.bf16_to_f32(want)
    assert (got != want).mean() <= max_fraction, (got != want).mean()
    # one bf16 ulp of the output, or of an operand of the final sum / product (magnitudes up to 4 in these cases)
    assert np.all(np.abs(g - w) <= np.maximum(2.0 ** -7 * np.abs(w), 2.0 ** -5))


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_oracle_projections_match_reference_prefill_kernels(name):
    c = cases.ProjectionCase(*cases.CASES[name])
    last_bit_only(oracle.linear(c.x, c.w, mode="f64"), GOLDEN[f"{name}_linear"])
    last_bit_only(oracle.linear(c.x, c.w, c.bias, c.residual, mode="f64"), GOLDEN[f"{name}_linear_bias_residual"])
    last_bit_only(oracle.gate_up_swiglu(c.x, c.w, c.up_w, mode="f64"), GOLDEN[f"{name}_swiglu"])
