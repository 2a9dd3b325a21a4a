"""GPU parity of the many-row projections (the prefill loop's linear_generic, launch_add and launch_swiglu,
devices/rtx4090-24g/qwen3_tts_1_7b.cu:16730-16860) against the double-precision oracle, under the bf16 tolerance used
for the decode-time projections (max-abs 2e-2, mean-relative 1e-2), and against the decode-time kernels on the same
rows: both accumulate in fp32, so they may differ by a last bf16 bit in a small fraction of the outputs only."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import prefill_projection_cases as cases
import scenario

pytestmark = pytest.mark.gpu
TOL_MAX_ABS = 2e-2
TOL_MEAN_REL = 1e-2


def engine(qm):
    return qm.TalkerAttention(layers=1, num_pages=1, max_positions=8)


def dev(bits):
    import torch

    return scenario._bf16_tensor(torch, bits)


def close(got_bits, want_bits, scale=1.0):
    m = oracle.error_metrics(oracle.bf16_to_f32(got_bits), oracle.bf16_to_f32(want_bits))
    assert m["max_abs"] <= TOL_MAX_ABS * scale and m["mean_rel"] <= TOL_MEAN_REL, m
    return m


# row tails (1, 130, 257), column tails (64, 320 = 256 + 64, 384 = 256 + 128), one and many K chunks, and a case
# with more output tiles (16 x 16) than SMs so that every CTA walks several tiles through both accumulators
@pytest.mark.parametrize("rows,out_features,in_features", [(1, 64, 64), (130, 320, 128), (257, 384, 2048),
                                                           (300, 2048, 2048), (1000, 1024, 6144), (2000, 4096, 2048)])
def test_linear_rows_matches_double_precision_oracle(qm, rows, out_features, in_features):
    import torch

    x = oracle.normal_bf16(41 + rows, (rows, in_features))
    w = oracle.scaled_normal_bf16(42 + rows, (out_features, in_features), 0.02)
    bias = oracle.scaled_normal_bf16(43, (out_features,), 0.1)
    residual = oracle.normal_bf16(44, (rows, out_features))
    eng = engine(qm)
    try:
        plain = scenario._bits(eng.linear_generic(dev(x), dev(w)))
        full = scenario._bits(eng.linear_generic(dev(x), dev(w), dev(bias), dev(residual)))
        torch.cuda.synchronize()
        assert eng.status() == 0
        close(plain, oracle.linear(x, w, mode="f64"), scale=max(1.0, (in_features / 2048) ** 0.5))
        close(full, oracle.linear(x, w, bias, residual, mode="f64"), scale=2.0)
        again = scenario._bits(eng.linear_generic(dev(x), dev(w)))
        assert np.array_equal(plain, again)
    finally:
        eng.close()


@pytest.mark.parametrize("rows,hidden,intermediate", [(129, 128, 64), (200, 2048, 320), (500, 2048, 6144)])
def test_gate_up_swiglu_rows_matches_double_precision_oracle(qm, rows, hidden, intermediate):
    import torch

    x = oracle.normal_bf16(51 + rows, (rows, hidden))
    gate = oracle.scaled_normal_bf16(52, (intermediate, hidden), 0.02)
    up = oracle.scaled_normal_bf16(53, (intermediate, hidden), 0.02)
    eng = engine(qm)
    try:
        got = scenario._bits(eng.gate_up_swiglu_rows(dev(x), dev(gate), dev(up)))
        torch.cuda.synchronize()
        assert eng.status() == 0
        want = oracle.gate_up_swiglu(x, gate, up, mode="f64")
        # millions of outputs: allow the one-ulp flip of the largest bf16 outputs (an ulp is 2^-7 of the value or less)
        largest = float(np.max(np.abs(oracle.bf16_to_f32(want))))
        close(got, want, scale=max(1.0, largest * 2.0 ** -7 / TOL_MAX_ABS))
    finally:
        eng.close()


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_against_reference_prefill_kernel_outputs(qm, name):
    """The reference's own linear_bf16 / launch_add / launch_swiglu outputs on the same inputs (golden file made on a
    B200): the tensor-core accumulation order differs from the reference's 32-lane sums, so the comparison is the
    bf16 tolerance, and the fraction of outputs that differ at all stays small."""
    import torch
    from pathlib import Path

    golden = np.load(Path(__file__).resolve().parent / "golden" / "reference_prefill_projection_golden.npz")
    c = cases.ProjectionCase(*cases.CASES[name])
    eng = engine(qm)
    try:
        plain = scenario._bits(eng.linear_generic(dev(c.x), dev(c.w)))
        full = scenario._bits(eng.linear_generic(dev(c.x), dev(c.w), dev(c.bias), dev(c.residual)))
        act = scenario._bits(eng.gate_up_swiglu_rows(dev(c.x), dev(c.w), dev(c.up_w)))
        torch.cuda.synchronize()
        assert eng.status() == 0
        for got, key in ((plain, "linear"), (full, "linear_bias_residual"), (act, "swiglu")):
            want = golden[f"{name}_{key}"]
            close(got, want, scale=2.0)
            assert (got != want).mean() <= 5e-3, (key, (got != want).mean())
    finally:
        eng.close()


def test_many_row_and_decode_time_kernels_agree(qm):
    """The same 64 rows through both kernels: equal up to a last bf16 bit in a small fraction of the outputs."""
    import torch

    rows, hidden, out_features = 64, 2048, 1024
    x = oracle.normal_bf16(61, (rows, hidden))
    w = oracle.scaled_normal_bf16(62, (out_features, hidden), 0.02)
    bias = oracle.scaled_normal_bf16(63, (out_features,), 0.1)
    eng = engine(qm)
    try:
        a = oracle.bf16_to_f32(scenario._bits(eng.linear_generic(dev(x), dev(w), dev(bias))))
        b = oracle.bf16_to_f32(scenario._bits(eng.launch_linear_m1(dev(x), dev(w), dev(bias))))
        torch.cuda.synchronize()
        assert eng.status() == 0
        differing = np.mean(a != b)
        assert differing < 0.05, differing
        assert np.max(np.abs(a - b)) <= 2.0 ** -7 * max(1.0, float(np.max(np.abs(a))))
    finally:
        eng.close()


def test_rows_inside_a_partial_tile_are_left_alone(qm):
    """Rows past `rows` in the last 128-row tile and columns past `out_features` are never written."""
    import torch

    rows, hidden, out_features = 70, 128, 64
    x = dev(oracle.normal_bf16(71, (rows, hidden)))
    w = dev(oracle.scaled_normal_bf16(72, (out_features, hidden), 0.02))
    eng = engine(qm)
    try:
        out = torch.full((rows + 58, out_features), 7.0, dtype=torch.bfloat16, device="cuda")
        eng.linear_generic(x, w, out=out[:rows])
        torch.cuda.synchronize()
        assert eng.status() == 0
        assert bool((out[rows:] == 7.0).all())
    finally:
        eng.close()


def test_argument_errors(qm):
    import torch

    eng = engine(qm)
    try:
        def z(*shape):
            return torch.zeros(*shape, dtype=torch.bfloat16, device="cuda")

        with pytest.raises(qm.QmError) as e:
            eng.linear_generic(z(200, 128), z(100, 128))            # output width not a multiple of 64
        assert e.value.code == qm.QM_EINVAL
        with pytest.raises(qm.QmError) as e:
            eng.linear_generic(z(200, 100), z(64, 100))             # reduction width not a multiple of 64
        assert e.value.code == qm.QM_EINVAL
        with pytest.raises(qm.QmError) as e:
            eng.gate_up_swiglu_rows(z(200, 128), z(96, 128), z(96, 128))
        assert e.value.code == qm.QM_EINVAL
        assert eng.linear_generic(z(0, 128), z(64, 128)).shape == (0, 64)      # no rows: nothing to do
    finally:
        eng.close()
