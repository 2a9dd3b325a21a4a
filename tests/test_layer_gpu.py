"""GPU parity of the non-attention operators of the talker layer (rows of tokens instead of the reference's M = 1).

RMSNorm and add+post-norm keep the reference's reduction order and roundings: compared with the oracle's
bit-faithful mode (only the device rsqrtf may flip a last bit).  The projections accumulate on the tensor cores in
fp32 in a different order than the reference's lane-strided chains: compared with the double-precision oracle under
the bf16 tolerance used everywhere else (max-abs 2e-2, mean-relative 1e-2)."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import layer_cases
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


def nearly_identical(got, want, max_fraction=2e-3):
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -5, diff.max()
    assert (got != want).mean() <= max_fraction, (got != want).mean()


@pytest.mark.parametrize("name", sorted(layer_cases.CASES))
def test_norm_kernels_match_the_bit_faithful_oracle(qm, name):
    import torch

    seed, rows = layer_cases.CASES[name]
    c = layer_cases.LayerCase(seed, rows)
    eng = engine(qm)
    try:
        got = scenario._bits(eng.launch_rmsnorm(dev(c.x), dev(c.norm_w)))
        nearly_identical(got, oracle.rmsnorm(c.x, c.norm_w))
        res, nrm = eng.launch_add_postnorm_m1(dev(c.x), dev(c.attn), dev(c.norm_w))
        torch.cuda.synchronize()
        want_res, want_nrm = oracle.add_postnorm(c.x, c.attn, c.norm_w)
        assert np.array_equal(scenario._bits(res), want_res), "residual add is exact bf16 arithmetic"
        nearly_identical(scenario._bits(nrm), want_nrm)
    finally:
        eng.close()


@pytest.mark.parametrize("rows,dim", [(5, 2048), (300, 1024), (3, 4104)])
def test_vector_and_scalar_norm_paths_give_the_same_bits(qm, rows, dim):
    """16-byte aligned rows take the vector kernel, a view shifted by one element the scalar one: same bits."""
    import torch

    x = oracle.normal_bf16(201 + rows, (rows, dim))
    h = oracle.normal_bf16(202 + rows, (rows, dim))
    x[0, 5] = 0x7f80          # +inf: the row's outputs become NaN / 0 exactly as in the scalar kernel
    x[1, 7] = 0x7fc1          # a NaN with a payload
    h[2, 9] = 0xff80          # -inf in the residual branch only
    w = oracle.scaled_normal_bf16(203, (dim,), 0.5)
    eng = engine(qm)
    try:
        def shifted(bits):
            flat = torch.zeros(bits.size + 1, dtype=torch.bfloat16, device="cuda")
            view = flat[1:].view(bits.shape)
            view.copy_(dev(bits))
            return view

        aligned = scenario._bits(eng.launch_rmsnorm(dev(x), dev(w)))
        unaligned = scenario._bits(eng.launch_rmsnorm(shifted(x), dev(w), out=shifted(x)))
        assert np.array_equal(aligned, unaligned)
        res_a, nrm_a = eng.launch_add_postnorm_m1(dev(h), dev(x), dev(w))
        res_u, nrm_u = eng.launch_add_postnorm_m1(shifted(h), shifted(x), dev(w), residual=shifted(x), normalized=shifted(x))
        torch.cuda.synchronize()
        assert np.array_equal(scenario._bits(res_a), scenario._bits(res_u))
        assert np.array_equal(scenario._bits(nrm_a), scenario._bits(nrm_u))
        if rows > 3:      # the rows without non-finite values, against the bit-faithful oracle
            nearly_identical(aligned[3:], oracle.rmsnorm(x, w)[3:])
    finally:
        eng.close()


@pytest.mark.parametrize("rows,out_features,in_features", [(3, 384, 2048), (33, 384, 2048), (32, 4096, 2048),
                                                           (64, 2048, 6144), (1, 100, 64), (17, 3072, 2048)])
def test_projection_matches_double_precision_oracle(qm, rows, out_features, in_features):
    import torch

    x = oracle.normal_bf16(11 + rows, (rows, in_features))
    w = oracle.scaled_normal_bf16(12 + rows, (out_features, in_features), 0.02)
    bias = oracle.scaled_normal_bf16(13, (out_features,), 0.1)
    residual = oracle.normal_bf16(14, (rows, out_features))
    eng = engine(qm)
    try:
        plain = scenario._bits(eng.launch_linear_m1(dev(x), dev(w)))
        full = scenario._bits(eng.launch_linear_m1(dev(x), dev(w), dev(bias), dev(residual)))
        torch.cuda.synchronize()
        assert eng.status() == 0
        close(plain, oracle.linear(x, w, mode="f64"), scale=max(1.0, (in_features / 2048) ** 0.5))
        close(full, oracle.linear(x, w, bias, residual, mode="f64"), scale=2.0)
        # determinism: cluster-rank-ordered fold
        again = scenario._bits(eng.launch_linear_m1(dev(x), dev(w)))
        assert np.array_equal(plain, again)
    finally:
        eng.close()


@pytest.mark.parametrize("rows,hidden,intermediate", [(3, 2048, 320), (33, 2048, 320), (32, 2048, 6144), (5, 128, 70)])
def test_gate_up_swiglu_matches_double_precision_oracle(qm, rows, hidden, intermediate):
    import torch

    x = oracle.normal_bf16(21 + rows, (rows, hidden))
    gate = oracle.scaled_normal_bf16(22, (intermediate, hidden), 0.02)
    up = oracle.scaled_normal_bf16(23, (intermediate, hidden), 0.02)
    eng = engine(qm)
    try:
        got = scenario._bits(eng.launch_gate_up_swiglu_m1(dev(x), dev(gate), dev(up)))
        torch.cuda.synchronize()
        assert eng.status() == 0
        close(got, oracle.gate_up_swiglu(x, gate, up, mode="f64"))
    finally:
        eng.close()


def test_projection_argument_errors(qm):
    import torch

    eng = engine(qm)
    try:
        x = torch.zeros(65, 128, dtype=torch.bfloat16, device="cuda")
        w = torch.zeros(16, 128, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(qm.QmError) as e:
            eng.launch_linear_m1(x, w)
        assert e.value.code == qm.QM_ECAPACITY
        with pytest.raises(qm.QmError) as e:
            eng.launch_linear_m1(torch.zeros(2, 100, dtype=torch.bfloat16, device="cuda"),
                                 torch.zeros(16, 100, dtype=torch.bfloat16, device="cuda"))
        assert e.value.code == qm.QM_EINVAL
    finally:
        eng.close()


@pytest.mark.parametrize("name", sorted(layer_cases.CASES))
def test_against_reference_kernel_bits(qm, name):
    """Norm kernels must EQUAL the reference kernels' bits; projections sit within the bf16 tolerance of them."""
    import torch
    from pathlib import Path

    golden = np.load(Path(__file__).resolve().parent / "golden" / "reference_layer_golden.npz")
    seed, rows = layer_cases.CASES[name]
    c = layer_cases.LayerCase(seed, rows)
    eng = engine(qm)
    try:
        assert np.array_equal(scenario._bits(eng.launch_rmsnorm(dev(c.x), dev(c.norm_w))), golden[f"{name}_rmsnorm"])
        res, nrm = eng.launch_add_postnorm_m1(dev(c.x), dev(c.attn), dev(c.norm_w))
        assert np.array_equal(scenario._bits(res), golden[f"{name}_residual"])
        assert np.array_equal(scenario._bits(nrm), golden[f"{name}_postnorm"])
        close(scenario._bits(eng.launch_linear_m1(dev(c.x), dev(c.w))), golden[f"{name}_linear"])
        close(scenario._bits(eng.launch_linear_m1(dev(c.x), dev(c.w), dev(c.bias), dev(c.residual))),
              golden[f"{name}_linear_bias_residual"], scale=2.0)
        close(scenario._bits(eng.launch_gate_up_swiglu_m1(dev(c.x), dev(c.gate_w), dev(c.up_w))), golden[f"{name}_swiglu"])
        torch.cuda.synchronize()
    finally:
        eng.close()


def test_fused_qkv_projection_writes_three_outputs(qm):
    import torch

    rows, hidden, q_dim, kv_dim = 32, 2048, 2048, 1024
    x = oracle.normal_bf16(31, (rows, hidden))
    wq = oracle.scaled_normal_bf16(32, (q_dim, hidden), 0.02)
    wk = oracle.scaled_normal_bf16(33, (kv_dim, hidden), 0.02)
    wv = oracle.scaled_normal_bf16(34, (kv_dim, hidden), 0.02)
    bk = oracle.scaled_normal_bf16(35, (kv_dim,), 0.1)
    eng = engine(qm)
    try:
        q, k, v = eng.launch_qkv_m1(dev(x), dev(wq), dev(wk), dev(wv), k_bias=dev(bk))
        torch.cuda.synchronize()
        assert eng.status() == 0
        close(scenario._bits(q), oracle.linear(x, wq, mode="f64"))
        close(scenario._bits(k), oracle.linear(x, wk, bk, mode="f64"))
        close(scenario._bits(v), oracle.linear(x, wv, mode="f64"))
        # same bits as three separate projections
        assert np.array_equal(scenario._bits(q), scenario._bits(eng.launch_linear_m1(dev(x), dev(wq))))
    finally:
        eng.close()
