"""The library's kernels on the code predictor's shapes against the REFERENCE's own predictor kernels
(tests/golden/reference_predictor_golden.npz; 17.cu:12063-12830), one kernel at a time: bit for bit where the
arithmetic is element-wise or keeps the reference's reduction order (head norm + RoPE + append, residual add,
post-norm), under the path's tolerance (max-abs 2e-2, mean-relative 1e-2) where the tensor cores or the fp32 softmax
sum in another order (projections, SwiGLU, attention)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import predictor_cases as pc
import scenario

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_predictor_golden.npz")
TOL_MAX_ABS, TOL_MEAN_REL = 2e-2, 1e-2


def dev(bits):
    import torch

    return scenario._bf16_tensor(torch, np.ascontiguousarray(bits))


def close(got_bits, want_bits, scale=1.0):
    m = oracle.error_metrics(oracle.bf16_to_f32(got_bits), oracle.bf16_to_f32(want_bits))
    assert m["max_abs"] <= TOL_MAX_ABS * scale and m["mean_rel"] <= TOL_MEAN_REL, m


def nearly_identical(got, want, max_fraction=2e-3):
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -5, diff.max()
    assert (got != want).mean() <= max_fraction, (got != want).mean()


@pytest.mark.parametrize("seed", pc.SEEDS)
def test_projections_norms_and_swiglu_against_the_predictor_kernels(qm, seed):
    import torch

    c, name = pc.PredictorCase(seed), f"p{seed}"
    eng = qm.TalkerAttention(layers=1, num_pages=1, max_positions=16)
    try:
        x = dev(c.x.reshape(1, -1))
        q, k, v = eng.launch_qkv_m1(x, dev(c.q_w), dev(c.k_w), dev(c.v_w))
        # outputs are O(1): the tolerance is scaled to a bf16 ulp at that magnitude, as in the talker layer tests
        close(scenario._bits(q)[0], GOLDEN[f"{name}_q"], scale=2.0)
        close(scenario._bits(k)[0], GOLDEN[f"{name}_k"], scale=2.0)
        close(scenario._bits(v)[0], GOLDEN[f"{name}_v"], scale=2.0)
        o = eng.launch_linear_m1(dev(c.context.reshape(1, -1)), dev(c.o_w))
        close(scenario._bits(o)[0], GOLDEN[f"{name}_o"], scale=2.0)
        down = eng.launch_linear_m1(dev(c.act.reshape(1, -1)), dev(c.down_w), residual=dev(c.residual.reshape(1, -1)))
        close(scenario._bits(down)[0], GOLDEN[f"{name}_down"], scale=2.0)
        res, nrm = eng.launch_add_postnorm_m1(x, dev(c.attention.reshape(1, -1)), dev(c.post_norm_w))
        act = eng.launch_gate_up_swiglu_m1(x, dev(c.gate_w), dev(c.up_w))
        torch.cuda.synchronize()
        assert eng.status() == 0
        assert np.array_equal(scenario._bits(res)[0], GOLDEN[f"{name}_residual"])
        nearly_identical(scenario._bits(nrm)[0], GOLDEN[f"{name}_postnorm"])
        close(scenario._bits(act)[0], GOLDEN[f"{name}_swiglu"], scale=2.0)
    finally:
        eng.close()


@pytest.mark.parametrize("seed", pc.SEEDS)
@pytest.mark.parametrize("pos", pc.POSITIONS)
def test_append_and_short_context_attention_against_the_predictor_kernels(qm, seed, pos):
    """The predictor's 16 positions fit one page: the two-launch path and the fused step both take the
    short-context kernel."""
    import torch

    c, name = pc.PredictorCase(seed), f"p{seed}_pos{pos}"
    for fused in (False, True):
        eng = qm.TalkerAttention(layers=1, num_pages=1, max_positions=pc.MAX_CACHE)
        try:
            kc, vc = c.caches_before(pos)
            kpool = np.zeros((1, pc.HKV, 64, pc.D), dtype=np.uint16)
            vpool = np.zeros_like(kpool)
            kpool[0, :, :pc.MAX_CACHE], vpool[0, :, :pc.MAX_CACHE] = kc, vc
            kview, vview = eng.pool_view(0)
            kview.copy_(dev(kpool))
            vview.copy_(dev(vpool))
            table = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
            positions = torch.tensor([pos], dtype=torch.int32, device="cuda")
            q, k, v = dev(c.q[None]), dev(c.k[None]), dev(c.v[None])
            if fused:
                ctx = eng.decode_step(0, q, k, v, dev(c.q_norm_w), dev(c.k_norm_w), positions, table)
            else:
                q_rot = eng.launch_qk_norm_rope_cache_m1(0, q, k, v, dev(c.q_norm_w), dev(c.k_norm_w), positions, table)
                ctx = eng.launch_attention(0, q_rot, positions + 1, table)
                assert np.array_equal(scenario._bits(q_rot)[0], GOLDEN[f"{name}_q_rot"])
            torch.cuda.synchronize()
            assert eng.status() == 0
            assert np.array_equal(scenario._bits(kview)[0, :, pos], GOLDEN[f"{name}_k_row"])
            assert np.array_equal(scenario._bits(vview)[0, :, pos], GOLDEN[f"{name}_v_row"])
            close(scenario._bits(ctx)[0], GOLDEN[f"{name}_context"])
        finally:
            eng.close()
