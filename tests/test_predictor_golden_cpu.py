"""Pins the oracle's operators to the reference's own CODE PREDICTOR kernels (17.cu:12063-12830) on the predictor's
shapes: tests/golden/reference_predictor_golden.npz holds what predictor_qkv_m1_fused_kernel,
predictor_qk_norm_rope_cache_m1_kernel, predictor_attention_gqa2_m1_kernel, predictor_linear_m1_fused_kernel,
predictor_add_postnorm_m1_kernel and predictor_gate_up_swiglu_m1_kernel produced on a B200
(tests/golden/make_reference_predictor_golden.py).  The restatements were written from the talker's kernels; this
shows they describe the predictor's kernels as well, so a predictor frame can be checked against their chain."""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import predictor_cases as pc

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_predictor_golden.npz")


def nearly_identical(got, want, max_fraction=2e-3):
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -5, diff.max()
    assert (got != want).mean() <= max_fraction, (got != want).mean()


@pytest.mark.parametrize("seed", pc.SEEDS)
def test_oracle_projections_and_norms_match_the_predictor_kernels(seed):
    c, name = pc.PredictorCase(seed), f"p{seed}"
    x1 = c.x.reshape(1, -1)
    assert np.array_equal(oracle.linear(x1, c.q_w)[0], GOLDEN[f"{name}_q"])
    assert np.array_equal(oracle.linear(x1, c.k_w)[0], GOLDEN[f"{name}_k"])
    assert np.array_equal(oracle.linear(x1, c.v_w)[0], GOLDEN[f"{name}_v"])
    assert np.array_equal(oracle.linear(c.context.reshape(1, -1), c.o_w)[0], GOLDEN[f"{name}_o"])
    assert np.array_equal(oracle.linear(c.act.reshape(1, -1), c.down_w, residual=c.residual.reshape(1, -1))[0], GOLDEN[f"{name}_down"])
    res, nrm = oracle.add_postnorm(x1, c.attention.reshape(1, -1), c.post_norm_w)
    assert np.array_equal(res[0], GOLDEN[f"{name}_residual"])
    nearly_identical(nrm[0], GOLDEN[f"{name}_postnorm"])
    nearly_identical(oracle.gate_up_swiglu(x1, c.gate_w, c.up_w)[0], GOLDEN[f"{name}_swiglu"])


@pytest.mark.parametrize("seed", pc.SEEDS)
@pytest.mark.parametrize("pos", pc.POSITIONS)
def test_oracle_attention_path_matches_the_predictor_kernels(seed, pos):
    c, name = pc.PredictorCase(seed), f"p{seed}_pos{pos}"
    kc, vc = c.caches_before(pos)
    q_rot = oracle.append(c.q[None], c.k[None], c.v[None], c.q_norm_w, c.k_norm_w, c.cos[pos:pos + 1], c.sin[pos:pos + 1], pos, kc, vc)[0]
    nearly_identical(q_rot, GOLDEN[f"{name}_q_rot"])
    nearly_identical(kc[:, pos], GOLDEN[f"{name}_k_row"])
    assert np.array_equal(vc[:, pos], GOLDEN[f"{name}_v_row"])
    # attention on the reference's own q_rot and K row, so that a last-bit difference above does not leak in
    kc[:, pos] = GOLDEN[f"{name}_k_row"]
    ctx = oracle.decode_attention(GOLDEN[f"{name}_q_rot"][None], [kc], [vc], [pos + 1], mode="ref")[0]
    nearly_identical(ctx, GOLDEN[f"{name}_context"], max_fraction=5e-3)
