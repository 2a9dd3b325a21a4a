"""The one-launch decode step (qm_decode_step) against the two-call path it replaces.

Same inputs, fresh pools: the context bits and every byte of both pools must be equal, and the result must sit
within the stated bf16 tolerance of the fp32 oracle."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu
TOL_MAX_ABS = 2e-2
TOL_MEAN_REL = 1e-2


def run_fused(qm, sc):
    import torch

    tb = scenario._bf16_tensor
    eng = qm.TalkerAttention(layers=1, num_pages=sc.num_pages, q_heads=sc.q_heads, kv_heads=sc.kv_heads,
                             max_positions=sc.max_pos)
    try:
        kp, vp = sc.pools()
        kview, vview = eng.pool_view(0)
        kview.copy_(tb(torch, kp))
        vview.copy_(tb(torch, vp))
        out = eng.decode_step(0, tb(torch, sc.q), tb(torch, sc.k), tb(torch, sc.v), tb(torch, sc.q_w), tb(torch, sc.k_w),
                              torch.from_numpy(sc.lengths).cuda(), torch.from_numpy(np.maximum(sc.page_table, 0)).cuda())
        torch.cuda.synchronize()
        assert eng.status() == 0
        return scenario._bits(out), scenario._bits(kview), scenario._bits(vview)
    finally:
        eng.close()


@pytest.mark.parametrize("lengths,heads", [([512], (16, 8)), ([0, 1, 63, 64, 65, 127, 128], (16, 8)),
                                           ([9000, 3, 4100, 700], (16, 8)), ([5] * 200 + [130] * 9, (16, 8)),
                                           ([0, 1, 15, 16, 31, 40, 62, 63, 7, 33], (16, 8)),    # one page per stream: short-context kernel
                                           ([2, 63], (4, 2)),
                                           ([100, 257], (4, 2))])
def test_fused_step_equals_append_then_attention(qm, lengths, heads):
    sc = scenario.DecodeScenario(seed=70 + len(lengths), lengths=lengths, q_heads=heads[0], kv_heads=heads[1],
                                 random_weights=True)
    out, kpool, vpool = run_fused(qm, sc)
    two = scenario.run_decode_on_gpu(qm, sc)
    assert np.array_equal(kpool, two["key_pool"]), "fused step wrote different K bits"
    assert np.array_equal(vpool, two["value_pool"]), "fused step wrote different V bits"
    assert np.array_equal(out, two["out"]), "fused step context differs from the two-call path"
    m = oracle.error_metrics(oracle.bf16_to_f32(out), sc.expected()["out_fp32"])
    assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m


def test_fused_step_ragged_batch_of_64(qm):
    lengths = oracle.uniform_int(4242, 0, 1200, 64)
    sc = scenario.DecodeScenario(seed=5, lengths=lengths)
    out, _, _ = run_fused(qm, sc)
    two = scenario.run_decode_on_gpu(qm, sc)
    assert np.array_equal(out, two["out"])
