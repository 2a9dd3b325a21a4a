"""Decode attention through the entry point that allocates nothing.

Some hosts of this library may not allocate device memory on the decode path: a resident serving loop that
budgeted its memory at start-up and must not trigger the device-wide synchronisation that cudaMalloc / cudaFree
imply (it would stall the audio decoder running on a second stream), or an engine whose own allocator already
owns the whole GPU.  qm_decode_attention_static serves them from a scratch array that is part of the library.

The check: on the same inputs it must give what qm_decode_attention gives with caller-provided workspace, on two
calls in a row with different batches (the second call finds the first call's leftovers in the shared scratch).
This file is collected last so that a run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu

TOL_MAX_ABS = 2e-2      # the bf16 tolerance the other attention tests use
TOL_MEAN_REL = 1e-2


def run_both(qm, sc):
    import torch

    eng = qm.TalkerAttention(layers=1, num_pages=sc.num_pages, q_heads=sc.q_heads, kv_heads=sc.kv_heads,
                             max_positions=sc.max_pos)
    try:
        kp, vp = sc.pools()
        kview, vview = eng.pool_view(0)
        kview.copy_(scenario._bf16_tensor(torch, kp))
        vview.copy_(scenario._bf16_tensor(torch, vp))
        q, k, v = (scenario._bf16_tensor(torch, x) for x in (sc.q, sc.k, sc.v))
        qw, kw = scenario._bf16_tensor(torch, sc.q_w), scenario._bf16_tensor(torch, sc.k_w)
        positions = torch.from_numpy(sc.lengths).cuda()
        page_table = torch.from_numpy(np.maximum(sc.page_table, 0)).cuda()
        seq_lens = torch.from_numpy(sc.lengths + 1).cuda()
        q_rot = eng.launch_qk_norm_rope_cache_m1(0, q, k, v, qw, kw, positions, page_table)
        with_workspace = eng.launch_attention(0, q_rot, seq_lens, page_table)
        out = torch.empty_like(q_rot)          # the caller's output buffer, allocated before the call under test
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        builtin_scratch = eng.launch_attention_static(0, q_rot, seq_lens, page_table, out=out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert eng.status() == 0
        return scenario._bits(with_workspace), scenario._bits(builtin_scratch)
    finally:
        eng.close()


def test_static_scratch_entry_point_matches_the_workspace_one_twice_in_a_row(qm):
    first = scenario.DecodeScenario(seed=31, lengths=[3000, 40, 700, 64, 1999, 5], random_weights=True)
    second = scenario.DecodeScenario(seed=32, lengths=list(oracle.uniform_int(77, 0, 900, 64)))
    for sc in (first, second):
        want_bits, got_bits = run_both(qm, sc)
        m = oracle.error_metrics(oracle.bf16_to_f32(got_bits), oracle.bf16_to_f32(want_bits))
        assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m
        # same kernels, same split, same fold order: the bits agree as well
        assert np.array_equal(got_bits, want_bits)
        # and both sit within tolerance of exact arithmetic
        m = oracle.error_metrics(oracle.bf16_to_f32(got_bits), sc.expected()["out_fp32"])
        assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m


def test_static_scratch_entry_point_rejects_batches_beyond_its_limit(qm):
    import torch

    eng = qm.TalkerAttention(layers=1, num_pages=4, max_positions=64)
    try:
        q_rot = torch.zeros(65, 16, 128, device="cuda", dtype=torch.bfloat16)
        lens = torch.ones(65, dtype=torch.int32, device="cuda")
        table = torch.zeros((65, 1), dtype=torch.int32, device="cuda")
        with pytest.raises(qm.QmError) as err:
            eng.launch_attention_static(0, q_rot, lens, table)
        assert err.value.code == qm.QM_ECAPACITY
        assert "at most 64 streams" in str(err.value)
    finally:
        eng.close()
