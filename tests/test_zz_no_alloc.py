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
        out = torch.empty_like(q_rot)          # the caller's output buffer, allocated before the calls under test
        # A first call so that everything that happens once per process or device (loading the kernel image,
        # looking up the scratch array's address) is behind us; the second call is the one that is measured.
        eng.launch_attention_static(0, q_rot, seq_lens, page_table, out=out)
        torch.cuda.synchronize()
        # Free device memory as the driver counts it: a cudaMalloc inside the library would show up here, whereas
        # torch's own counters only see torch's allocator.
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        builtin_scratch = eng.launch_attention_static(0, q_rot, seq_lens, page_table, out=out)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, (free_before, free_after)
        assert torch.cuda.memory_allocated() == torch_before
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


def test_static_scratch_is_usable_again_after_a_reported_timeout_and_a_reset(qm):
    """A device-side wait that gives up may leave arrival counters behind in the shared scratch.  The recipe the
    header gives - read the status, reset the scratch, carry on - must leave the entry point correct."""
    import torch

    sc = scenario.DecodeScenario(seed=33, lengths=[2500, 130, 64, 900])
    eng = qm.TalkerAttention(layers=1, num_pages=sc.num_pages, max_positions=sc.max_pos)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        assert eng.lib.qm_selftest_wait_timeout(eng.pool, stream) == qm.QM_OK
        assert eng.status() == qm.DEVSTAT_TIMEOUT
        assert eng.lib.qm_decode_static_scratch_reset(eng.pool, stream) == qm.QM_OK
    finally:
        eng.close()
    want_bits, got_bits = run_both(qm, sc)
    assert np.array_equal(got_bits, want_bits)


def test_static_entry_points_need_the_pools_device_to_be_current(qm):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs a second GPU to make another device current")
    eng = qm.TalkerAttention(layers=1, num_pages=4, max_positions=64)
    try:
        with torch.cuda.device(1):
            assert eng.lib.qm_decode_static_scratch_reset(eng.pool, None) == qm.QM_EINVAL
    finally:
        eng.close()
