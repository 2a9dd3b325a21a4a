"""GPU parity of the decode step: fused norm + RoPE + paged append, split-KV attention, partial + combine.

Everything goes through the C ABI (ctypes).  Bit-exact where the work is integer/byte (V rows, page
indexing, untouched pool bytes); the roped K/Q rows keep the reference's five roundings and may differ
from the CPU oracle by one bf16 ulp where the device rsqrtf differs from 1/sqrtf (the count is bounded
below); attention is compared with the fp32 oracle under the stated bf16 tolerance.
"""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu

TOL_MAX_ABS = 2e-2
TOL_MEAN_REL = 1e-2
MAX_ULP_MISMATCH_FRACTION = 0.002  # roped rows: share of elements allowed to differ from the CPU oracle


def ulp_distance(a, b):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + (x & 0x7FFF))
    return np.abs(key(a) - key(b))


def check_roped(got, want):
    # device rsqrtf vs the oracle's 1/sqrtf flips the first rounding of a few rows; after RoPE's a*cos + b*sin
    # the flipped ulp is an absolute error of at most one ulp of the normalised value (|x| < 8 -> 2^-5), which
    # near a cancellation can be many ulps of the small result.  Exact equality with the reference kernels' own
    # bits is asserted in test_golden_gpu.py.
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -5, diff.max()
    frac = float((got != want).mean())
    assert frac <= MAX_ULP_MISMATCH_FRACTION, f"{frac:.4f} of elements differ"
    return frac


def check_step(qm, sc):
    got = scenario.run_decode_on_gpu(qm, sc)
    want = sc.expected()
    assert got["status"] == 0
    # RoPE table: same host recipe -> identical bits
    cos, sin = oracle.make_rope(sc.max_pos)
    assert np.array_equal(got["rope_cos"], cos) and np.array_equal(got["rope_sin"], sin)
    # append: V rows and page indexing bit-exact
    assert np.array_equal(got["value_pool_new_rows"], want["value_rows"])
    check_roped(got["q_rot"], want["q_rot"])
    check_roped(got["key_pool_new_rows"], want["key_rows"])
    # gather through the page table == reference layout, and nothing else in the pool moved
    kp0, vp0 = sc.pools()
    for s in range(sc.batch):
        n = int(sc.lengths[s])
        gathered_v = oracle.gather_paged(got["value_pool"], sc.page_table[s], n + 1, sc.max_cache)
        assert np.array_equal(gathered_v[:, :n + 1], want["value_caches"][s][:, :n + 1])
        gathered_k = oracle.gather_paged(got["key_pool"], sc.page_table[s], n, sc.max_cache)
        assert np.array_equal(gathered_k[:, :n], want["key_caches"][s][:, :n])
    changed_v = (got["value_pool"] != vp0).any(axis=3)
    expect_changed = np.zeros_like(changed_v)
    for s in range(sc.batch):
        t = int(sc.lengths[s])
        expect_changed[sc.page_table[s, t >> 6], :, t & 63] = True
    assert not (changed_v & ~expect_changed).any(), "append touched rows it does not own"
    # attention vs fp32 oracle
    m = oracle.error_metrics(oracle.bf16_to_f32(got["out"]), want["out_fp32"])
    assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m
    # partial + combine must agree with the direct path (same fp32 state, one rounding)
    m2 = oracle.error_metrics(oracle.bf16_to_f32(got["out_from_partial"]), oracle.bf16_to_f32(got["out"]))
    assert m2["max_abs"] <= 2.0 ** -7, m2
    # and the partial state itself: o / l is the fp32 result
    p = got["partial"]
    recon = p[:, :, 2:] / p[:, :, 1:2]
    m3 = oracle.error_metrics(recon, want["out_fp32"])
    assert m3["max_abs"] <= 2e-3, m3
    return m


def test_config1_single_stream_512(qm):
    m = check_step(qm, scenario.DecodeScenario(seed=0, lengths=[512]))
    print("config1", m)


@pytest.mark.parametrize("length", [0, 1, 2, 62, 63, 64, 65, 126, 127, 128, 129, 191, 192])
def test_page_boundaries(qm, length):
    check_step(qm, scenario.DecodeScenario(seed=20 + length, lengths=[length]))


def test_ragged_batch_random_weights(qm):
    lengths = oracle.uniform_int(1001, 0, 700, 24)
    check_step(qm, scenario.DecodeScenario(seed=1, lengths=lengths, random_weights=True))


def test_long_stream_spans_many_ctas(qm):
    check_step(qm, scenario.DecodeScenario(seed=6, lengths=[9000, 3, 4100]))


def test_many_short_streams(qm):
    check_step(qm, scenario.DecodeScenario(seed=8, lengths=[5] * 300 + [130] * 20))


def test_other_head_counts(qm):
    check_step(qm, scenario.DecodeScenario(seed=12, lengths=[100, 257], q_heads=4, kv_heads=2))


def test_deterministic_across_runs(qm):
    sc = scenario.DecodeScenario(seed=13, lengths=[2000, 77, 640, 1500])
    a = scenario.run_decode_on_gpu(qm, sc)
    b = scenario.run_decode_on_gpu(qm, sc)
    assert np.array_equal(a["out"], b["out"]) and np.array_equal(a["key_pool"], b["key_pool"])


def test_zero_length_stream_gives_zero_row(qm):
    import torch

    eng = qm.TalkerAttention(layers=1, num_pages=4, max_positions=64)
    q_rot = torch.randn(2, 16, 128, device="cuda").to(torch.bfloat16)
    seq_lens = torch.tensor([0, 0], dtype=torch.int32, device="cuda")
    table = torch.zeros((2, 1), dtype=torch.int32, device="cuda")
    out = eng.launch_attention(0, q_rot, seq_lens, table)
    torch.cuda.synchronize()
    assert not out.float().abs().max().item()
    eng.close()


def test_bad_page_and_position_set_status_bits(qm):
    import torch

    eng = qm.TalkerAttention(layers=1, num_pages=4, max_positions=256)
    q = torch.randn(2, 16, 128, device="cuda").to(torch.bfloat16)
    kv = torch.randn(2, 8, 128, device="cuda").to(torch.bfloat16)
    w = torch.ones(128, device="cuda", dtype=torch.bfloat16)
    table = torch.tensor([[0, 99], [1, 2]], dtype=torch.int32, device="cuda")   # page 99 is outside the pool
    positions = torch.tensor([70, 200], dtype=torch.int32, device="cuda")       # 200 >= 2 pages * 64
    kbefore = eng.pool_view(0)[0].clone()
    eng.launch_qk_norm_rope_cache_m1(0, q, kv, kv, w, w, positions, table)
    bits = eng.status()
    assert bits & qm.DEVSTAT_BAD_PAGE and bits & qm.DEVSTAT_BAD_POS
    assert torch.equal(kbefore, eng.pool_view(0)[0]), "a rejected row must not be written"
    assert eng.status() == 0   # reading clears
    eng.close()


def test_argument_validation_on_gpu(qm):
    import torch

    eng = qm.TalkerAttention(layers=2, num_pages=4, max_positions=64)
    q_rot = torch.zeros(1, 16, 128, device="cuda", dtype=torch.bfloat16)
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    table = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    with pytest.raises(qm.QmError) as e:
        eng.launch_attention(5, q_rot, lens, table)
    assert e.value.code == qm.QM_EINVAL
    eng.q_heads = 24
    with pytest.raises(qm.QmError):
        eng.launch_attention(0, torch.zeros(1, 24, 128, device="cuda", dtype=torch.bfloat16), lens, table)
    eng.close()


def test_reset_request_zeroes_the_pool(qm):
    import torch

    eng = qm.TalkerAttention(layers=2, num_pages=3, max_positions=64)
    for layer in range(2):
        k, v = eng.pool_view(layer)
        k.fill_(1.0)
        v.fill_(2.0)
    eng.reset_request()
    for layer in range(2):
        k, v = eng.pool_view(layer)
        assert not k.view(torch.int16).any().item() and not v.view(torch.int16).any().item()
    eng.close()


def test_batch_larger_than_one_launch_chunk(qm):
    # more streams than one launch takes (256): the host splits the batch into several launches that share the workspace
    lengths = [int(x) for x in oracle.uniform_int(555, 0, 150, 700)]
    check_step(qm, scenario.DecodeScenario(seed=14, lengths=lengths))


def test_lengths_written_by_the_launch_just_before(qm):
    """The decode kernel works out its unit partition before its dependency wait and keeps it only if the lengths
    still hold afterwards.  Here the launch immediately before it (qm_embedding_gather, which lets its successor
    start early) overwrites seq_lens, so the early guess may be made from the OLD lengths; the result must be the
    one for the NEW lengths, bit for bit the same as when the lengths were in place all along."""
    import torch

    sc = scenario.DecodeScenario(seed=21, lengths=[300, 17, 129, 64, 1000, 5, 640, 77])
    b = sc.batch
    eng = qm.TalkerAttention(layers=1, num_pages=sc.num_pages, q_heads=sc.q_heads, kv_heads=sc.kv_heads, max_positions=sc.max_pos)
    try:
        tb = scenario._bf16_tensor
        kp, vp = sc.pools()
        kview, vview = eng.pool_view(0)
        kview.copy_(tb(torch, kp))
        vview.copy_(tb(torch, vp))
        page_table = torch.from_numpy(np.maximum(sc.page_table, 0)).cuda()
        positions = torch.from_numpy(sc.lengths).cuda()
        q_rot = eng.launch_qk_norm_rope_cache_m1(0, tb(torch, sc.q), tb(torch, sc.k), tb(torch, sc.v), tb(torch, sc.q_w),
                                                 tb(torch, sc.k_w), positions, page_table)
        new_lens = torch.from_numpy(sc.lengths + 1).cuda()
        want = eng.launch_attention(0, q_rot, new_lens, page_table).clone()
        # the "table" holds two rows of raw bytes: the new lengths and a set of much shorter old ones
        old_lens = torch.clamp(new_lens // 3, min=1)
        table = torch.stack([new_lens, old_lens]).view(torch.bfloat16)            # [2][2 * b] bf16
        seq_lens = torch.empty(b, dtype=torch.int32, device="cuda")
        rows = torch.tensor([[1], [0]], dtype=torch.int32, device="cuda")
        for _ in range(20):
            eng.embedding_gather(table, rows[0], out=seq_lens.view(torch.bfloat16).view(1, 2 * b))   # old lengths
            torch.cuda.synchronize()
            eng.embedding_gather(table, rows[1], out=seq_lens.view(torch.bfloat16).view(1, 2 * b))   # new, just in time
            got = eng.launch_attention(0, q_rot, seq_lens, page_table)
            assert torch.equal(got, want)
        assert eng.status() == 0
    finally:
        eng.close()


def test_short_contexts_one_page_per_stream(qm):
    """Every stream within one page: the dedicated short-context kernel (one CTA per stream and KV head) serves the
    call - same checks as any other step, including the partial + combine path and an empty stream."""
    check_step(qm, scenario.DecodeScenario(seed=31, lengths=[0, 1, 5, 16, 17, 33, 62, 63, 40, 2, 31, 32]))
    check_step(qm, scenario.DecodeScenario(seed=32, lengths=[63] * 70, random_weights=True))
