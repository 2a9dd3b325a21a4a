"""GPU parity of the prefill path: fused varlen norm + RoPE + paged append, then tcgen05 causal attention.

The append must equal the oracle's bit-faithful mode up to the rsqrtf ulp cases (and equals the reference
kernels' bits in test_golden_gpu.py); attention is compared with the fp32 oracle under the stated bf16 tolerance
(max-abs <= 2e-2, mean-relative <= 1e-2) and with the reference kernels' own output from the golden file.
"""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario
from golden.make_reference_golden import PREFILL_CASES

pytestmark = pytest.mark.gpu
TOL_MAX_ABS = 2e-2
TOL_MEAN_REL = 1e-2
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_kernels_golden.npz")


def ulp_distance(a, b):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + (x & 0x7FFF))
    return np.abs(key(a) - key(b))


def assert_roped_close(got, want):
    # device rsqrtf vs the oracle's 1/sqrtf flips the first rounding of a few rows; after RoPE's a*cos + b*sin
    # the flipped ulp is an absolute error of at most one ulp of the normalised value (|x| < 8 -> 2^-5)
    if got.size == 0:
        return
    diff = np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))
    assert diff.max() <= 2.0 ** -5, diff.max()
    assert (got != want).mean() <= 1e-3, (got != want).mean()


def check_append(ps, got):
    q_rot, kcs, vcs = ps.expected_append()
    assert_roped_close(got["q_rot"], q_rot)
    for s in range(ps.batch):
        n = int(ps.lengths[s])
        gk = oracle.gather_paged(got["key_pool"], ps.page_table[s], n, ps.max_cache)
        gv = oracle.gather_paged(got["value_pool"], ps.page_table[s], n, ps.max_cache)
        assert np.array_equal(gv[:, :n], vcs[s][:, :n]), "V rows / page indexing must be bit-exact"
        assert_roped_close(gk[:, :n], kcs[s][:, :n])


def check_prefill(qm, ps, rows_per_stream=None):
    got = scenario.run_prefill_on_gpu(qm, ps)
    assert got["status"] == 0
    check_append(ps, got)
    want, mask = ps.expected_attention(mode="fp32", rows_per_stream=rows_per_stream)
    m = oracle.error_metrics(oracle.bf16_to_f32(got["out"])[mask], want[mask])
    assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m
    return m, got


@pytest.mark.parametrize("lengths", [[70], [128], [129], [1], [1, 2, 3], [64, 65, 127], [300, 257, 64, 5]])
def test_small_sequences(qm, lengths):
    check_prefill(qm, scenario.PrefillScenario(seed=40 + len(lengths) + lengths[0], lengths=lengths, random_weights=True))


def test_unshuffled_pages_and_unit_weights(qm):
    check_prefill(qm, scenario.PrefillScenario(seed=3, lengths=[200, 131], shuffle_pages=False))


def test_one_long_sequence(qm):
    m, _ = check_prefill(qm, scenario.PrefillScenario(seed=2, lengths=[1500]))
    print("prefill L=1500", m)


def test_ragged_batch_sampled_rows(qm):
    # the config-3 shape at reduced lengths; the oracle checks the first and last 96 rows of every sequence
    lengths = [int(x) for x in oracle.uniform_int(2 * 1000 + 99, 1024, 3000, 4)]
    ps = scenario.PrefillScenario(seed=2, lengths=lengths)
    got = scenario.run_prefill_on_gpu(qm, ps)
    assert got["status"] == 0
    for part in ("head", "tail"):
        rows = {s: ((0, 96) if part == "head" else (n - 96, n)) for s, n in enumerate(lengths)}
        want, mask = ps.expected_attention(mode="fp32", rows_per_stream=rows)
        m = oracle.error_metrics(oracle.bf16_to_f32(got["out"])[mask], want[mask])
        assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, (part, m)


def test_empty_sequence_in_batch(qm):
    check_prefill(qm, scenario.PrefillScenario(seed=5, lengths=[0, 40, 0, 129]))


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_attention_against_reference_kernel_output(qm, name):
    seed, lengths, rw = PREFILL_CASES[name]
    ps = scenario.PrefillScenario(seed=seed, lengths=lengths, random_weights=rw)
    got = scenario.run_prefill_on_gpu(qm, ps)
    m = oracle.error_metrics(oracle.bf16_to_f32(got["out"]), oracle.bf16_to_f32(GOLDEN[f"{name}_context"]))
    assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m


def test_prefill_then_decode_share_the_cache(qm):
    """Prefill writes the pages, a decode step then attends over them plus its own token."""
    import torch

    ps = scenario.PrefillScenario(seed=9, lengths=[100, 63], spare_pages=4)
    q_rot, kcs, vcs = ps.expected_append()
    eng = qm.TalkerAttention(layers=1, num_pages=ps.num_pages, max_positions=256)
    try:
        tb = scenario._bf16_tensor
        cu = torch.from_numpy(ps.cu_seqlens).cuda()
        # give stream 1 (63 tokens) room for position 63: still page 0; stream 0 position 100: page 1
        table = torch.from_numpy(np.maximum(ps.page_table, 0)).cuda()
        eng.prefill_norm_rope_scatter(0, tb(torch, ps.q), tb(torch, ps.k), tb(torch, ps.v), tb(torch, ps.q_w),
                                      tb(torch, ps.k_w), cu, table)
        newq = oracle.normal_bf16(991, (2, 16, 128))
        newk = oracle.normal_bf16(992, (2, 8, 128))
        newv = oracle.normal_bf16(993, (2, 8, 128))
        positions = torch.from_numpy(ps.lengths).cuda()
        qr = eng.launch_qk_norm_rope_cache_m1(0, tb(torch, newq), tb(torch, newk), tb(torch, newv), tb(torch, ps.q_w),
                                              tb(torch, ps.k_w), positions, table)
        out = eng.launch_attention(0, qr, torch.from_numpy(ps.lengths + 1).cuda(), table)
        torch.cuda.synchronize()
        assert eng.status() == 0
        cos, sin = oracle.make_rope(256)
        want_rows = []
        for s in range(2):
            pos = int(ps.lengths[s])
            kc, vc = kcs[s].copy(), vcs[s].copy()
            qrs = oracle.append(newq[s:s + 1], newk[s:s + 1], newv[s:s + 1], ps.q_w, ps.k_w, cos[pos:pos + 1],
                                sin[pos:pos + 1], pos, kc, vc)
            want_rows.append(oracle.decode_attention(qrs, [kc], [vc], [pos + 1], mode="fp32")[0])
        m = oracle.error_metrics(oracle.bf16_to_f32(scenario._bits(out)), np.stack(want_rows))
        assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m
    finally:
        eng.close()


def test_second_chunk_attends_the_cache_of_the_first(qm):
    """Chunked prefill: rows of the second call start at position start_positions[s] and attend every cached key
    before them (the reference's cache_before, 17.cu:15832-15852)."""
    import torch

    lengths = [200, 77]
    first = [130, 64]                      # tokens of each sequence that go in with the first call
    ps = scenario.PrefillScenario(seed=17, lengths=lengths, random_weights=True, spare_pages=2)
    q_rot_all, kcs, vcs = ps.expected_append()
    tb = scenario._bf16_tensor
    eng = qm.TalkerAttention(layers=1, num_pages=ps.num_pages, max_positions=256)
    try:
        table = torch.from_numpy(np.maximum(ps.page_table, 0)).cuda()
        qw, kw = tb(torch, ps.q_w), tb(torch, ps.k_w)

        def rows(lo_hi):
            idx = np.concatenate([np.arange(ps.cu_seqlens[s] + a, ps.cu_seqlens[s] + b) for s, (a, b) in enumerate(lo_hi)])
            return idx

        for part, spans in (("first", [(0, first[0]), (0, first[1])]), ("second", [(first[0], lengths[0]), (first[1], lengths[1])])):
            idx = rows(spans)
            n = [b - a for a, b in spans]
            cu = torch.tensor(np.concatenate([[0], np.cumsum(n)]).astype(np.int32)).cuda()
            start = torch.tensor(np.array([a for a, _ in spans], dtype=np.int32)).cuda()
            q, k, v = (tb(torch, np.ascontiguousarray(x[idx])) for x in (ps.q, ps.k, ps.v))
            q_rot = eng.prefill_norm_rope_scatter(0, q, k, v, qw, kw, cu, table, start_positions=start)
            out = eng.launch_attention_prefill(0, q_rot, cu, table, max(n), start_positions=start)
            torch.cuda.synchronize()
            assert eng.status() == 0
            got = oracle.bf16_to_f32(scenario._bits(out))
            want = []
            for s, (a, b) in enumerate(spans):
                c0 = int(ps.cu_seqlens[s])
                res = oracle.prefill_attention(q_rot_all[c0 + a:c0 + b], kcs[s], vcs[s], b - a, cache_before=a, mode="fp32")
                want.append(res)
            m = oracle.error_metrics(got, np.concatenate(want))
            assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, (part, m)
    finally:
        eng.close()


def test_eight_rows_per_warp_equals_four_rows_per_warp(qm):
    """With 16 + 8 heads a warp of the append kernels takes eight head rows and reduces their sums of squares
    together; with 8 + 4 heads it takes four and reduces each on its own.  The same rows through both must give the same bits, non-finite rows and rows whose
    squares overflow included, and such a row must not leak into its seven neighbours."""
    big = scenario.PrefillScenario(41, [37, 5, 64], q_heads=16, kv_heads=8, random_weights=True)
    big.q[3, 2, 17] = 0x7F80            # +inf
    big.q[3, 5, 0] = 0x7FC1             # NaN with a payload
    big.q[9, 11, 127] = 0xFF80          # -inf
    big.q[20, 1, :] = 0x7F00            # 1.7e38: every square overflows
    big.k[3, 0, 64] = 0x7F80
    big.k[9, 3, 1] = 0xFFC0
    big.k[30, 2, 5] = 0x7E80            # one overflowing square in an otherwise ordinary row
    small = scenario.PrefillScenario(41, [37, 5, 64], q_heads=8, kv_heads=4, random_weights=True)
    small.q, small.k, small.v = (np.ascontiguousarray(x) for x in (big.q[:, :8], big.k[:, :4], big.v[:, :4]))
    small.q_w, small.k_w, small.page_table = big.q_w, big.k_w, big.page_table
    assert small.num_pages == big.num_pages
    got_big = scenario.run_prefill_on_gpu(qm, big, attention=False)
    got_small = scenario.run_prefill_on_gpu(qm, small, attention=False)
    assert got_big["status"] == 0 and got_small["status"] == 0
    assert np.array_equal(got_big["q_rot"][:, :8], got_small["q_rot"])
    kb = got_big["key_pool"].reshape(big.num_pages, 8, 64, 128)
    ks = got_small["key_pool"].reshape(big.num_pages, 4, 64, 128)
    vb = got_big["value_pool"].reshape(big.num_pages, 8, 64, 128)
    vs = got_small["value_pool"].reshape(big.num_pages, 4, 64, 128)
    assert np.array_equal(kb[:, :4], ks) and np.array_equal(vb[:, :4], vs)
    # the rows next to a non-finite one are ordinary numbers, and the heads the small run does not have agree with
    # the oracle like any other row
    finite_rows = np.ones(big.q.shape[:2], dtype=bool)
    for t, h in ((3, 2), (3, 5), (9, 11), (20, 1)):
        finite_rows[t, h] = False
    want_q, _, _ = big.expected_append()
    assert_roped_close(got_big["q_rot"][finite_rows], want_q[finite_rows])
    assert np.isfinite(oracle.bf16_to_f32(got_big["q_rot"][finite_rows])).all()


@pytest.mark.parametrize("lengths", [[150, 3, 77], [5192, 4730, 1554, 3417]])
def test_inputs_a_bulk_copy_cannot_read_take_the_one_shot_kernel_with_the_same_bits(qm, lengths):
    """Packed prompts go through the ring of bulk copies when q, k and v start on 16-byte boundaries; inputs that
    are only 8-byte aligned (the ABI's requirement) go through the one-shot kernel.  Same rows, same bits."""
    import torch

    ps = scenario.PrefillScenario(43, lengths, random_weights=True)      # the second case: 14 893 tokens, 4 prompts of the bench's 8
    aligned = scenario.run_prefill_on_gpu(qm, ps, attention=False)
    eng = qm.TalkerAttention(layers=1, num_pages=ps.num_pages, q_heads=ps.q_heads, kv_heads=ps.kv_heads,
                             max_positions=max(ps.max_pos, 1))
    try:
        def shifted(bits):
            flat = torch.zeros(bits.size + 4, dtype=torch.bfloat16, device="cuda")
            view = flat[4:].view(*bits.shape)            # starts 8 bytes after a 16-byte boundary
            view.copy_(scenario._bf16_tensor(torch, bits))
            assert view.data_ptr() % 16 == 8
            return view
        q, k, v = shifted(ps.q), shifted(ps.k), shifted(ps.v)
        qw, kw = scenario._bf16_tensor(torch, ps.q_w), scenario._bf16_tensor(torch, ps.k_w)
        cu = torch.from_numpy(ps.cu_seqlens).cuda()
        page_table = torch.from_numpy(np.maximum(ps.page_table, 0)).cuda()
        q_rot = eng.prefill_norm_rope_scatter(0, q, k, v, qw, kw, cu, page_table)
        torch.cuda.synchronize()
        kview, vview = eng.pool_view(0)
        assert eng.status() == 0
        assert np.array_equal(scenario._bits(q_rot), aligned["q_rot"])
        assert np.array_equal(scenario._bits(kview), aligned["key_pool"])
        assert np.array_equal(scenario._bits(vview), aligned["value_pool"])
    finally:
        eng.close()


def test_prefill_append_rejects_bad_pages_and_positions_without_writing(qm):
    """A page id outside the pool, a prompt longer than its page table and a position past the RoPE table set their
    status bits; the rows concerned are not written, every other row is."""
    import torch

    eng = qm.TalkerAttention(layers=1, num_pages=6, max_positions=160)
    try:
        lengths = [130, 70, 200]                       # stream 2 runs past the 160 RoPE rows
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)).cuda()
        total = int(sum(lengths))
        q = torch.randn(total, 16, 128, device="cuda").to(torch.bfloat16)
        k = torch.randn(total, 8, 128, device="cuda").to(torch.bfloat16)
        v = torch.randn(total, 8, 128, device="cuda").to(torch.bfloat16)
        w = torch.ones(128, device="cuda", dtype=torch.bfloat16)
        # stream 0: second page id outside the pool, no third page (its tokens 128, 129 have nowhere to go);
        # stream 1: fine; stream 2: pages 3, 4 only
        table = torch.tensor([[0, 99], [1, 2], [3, 4]], dtype=torch.int32, device="cuda")
        q_rot = torch.full_like(q, 7.0)
        eng.prefill_norm_rope_scatter(0, q, k, v, w, w, cu, table, q_rot=q_rot)
        torch.cuda.synchronize()
        bits = eng.status()
        assert bits & qm.DEVSTAT_BAD_PAGE and bits & qm.DEVSTAT_BAD_POS and not bits & qm.DEVSTAT_TIMEOUT
        kview, vview = eng.pool_view(0)
        kview = kview.view(6, 8, 64, 128)
        vview = vview.view(6, 8, 64, 128)
        # stream 1 landed whole: V rows are copies
        want = v[130:200].permute(1, 0, 2)
        assert torch.equal(vview[1, :, :64], want[:, :64]) and torch.equal(vview[2, :, :6], want[:, 64:70])
        # stream 0: first page written, nothing anywhere else for it (page 5 is nobody's and stays zero)
        assert torch.equal(vview[0], v[0:64].permute(1, 0, 2))
        assert not vview[5].float().abs().max().item() and not kview[5].float().abs().max().item()
        # stream 2: positions 0 .. 127 written (pages 3, 4), positions 128 .. 159 roped but without a cache row,
        # positions >= 160 untouched (q_rot keeps its fill)
        assert torch.equal(vview[3], v[200:264].permute(1, 0, 2)) and torch.equal(vview[4], v[264:328].permute(1, 0, 2))
        assert (q_rot[200 + 160:] == 7.0).all()
        assert not (q_rot[200:200 + 160] == 7.0).all(dim=-1).any()
    finally:
        eng.close()
