"""Seeded synthetic workloads for the parity tests, and the expected results computed by the CPU oracle.

Input recipe: SplitMix64 -> Box-Muller -> bf16, one RNG stream per (seed, tensor) seeded seed*1000 + tensor id;
q/k/v are pre-norm projections ~ N(0,1); norm weights are bf16(1.0) unless `random_weights`; eps 1e-6;
RoPE theta 1e6; pages of 64 tokens with a Fisher-Yates-shuffled page table.  The cache content that exists
before the measured call is produced by the oracle's own append over positions 0..L-1.
"""
from __future__ import annotations

import numpy as np

from oracle import qm_oracle as oracle

D = 128
PAGE = 64

T_Q, T_K, T_V, T_KPREV, T_VPREV, T_QW, T_KW, T_PAGES = range(1, 9)


def _norm_weights(seed, random_weights):
    if not random_weights:
        one = oracle.f32_to_bf16(np.ones(D, dtype=np.float32))
        return one.copy(), one.copy()
    qw = oracle.f32_to_bf16(1.0 + 0.25 * oracle.bf16_to_f32(oracle.normal_bf16(seed * 1000 + T_QW, (D,))))
    kw = oracle.f32_to_bf16(1.0 + 0.25 * oracle.bf16_to_f32(oracle.normal_bf16(seed * 1000 + T_KW, (D,))))
    return qw, kw


class DecodeScenario:
    """`lengths[s]` tokens already cached for stream s; the measured step appends position lengths[s] and
    attends lengths[s] + 1 keys."""

    def __init__(self, seed, lengths, q_heads=16, kv_heads=8, random_weights=False, shuffle_pages=True,
                 spare_pages=3):
        self.seed, self.q_heads, self.kv_heads = seed, q_heads, kv_heads
        self.lengths = np.asarray(lengths, dtype=np.int32)
        b = self.batch = len(lengths)
        self.max_pos = int(self.lengths.max()) + 1
        self.pages_per_stream = (self.lengths + 1 + PAGE - 1) // PAGE
        self.max_pages = int(self.pages_per_stream.max())
        self.max_cache = self.max_pages * PAGE
        self.num_pages = int(self.pages_per_stream.sum()) + spare_pages
        self.q_w, self.k_w = _norm_weights(seed, random_weights)
        self.cos, self.sin = oracle.make_rope(self.max_pos)
        ids = oracle.shuffled_range(seed * 1000 + T_PAGES, self.num_pages) if shuffle_pages else np.arange(
            self.num_pages, dtype=np.int32)
        self.page_table = np.full((b, self.max_pages), -1, dtype=np.int32)
        cursor = 0
        for s in range(b):
            n = int(self.pages_per_stream[s])
            self.page_table[s, :n] = ids[cursor:cursor + n]
            cursor += n
        self.q = oracle.normal_bf16(seed * 1000 + T_Q, (b, q_heads, D))
        self.k = oracle.normal_bf16(seed * 1000 + T_K, (b, kv_heads, D))
        self.v = oracle.normal_bf16(seed * 1000 + T_V, (b, kv_heads, D))
        # existing cache content, reference layout per stream
        self.key_caches, self.value_caches = [], []
        total_prev = int(self.lengths.sum())
        k_prev = oracle.normal_bf16(seed * 1000 + T_KPREV, (total_prev, kv_heads, D))
        v_prev = oracle.normal_bf16(seed * 1000 + T_VPREV, (total_prev, kv_heads, D))
        dummy_q = np.zeros((1, q_heads, D), dtype=np.uint16)
        cursor = 0
        for s in range(b):
            n = int(self.lengths[s])
            kc = np.zeros((kv_heads, self.max_cache, D), dtype=np.uint16)
            vc = np.zeros_like(kc)
            if n:
                qz = np.zeros((n, q_heads, D), dtype=np.uint16)
                oracle.append(qz, k_prev[cursor:cursor + n], v_prev[cursor:cursor + n], self.q_w, self.k_w,
                              self.cos[:n], self.sin[:n], 0, kc, vc)
            cursor += n
            self.key_caches.append(kc)
            self.value_caches.append(vc)
        del dummy_q
        self._expected = None

    def pools(self):
        """(K pool, V pool) [num_pages][Hkv][64][128] holding the pre-existing tokens."""
        kp = np.zeros((self.num_pages, self.kv_heads, PAGE, D), dtype=np.uint16)
        vp = np.zeros_like(kp)
        for s in range(self.batch):
            n = int(self.lengths[s])
            oracle.scatter_paged(self.key_caches[s], self.page_table[s], n, kp)
            oracle.scatter_paged(self.value_caches[s], self.page_table[s], n, vp)
        return kp, vp

    def expected(self):
        if self._expected is not None:
            return self._expected
        b = self.batch
        q_rot = np.empty_like(self.q)
        kcs = [kc.copy() for kc in self.key_caches]
        vcs = [vc.copy() for vc in self.value_caches]
        for s in range(b):
            pos = int(self.lengths[s])
            q_rot[s:s + 1] = oracle.append(self.q[s:s + 1], self.k[s:s + 1], self.v[s:s + 1], self.q_w, self.k_w,
                                           self.cos[pos:pos + 1], self.sin[pos:pos + 1], pos, kcs[s], vcs[s])
        key_lens = self.lengths + 1
        self._expected = {
            "q_rot": q_rot,
            "key_caches": kcs,
            "value_caches": vcs,
            "key_rows": np.stack([kcs[s][:, int(self.lengths[s])] for s in range(b)]),
            "value_rows": np.stack([vcs[s][:, int(self.lengths[s])] for s in range(b)]),
            "out_ref": oracle.decode_attention(q_rot, kcs, vcs, key_lens, mode="ref"),
            "out_fp32": oracle.decode_attention(q_rot, kcs, vcs, key_lens, mode="fp32"),
        }
        return self._expected


def _bf16_tensor(torch, bits):
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def _bits(t):
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def run_decode_on_gpu(pkg, sc: DecodeScenario, layer=0, layers=1):
    """One decode step through the C ABI; returns raw bf16 bits of every output."""
    import torch

    eng = pkg.TalkerAttention(layers=layers, num_pages=sc.num_pages, q_heads=sc.q_heads, kv_heads=sc.kv_heads,
                              max_positions=sc.max_pos)
    try:
        kp, vp = sc.pools()
        kview, vview = eng.pool_view(layer)
        kview.copy_(_bf16_tensor(torch, kp))
        vview.copy_(_bf16_tensor(torch, vp))
        q, k, v = (_bf16_tensor(torch, x) for x in (sc.q, sc.k, sc.v))
        qw, kw = _bf16_tensor(torch, sc.q_w), _bf16_tensor(torch, sc.k_w)
        positions = torch.from_numpy(sc.lengths).cuda()
        page_table = torch.from_numpy(np.maximum(sc.page_table, 0)).cuda()
        seq_lens = torch.from_numpy(sc.lengths + 1).cuda()
        q_rot = eng.launch_qk_norm_rope_cache_m1(layer, q, k, v, qw, kw, positions, page_table)
        out = eng.launch_attention(layer, q_rot, seq_lens, page_table)
        partial = eng.launch_attention_partial(layer, q_rot, seq_lens, page_table)
        out_from_partial = eng.combine(partial.unsqueeze(0))
        torch.cuda.synchronize()
        status = eng.status()
        kp_after, vp_after = _bits(kview), _bits(vview)
        key_rows = np.stack([kp_after[sc.page_table[s, sc.lengths[s] // PAGE], :, sc.lengths[s] % PAGE]
                             for s in range(sc.batch)])
        value_rows = np.stack([vp_after[sc.page_table[s, sc.lengths[s] // PAGE], :, sc.lengths[s] % PAGE]
                               for s in range(sc.batch)])
        return {
            "q_rot": _bits(q_rot), "out": _bits(out), "out_from_partial": _bits(out_from_partial),
            "partial": partial.cpu().numpy(), "key_pool": kp_after, "value_pool": vp_after,
            "key_pool_new_rows": key_rows, "value_pool_new_rows": value_rows, "status": status,
            "rope_cos": _bits(eng.rope_cos), "rope_sin": _bits(eng.rope_sin),
        }
    finally:
        eng.close()


class PrefillScenario:
    """Packed varlen prompts starting from an empty cache."""

    def __init__(self, seed, lengths, q_heads=16, kv_heads=8, random_weights=False, shuffle_pages=True,
                 spare_pages=2):
        self.seed, self.q_heads, self.kv_heads = seed, q_heads, kv_heads
        self.lengths = np.asarray(lengths, dtype=np.int32)
        b = self.batch = len(lengths)
        self.cu_seqlens = np.concatenate([[0], np.cumsum(self.lengths)]).astype(np.int32)
        self.total = int(self.cu_seqlens[-1])
        self.max_seqlen = int(self.lengths.max())
        self.max_pos = self.max_seqlen
        self.pages_per_stream = (self.lengths + PAGE - 1) // PAGE
        self.max_pages = max(int(self.pages_per_stream.max()), 1)
        self.max_cache = self.max_pages * PAGE
        self.num_pages = int(self.pages_per_stream.sum()) + spare_pages
        self.q_w, self.k_w = _norm_weights(seed, random_weights)
        self.cos, self.sin = oracle.make_rope(max(self.max_pos, 1))
        ids = oracle.shuffled_range(seed * 1000 + T_PAGES, self.num_pages) if shuffle_pages else np.arange(
            self.num_pages, dtype=np.int32)
        self.page_table = np.full((b, self.max_pages), -1, dtype=np.int32)
        cursor = 0
        for s in range(b):
            n = int(self.pages_per_stream[s])
            self.page_table[s, :n] = ids[cursor:cursor + n]
            cursor += n
        self.q = oracle.normal_bf16(seed * 1000 + T_Q, (self.total, q_heads, D))
        self.k = oracle.normal_bf16(seed * 1000 + T_K, (self.total, kv_heads, D))
        self.v = oracle.normal_bf16(seed * 1000 + T_V, (self.total, kv_heads, D))
        self._append = None

    def expected_append(self):
        """q_rot [total][Hq][128] and per-stream reference-layout caches."""
        if self._append is None:
            q_rot = np.empty_like(self.q)
            kcs, vcs = [], []
            for s in range(self.batch):
                a, b = int(self.cu_seqlens[s]), int(self.cu_seqlens[s + 1])
                kc = np.zeros((self.kv_heads, self.max_cache, D), dtype=np.uint16)
                vc = np.zeros_like(kc)
                if b > a:
                    q_rot[a:b] = oracle.append(self.q[a:b], self.k[a:b], self.v[a:b], self.q_w, self.k_w,
                                               self.cos[:b - a], self.sin[:b - a], 0, kc, vc)
                kcs.append(kc)
                vcs.append(vc)
            self._append = (q_rot, kcs, vcs)
        return self._append

    def expected_attention(self, mode="fp32", rows_per_stream=None):
        """Oracle attention.  rows_per_stream: dict stream -> (begin, end) to limit the work; rows outside stay 0.
        Returns an array [total][Hq][128] and a boolean row mask of what was computed."""
        q_rot, kcs, vcs = self.expected_append()
        dtype = np.uint16 if mode == "ref" else np.float32
        out = np.zeros((self.total, self.q_heads, D), dtype=dtype)
        mask = np.zeros(self.total, dtype=bool)
        for s in range(self.batch):
            a, b = int(self.cu_seqlens[s]), int(self.cu_seqlens[s + 1])
            if b == a:
                continue
            rows = (0, b - a) if rows_per_stream is None else rows_per_stream.get(s)
            if rows is None:
                continue
            res = oracle.prefill_attention(q_rot[a:b], kcs[s], vcs[s], b - a, 0, rows=rows, mode=mode)
            out[a + rows[0]:a + rows[1]] = res[rows[0]:rows[1]]
            mask[a + rows[0]:a + rows[1]] = True
        return out, mask


def run_prefill_on_gpu(pkg, sc: PrefillScenario, layer=0, attention=True):
    import torch

    eng = pkg.TalkerAttention(layers=1, num_pages=sc.num_pages, q_heads=sc.q_heads, kv_heads=sc.kv_heads,
                              max_positions=max(sc.max_pos, 1))
    try:
        q, k, v = (_bf16_tensor(torch, x) for x in (sc.q, sc.k, sc.v))
        qw, kw = _bf16_tensor(torch, sc.q_w), _bf16_tensor(torch, sc.k_w)
        cu = torch.from_numpy(sc.cu_seqlens).cuda()
        page_table = torch.from_numpy(np.maximum(sc.page_table, 0)).cuda()
        q_rot = eng.prefill_norm_rope_scatter(layer, q, k, v, qw, kw, cu, page_table)
        result = {}
        if attention:
            out = eng.launch_attention_prefill(layer, q_rot, cu, page_table, sc.max_seqlen)
            result["out"] = _bits(out)
        torch.cuda.synchronize()
        kview, vview = eng.pool_view(layer)
        result.update({"q_rot": _bits(q_rot), "key_pool": _bits(kview), "value_pool": _bits(vview),
                       "status": eng.status()})
        return result
    finally:
        eng.close()
