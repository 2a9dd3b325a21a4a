"""Builds rank-local pools for the split-across-GPUs decode path from a DecodeScenario."""
import numpy as np

from oracle import qm_oracle as oracle

PAGE = 64


def rank_local_state(sc, exp, sh, world, rank, include_new_token=True):
    """Pools, page table and key counts of `rank` when every stream's keys are split contiguously over `world` ranks.

    The caches in `exp` already hold the new token at position lengths[s]; with include_new_token=False the owner's
    slice stops before it (for testing the append on the owner).
    Returns dict(kpool, vpool, table, local_lens, begins, num_pages, max_pages).
    """
    b = sc.batch
    spans = []
    for s in range(b):
        total = int(sc.lengths[s]) + 1
        begin, end = sh.slice_bounds(total, world, rank)
        if not include_new_token and end == total:
            end -= 1
        spans.append((begin, max(end, begin)))
    pages = [max((e - bgn + PAGE - 1) // PAGE, 1) for bgn, e in spans]
    # leave room for one more token on the owner
    pages = [p + (1 if (e - bgn) % PAGE == 0 else 0) for p, (bgn, e) in zip(pages, spans)]
    max_pages = max(pages)
    num_pages = sum(pages) + 1
    ids = oracle.shuffled_range(900 + rank, num_pages)
    table = np.zeros((b, max_pages), dtype=np.int32)
    kpool = np.zeros((num_pages, sc.kv_heads, PAGE, 128), dtype=np.uint16)
    vpool = np.zeros_like(kpool)
    cursor = 0
    for s in range(b):
        table[s, :pages[s]] = ids[cursor:cursor + pages[s]]
        cursor += pages[s]
        bgn, e = spans[s]
        n = e - bgn
        if n:
            kc = np.ascontiguousarray(exp["key_caches"][s][:, bgn:e])
            vc = np.ascontiguousarray(exp["value_caches"][s][:, bgn:e])
            oracle.scatter_paged(kc, table[s], n, kpool)
            oracle.scatter_paged(vc, table[s], n, vpool)
    return {"kpool": kpool, "vpool": vpool, "table": table,
            "local_lens": np.array([e - bgn for bgn, e in spans], dtype=np.int32),
            "begins": np.array([bgn for bgn, _ in spans], dtype=np.int32), "num_pages": num_pages,
            "max_pages": max_pages}
