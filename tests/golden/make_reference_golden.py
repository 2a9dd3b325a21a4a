"""Produces tests/golden/reference_kernels_golden.npz by launching the REFERENCE's own CUDA kernels
(through oracle/_ref/libqm_refkernels.so, built from the reference checkout by oracle/Makefile) on the seeded
scenarios of tests/scenario.py.  Needs a GPU and the prebuilt harness; it does not need the reference checkout.

    python tests/golden/make_reference_golden.py [output.npz]

Only outputs are stored; the inputs are regenerated from their seeds by the tests.  The script also prints how
far the CPU restatement (oracle "ref" mode) is from the reference's bits, and the reference kernels' time.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import scenario  # noqa: E402
from oracle import qm_oracle as oracle  # noqa: E402

DECODE_CASES = {  # name -> (seed, lengths, random_weights)
    "dec_a": (101, [0, 1, 63, 64, 65, 200], True),
    "dec_b": (0, [512], False),
    "dec_c": (102, [1000, 2500], True),
}
PREFILL_CASES = {"pre_a": (201, [70], True), "pre_b": (202, [130, 9], False)}


def mismatch(a, b):
    return int((a != b).sum()), a.size


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_kernels_golden.npz")
    store = {}
    for name, (seed, lengths, rw) in DECODE_CASES.items():
        sc = scenario.DecodeScenario(seed=seed, lengths=lengths, random_weights=rw)
        exp = sc.expected()
        q_rot_all, krow_all, ctx_all = [], [], []
        for s in range(sc.batch):
            pos = int(sc.lengths[s])
            kc, vc = sc.key_caches[s].copy(), sc.value_caches[s].copy()
            q_rot = oracle.ref_decode_append(sc.q[s], sc.k[s], sc.v[s], sc.q_w, sc.k_w, sc.cos[pos], sc.sin[pos],
                                             kc, vc, pos)
            assert np.array_equal(vc[:, pos], sc.v[s]), "reference V append is not a raw copy?"
            untouched = np.ones(kc.shape[1], dtype=bool)
            untouched[pos] = False
            assert np.array_equal(kc[:, untouched], sc.key_caches[s][:, untouched])
            ctx, ms = oracle.ref_attention(q_rot[None], kc, vc, 1, pos, iterations=20)
            q_rot_all.append(q_rot)
            krow_all.append(kc[:, pos].copy())
            ctx_all.append(ctx[0])
            print(f"{name} stream {s} L={pos + 1}: reference decode attention {ms * 1e3:.1f} us/launch")
        q_rot_all, krow_all, ctx_all = np.stack(q_rot_all), np.stack(krow_all), np.stack(ctx_all)
        store[f"{name}_q_rot"], store[f"{name}_key_rows"], store[f"{name}_context"] = q_rot_all, krow_all, ctx_all
        print(name, "q_rot mismatches vs oracle", mismatch(q_rot_all, exp["q_rot"]),
              "k rows", mismatch(krow_all, exp["key_rows"]))
        # attention of the oracle on the REFERENCE's q_rot / k row would be the cleanest comparison; the rows
        # differ in at most a few ulps, so compare directly and report
        print(name, "context mismatches vs oracle ref mode", mismatch(ctx_all, exp["out_ref"]),
              oracle.error_metrics(oracle.bf16_to_f32(ctx_all), oracle.bf16_to_f32(exp["out_ref"])))
        print(name, "reference vs fp32 oracle", oracle.error_metrics(oracle.bf16_to_f32(ctx_all), exp["out_fp32"]))
    for name, (seed, lengths, rw) in PREFILL_CASES.items():
        ps = scenario.PrefillScenario(seed=seed, lengths=lengths, random_weights=rw)
        q_rot_exp, kcs_exp, vcs_exp = ps.expected_append()
        out_exp, _ = ps.expected_attention(mode="ref")
        q_rot_all, ctx_all, kc_all = [], [], []
        for s in range(ps.batch):
            a, b = int(ps.cu_seqlens[s]), int(ps.cu_seqlens[s + 1])
            n = b - a
            kc = np.zeros((ps.kv_heads, ps.max_cache, 128), dtype=np.uint16)
            vc = np.zeros_like(kc)
            q_rot = oracle.ref_prefill_append(ps.q[a:b], ps.k[a:b], ps.v[a:b], ps.q_w, ps.k_w, ps.cos[:n],
                                              ps.sin[:n], kc, vc)
            assert np.array_equal(vc, vcs_exp[s])
            ctx, ms = oracle.ref_attention(q_rot, kc, vc, n, 0, iterations=5)
            print(f"{name} seq {s} len {n}: reference prefill attention {ms * 1e3:.1f} us/launch")
            q_rot_all.append(q_rot)
            ctx_all.append(ctx)
            kc_all.append(kc[:, :n].copy())
            print(name, s, "k cache mismatches vs oracle", mismatch(kc[:, :n], kcs_exp[s][:, :n]))
        q_rot_all, ctx_all = np.concatenate(q_rot_all), np.concatenate(ctx_all)
        store[f"{name}_q_rot"], store[f"{name}_context"] = q_rot_all, ctx_all
        for s, kc in enumerate(kc_all):
            store[f"{name}_key_cache_{s}"] = kc
        print(name, "q_rot mismatches", mismatch(q_rot_all, q_rot_exp), "context mismatches vs oracle ref mode",
              mismatch(ctx_all, out_exp),
              oracle.error_metrics(oracle.bf16_to_f32(ctx_all), oracle.bf16_to_f32(out_exp)))
    np.savez_compressed(out_path, **store)
    print("written", out_path, {k: v.shape for k, v in store.items()})

    # reference kernel time on the headline decode shapes (one stream at a time: the reference is batch 1)
    rng_lengths = oracle.uniform_int(1 * 1000 + 99, 256, 4096, 64)
    total_ms, total_bytes = 0.0, 0
    for length in rng_lengths[:8]:
        length = int(length)
        kc = oracle.normal_bf16(5, (8, length + 1, 128))
        vc = oracle.normal_bf16(6, (8, length + 1, 128))
        q = oracle.normal_bf16(7, (1, 16, 128))
        _, ms = oracle.ref_attention(q, kc, vc, 1, length, iterations=10)
        total_ms += ms
        total_bytes += (length + 1) * 4096
        print(f"reference gqa2 decode L={length + 1}: {ms * 1e3:.1f} us, {(length + 1) * 4096 / ms / 1e6:.1f} GB/s")
    print(f"reference decode, 8 streams of the ragged batch back to back: {total_ms * 1e3:.1f} us, "
          f"{total_bytes / total_ms / 1e6:.1f} GB/s")


if __name__ == "__main__":
    main()
