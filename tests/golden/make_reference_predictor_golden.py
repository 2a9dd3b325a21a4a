"""Produces tests/golden/reference_predictor_golden.npz: outputs of the REFERENCE's own code-predictor kernels
(predictor_qkv_m1_fused_kernel, predictor_qk_norm_rope_cache_m1_kernel, predictor_attention_gqa2_m1_kernel,
predictor_linear_m1_fused_kernel, predictor_add_postnorm_m1_kernel, predictor_gate_up_swiglu_m1_kernel; launched
through oracle/_ref/libqm_refkernels.so on a GPU) on the seeded cases of tests/predictor_cases.py, and prints how
far the CPU restatement is from them.

    python tests/golden/make_reference_predictor_golden.py [output.npz]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import predictor_cases as pc  # noqa: E402
from oracle import qm_oracle as oracle  # noqa: E402


def mismatch(a, b):
    return int((a != b).sum()), a.size


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_predictor_golden.npz")
    store = {}
    for seed in pc.SEEDS:
        c = pc.PredictorCase(seed)
        name = f"p{seed}"
        q, k, v = oracle.ref_predictor_qkv_m1(c.x, c.q_w, c.k_w, c.v_w)
        store[f"{name}_q"], store[f"{name}_k"], store[f"{name}_v"] = q, k, v
        x1 = c.x.reshape(1, -1)
        print(name, "qkv", mismatch(q, oracle.linear(x1, c.q_w)[0]), mismatch(k, oracle.linear(x1, c.k_w)[0]),
              mismatch(v, oracle.linear(x1, c.v_w)[0]))
        store[f"{name}_o"] = oracle.ref_predictor_linear_m1(c.context, c.o_w)
        store[f"{name}_down"] = oracle.ref_predictor_linear_m1(c.act, c.down_w, c.residual)
        print(name, "o", mismatch(store[f"{name}_o"], oracle.linear(c.context.reshape(1, -1), c.o_w)[0]),
              "down+residual", mismatch(store[f"{name}_down"],
                                        oracle.linear(c.act.reshape(1, -1), c.down_w, residual=c.residual.reshape(1, -1))[0]))
        res, nrm = oracle.ref_predictor_add_postnorm_m1(c.x, c.attention, c.post_norm_w)
        store[f"{name}_residual"], store[f"{name}_postnorm"] = res, nrm
        want_res, want_nrm = oracle.add_postnorm(x1, c.attention.reshape(1, -1), c.post_norm_w)
        print(name, "residual", mismatch(res, want_res[0]), "postnorm", mismatch(nrm, want_nrm[0]))
        store[f"{name}_swiglu"] = oracle.ref_predictor_gate_up_swiglu_m1(c.x, c.gate_w, c.up_w)
        print(name, "swiglu", mismatch(store[f"{name}_swiglu"], oracle.gate_up_swiglu(x1, c.gate_w, c.up_w)[0]))
        for pos in pc.POSITIONS:
            kc, vc = c.caches_before(pos)
            q_rot = oracle.ref_predictor_qk_norm_rope_cache_m1(c.q, c.k, c.v, c.q_norm_w, c.k_norm_w, c.cos[pos], c.sin[pos], kc, vc, pos)
            ctx = oracle.ref_predictor_attention_m1(q_rot, kc, vc, pos + 1)
            store[f"{name}_pos{pos}_q_rot"], store[f"{name}_pos{pos}_k_row"], store[f"{name}_pos{pos}_v_row"] = q_rot, kc[:, pos].copy(), vc[:, pos].copy()
            store[f"{name}_pos{pos}_context"] = ctx
            okc, ovc = c.caches_before(pos)
            oq = oracle.append(c.q[None], c.k[None], c.v[None], c.q_norm_w, c.k_norm_w, c.cos[pos:pos + 1], c.sin[pos:pos + 1], pos, okc, ovc)[0]
            octx = oracle.decode_attention(oq[None], [okc], [ovc], [pos + 1], mode="ref")[0]
            print(name, "position", pos, "q_rot", mismatch(q_rot, oq), "k row", mismatch(kc[:, pos], okc[:, pos]),
                  "v row", mismatch(vc[:, pos], ovc[:, pos]), "untouched rows equal", bool(np.array_equal(np.delete(kc, pos, 1), np.delete(okc, pos, 1))),
                  "context", mismatch(ctx, octx))
    np.savez_compressed(out_path, **store)
    print("written", out_path, {k: v.shape for k, v in store.items()})


if __name__ == "__main__":
    main()
