"""Produces tests/golden/reference_layer_golden.npz: outputs of the REFERENCE's own non-attention talker kernels
(rmsnorm, linear, add+postnorm, gate/up SwiGLU; launched through oracle/_ref/libqm_refkernels.so on a GPU) on the
seeded cases of tests/layer_cases.py, and prints how far the CPU restatement is from them.

    python tests/golden/make_reference_layer_golden.py [output.npz]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import layer_cases  # noqa: E402
from oracle import qm_oracle as oracle  # noqa: E402


def mismatch(a, b):
    return int((a != b).sum()), a.size


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_layer_golden.npz")
    store = {}
    for name, (seed, rows) in layer_cases.CASES.items():
        c = layer_cases.LayerCase(seed, rows)
        store[f"{name}_rmsnorm"] = oracle.ref_rmsnorm(c.x, c.norm_w)
        store[f"{name}_linear"] = oracle.ref_linear(c.x, c.w)
        store[f"{name}_linear_bias_residual"] = oracle.ref_linear(c.x, c.w, c.bias, c.residual)
        res, nrm = oracle.ref_add_postnorm(c.x, c.attn, c.norm_w)
        store[f"{name}_residual"], store[f"{name}_postnorm"] = res, nrm
        store[f"{name}_swiglu"] = oracle.ref_gate_up_swiglu(c.x, c.gate_w, c.up_w)
        print(name, "rmsnorm", mismatch(store[f"{name}_rmsnorm"], oracle.rmsnorm(c.x, c.norm_w)),
              "linear", mismatch(store[f"{name}_linear"], oracle.linear(c.x, c.w)),
              "linear+bias+res", mismatch(store[f"{name}_linear_bias_residual"], oracle.linear(c.x, c.w, c.bias, c.residual)),
              "residual", mismatch(res, oracle.add_postnorm(c.x, c.attn, c.norm_w)[0]),
              "postnorm", mismatch(nrm, oracle.add_postnorm(c.x, c.attn, c.norm_w)[1]),
              "swiglu", mismatch(store[f"{name}_swiglu"], oracle.gate_up_swiglu(c.x, c.gate_w, c.up_w)))
    np.savez_compressed(out_path, **store)
    print("written", out_path, {k: v.shape for k, v in store.items()})


if __name__ == "__main__":
    main()
