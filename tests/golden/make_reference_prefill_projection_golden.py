"""Produces tests/golden/reference_prefill_projection_golden.npz: outputs of the REFERENCE's own prefill-loop
projections (native_ops::linear_bf16, code_predictor::launch_add, code_predictor::launch_swiglu; launched through
oracle/_ref/libqm_refkernels.so on a GPU) on the seeded cases of tests/prefill_projection_cases.py, and prints how
far the CPU restatement (double-precision mode) is from them.

    python tests/golden/make_reference_prefill_projection_golden.py [output.npz]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import prefill_projection_cases as cases  # noqa: E402
from oracle import qm_oracle as oracle  # noqa: E402


def distance(a, b):
    m = oracle.error_metrics(oracle.bf16_to_f32(a), oracle.bf16_to_f32(b))
    return {"differing": int((a != b).sum()), "of": int(a.size), "max_abs": float(m["max_abs"]), "mean_rel": float(m["mean_rel"])}


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_prefill_projection_golden.npz")
    store = {}
    for name, spec in cases.CASES.items():
        c = cases.ProjectionCase(*spec)
        store[f"{name}_linear"] = oracle.ref_linear_generic(c.x, c.w)
        store[f"{name}_linear_bias_residual"] = oracle.ref_linear_generic(c.x, c.w, c.bias, c.residual)
        store[f"{name}_swiglu"] = oracle.ref_gate_up_swiglu_generic(c.x, c.w, c.up_w)
        print(name, "linear", distance(store[f"{name}_linear"], oracle.linear(c.x, c.w, mode="f64")),
              "linear+bias+res", distance(store[f"{name}_linear_bias_residual"], oracle.linear(c.x, c.w, c.bias, c.residual, mode="f64")),
              "swiglu", distance(store[f"{name}_swiglu"], oracle.gate_up_swiglu(c.x, c.w, c.up_w, mode="f64")))
    np.savez_compressed(out_path, **store)
    print("written", out_path, {k: v.shape for k, v in store.items()})


if __name__ == "__main__":
    main()
