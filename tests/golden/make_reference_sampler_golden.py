"""Produces tests/golden/reference_sampler_golden.npz: what the REFERENCE's own final-head kernels
(cast_final_head_logits, repetition_penalty, suppress_tokens, argmax_final_head / gpu_sample_topk_f32_kernel,
record_sampled_code_kernel; launched through oracle/_ref/libqm_refkernels.so on a GPU) return on the seeded cases
of tests/sampler_cases.py, and prints whether the CPU restatement agrees.

    python tests/golden/make_reference_sampler_golden.py [output.npz]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import sampler_cases  # noqa: E402
from oracle import qm_oracle as oracle  # noqa: E402


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_sampler_golden.npz")
    store = {}
    for name in sampler_cases.CASES:
        c = sampler_cases.SamplerCase(name)
        code, processed, state, history = oracle.ref_final_head(c.logits, c.history, c.generation_index, c.flags, c.top_k,
                                                               c.temperature, c.rng_state)
        store[f"{name}_code"] = np.int32(code)
        store[f"{name}_processed"] = processed
        store[f"{name}_state"] = np.uint64(state)
        store[f"{name}_recorded"] = np.int32(history[c.generation_index])
        mine = oracle.final_head_sample(c.logits, c.history, c.generation_index, c.flags, top_k=c.top_k,
                                        temperature=c.temperature, rng_state=c.rng_state)
        print(name, "reference code", code, "restatement", mine[0], "processed equal",
              bool(np.array_equal(processed.view(np.uint32), mine[1].view(np.uint32))), "state equal", state == mine[2])
    # a chain of draws from one state: the order of SplitMix64 draws over consecutive steps
    c = sampler_cases.SamplerCase("topk_processed")
    state, history, codes = c.rng_state, c.history.copy(), []
    for step in range(16):
        code, _, state, history = oracle.ref_final_head(c.logits, history, c.generation_index + step,
                                                        sampler_cases.REPETITION | sampler_cases.SUPPRESS | sampler_cases.RECORD,
                                                        c.top_k, c.temperature, state)
        codes.append(code)
    store["chain_codes"] = np.asarray(codes, dtype=np.int32)
    store["chain_state"] = np.uint64(state)
    np.savez_compressed(out_path, **store)
    print("written", out_path)


if __name__ == "__main__":
    main()
