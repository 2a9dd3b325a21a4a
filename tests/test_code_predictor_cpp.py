"""The C++ code-predictor driver (host/code_predictor_b200.hpp, counterpart of the reference's capture_step,
17.cu:13616-13905) against the chain of the CPU oracle's operators - which tests/test_predictor_golden_cpu.py pins
to the reference's own predictor kernels.  One frame at reduced widths (hidden 256, SwiGLU 512, 2 layers, 4 steps;
real head shape and vocabulary), with the two rows of step 0 once as two one-row positions and once through the
staged many-row path the reference uses for them.  Per step: the logits against the oracle chain (fed the driver's
own codes, so a near-tie cannot fork the two chains), and the code against the restated sampler on the driver's
own logits."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import test_predictor_gpu as chain

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qingming-qwen3-tts_b200"
BINARY = ROOT / "tests" / "cpp" / "code_predictor_test.bin"
HQ, HKV, D = 16, 8, 128
DIMS = dict(streams=3, outer=512, hidden=256, intermediate=512, layers=2, vocab=2048, steps=4)


def build(qm):
    qm.build_library()
    source = ROOT / "tests" / "cpp" / "code_predictor_test.cpp"
    stamp = max(p.stat().st_mtime for p in list((PKG / "host").glob("*.hpp")) + [source, ROOT / "include" / "qm_attention.h"])
    if BINARY.exists() and BINARY.stat().st_mtime >= stamp:
        return
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "-O2", "-Xcompiler=-pthread,-Wall,-Wextra",
           "-I", str(ROOT / "include"), "-I", str(PKG / "host"), str(source), "-o", str(BINARY), "-L", str(PKG / "lib"),
           "-lqm_attention_b200", "-Xlinker", f"-rpath={PKG / 'lib'}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0 and "warning" not in proc.stderr, proc.stdout + proc.stderr


def test_code_predictor_driver_compiles_as_cpp20(qm):
    build(qm)
    assert BINARY.exists()


def make_weights(seed):
    d = DIMS
    h, o, i, v = d["hidden"], d["outer"], d["intermediate"], d["vocab"]

    def norm_like(s, n):
        return oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(s, (n,))))

    w = {"projection": oracle.scaled_normal_bf16(seed + 1, (h, o), 0.06), "projection_bias": oracle.scaled_normal_bf16(seed + 2, (h,), 0.06),
         "final_norm": norm_like(seed + 3, h), "layers": [], "heads": [], "embeddings": []}
    for layer in range(d["layers"]):
        s = seed + 100 * (layer + 1)
        w["layers"].append({
            "in_norm": norm_like(s, h), "post_norm": norm_like(s + 1, h), "q_norm": norm_like(s + 2, D), "k_norm": norm_like(s + 3, D),
            "q": oracle.scaled_normal_bf16(s + 4, (HQ * D, h), 0.06), "k": oracle.scaled_normal_bf16(s + 5, (HKV * D, h), 0.06),
            "v": oracle.scaled_normal_bf16(s + 6, (HKV * D, h), 0.06), "o": oracle.scaled_normal_bf16(s + 7, (h, HQ * D), 0.06),
            "gate": oracle.scaled_normal_bf16(s + 8, (i, h), 0.06), "up": oracle.scaled_normal_bf16(s + 9, (i, h), 0.06),
            "down": oracle.scaled_normal_bf16(s + 10, (h, i), 0.06)})
    for step in range(d["steps"]):
        w["heads"].append(oracle.scaled_normal_bf16(seed + 1000 + step, (v, h), 0.06))
        w["embeddings"].append(oracle.normal_bf16(seed + 2000 + step, (v, o)))
    return w


FILE_NAMES = {"in_norm": "input_norm", "post_norm": "post_norm", "q_norm": "q_norm", "k_norm": "k_norm", "q": "q", "k": "k", "v": "v",
              "o": "o", "gate": "gate", "up": "up", "down": "down"}


@pytest.mark.gpu
@pytest.mark.parametrize("top_k", [0, 50])
def test_cpp_code_predictor_frame_matches_oracle_chain(qm, tmp_path, top_k):
    build(qm)
    d = DIMS
    streams, steps, vocab = d["streams"], d["steps"], d["vocab"]
    w = make_weights(900)
    for name in ("projection", "projection_bias", "final_norm"):
        w[name].tofile(tmp_path / f"{name}.bin")
    for index, layer in enumerate(w["layers"]):
        for key, value in layer.items():
            value.tofile(tmp_path / f"l{index}_{FILE_NAMES[key]}.bin")
    for step in range(steps):
        w["heads"][step].tofile(tmp_path / f"head{step}.bin")
        w["embeddings"][step].tofile(tmp_path / f"embedding{step}.bin")
    talker_hidden = oracle.normal_bf16(951, (streams, d["outer"]))
    first_embedding = oracle.normal_bf16(952, (streams, d["outer"]))
    talker_hidden.tofile(tmp_path / "talker_hidden.bin")
    first_embedding.tofile(tmp_path / "first_embedding.bin")
    states_before = np.array([11, 22, 33], dtype=np.uint64)
    states_before.tofile(tmp_path / "rng.bin")
    proc = subprocess.run([str(BINARY), str(tmp_path)] + [f"{k}={v}" for k, v in d.items()] + [f"top_k={top_k}"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "CODE_PREDICTOR_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]

    cos, sin = oracle.make_rope(64)
    results = {}
    for mode in ("positions", "staged"):
        codes = np.fromfile(tmp_path / f"codes_{mode}.bin", dtype=np.int32).reshape(steps, streams)
        logits = np.fromfile(tmp_path / f"logits_{mode}.bin", dtype=np.uint16).reshape(steps, streams, vocab)
        key_caches = [[np.zeros((HKV, 64, D), dtype=np.uint16) for _ in range(streams)] for _ in range(d["layers"])]
        value_caches = [[np.zeros((HKV, 64, D), dtype=np.uint16) for _ in range(streams)] for _ in range(d["layers"])]
        chain.oracle_token_step(w, talker_hidden, 0, key_caches, value_caches, cos, sin)
        row_input = first_embedding
        state = [int(x) for x in states_before]
        for step in range(steps):
            last = chain.oracle_token_step(w, row_input, step + 1, key_caches, value_caches, cos, sin)
            want = oracle.linear(oracle.rmsnorm(last, w["final_norm"]), w["heads"][step])
            m = oracle.error_metrics(oracle.bf16_to_f32(logits[step]), oracle.bf16_to_f32(want))
            print(f"{mode} step {step}: max_abs {m['max_abs']:.4f} mean_rel {m['mean_rel']:.5f}")
            # per-step budget: the path's mean-relative tolerance (1e-2), and at most 5e-2 absolute on logits that
            # reach 4 (a bf16 ulp is 0.016 at 2 and 0.031 at 4; two layers of one-ulp differences add up to two or
            # three); every step is teacher-forced with the driver's own codes
            scale = float(np.abs(oracle.bf16_to_f32(want)).max())
            assert m["max_abs"] <= 5e-2 and m["mean_rel"] <= 1e-2, (mode, step, m, scale)
            for s in range(streams):
                code, _, state[s], _ = oracle.final_head_sample(logits[step][s], flags=0, top_k=top_k, temperature=0.9, rng_state=state[s])
                assert code == codes[step][s], (mode, step, s)
            row_input = w["embeddings"][step][codes[step]]
        if top_k:
            assert [int(x) for x in np.fromfile(tmp_path / f"rng_{mode}.bin", dtype=np.uint64)] == state
        results[mode] = (codes, logits)
    # the two spellings of step 0 agree with each other as closely as each agrees with the oracle
    m = oracle.error_metrics(oracle.bf16_to_f32(results["staged"][1][0]), oracle.bf16_to_f32(results["positions"][1][0]))
    assert m["max_abs"] <= 5e-2 and m["mean_rel"] <= 1e-2, m
