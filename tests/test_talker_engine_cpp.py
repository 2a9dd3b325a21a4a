"""The C++ host drivers: NativeTalkerEngineB200::decode_device / prefill (host/talker_engine_b200.hpp, counterparts of
the reference's 17.cu:17189-17435 and :16654-16912), the resident serving loop (host/resident_loop_b200.hpp) and the
b200-sxm device directory's main.cu.

On the CPU: everything compiles with the reference's own language level (-std=c++20) in the place the integration
gives it, and the request / result protocol helpers behave.  On the GPU: a two-layer decode step at batch 1 with an
identity page table and at batch 8 with shuffled pages, and a two-layer packed prefill, each against the chain of
the CPU oracle's bit-faithful operators; the profiled path fills the reference's buckets and gives the same bits;
the serving binary answers a request file."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qingming-qwen3-tts_b200"
CPP = ROOT / "tests" / "cpp"
ENGINE_BIN = CPP / "talker_engine_test.bin"
PROTOCOL_BIN = CPP / "resident_protocol_test.bin"
SERVER_BIN = {family: CPP / f"qingming-qwen3-tts_b200-sxm_{family}.bin" for family in ("1.7b", "0.6b")}
HQ, HKV, D = 16, 8, 128


def nvcc(source, binary, extra=()):
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "-O2", "-Xcompiler=-pthread,-Wall,-Wextra",
           "-I", str(ROOT / "include"), "-I", str(PKG / "host"), "-I", str(PKG / "devices" / "b200-sxm"), *extra,
           str(source), "-o", str(binary), "-L", str(PKG / "lib"), "-lqm_attention_b200",
           "-Xlinker", f"-rpath={PKG / 'lib'}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "warning" not in proc.stderr, proc.stderr


def build_all(qm):
    qm.build_library()
    stamp = max(p.stat().st_mtime for p in list((PKG / "host").glob("*.hpp")) + list((PKG / "devices" / "b200-sxm").iterdir())
                + [CPP / "talker_engine_test.cpp", CPP / "resident_protocol_test.cpp", ROOT / "include" / "qm_attention.h"])
    if not ENGINE_BIN.exists() or ENGINE_BIN.stat().st_mtime < stamp:
        nvcc(CPP / "talker_engine_test.cpp", ENGINE_BIN)
    if not PROTOCOL_BIN.exists() or PROTOCOL_BIN.stat().st_mtime < stamp:
        nvcc(CPP / "resident_protocol_test.cpp", PROTOCOL_BIN)
    for family, binary in SERVER_BIN.items():
        if not binary.exists() or binary.stat().st_mtime < stamp:
            define = "-DQINGMING_MODEL_FAMILY_1_7B=1" if family == "1.7b" else "-DQINGMING_MODEL_FAMILY_0_6B=1"
            nvcc(PKG / "devices" / "b200-sxm" / "main.cu", binary, extra=(define,))


def test_drivers_and_device_directory_compile_as_cpp20(qm):
    build_all(qm)
    assert ENGINE_BIN.exists() and all(b.exists() for b in SERVER_BIN.values())


def test_cmake_branch_names_the_files_that_exist():
    text = (PKG / "devices" / "b200-sxm" / "b200-sxm.cmake").read_text()
    assert 'QINGMING_DEVICE STREQUAL "b200-sxm"' in text and "sm_100a" in text and "-std=c++20" in text
    assert "qingming-qwen3-tts_b200-sxm_${QINGMING_MODEL_FAMILY}" in text
    for name in ("devices/b200-sxm/main.cu", "devices/b200-sxm/device.h", "host/talker_engine_b200.hpp",
                 "host/resident_loop_b200.hpp"):
        assert name in text and (PKG / name).exists()


def test_resident_protocol_helpers_on_cpu(qm):
    build_all(qm)
    proc = subprocess.run([str(PROTOCOL_BIN)], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "RESIDENT_PROTOCOL_OK" in proc.stdout


# ------------------------------------------------------------------------------------------------ GPU

def layer_weights(seed, layers, hidden, inter):
    out = []
    for layer in range(layers):
        s = seed + 20 * (layer + 1)
        out.append({
            "input_norm": oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(s, (hidden,)))),
            "post_norm": oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(s + 1, (hidden,)))),
            "q": oracle.scaled_normal_bf16(s + 2, (HQ * D, hidden), 0.06), "k": oracle.scaled_normal_bf16(s + 3, (HKV * D, hidden), 0.06),
            "v": oracle.scaled_normal_bf16(s + 4, (HKV * D, hidden), 0.06), "o": oracle.scaled_normal_bf16(s + 5, (hidden, HQ * D), 0.02),
            "gate": oracle.scaled_normal_bf16(s + 6, (inter, hidden), 0.06), "up": oracle.scaled_normal_bf16(s + 7, (inter, hidden), 0.06),
            "down": oracle.scaled_normal_bf16(s + 8, (hidden, inter), 0.04),
        })
    final_norm = oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(seed + 7, (hidden,))))
    return out, final_norm


def write_weights(directory, weights, final_norm, q_norms, k_norms):
    for index, w in enumerate(weights):
        for name, value in w.items():
            value.tofile(directory / f"l{index}_{name}.bin")
        q_norms[index].tofile(directory / f"l{index}_q_norm.bin")
        k_norms[index].tofile(directory / f"l{index}_k_norm.bin")
    final_norm.tofile(directory / "final_norm.bin")


def run_engine(directory, **options):
    args = [str(ENGINE_BIN), str(directory)] + [f"{k}={v}" for k, v in options.items()]
    proc = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "TALKER_ENGINE_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]
    return proc.stdout


def decode_case(qm, tmp_path, lengths, shuffle_pages, seed):
    hidden, inter, layers = 256, 512, 2
    b = len(lengths)
    weights, final_norm = layer_weights(seed, layers, hidden, inter)
    scs = [scenario.DecodeScenario(seed=seed + layer, lengths=lengths, random_weights=True, shuffle_pages=shuffle_pages)
           for layer in range(layers)]
    sc0 = scs[0]
    # the engine has ONE page table for all layers: every layer's pool is laid out by the first scenario's table
    table = np.maximum(sc0.page_table, 0).astype(np.int32)
    x0 = oracle.normal_bf16(seed + 3, (b, hidden))
    cur = x0
    expected_rows = []
    for layer in range(layers):
        w, sc = weights[layer], scs[layer]
        normed = oracle.rmsnorm(cur, w["input_norm"])
        q = oracle.linear(normed, w["q"]).reshape(b, HQ, D)
        k = oracle.linear(normed, w["k"]).reshape(b, HKV, D)
        v = oracle.linear(normed, w["v"]).reshape(b, HKV, D)
        ctx = np.empty((b, HQ, D), dtype=np.uint16)
        rows = []
        for s in range(b):
            pos = int(sc.lengths[s])
            kc, vc = sc.key_caches[s].copy(), sc.value_caches[s].copy()
            qr = oracle.append(q[s:s + 1], k[s:s + 1], v[s:s + 1], sc.q_w, sc.k_w, sc.cos[pos:pos + 1], sc.sin[pos:pos + 1], pos, kc, vc)
            ctx[s] = oracle.decode_attention(qr, [kc], [vc], [pos + 1], mode="ref")[0]
            rows.append((kc[:, pos].copy(), vc[:, pos].copy()))
        expected_rows.append(rows)
        attn = oracle.linear(ctx.reshape(b, HQ * D), w["o"])
        residual, post = oracle.add_postnorm(cur, attn, w["post_norm"])
        act = oracle.gate_up_swiglu(post, w["gate"], w["up"])
        cur = oracle.linear(act, w["down"], residual=residual)
    want = oracle.rmsnorm(cur, final_norm)

    write_weights(tmp_path, weights, final_norm, [sc.q_w for sc in scs], [sc.k_w for sc in scs])
    x0.tofile(tmp_path / "x.bin")
    sc0.lengths.astype(np.int32).tofile(tmp_path / "positions.bin")
    table.tofile(tmp_path / "page_table.bin")
    for layer, sc in enumerate(scs):
        kp = np.zeros((sc0.num_pages, HKV, 64, D), dtype=np.uint16)
        vp = np.zeros_like(kp)
        for s in range(b):
            oracle.scatter_paged(sc.key_caches[s], table[s], int(sc.lengths[s]), kp)
            oracle.scatter_paged(sc.value_caches[s], table[s], int(sc.lengths[s]), vp)
        kp.tofile(tmp_path / f"kpool{layer}.bin")
        vp.tofile(tmp_path / f"vpool{layer}.bin")
    common = dict(mode="decode", layers=layers, hidden=hidden, intermediate=inter, num_pages=sc0.num_pages,
                  max_pages=sc0.max_pages, batch=b, rope_rows=sc0.max_pos)
    results = {}
    for profile in (0, 1):
        text = run_engine(tmp_path, profile=profile, **common)
        got = np.fromfile(tmp_path / "out_final.bin", dtype=np.uint16).reshape(b, hidden)
        pools = [(np.fromfile(tmp_path / f"out_kpool{layer}.bin", dtype=np.uint16).reshape(sc0.num_pages, HKV, 64, D),
                  np.fromfile(tmp_path / f"out_vpool{layer}.bin", dtype=np.uint16).reshape(sc0.num_pages, HKV, 64, D))
                 for layer in range(layers)]
        results[profile] = (got, pools, text)
    # the fused step and the two-launch profiled path give the same bits
    assert np.array_equal(results[0][0], results[1][0])
    for layer in range(layers):
        assert np.array_equal(results[0][1][layer][0], results[1][1][layer][0])
        assert np.array_equal(results[0][1][layer][1], results[1][1][layer][1])
    got, pools, _ = results[0]
    m = oracle.error_metrics(oracle.bf16_to_f32(got), oracle.bf16_to_f32(want))
    assert m["max_abs"] <= 8e-2 and m["mean_rel"] <= 2e-2, m
    # layer 0's appended rows land where the page table says; their values come from the tensor-core projections,
    # which differ from the oracle's lane-strided sums by a bf16 ulp here and there
    for s in range(b):
        pos = int(sc0.lengths[s])
        page, slot = table[s, pos // 64], pos % 64
        dv = np.abs(oracle.bf16_to_f32(pools[0][1][page, :, slot]) - oracle.bf16_to_f32(expected_rows[0][s][1]))
        dk = np.abs(oracle.bf16_to_f32(pools[0][0][page, :, slot]) - oracle.bf16_to_f32(expected_rows[0][s][0]))
        assert dv.max() <= 2.0 ** -4 and dk.max() <= 2.0 ** -4
        assert (pools[0][1][page, :, slot] == expected_rows[0][s][1]).mean() >= 0.85
    # and nothing else in the pools moved: every other row is what was uploaded
    for layer, sc in enumerate(scs):
        for which, name in ((0, "kpool"), (1, "vpool")):
            before = np.fromfile(tmp_path / f"{name}{layer}.bin", dtype=np.uint16).reshape(sc0.num_pages, HKV, 64, D)
            after = pools[layer][which].copy()
            for s in range(b):
                pos = int(sc0.lengths[s])
                after[table[s, pos // 64], :, pos % 64] = before[table[s, pos // 64], :, pos % 64]
            assert np.array_equal(after, before)
    # the profiled run reports the reference's buckets, each one measured
    text = results[1][2]
    keys = json.loads([line for line in text.splitlines() if line.startswith("{")][-1])
    for name in ("decode", "input_norm", "qkv", "qk_norm_rope_cache", "attention", "o_projection", "residual_postnorm",
                 "gate_up_swiglu", "down_residual", "final_norm"):
        assert keys[f"profile_talker_{name}_ms"] > 0.0, name
        label = "decode" if name == "decode" else name
        assert f"generation_profile_talker_{label}_mean_ms: " in text
    parts = sum(keys[f"profile_talker_{n}_ms"] for n in ("input_norm", "qkv", "qk_norm_rope_cache", "attention", "o_projection",
                                                          "residual_postnorm", "gate_up_swiglu", "down_residual", "final_norm"))
    assert parts <= keys["profile_talker_decode_ms"] * 1.05


@pytest.mark.gpu
def test_cpp_decode_device_batch_1_identity_page_table(qm, tmp_path):
    build_all(qm)
    decode_case(qm, tmp_path, lengths=[200], shuffle_pages=False, seed=700)


@pytest.mark.gpu
def test_cpp_decode_device_batch_8_paged(qm, tmp_path):
    build_all(qm)
    decode_case(qm, tmp_path, lengths=[70, 5, 129, 0, 640, 63, 64, 300], shuffle_pages=True, seed=720)


@pytest.mark.gpu
def test_cpp_prefill_two_layers_packed_varlen(qm, tmp_path):
    build_all(qm)
    hidden, inter, layers, seed = 256, 512, 2, 740
    lengths = [150, 64, 9]
    weights, final_norm = layer_weights(seed, layers, hidden, inter)
    scs = [scenario.PrefillScenario(seed=seed + layer, lengths=lengths, random_weights=True) for layer in range(layers)]
    sc0 = scs[0]
    table = np.maximum(sc0.page_table, 0).astype(np.int32)
    total, b = sc0.total, sc0.batch
    x0 = oracle.normal_bf16(seed + 3, (total, hidden))
    cur = x0
    caches = []
    for layer in range(layers):
        w, sc = weights[layer], scs[layer]
        normed = oracle.rmsnorm(cur, w["input_norm"])
        q = oracle.linear(normed, w["q"]).reshape(total, HQ, D)
        k = oracle.linear(normed, w["k"]).reshape(total, HKV, D)
        v = oracle.linear(normed, w["v"]).reshape(total, HKV, D)
        ctx = np.empty((total, HQ, D), dtype=np.uint16)
        layer_caches = []
        for s in range(b):
            a, e = int(sc0.cu_seqlens[s]), int(sc0.cu_seqlens[s + 1])
            kc = np.zeros((HKV, sc0.max_cache, D), dtype=np.uint16)
            vc = np.zeros_like(kc)
            qr = oracle.append(q[a:e], k[a:e], v[a:e], sc.q_w, sc.k_w, sc0.cos[:e - a], sc0.sin[:e - a], 0, kc, vc)
            ctx[a:e] = oracle.prefill_attention(qr, kc, vc, e - a, 0, mode="ref")
            layer_caches.append((kc, vc))
        caches.append(layer_caches)
        attn = oracle.linear(ctx.reshape(total, HQ * D), w["o"], residual=cur)
        post = oracle.rmsnorm(attn, w["post_norm"])
        act = oracle.gate_up_swiglu(post, w["gate"], w["up"])
        cur = oracle.linear(act, w["down"], residual=attn)
    want = oracle.rmsnorm(cur, final_norm)
    last = (sc0.cu_seqlens[1:] - 1).astype(np.int32)

    write_weights(tmp_path, weights, final_norm, [sc.q_w for sc in scs], [sc.k_w for sc in scs])
    x0.tofile(tmp_path / "x.bin")
    sc0.cu_seqlens.astype(np.int32).tofile(tmp_path / "cu_seqlens.bin")
    table.tofile(tmp_path / "page_table.bin")
    last.tofile(tmp_path / "last_rows.bin")
    run_engine(tmp_path, mode="prefill", layers=layers, hidden=hidden, intermediate=inter, num_pages=sc0.num_pages,
               max_pages=sc0.max_pages, batch=b, rope_rows=sc0.max_pos, total=total, max_seqlen=sc0.max_seqlen)
    got = np.fromfile(tmp_path / "out_final.bin", dtype=np.uint16).reshape(total, hidden)
    m = oracle.error_metrics(oracle.bf16_to_f32(got), oracle.bf16_to_f32(want))
    assert m["max_abs"] <= 8e-2 and m["mean_rel"] <= 2e-2, m
    got_last = np.fromfile(tmp_path / "out_last.bin", dtype=np.uint16).reshape(b, hidden)
    assert np.array_equal(got_last, got[last])
    # layer 0's cache holds every prompt row where the page table says (values within a bf16 ulp or two of the
    # oracle's: they come from the tensor-core projections)
    kp = np.fromfile(tmp_path / "out_kpool0.bin", dtype=np.uint16).reshape(sc0.num_pages, HKV, 64, D)
    vp = np.fromfile(tmp_path / "out_vpool0.bin", dtype=np.uint16).reshape(sc0.num_pages, HKV, 64, D)
    for s in range(b):
        n = int(lengths[s])
        kc, vc = caches[0][s]
        dv = np.abs(oracle.bf16_to_f32(oracle.gather_paged(vp, table[s], n, sc0.max_cache)[:, :n]) - oracle.bf16_to_f32(vc[:, :n]))
        dk = np.abs(oracle.bf16_to_f32(oracle.gather_paged(kp, table[s], n, sc0.max_cache)[:, :n]) - oracle.bf16_to_f32(kc[:, :n]))
        assert dv.max() <= 2.0 ** -4 and dk.max() <= 2.0 ** -4


@pytest.mark.gpu
def test_serving_binary_answers_a_request_file(qm, tmp_path):
    build_all(qm)
    requests = tmp_path / "requests.jsonl"
    lines = [
        {"prompt_rows": 70, "seed": 1, "max_new_tokens": 9, "output": str(tmp_path / "a.bin")},
        {"text": "hello there", "seed": 2, "max_new_tokens": 5, "output": str(tmp_path / "b.bin")},
        {"prompt_rows": 200, "seed": 3, "max_new_tokens": 12, "output": "-"},
        {"prompt_rows": 10, "seed": 4, "output": "-"},                                   # no max_new_tokens: an error line
        {"prompt_rows": 130, "seed": 5, "max_new_tokens": 7, "output": str(tmp_path / "e.bin")},
    ]
    requests.write_text("".join(json.dumps(x) + "\n" for x in lines))
    small = ["--layers", "2", "--hidden", "256", "--intermediate", "512", "--max-streams", "3", "--num-pages", "64",
             "--max-pages", "8", "--eos-check-interval", "3", "--max-prefill-rows", "1024"]

    def serve(extra=()):
        proc = subprocess.run([str(SERVER_BIN["1.7b"]), "--lifecycle", "resident", "--requests", str(requests), *small, *extra],
                              capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
        return [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")], proc.stderr

    results, log = serve()
    assert "resident_ready: True" in log
    by_index = {r["request_index"]: r for r in results if "request_index" in r}
    assert sorted(by_index) == [0, 1, 2, 3, 4]
    assert by_index[3]["status"] == "error" and "max_new_tokens" in by_index[3]["error"]
    for index in (0, 1, 2, 4):
        r, req = by_index[index], lines[index]
        assert r["status"] == "ok" and r["device"] == "b200-sxm" and r["family"] == "1.7b" and r["lifecycle"] == "resident"
        assert r["seed"] == req["seed"] and r["max_new_tokens"] == req["max_new_tokens"] and r["max_new_tokens_capacity"] == 256
        assert 0 <= r["frames"] <= req["max_new_tokens"]
        assert r["eos"] == (r["eos_frame"] >= 0) and (not r["eos"] or r["eos_frame"] == r["frames"])
        assert r["eos"] or r["frames"] == req["max_new_tokens"]
        assert r["ttft_ms"] > 0 and r["generation_ms"] >= r["ttft_ms"] and r["e2e_ms"] >= r["generation_ms"]
        if req["output"] != "-":
            codes = np.fromfile(req["output"], dtype=np.int32)
            assert len(codes) == r["frames"] and ((codes >= 0) & (codes < 3072)).all()
            value = 1469598103934665603
            for byte in codes.tobytes():
                value = ((value ^ byte) * 1099511628211) & ((1 << 64) - 1)
            assert str(value) == r["codec_fnv1a64"]
    assert by_index[1]["prompt_rows"] == 9 + len("hello there")
    # three slots, four valid requests: the fourth had to wait for a stream to retire
    assert by_index[4]["queue_ms"] > 0
    # the same file again gives the same codes (a request file is consumed in a fixed order)
    again, _ = serve()
    for index in (0, 1, 2, 4):
        assert {r["request_index"]: r for r in again if "request_index" in r}[index]["codec_fnv1a64"] == by_index[index]["codec_fnv1a64"]
    # with the profile on, the reference's buckets are reported and the codes do not change
    profiled, log = serve(["--generation-profile"])
    summary = [r for r in profiled if r.get("status") == "profile"][0]
    assert summary["profile_talker_attention_ms"] > 0 and summary["profile_talker_qk_norm_rope_cache_ms"] > 0
    assert "generation_profile_talker_attention_mean_ms: " in log
    for index in (0, 1, 2, 4):
        assert {r["request_index"]: r for r in profiled if "request_index" in r}[index]["codec_fnv1a64"] == by_index[index]["codec_fnv1a64"]
    # the once lifecycle
    proc = subprocess.run([str(SERVER_BIN["1.7b"]), "--lifecycle", "once", "--prompt-rows", "70", "--seed", "1", "--max-new-tokens", "9",
                           "--output", "-", *small], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    once = json.loads([line for line in proc.stdout.splitlines() if line.startswith("{")][0])
    assert once["status"] == "ok" and once["frames"] <= 9
