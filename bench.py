#!/usr/bin/env python
"""Benchmark of the talker attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at N = 1 ("ragged_decode_b64"): batched ragged decode attention in the Qwen3-TTS 1.7B talker shape -
64 streams, KV lengths uniform in [256, 4096] (SplitMix64 seed 1), 16 query / 8 KV heads, head_dim 128, paged bf16
KV cache with 64-token pages and a shuffled page table, QK-RMSNorm + RoPE (theta 1e6) fused into the append.
One step = one decode token through all 28 layers' attention path: per layer the fused norm + RoPE + paged append
and the split-KV attention over every stream.  Each layer has its own pools (about 0.57 GB of KV per layer), so
consecutive launches never find their input in the 126 MB L2.

With N > 1 every rank runs the same workload on its own streams and pool (streams are independent: no collective
on the data path); the reported value is all ranks' bytes over the slowest rank's time (weak scaling).

`--impl reference` times the CPU restatement of the reference's attention (the reference has no CPU
implementation of its own; see the oracle's header) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

Q_HEADS, KV_HEADS, D, PAGE = 16, 8, 128, 64
LAYERS = 28
BATCH = 64
LEN_LO, LEN_HI = 256, 4096
METRIC = "decode attn HBM GB/s"
WORKLOAD = "ragged_decode_b64"


def splitmix64_ints(seed, lo, hi, n):
    """lo + next_u64() % (hi - lo + 1), SplitMix64 - same recipe as the tests, in pure Python for the bench."""
    mask = (1 << 64) - 1
    state, out = seed & mask, []
    for _ in range(n):
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        out.append(lo + z % (hi - lo + 1))
    return np.array(out, dtype=np.int32)


def workload_lengths(rank=0):
    """Existing KV length per stream; the timed step appends one token and attends length + 1 keys.  Every rank
    serves its own 64 streams with the same length draw (its cache contents, page ids and activations differ), so
    that the work per GPU is the same at every N - what weak scaling means."""
    del rank
    return splitmix64_ints(1 * 1000 + 99, LEN_LO, LEN_HI, BATCH)


def algorithmic_bytes_per_layer(lengths):
    # K and V rows of every attended key (2 * 8 heads * 128 * 2 B = 4096 B per key) + q, out, appended rows
    return int((lengths.astype(np.int64) + 1).sum()) * 4096 + len(lengths) * 12288


def workload_config(world):
    """The `config` object of the JSON line - the same in both arms, since both run this workload."""
    return {"workload": WORKLOAD, "streams_per_gpu": BATCH, "kv_len": [LEN_LO, LEN_HI], "q_heads": Q_HEADS,
            "kv_heads": KV_HEADS, "head_dim": D, "page_tokens": PAGE, "layers_per_step": LAYERS,
            "parallelism": f"streams x{world}",
            "l2": "each layer reads its own 0.57 GB of KV; inputs larger than the 126 MB L2"}


def _s64(v):
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def recipe_normal_bf16(seed, shape, device):
    """The input recipe of every test and of both arms, as torch ops: draw k of SplitMix64(seed) is a function of
    seed + (k + 1) * 0x9E3779B97F4A7C15 alone, so the whole tensor is computed in parallel; pairs of 53-bit
    uniforms go through Box-Muller in float64, then float32, then bf16 (round to nearest even), row-major.
    uint64 arithmetic is done in int64 (wrapping multiply and add; logical shifts by masking the sign extension)."""
    import math

    import torch

    n = math.prod(shape)
    out = torch.empty(n + (n & 1), dtype=torch.bfloat16, device=device)
    chunk = 1 << 24                                   # pairs per pass: bounds the int64 / float64 temporaries
    gamma = _s64(0x9E3779B97F4A7C15)

    def draw(idx):
        z = (idx + 1) * gamma + _s64(seed)
        z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _s64(0xBF58476D1CE4E5B9)
        z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _s64(0x94D049BB133111EB)
        z = z ^ ((z >> 31) & ((1 << 33) - 1))
        return ((z >> 11) & ((1 << 53) - 1)).to(torch.float64) * (1.0 / 9007199254740992.0)

    pairs = (n + 1) // 2
    for begin in range(0, pairs, chunk):
        k = torch.arange(begin, min(begin + chunk, pairs), dtype=torch.int64, device=device) * 2
        radius = torch.sqrt(-2.0 * torch.log(draw(k).clamp_min(1e-300)))
        angle = 6.283185307179586476925286766559 * draw(k + 1)
        both = torch.stack((radius * torch.cos(angle), radius * torch.sin(angle)), dim=1).reshape(-1)
        out[2 * begin:2 * begin + both.numel()] = both.to(torch.float32).to(torch.bfloat16)
    return out[:n].view(shape)


def splitmix64_shuffle(seed, n):
    """Fisher-Yates shuffle of 0 .. n-1 driven by SplitMix64(seed), as the tests shuffle page ids."""
    mask = (1 << 64) - 1
    state = seed & mask
    ids = list(range(n))
    for i in range(n - 1, 0, -1):
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        j = z % (i + 1)
        ids[i], ids[j] = ids[j], ids[i]
    return np.array(ids, dtype=np.int32)


def workload_page_table(lengths, rank=0):
    """Page table [BATCH][max_pages] with Fisher-Yates-shuffled page ids, and the number of pages in the pool."""
    pages_per_stream = (lengths + 1 + PAGE - 1) // PAGE
    max_pages, num_pages = int(pages_per_stream.max()), int(pages_per_stream.sum())
    perm = splitmix64_shuffle(1 * 1000 + 8 + 100 * rank, num_pages)
    table = np.zeros((len(lengths), max_pages), dtype=np.int32)
    cursor = 0
    for s, n in enumerate(pages_per_stream):
        table[s, :int(n)] = perm[cursor:cursor + int(n)]
        cursor += int(n)
    return table, num_pages


def layer_tensor_seed(rank, layer, tensor):
    """One RNG stream per (rank, layer, tensor): seed 1 of the workload * 1000 + tensor id, spread over layers and ranks."""
    return 1 * 1000 + tensor + 16 * layer + 1000003 * rank


T_Q, T_K, T_V, T_KPOOL, T_VPOOL = 1, 2, 3, 4, 5


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            cols = [c.strip() for c in line.split(",")]
            if len(cols) < 9:
                continue
            try:
                sm.append(float(cols[1]))
                smax.append(float(cols[2]))
            except ValueError:
                continue
            for name, col in zip(names, cols[5:9]):
                if col.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons),
                "samples": len(sm)}


def five_numbers(samples):
    """min / mean / p50 / p95 / max of a list of samples."""
    x = np.asarray(samples, dtype=np.float64)
    return {"min": float(x.min()), "mean": float(x.mean()), "p50": float(np.percentile(x, 50)),
            "p95": float(np.percentile(x, 95)), "max": float(x.max()), "n": int(x.size)}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------- reference arm (CPU)

def cpu_attention_sample(q_rot_bits, key_caches, value_caches, key_lens, repeats):
    """Times the oracle's reference-faithful decode attention (all host threads) on the given streams."""
    from oracle import qm_oracle as oracle

    best = float("inf")
    out = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = oracle.decode_attention(q_rot_bits, key_caches, value_caches, key_lens, mode="ref")
        best = min(best, time.perf_counter() - t0)
    return best, out


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def use_all_host_threads():
    """The CPU legs run OpenMP loops; a launcher (torchrun) may have exported OMP_NUM_THREADS=1 for its workers.
    Returns the thread count in use."""
    import ctypes

    cores = host_cores()
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        cores = int(os.environ.get("OMP_NUM_THREADS", cores))
    return cores


def layer0_inputs(device, rank=0):
    """Layer 0 of the workload, drawn by the input recipe: pools [num_pages][8][64][128] (the tokens already cached,
    placed through the page table - a page's unused slots hold draws too, nobody reads them), the new token's q, k,
    v, the lengths and the page table.  Both arms call this, so they see the same tensors."""
    lengths = workload_lengths(rank)
    table, num_pages = workload_page_table(lengths, rank)
    kpool = recipe_normal_bf16(layer_tensor_seed(rank, 0, T_KPOOL), (num_pages, KV_HEADS, PAGE, D), device)
    vpool = recipe_normal_bf16(layer_tensor_seed(rank, 0, T_VPOOL), (num_pages, KV_HEADS, PAGE, D), device)
    q = recipe_normal_bf16(layer_tensor_seed(rank, 0, T_Q), (BATCH, Q_HEADS, D), device)
    k = recipe_normal_bf16(layer_tensor_seed(rank, 0, T_K), (BATCH, KV_HEADS, D), device)
    v = recipe_normal_bf16(layer_tensor_seed(rank, 0, T_V), (BATCH, KV_HEADS, D), device)
    return {"lengths": lengths, "table": table, "num_pages": num_pages, "kpool": kpool, "vpool": vpool, "q": q, "k": k, "v": v}


def _bits(t):
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def oracle_decode_step_inputs(inputs):
    """What the reference's decode step sees for layer 0, in the reference's own cache layout: per stream the
    contiguous [kv_head][max_cache][128] caches gathered through the page table, with the new token appended by the
    oracle's restatement of the fused norm + RoPE + append kernel, and the normed, roped queries."""
    from oracle import qm_oracle as oracle

    lengths, table = inputs["lengths"], inputs["table"]
    kpool, vpool = _bits(inputs["kpool"]), _bits(inputs["vpool"])
    q, k, v = _bits(inputs["q"]), _bits(inputs["k"]), _bits(inputs["v"])
    ones = oracle.f32_to_bf16(np.ones(D, dtype=np.float32))
    cos, sin = oracle.make_rope(LEN_HI + 2)
    q_rot = np.empty_like(q)
    key_caches, value_caches = [], []
    for s in range(len(lengths)):
        pos = int(lengths[s])
        kc = oracle.gather_paged(kpool, table[s], pos, pos + 1)
        vc = oracle.gather_paged(vpool, table[s], pos, pos + 1)
        q_rot[s:s + 1] = oracle.append(q[s:s + 1], k[s:s + 1], v[s:s + 1], ones, ones, cos[pos:pos + 1], sin[pos:pos + 1], pos, kc, vc)
        key_caches.append(kc)
        value_caches.append(vc)
    return q_rot, key_caches, value_caches


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import qm_oracle as oracle

    oracle.lib()
    cores = use_all_host_threads()
    # the same tensors as the GPU arm's layer 0 (drawn on the GPU when there is one: the draw is not what is timed)
    inputs = layer0_inputs("cuda" if torch.cuda.is_available() else "cpu")
    lens = inputs["lengths"]
    q_rot, key_caches, value_caches = oracle_decode_step_inputs(inputs)
    bytes_per_step = algorithmic_bytes_per_layer(lens)
    for _ in range(args.warmup):
        oracle.decode_attention(q_rot, key_caches, value_caches, lens + 1, mode="ref")
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.decode_attention(q_rot, key_caches, value_caches, lens + 1, mode="ref")
    seconds = time.perf_counter() - t0
    gbs = bytes_per_step * args.steps / seconds / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"one layer of all {BATCH} streams per step (1/{LAYERS} of a GPU step), on the GPU arm's "
                                   "layer-0 tensors; bf16-faithful restatement of the reference kernels, OpenMP over "
                                   "(stream, kv head)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- our arm (GPU)

def run_ours(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = entry.load_package()
    pkg.load_library()

    # Inputs by the recipe of the tests (SplitMix64 -> Box-Muller -> bf16), one RNG stream per (rank, layer, tensor);
    # layer 0 of rank 0 is what the reference arm and the CPU-baseline leg run on.
    first = layer0_inputs("cuda", rank)
    lengths, table, num_pages = first["lengths"], first["table"], first["num_pages"]
    max_pages = table.shape[1]
    eng = pkg.TalkerAttention(layers=LAYERS, num_pages=num_pages, q_heads=Q_HEADS, kv_heads=KV_HEADS,
                              max_positions=LEN_HI + 2)
    q = torch.empty((LAYERS, BATCH, Q_HEADS, D), dtype=torch.bfloat16, device="cuda")
    k = torch.empty((LAYERS, BATCH, KV_HEADS, D), dtype=torch.bfloat16, device="cuda")
    v = torch.empty_like(k)
    for layer in range(LAYERS):
        kview, vview = eng.pool_view(layer)
        if layer == 0:
            kview.copy_(first["kpool"]); vview.copy_(first["vpool"])
            q[0].copy_(first["q"]); k[0].copy_(first["k"]); v[0].copy_(first["v"])
        else:
            kview.copy_(recipe_normal_bf16(layer_tensor_seed(rank, layer, T_KPOOL), tuple(kview.shape), "cuda"))
            vview.copy_(recipe_normal_bf16(layer_tensor_seed(rank, layer, T_VPOOL), tuple(vview.shape), "cuda"))
            q[layer].copy_(recipe_normal_bf16(layer_tensor_seed(rank, layer, T_Q), (BATCH, Q_HEADS, D), "cuda"))
            k[layer].copy_(recipe_normal_bf16(layer_tensor_seed(rank, layer, T_K), (BATCH, KV_HEADS, D), "cuda"))
            v[layer].copy_(recipe_normal_bf16(layer_tensor_seed(rank, layer, T_V), (BATCH, KV_HEADS, D), "cuda"))
    del first
    torch.cuda.empty_cache()
    page_table = torch.from_numpy(table).cuda()
    positions = torch.from_numpy(lengths).cuda()
    seq_lens = torch.from_numpy(lengths + 1).cuda()
    ones = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    q_rot = torch.empty_like(q)
    out = torch.empty_like(q)
    eng.workspace(BATCH)

    def step_device():
        # one launch per layer: QK-RMSNorm + RoPE + paged append + split-KV attention (qm_decode_step)
        for layer in range(LAYERS):
            eng.decode_step(layer, q[layer], k[layer], v[layer], ones, ones, positions, page_table, out=out[layer])

    # Host-buffer path.  The step's q/k/v (all layers) live in pinned host memory and the contexts go back to pinned
    # host memory, inside the timed region.  Copies are issued per chunk of layers on their own streams so that
    # the transfer of one chunk overlaps the kernels of another, as a serving loop would do; every copy and kernel
    # of the K timed steps still lies between the two timing events.
    # Chunk sizes grow from one layer (so that only a small copy stands before the step's first kernel, and the
    # copy of a chunk is finished before the kernels of the chunks ahead of it are) and shrink again towards the
    # end (so that only a small read-back is left when the last kernel ends).
    if LAYERS >= 16:
        bounds = sorted({0, 1, 3, 8, LAYERS // 2 + 4, LAYERS - 4, LAYERS - 1, LAYERS})
    elif LAYERS >= 6:
        bounds = [0, 1, LAYERS // 2, LAYERS - 1, LAYERS]
    else:
        bounds = [0, LAYERS]
    n_chunks = len(bounds) - 1
    per_layer = BATCH * (Q_HEADS + 2 * KV_HEADS) * D
    qkv_host = torch.empty((LAYERS, per_layer), dtype=torch.bfloat16).pin_memory()
    nq, nk = BATCH * Q_HEADS * D, BATCH * KV_HEADS * D
    qkv_host[:, :nq].copy_(q.reshape(LAYERS, -1).cpu())
    qkv_host[:, nq:nq + nk].copy_(k.reshape(LAYERS, -1).cpu())
    qkv_host[:, nq + nk:].copy_(v.reshape(LAYERS, -1).cpu())
    out_host = torch.empty((LAYERS, BATCH, Q_HEADS, D), dtype=torch.bfloat16).pin_memory()
    qkv_dev = torch.empty((LAYERS, per_layer), dtype=torch.bfloat16, device="cuda")
    h2d_bytes = qkv_dev.numel() * 2
    d2h_bytes = out_host.numel() * 2
    h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
    ev_h2d = [torch.cuda.Event() for _ in range(n_chunks)]
    ev_comp = [torch.cuda.Event() for _ in range(n_chunks)]
    ev_d2h = [torch.cuda.Event() for _ in range(n_chunks)]

    def step_e2e():
        main = torch.cuda.current_stream()
        h2d_stream.wait_stream(main)
        for c in range(n_chunks):
            lo, hi = bounds[c], bounds[c + 1]
            with torch.cuda.stream(h2d_stream):
                h2d_stream.wait_event(ev_comp[c])          # the previous step's kernels have consumed this chunk
                qkv_dev[lo:hi].copy_(qkv_host[lo:hi], non_blocking=True)
                ev_h2d[c].record(h2d_stream)
            main.wait_event(ev_h2d[c])
            main.wait_event(ev_d2h[c])                     # the previous step's context of this chunk has left
            for layer in range(lo, hi):
                row = qkv_dev[layer]
                eng.decode_step(layer, row[:nq].view(BATCH, Q_HEADS, D), row[nq:nq + nk].view(BATCH, KV_HEADS, D),
                                row[nq + nk:].view(BATCH, KV_HEADS, D), ones, ones, positions, page_table,
                                out=out[layer])
            ev_comp[c].record(main)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(ev_comp[c])
                out_host[lo:hi].copy_(out[lo:hi], non_blocking=True)
                ev_d2h[c].record(d2h_stream)
        # The read-back of the last chunk may still run while the next step starts (the wait on ev_d2h above keeps
        # a context from being overwritten before it has left); the barrier that ends the timed region waits for it.

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, before_end=None):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            fn()
        if before_end is not None:
            before_end()          # work on side streams joins the timing stream before the end event
        end.record()
        barrier()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step_device()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    total_ms = timed(step_device, args.steps)
    # the dominant kernel alone (the fused decode step), per launch, CUDA events on the launching stream
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(LAYERS)]
    attn_samples = []
    for _ in range(max(2, min(args.steps, 5))):
        torch.cuda.synchronize()
        for layer in range(LAYERS):
            ev[layer][0].record()
            eng.decode_step(layer, q[layer], k[layer], v[layer], ones, ones, positions, page_table, out=out[layer])
            ev[layer][1].record()
        torch.cuda.synchronize()
        attn_samples += [a.elapsed_time(b) for a, b in ev]
    # q_rot of layer 0, for the parity check against the oracle (same bits as the fused step uses internally)
    eng.launch_qk_norm_rope_cache_m1(0, q[0], k[0], v[0], ones, ones, positions, page_table, q_rot=q_rot[0])
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps, before_end=lambda: torch.cuda.current_stream().wait_stream(d2h_stream))
    clocks = sampler.stop()
    status = eng.status()

    layer_bytes = algorithmic_bytes_per_layer(lengths)
    if world > 1:
        t = torch.tensor([float(layer_bytes)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)
        total_layer_bytes = float(t.item())
    else:
        total_layer_bytes = float(layer_bytes)
    ms_per_step = total_ms / args.steps
    value = total_layer_bytes * LAYERS / (ms_per_step * 1e-3) / 1e9
    e2e_value = total_layer_bytes * LAYERS / (e2e_ms / args.steps * 1e-3) / 1e9
    attn_ms = float(np.mean(attn_samples))
    attn_bytes = layer_bytes                         # K/V rows of every attended key, q/k/v in, appended rows and context out
    peak, peak_kind = load_peaks()
    # the timed region launches this one kernel LAYERS times per step and nothing else, so its average launch
    # duration there is the step time over LAYERS; the per-launch event samples (launches serialised by the
    # events between them) are reported beside it
    traffic, traffic_note = stored_traffic()
    launch_ms = ms_per_step / LAYERS
    achieved = attn_bytes / (launch_ms * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world),
        "us_per_layer": ms_per_step * 1e3 / LAYERS,
        "attention_us_per_layer": attn_ms * 1e3,
        "launch_us_distribution": five_numbers([x * 1e3 for x in attn_samples]),
        "pct_of_measured_hbm_peak": 100.0 * value / world / peak,
        "pct_of_nominal_8tbs": 100.0 * value / world / 8000.0,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": e2e_ms / args.steps,
                "note": "every layer's q/k/v copied from pinned host memory and every context copied back inside the "
                        "timed region, in chunks of layers (small at both ends of the step) on copy streams so transfers overlap kernels, the last read-back overlapping the next step's first kernels; the KV "
                        "cache is device-resident state by design"},
        "gpu_launches": args.steps * LAYERS,
        "roofline": {"bound": "hbm", "kernel": "qm_decode_splitkv_kernel<fused>", "achieved": achieved,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_note": traffic_note, "bytes_per_launch": attn_bytes, "us_per_launch": launch_ms * 1e3,
                     "us_per_launch_isolated": attn_ms * 1e3},
        "clocks": clocks,
        "device_status": status,
    }

    if rank == 0 and not args.no_cpu_baseline:
        line["cpu_baseline"], line["parity"] = cpu_baseline_and_parity(eng, q_rot[0], out[0], lengths, table)
        line["reference_gpu_kernel"] = reference_gpu_kernel_timing(eng, q_rot[0], lengths, table)
    eng.close()
    del q, k, v, q_rot, out
    torch.cuda.empty_cache()
    def guarded(name, section):
        """A secondary section that raises must not take the primary line down with it: its entry then holds the
        error text instead of figures (every rank takes the same path when the error is one every rank meets)."""
        try:
            return section()
        except Exception as exc:
            sys.stderr.write(f"bench.py: section {name} failed: {type(exc).__name__}: {exc}\n")
            return {"error": f"{type(exc).__name__}: {exc}"[:400]}

    def summed_over_ranks(entry, key, total_key):
        if world > 1:
            t = torch.tensor([entry.get(key, 0.0) or 0.0], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)
            entry[total_key] = float(t.item())

    if not args.no_prefill:
        prefill = guarded("prefill", lambda: run_prefill_section(pkg, max(3, min(args.steps, 10)), args.warmup, check=rank == 0))
        summed_over_ranks(prefill, "tflops", "tflops_all_gpus")
        line["prefill"] = prefill
    if not args.no_long_context:
        line["long_context"] = guarded("long_context", lambda: run_long_context_section(pkg, world, rank, args.steps))
    if not args.no_single_stream and rank == 0:
        line["single_stream"] = guarded("single_stream", lambda: run_single_stream_section(pkg, args.steps))
    if not args.no_talker_step and rank == 0:
        line["code_predictor"] = guarded("code_predictor", lambda: run_code_predictor_section(pkg, args.steps))
    if not args.no_talker_step:
        talker = guarded("talker_step", lambda: run_talker_step_section(pkg, args.steps))
        summed_over_ranks(talker, "tokens_per_s", "tokens_per_s_all_gpus")
        line["talker_step"] = talker
    if rank == 0:
        # the figures a reader looks for first, ahead of everything else on the line
        lc, pf, tk = line.get("long_context", {}), line.get("prefill", {}), line.get("talker_step", {})
        summary = {
            "decode_gbs": line["value"], "decode_frac_of_measured_hbm": line["roofline"]["frac"],
            "decode_parity_ok": line.get("parity", {}).get("ok"),
            "prefill_tflops": pf.get("tflops"), "prefill_parity_ok": pf.get("parity", {}).get("ok"),
            "long_context_us": lc.get("us_per_layer"), "long_context_us_nccl": lc.get("us_per_layer_nccl_all_gather"),
            "long_context_us_two_launch": lc.get("us_per_layer_two_launch_peer_exchange"),
            "long_context_us_fused": lc.get("us_per_layer_fused_peer_exchange"),
            "long_context_parity_ok": lc.get("parity", {}).get("ok"),
            "talker_tok_s_all_gpus": tk.get("tokens_per_s_all_gpus", tk.get("tokens_per_s")),
            "talker_ms_per_step": tk.get("ms_per_step"),
            "profile_talker_attention_ms": tk.get("profile_talker_attention_ms"),
            "profile_talker_qk_norm_rope_cache_ms": tk.get("profile_talker_qk_norm_rope_cache_ms"),
            "code_predictor_ms_per_frame": line.get("code_predictor", {}).get("ms_per_frame"),
        }
        print(json.dumps({"summary": summary, **line}))
    if world > 1:
        dist.destroy_process_group()


def stored_traffic():
    """DRAM bytes (read + write) per launch of the decode kernel on this workload, from the ncu capture summarised in
    profiles/decode_step_traffic.txt.  The file records the SHA-256 of the kernel source it was captured on; when the
    source has changed since, the number is withheld rather than reported stale."""
    import hashlib

    path = ROOT / "profiles" / "decode_step_traffic.txt"
    if not path.exists():
        return None, "no capture on file"
    record = json.loads(path.read_text())
    source = ROOT / "qingming-qwen3-tts_b200" / "csrc" / "qm_decode.cu"
    current = hashlib.sha256(source.read_bytes()).hexdigest() if source.exists() else None
    if record.get("kernel_source_sha256") != current:
        return None, "the capture on file was taken on another version of qm_decode.cu"
    return record["dram_bytes_read"] + record["dram_bytes_write"], "ncu dram__bytes_read.sum + dram__bytes_write.sum, 2-layer capture"


def reference_gpu_kernel_timing(eng, q_rot0, lengths, table):
    """The reference's own decode attention kernel (talker_attention_gqa2_m1_locality_kernel, 8 CTAs, one stream per
    launch) timed on this GPU through the harness built from the reference's sources, on three streams of the
    workload's layer 0.  Reported beside the CPU baseline; `unavailable` where the harness was not built."""
    from oracle import qm_oracle as oracle

    if not oracle.ref_available():
        return {"unavailable": "the harness around the reference's kernels is not built here (it needs the reference's sources at build time)"}
    import torch

    try:
        kview, vview = eng.pool_view(0)
        kpool, vpool = _bits(kview), _bits(vview)
        q_bits = _bits(q_rot0)
        order = np.argsort(lengths)
        picks = [int(order[0]), int(order[len(order) // 2]), int(order[-1])]
        rows = []
        for s in picks:
            n = int(lengths[s]) + 1
            kc = oracle.gather_paged(kpool, table[s], n, n)
            vc = oracle.gather_paged(vpool, table[s], n, n)
            _, ms = oracle.ref_attention(q_bits[s:s + 1], kc, vc, 1, n - 1, iterations=20)
            rows.append({"keys": n, "us": ms * 1e3, "gbs": (n * 4096 + 12288) / (ms * 1e-3) / 1e9})
        torch.cuda.synchronize()
        return {"kernel": "talker_attention_gqa2_m1_locality_kernel (reference, batch 1, 8 CTAs)", "streams": rows,
                "gbs_mean": float(np.mean([r["gbs"] for r in rows]))}
    except Exception as exc:        # the harness is optional: never let it take the bench line down
        return {"unavailable": f"{type(exc).__name__}: {exc}"}


def prefill_lengths():
    """Prompt lengths of the prefill workload: 8 sequences, uniform in [1024, 8192], SplitMix64 seed 2."""
    return splitmix64_ints(2 * 1000 + 99, 1024, 8192, 8)


def run_prefill_section(pkg, steps, warmup, n_seqs=8, check=True):
    """Secondary measurement: varlen causal prefill (fused append + tcgen05 attention), 1.7B talker shape."""
    import torch

    lengths = prefill_lengths()[:n_seqs]
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    total = int(cu[-1])
    pages_per_seq = (lengths + PAGE - 1) // PAGE
    max_pages = int(pages_per_seq.max())
    num_pages = int(pages_per_seq.sum())
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2000)
    eng = pkg.TalkerAttention(layers=1, num_pages=num_pages, q_heads=Q_HEADS, kv_heads=KV_HEADS,
                              max_positions=int(lengths.max()))
    perm = splitmix64_shuffle(2 * 1000 + 8, num_pages)
    table = np.zeros((len(lengths), max_pages), dtype=np.int32)
    cursor = 0
    for s, n in enumerate(pages_per_seq):
        table[s, :n] = perm[cursor:cursor + n]
        cursor += int(n)
    page_table = torch.from_numpy(table).cuda()
    cu_dev = torch.from_numpy(cu).cuda()
    # pre-norm projections ~ N(0, 1) by the input recipe, seed 2 (one RNG stream per tensor)
    q = recipe_normal_bf16(2 * 1000 + 1, (total, Q_HEADS, D), "cuda")
    k = recipe_normal_bf16(2 * 1000 + 2, (total, KV_HEADS, D), "cuda")
    v = recipe_normal_bf16(2 * 1000 + 3, (total, KV_HEADS, D), "cuda")
    ones = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    q_rot = torch.empty_like(q)
    out = torch.empty_like(q)
    max_len = int(lengths.max())

    def step():
        eng.prefill_norm_rope_scatter(0, q, k, v, ones, ones, cu_dev, page_table, q_rot=q_rot)
        eng.launch_attention_prefill(0, q_rot, cu_dev, page_table, max_len, out=out)

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    append_ms, attn_ms = [], []
    for _ in range(steps):
        e[0].record()
        eng.prefill_norm_rope_scatter(0, q, k, v, ones, ones, cu_dev, page_table, q_rot=q_rot)
        e[1].record()
        eng.launch_attention_prefill(0, q_rot, cu_dev, page_table, max_len, out=out)
        e[2].record()
        torch.cuda.synchronize()
        append_ms.append(e[0].elapsed_time(e[1]))
        attn_ms.append(e[1].elapsed_time(e[2]))
    parity = prefill_parity(eng, q_rot, out, lengths, cu, table) if check else None
    # ---- one whole decoder layer of the prefill loop over the same tokens (17.cu:16700-16880): input norm, q/k/v
    # projections, norm + RoPE + scatter, attention, o-projection + residual, post-norm, gate/up + SwiGLU,
    # down-projection + residual; weights ~ N(0, 0.02) in the 1.7B talker shape
    hidden_dim, inter = 2048, 6144
    nq, nk = Q_HEADS * D, KV_HEADS * D

    def weight(*shape):
        return (torch.randn(*shape, generator=gen, device="cuda") * 0.02).to(torch.bfloat16)

    w_q, w_k, w_v, w_o = weight(nq, hidden_dim), weight(nk, hidden_dim), weight(nk, hidden_dim), weight(hidden_dim, nq)
    w_gate, w_up, w_down = weight(inter, hidden_dim), weight(inter, hidden_dim), weight(hidden_dim, inter)
    norm_w = torch.ones(hidden_dim, dtype=torch.bfloat16, device="cuda")
    hidden_rows = torch.randn(total, hidden_dim, generator=gen, device="cuda").to(torch.bfloat16)

    def buf(cols):
        return torch.empty((total, cols), dtype=torch.bfloat16, device="cuda")

    normed, residual, post, act, nxt = buf(hidden_dim), buf(hidden_dim), buf(hidden_dim), buf(inter), buf(hidden_dim)
    ql, kl, vl = buf(nq), buf(nk), buf(nk)

    def layer():
        eng.launch_rmsnorm(hidden_rows, norm_w, out=normed)
        eng.linear_generic(normed, w_q, out=ql)
        eng.linear_generic(normed, w_k, out=kl)
        eng.linear_generic(normed, w_v, out=vl)
        eng.prefill_norm_rope_scatter(0, ql.view(total, Q_HEADS, D), kl.view(total, KV_HEADS, D), vl.view(total, KV_HEADS, D),
                                      ones, ones, cu_dev, page_table, q_rot=q_rot)
        eng.launch_attention_prefill(0, q_rot, cu_dev, page_table, max_len, out=out)
        eng.linear_generic(out.view(total, nq), w_o, residual=hidden_rows, out=residual)
        eng.launch_rmsnorm(residual, norm_w, out=post)
        eng.gate_up_swiglu_rows(post, w_gate, w_up, out=act)
        eng.linear_generic(act, w_down, residual=residual, out=nxt)

    for _ in range(3):
        layer()
    torch.cuda.synchronize()
    layer_ms = []
    for _ in range(steps):
        e[0].record()
        layer()
        e[1].record()
        torch.cuda.synchronize()
        layer_ms.append(e[0].elapsed_time(e[1]))
    status = eng.status()
    flops = float(sum(4096 * int(n) * (int(n) + 1) for n in lengths))
    projection_flops = 2.0 * total * (hidden_dim * (nq + 2 * nk) + nq * hidden_dim + 3 * hidden_dim * inter)
    layer_mean = float(np.mean(layer_ms))
    attn = float(np.mean(attn_ms))
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    burst = float(peaks.get("bf16_tflops", 1590.0))
    sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))
    tflops = flops / (attn * 1e-3) / 1e12
    result = {
        "workload": "varlen_causal_prefill_b8", "prompt_lengths": [int(n) for n in lengths], "tokens": total,
        "algorithmic_flops": flops, "attention_ms": attn, "attention_ms_min": float(np.min(attn_ms)),
        "append_ms": float(np.mean(append_ms)), "tflops": tflops,
        "frac_of_measured_burst_peak": tflops / burst, "frac_of_measured_sustained_peak": tflops / sustained,
        "peak_tflops_burst": burst, "peak_tflops_sustained": sustained, "device_status": status, "parity": parity,
        "append_gbs": total * (Q_HEADS + 2 * KV_HEADS) * D * 2 * 2 / (float(np.mean(append_ms)) * 1e-3) / 1e9,
        "layer": {"what": "one whole prefill decoder layer on the same tokens, 10 launches of this library",
                  "ms": layer_mean, "projection_flops": projection_flops,
                  "tflops": (flops + projection_flops) / (layer_mean * 1e-3) / 1e12,
                  "prompt_tokens_per_s_28_layers": total / (28 * layer_mean * 1e-3)},
    }
    eng.close()
    return result


def prefill_parity(eng, q_rot, out, lengths, cu, table, block=96):
    """Checks the prefill attention output of EVERY prompt of the workload against the fp32 oracle on the first,
    the middle and the last `block` query rows (each row attends all keys up to its own position, so the last rows
    exercise the whole cache of a prompt of up to 8 192 tokens), using the cache bits the append kernel wrote."""
    import torch

    from oracle import qm_oracle as oracle

    oracle.lib()
    use_all_host_threads()
    kview, vview = eng.pool_view(0)
    kpool, vpool = _bits(kview), _bits(vview)
    q_bits, out_bits = _bits(q_rot), _bits(out)
    worst = {"max_abs": 0.0, "mean_rel": 0.0, "mean_rel_elementwise": 0.0}
    num = den = 0.0
    rows_checked = 0
    for s, n in enumerate(int(x) for x in lengths):
        a = int(cu[s])
        kc = oracle.gather_paged(kpool, table[s], n, n)
        vc = oracle.gather_paged(vpool, table[s], n, n)
        spans = {(0, min(block, n)), (max(0, n // 2 - block // 2), min(n, n // 2 + block // 2)), (max(0, n - block), n)}
        for begin, end in sorted(spans):
            want = oracle.prefill_attention(q_bits[a:a + n], kc, vc, n, 0, rows=(begin, end), mode="fp32")[begin:end]
            got = oracle.bf16_to_f32(out_bits[a + begin:a + end])
            diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
            worst["max_abs"] = max(worst["max_abs"], float(diff.max()))
            num += float(diff.sum())
            den += float(np.abs(want).astype(np.float64).sum())
            rows_checked += end - begin
    worst["mean_rel"] = num / max(den, 1e-30)
    del worst["mean_rel_elementwise"]
    return {"against": "fp32 oracle on the cache bits the append kernel wrote", "prompts_checked": len(lengths),
            "rows_checked": rows_checked, "rows": f"first, middle and last {block} rows of every prompt", **worst,
            "tolerance": {"max_abs": 2e-2, "mean_rel": 1e-2},
            "ok": bool(worst["max_abs"] <= 2e-2 and worst["mean_rel"] <= 1e-2)}


def run_talker_step_section(pkg, steps):
    """Secondary measurement: one greedy decode step of a random-init Qwen3 decoder in the 1.7B talker shape
    (28 layers, hidden 2048, 16 q / 8 kv heads, head_dim 128, SwiGLU 6144, RMSNorm, QK-norm, RoPE 1e6, codec vocab
    3072), 32 streams per GPU at context 2048, weights ~ N(0, 0.02).  Every layer runs through this library's
    entry points in the reference's decode_device order (17.cu:17247-17397): RMSNorm, fused QKV projection,
    qm_decode_step, o-projection, add + post-norm, gate/up SwiGLU, down-projection + residual; then the final norm
    and the codec head projection; the next code comes from qm_final_head_sample (greedy, with the reference's
    repetition penalty and token suppression) and its embedding row from qm_embedding_gather.  The step is
    captured in one CUDA graph."""
    import torch

    hidden, inter, vocab, layers, streams, context = 2048, 6144, 3072, 28, 32, 2048
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4000)

    def weight(*shape):
        return (torch.randn(*shape, generator=gen, device="cuda") * 0.02).to(torch.bfloat16)

    nq, nk = Q_HEADS * D, KV_HEADS * D
    w_q = [weight(nq, hidden) for _ in range(layers)]
    w_k = [weight(nk, hidden) for _ in range(layers)]
    w_v = [weight(nk, hidden) for _ in range(layers)]
    w_o = [weight(hidden, nq) for _ in range(layers)]
    w_gate = [weight(inter, hidden) for _ in range(layers)]
    w_up = [weight(inter, hidden) for _ in range(layers)]
    w_down = [weight(hidden, inter) for _ in range(layers)]
    norm_w = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    head = weight(vocab, hidden)
    embed = weight(vocab, hidden)
    ones = torch.ones(D, dtype=torch.bfloat16, device="cuda")

    max_new = 64
    pages_per_stream = (context + max_new + PAGE - 1) // PAGE
    num_pages = streams * pages_per_stream
    eng = pkg.TalkerAttention(layers=layers, num_pages=num_pages, q_heads=Q_HEADS, kv_heads=KV_HEADS,
                              max_positions=context + max_new + 1)
    for layer in range(layers):
        for view in eng.pool_view(layer):
            view.normal_(generator=gen)
    page_table = torch.randperm(num_pages, generator=gen, device="cuda").to(torch.int32).view(streams, pages_per_stream)
    positions = torch.full((streams,), context, dtype=torch.int32, device="cuda")
    tokens = torch.randint(0, vocab, (streams,), generator=gen, device="cuda").to(torch.int32)
    eng.workspace(streams)

    def buf(cols):
        return torch.empty((streams, cols), dtype=torch.bfloat16, device="cuda")

    x_a, x_b, normed, attn_proj, residual, post, act = buf(hidden), buf(hidden), buf(hidden), buf(hidden), buf(hidden), buf(hidden), buf(inter)
    q, k, v = buf(nq), buf(nk), buf(nk)
    context_out = torch.zeros((streams, Q_HEADS, D), dtype=torch.bfloat16, device="cuda")
    logits = buf(vocab)

    history = torch.zeros((streams, 8192), dtype=torch.int32, device="cuda")
    generation = torch.zeros((streams,), dtype=torch.int32, device="cuda")
    sample_flags = pkg.QM_SAMPLE_REPETITION | pkg.QM_SAMPLE_SUPPRESS | pkg.QM_SAMPLE_RECORD

    q_rot = torch.empty((streams, Q_HEADS, D), dtype=torch.bfloat16, device="cuda")
    seq_lens = torch.empty((streams,), dtype=torch.int32, device="cuda")
    spans = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(layers)]

    def one_step(with_attention=True, profile=False):
        cur, nxt = x_a, x_b
        eng.embedding_gather(embed, tokens, out=cur)
        if profile:
            torch.add(positions, 1, out=seq_lens)
        for layer in range(layers):
            eng.launch_rmsnorm(cur, norm_w, out=normed)
            eng.launch_qkv_m1(normed, w_q[layer], w_k[layer], w_v[layer], out=(q, k, v))
            if profile:
                # the attention path as the reference's two launches, each inside its own event span
                spans[layer][0].record()
                eng.launch_qk_norm_rope_cache_m1(layer, q.view(streams, Q_HEADS, D), k.view(streams, KV_HEADS, D),
                                                 v.view(streams, KV_HEADS, D), ones, ones, positions, page_table, q_rot=q_rot)
                spans[layer][1].record()
                eng.launch_attention(layer, q_rot, seq_lens, page_table, out=context_out)
                spans[layer][2].record()
            elif with_attention:
                eng.decode_step(layer, q.view(streams, Q_HEADS, D), k.view(streams, KV_HEADS, D),
                                v.view(streams, KV_HEADS, D), ones, ones, positions, page_table, out=context_out)
            eng.launch_linear_m1(context_out.view(streams, nq), w_o[layer], out=attn_proj)
            eng.launch_add_postnorm_m1(cur, attn_proj, norm_w, residual=residual, normalized=post)
            eng.launch_gate_up_swiglu_m1(post, w_gate[layer], w_up[layer], out=act)
            eng.launch_linear_m1(act, w_down[layer], residual=residual, out=nxt)
            cur, nxt = nxt, cur
        eng.launch_rmsnorm(cur, norm_w, out=normed)
        eng.launch_linear_m1(normed, head, out=logits)
        # greedy: cast, repetition penalty, token suppression, argmax, record - one launch for all streams
        eng.final_head_sample(logits, generation, history, flags=sample_flags, top_k=0, codes=tokens)
        positions.add_(1)
        generation.add_(1)

    def capture(with_attention):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                one_step(with_attention)
            positions.fill_(context)
            generation.zero_()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_step(with_attention)
        positions.fill_(context)
        generation.zero_()
        return graph

    def time_graph(graph, n):
        for _ in range(3):
            graph.replay()
        positions.fill_(context)
        generation.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        positions.fill_(context)
        generation.zero_()
        return a.elapsed_time(b) / n

    n = max(5, min(steps, 30))
    full_ms = time_graph(capture(True), n)
    rest_ms = time_graph(capture(False), n)
    # The two buckets of the reference's profile that cover this path (TalkerLayerProfileSpans::qk_norm_rope_cache and
    # ::attention, 17.cu:16465-16466; summed over the layers as at :17407-17426): the step launch by launch, not as a
    # graph, with cudaEvent spans, mean of three steps after one warm-up.
    bucket_append, bucket_attention = [], []
    for trial in range(4):
        positions.fill_(context)
        generation.zero_()
        one_step(profile=True)
        torch.cuda.synchronize()
        if trial:
            bucket_append.append(sum(e[0].elapsed_time(e[1]) for e in spans))
            bucket_attention.append(sum(e[1].elapsed_time(e[2]) for e in spans))
    positions.fill_(context)
    generation.zero_()
    status = eng.status()
    eng.close()
    kv_bytes = layers * streams * (context + 1) * 4096
    weight_bytes = 2 * (layers * ((nq + 2 * nk) * hidden + hidden * nq + 3 * inter * hidden) + vocab * hidden)
    peak, _ = load_peaks()
    return {"workload": "talker_decode_step_1p7b_shape", "streams_per_gpu": streams, "context": context,
            "ms_per_step": full_ms, "tokens_per_s": streams / (full_ms * 1e-3),
            "attention_ms": full_ms - rest_ms, "attention_share": (full_ms - rest_ms) / full_ms,
            "non_attention_ms": rest_ms, "kv_bytes_per_step": kv_bytes, "weight_bytes_per_step": weight_bytes,
            "weights_gbs": weight_bytes / (rest_ms * 1e-3) / 1e9,
            "hbm_bound_ms": (kv_bytes + weight_bytes) / (peak * 1e9) * 1e3, "device_status": status,
            "profile_talker_qk_norm_rope_cache_ms": float(np.mean(bucket_append)),
            "profile_talker_attention_ms": float(np.mean(bucket_attention)),
            "kernel_launches_per_step": layers * 7 + 4,
            "note": "every operator is this library's: embedding gather, norms, tcgen05 projections, fused decode step, "
                    "codec head, and the final-head chain (repetition penalty, suppression, greedy argmax, history "
                    "record) in one launch for all streams; only the two counter increments are torch ops; whole step "
                    "replayed as one CUDA graph; attention_ms = step with minus step without the qm_decode_step launches"}


def run_single_stream_section(pkg, steps):
    """Secondary measurement: the reference's own operating point - ONE stream, 512 cached tokens (the 0.6B / 1.7B
    talker attention shape is the same), one new token per step, 28 layers.  2.1 MB of KV per layer, so this is a
    latency figure: microseconds per layer of the fused decode step, replayed as a CUDA graph of 28 launches and
    also launched one by one."""
    import torch

    layers, length = 28, 512
    pages = (length + 1 + PAGE - 1) // PAGE
    gen = torch.Generator(device="cuda")
    gen.manual_seed(100)
    eng = pkg.TalkerAttention(layers=layers, num_pages=pages, q_heads=Q_HEADS, kv_heads=KV_HEADS, max_positions=length + 2)
    for layer in range(layers):
        for view in eng.pool_view(layer):
            view.normal_(generator=gen)
    table = torch.randperm(pages, generator=gen, device="cuda").to(torch.int32).view(1, pages)
    positions = torch.full((1,), length, dtype=torch.int32, device="cuda")
    ones = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    q = torch.randn(layers, 1, Q_HEADS, D, generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn(layers, 1, KV_HEADS, D, generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn(layers, 1, KV_HEADS, D, generator=gen, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    eng.workspace(1)

    def step():
        for layer in range(layers):
            eng.decode_step(layer, q[layer], k[layer], v[layer], ones, ones, positions, table, out=out[layer])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n / layers * 1e3

    n = max(10, min(steps, 50))
    graph_us = timed(graph.replay, n)
    eager_us = timed(step, n)
    status = eng.status()
    eng.close()
    layer_bytes = (length + 1) * 4096 + 12288
    return {"workload": "single_stream_decode_b1_l512", "kv_len": length, "layers": layers,
            "us_per_layer_graph": graph_us, "us_per_layer_eager_launches": eager_us,
            "gbs_graph": layer_bytes / (graph_us * 1e-6) / 1e9, "bytes_per_layer": layer_bytes, "device_status": status,
            "note": "2.1 MB per layer: launch and memory latency, not bandwidth, set this number"}


def run_code_predictor_section(pkg, steps):
    """Secondary measurement: one frame of the reference's code predictor (15 steps of a 5-layer decoder, hidden
    1024, same 16 / 8 x 128 attention shape, at most 16 cached positions; 17.cu:13616-13905) for 32 streams, on the
    same kernels as the talker step, random-init weights in the checkpoint's shapes, one CUDA graph per frame as in
    the reference; timed greedy and with the reference's default sampling (top-k 50, temperature 0.9)."""
    import importlib

    import torch

    predictor = importlib.import_module("qingming_qwen3_tts_b200.predictor")
    streams = 32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5000)
    weights = predictor.random_weights(predictor.PredictorDims(), gen)
    runner = predictor.CodePredictor(pkg, streams, weights)
    talker_hidden = torch.randn(streams, predictor.OUTER_HIDDEN, generator=gen, device="cuda").to(torch.bfloat16)
    first_embedding = torch.randn(streams, predictor.OUTER_HIDDEN, generator=gen, device="cuda").to(torch.bfloat16)
    rng_state = torch.arange(1, streams + 1, dtype=torch.int64, device="cuda")

    def frame_ms(**sampling):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                runner.frame(talker_hidden, first_embedding, **sampling)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            runner.frame(talker_hidden, first_embedding, **sampling)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        n = max(5, min(steps, 20))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    ms = frame_ms()
    # the reference's default for the predictor: subtalker_dosample, top_k 50, temperature 0.9 (17.cu:7139)
    ms_sampling = frame_ms(rng_state=rng_state, top_k=50, temperature=0.9)
    status = runner.engine.status()
    runner.close()
    d = predictor.PredictorDims()
    nq, nk = Q_HEADS * D, KV_HEADS * D
    layer_weights = 2 * ((nq + 2 * nk) * d.hidden + d.hidden * nq + 3 * d.intermediate * d.hidden)
    token_steps = d.steps + 1
    weight_bytes = token_steps * (d.layers * layer_weights + 2 * d.hidden * d.outer_hidden) + d.steps * 2 * d.vocab * d.hidden
    launches = token_steps * (d.layers * 7 + 2) + d.steps * 4
    peak, _ = load_peaks()
    return {"workload": "code_predictor_frame_1p7b_shape", "streams_per_gpu": streams, "steps_per_frame": d.steps,
            "ms_per_frame": ms, "frames_per_s": streams / (ms * 1e-3), "ms_per_frame_top_k_50_sampling": ms_sampling,
            "kernel_launches_per_frame": launches,
            "us_per_launch": ms * 1e3 / launches, "weight_bytes_per_frame": weight_bytes,
            "hbm_bound_ms": weight_bytes / (peak * 1e9) * 1e3, "device_status": status,
            "note": "every operator is this library's; 16 token rows per stream and frame through 5 layers; the "
                    "weights of a layer (29 MB) are small enough to stay in L2 between steps, so launch latency "
                    "sets the frame time"}


def run_long_context_section(pkg, world, rank, steps):
    """Secondary measurement: 4 streams of 65 536 keys each, keys split contiguously over the ranks; per layer every
    rank runs the split-KV kernel on its slice and the (m, l, o) partials are exchanged and combined - once with an
    NCCL all-gather and the combine kernel, once with the one-kernel exchange over peer memory.

    Layer 0 doubles as the parity case at the stated size.  Its 4 x 65 536 keys and values and the queries come from
    ONE seeded draw (the input recipe, seed 3) that every rank makes in full and slices, so the ranks hold pieces of
    the same cache.  Checked: every rank ends with the same bits; the peer-memory exchange and the NCCL path give the
    same bits; the result agrees with the single-GPU kernel run on the whole cache (rank 0 keeps a full copy for
    that) and, for two of the streams, with the fp32 oracle on the CPU."""
    import importlib

    import torch
    import torch.distributed as dist

    sh = importlib.import_module("qingming_qwen3_tts_b200.sharded")
    streams, length, layers = 4, 65536, 4
    begin, end = sh.slice_bounds(length, world, rank)
    local = end - begin
    pages_per_stream = (local + PAGE - 1) // PAGE
    num_pages = streams * pages_per_stream
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3000 + rank)
    eng = pkg.TalkerAttention(layers=layers, num_pages=num_pages, q_heads=Q_HEADS, kv_heads=KV_HEADS, max_positions=64)
    perm = torch.randperm(num_pages, generator=gen, device="cuda").to(torch.int32)
    page_table = perm.view(streams, pages_per_stream).contiguous()
    seq_lens = torch.full((streams,), local, dtype=torch.int32, device="cuda")
    q_rot = recipe_normal_bf16(3 * 1000 + 1, (streams, Q_HEADS, D), "cuda")        # the same on every rank
    full_lens = torch.full((streams,), length, dtype=torch.int32, device="cuda")
    eng_full = full_table = None
    for layer in range(layers):
        kview, vview = eng.pool_view(layer)
        if layer > 0:
            kview.normal_(generator=gen)
            vview.normal_(generator=gen)
            continue
        for tensor_id, view in ((2, kview), (3, vview)):
            # [streams][kv_heads][length][128] in the reference's cache layout, the whole of it on every rank
            whole = recipe_normal_bf16(3 * 1000 + tensor_id, (streams, KV_HEADS, length, D), "cuda")
            mine = whole[:, :, begin:end].reshape(streams, KV_HEADS, pages_per_stream, PAGE, D).permute(0, 2, 1, 3, 4)
            view[page_table.reshape(-1).long()] = mine.reshape(num_pages, KV_HEADS, PAGE, D)
            if rank == 0:
                if eng_full is None:
                    full_pages = length // PAGE
                    eng_full = pkg.TalkerAttention(layers=1, num_pages=streams * full_pages, q_heads=Q_HEADS, kv_heads=KV_HEADS,
                                                   max_positions=64)
                    full_table = torch.arange(streams * full_pages, dtype=torch.int32, device="cuda").view(streams, full_pages)
                target = eng_full.pool_view(0)[0 if tensor_id == 2 else 1]
                target.copy_(whole.reshape(streams, KV_HEADS, length // PAGE, PAGE, D).permute(0, 2, 1, 3, 4)
                             .reshape(streams * (length // PAGE), KV_HEADS, PAGE, D))
            del whole, mine
    torch.cuda.empty_cache()
    out = torch.empty_like(q_rot)
    exchange = None
    if world > 1:
        runner = sh.ShardedDecode()
        try:
            exchange = sh.PeerExchange(eng, rows_capacity=streams * Q_HEADS)
        except Exception as exc:       # symmetric memory not available: NCCL path only
            exchange_error = f"{type(exc).__name__}: {exc}"

    def layer_nccl(layer):
        sh.sharded_decode_attention(eng, runner, layer, q_rot, seq_lens, page_table, out=out)

    def layer_peer(layer):
        sh.sharded_decode_attention_peer(eng, exchange, layer, q_rot, seq_lens, page_table, out=out)

    def layer_fused(layer):
        exchange.run_fused(layer, q_rot, seq_lens, page_table, out=out)

    def layer_single(layer):
        eng.launch_attention(layer, q_rot, seq_lens, page_table, out=out)

    # ---- parity on layer 0, before any timing
    parity = {"streams": streams, "kv_len": length, "ranks": world}
    one_ulp = 2.0 ** -7            # outputs are O(0.1): one bf16 ulp is far below this

    def max_abs_bits(a, b):
        return float((a.float() - b.float()).abs().max().item())

    if world > 1:
        layer_nccl(0)
        via_nccl = out.clone()
        gathered = [torch.empty_like(via_nccl) for _ in range(world)]
        dist.all_gather(gathered, via_nccl.contiguous())
        parity["all_ranks_same_bits"] = all(bool(torch.equal(g.view(torch.int16), gathered[0].view(torch.int16))) for g in gathered)
        result = via_nccl
        if exchange is not None:
            layer_peer(0)
            parity["peer_exchange_equals_nccl_bits"] = bool(torch.equal(out.view(torch.int16), via_nccl.view(torch.int16)))
            out.zero_()
            layer_fused(0)
            parity["fused_exchange_equals_nccl_bits"] = bool(torch.equal(out.view(torch.int16), via_nccl.view(torch.int16)))
    else:
        layer_single(0)
        result = out.clone()
    ok = (parity.get("all_ranks_same_bits", True) and parity.get("peer_exchange_equals_nccl_bits", True)
          and parity.get("fused_exchange_equals_nccl_bits", True))
    if rank == 0:
        single = eng_full.launch_attention(0, q_rot, full_lens, full_table)
        parity["max_abs_vs_single_gpu_kernel"] = max_abs_bits(result, single)
        ok = ok and parity["max_abs_vs_single_gpu_kernel"] <= one_ulp
        from oracle import qm_oracle as oracle

        oracle.lib()
        use_all_host_threads()
        kfull, vfull = eng_full.pool_view(0)
        checked = [0, streams - 1]
        key_caches, value_caches = [], []
        for s_index in checked:
            pages = full_table[s_index].long()
            key_caches.append(_bits(kfull[pages].permute(1, 0, 2, 3).reshape(KV_HEADS, length, D)))
            value_caches.append(_bits(vfull[pages].permute(1, 0, 2, 3).reshape(KV_HEADS, length, D)))
        want = oracle.decode_attention(_bits(q_rot[checked]), key_caches, value_caches, np.full(len(checked), length, dtype=np.int32),
                                       mode="fp32")
        m = oracle.error_metrics(oracle.bf16_to_f32(_bits(result[checked])), want)
        parity.update({"against": "fp32 oracle, streams 0 and 3, all 16 query heads, 65 536 keys each", "max_abs": m["max_abs"],
                       "mean_rel": m["mean_rel"], "tolerance": {"max_abs": 2e-2, "mean_rel": 1e-2}})
        ok = ok and m["max_abs"] <= 2e-2 and m["mean_rel"] <= 1e-2
        eng_full.close()
        del kfull, vfull, eng_full
        torch.cuda.empty_cache()
    if world > 1:
        flag = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
    parity["ok"] = bool(ok)

    def measure(one_layer):
        # the per-layer host work (two ctypes calls) would otherwise dominate a 20-60 us layer: replay a CUDA graph
        reps = 4
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(2 * layers):
                one_layer(i % layers)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps * layers):
                one_layer(i % layers)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        replays = max(steps, 5)
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / (replays * reps * layers)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    extra = {}
    if world == 1:
        ms = measure(layer_single)
    else:
        nccl_ms = measure(layer_nccl)
        extra["us_per_layer_nccl_all_gather"] = nccl_ms * 1e3
        if exchange is not None:
            two_launch_ms = measure(layer_peer)
            fused_ms = measure(layer_fused)
            extra["us_per_layer_two_launch_peer_exchange"] = two_launch_ms * 1e3
            extra["us_per_layer_fused_peer_exchange"] = fused_ms * 1e3
            ms = min(two_launch_ms, fused_ms)
            extra["exchange"] = ("us_per_layer is the faster of the two peer-memory forms: fused = inside the split-KV kernel's "
                                 "launch (qm_decode_attention_exchange), two_launch = partial kernel + qm_attention_exchange_combine")
            # after the timed replays the exchange must still be in step on every rank: same bits as before
            out.zero_()
            layer_fused(0)
            still = bool(torch.equal(out.view(torch.int16), via_nccl.view(torch.int16)))
            flag = torch.tensor([1 if still else 0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            parity["peer_exchange_after_graph_replays"] = bool(flag.item())
            parity["ok"] = parity["ok"] and parity["peer_exchange_after_graph_replays"]
        else:
            ms = nccl_ms
            extra["exchange"] = "NCCL all-gather + combine kernel (" + exchange_error + ")"
    status = eng.status()
    if world > 1:
        dist.barrier()
        exchange = None
    eng.close()
    total_bytes = streams * length * 4096
    peak, _ = load_peaks()
    return {"workload": "long_context_split_kv_b4_l65536", "streams": streams, "kv_len": length, "gpus": world,
            "us_per_layer": ms * 1e3, "aggregate_gbs": total_bytes / (ms * 1e-3) / 1e9,
            "frac_of_measured_hbm_peak_per_gpu": total_bytes / world / (ms * 1e-3) / 1e9 / peak,
            "exchange_bytes_per_rank": streams * Q_HEADS * 130 * 4 if world > 1 else 0, "device_status": status,
            "parity": parity, **extra}


def cpu_baseline_and_parity(eng, q_rot0, out0, lengths, table):
    """CPU-baseline leg: times the oracle on a sample of layer 0 and uses its fp32 mode to check the GPU result."""
    import torch

    from oracle import qm_oracle as oracle

    oracle.lib()
    use_all_host_threads()
    sample = list(range(BATCH))
    kview, vview = eng.pool_view(0)
    kpool = kview.view(torch.int16).cpu().numpy().view(np.uint16)
    vpool = vview.view(torch.int16).cpu().numpy().view(np.uint16)
    q_bits = q_rot0.view(torch.int16).cpu().numpy().view(np.uint16)
    out_bits = out0.view(torch.int16).cpu().numpy().view(np.uint16)
    lens = lengths[sample] + 1
    key_caches = [oracle.gather_paged(kpool, table[s], int(lengths[s]) + 1, int(lengths[s]) + 1) for s in sample]
    value_caches = [oracle.gather_paged(vpool, table[s], int(lengths[s]) + 1, int(lengths[s]) + 1) for s in sample]
    q_sample = np.ascontiguousarray(q_bits[sample])
    seconds, _ = cpu_attention_sample(q_sample, key_caches, value_caches, lens, repeats=5)
    sample_bytes = algorithmic_bytes_per_layer(lengths[sample])
    want = oracle.decode_attention(q_sample, key_caches, value_caches, lens, mode="fp32")
    metrics = oracle.error_metrics(oracle.bf16_to_f32(out_bits[sample]), want)
    cpu = {"value": sample_bytes / seconds / 1e9, "unit": "GB/s", "cores": host_cores(), "kind": "port",
           "sample": f"layer 0 of all {BATCH} streams (1/28 of a GPU step), best of 5, bf16-faithful restatement "
                     "of the reference kernels, OpenMP over (stream, kv head)",
           "seconds": seconds}
    parity = {"against": "fp32 oracle on the same cache bits", "streams_checked": len(sample), **metrics,
              "tolerance": {"max_abs": 2e-2, "mean_rel": 1e-2},
              "ok": bool(metrics["max_abs"] <= 2e-2 and metrics["mean_rel"] <= 1e-2)}
    return cpu, parity


def main():
    global LAYERS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary prefill measurement")
    ap.add_argument("--only-prefill", action="store_true", help="run only the prefill section (profiling aid)")
    ap.add_argument("--prefill-seqs", type=int, default=8, help="with --only-prefill: use the first N prompts")
    ap.add_argument("--only-talker-step", action="store_true", help="run only the whole-decoder-step section (profiling aid)")
    ap.add_argument("--only-code-predictor", action="store_true", help="run only the code-predictor frame section (profiling aid)")
    ap.add_argument("--no-talker-step", action="store_true", help="skip the secondary whole-decoder-step measurement")
    ap.add_argument("--no-long-context", action="store_true", help="skip the secondary split-KV long-context measurement")
    ap.add_argument("--no-single-stream", action="store_true", help="skip the secondary one-stream latency measurement")
    ap.add_argument("--layers", type=int, default=LAYERS,
                    help="layers per step (default: the talker's 28); a smaller value gives a small case for profiling")
    args = ap.parse_args()
    LAYERS = args.layers
    if args.only_prefill:
        import torch

        import __graft_entry__ as entry

        torch.cuda.set_device(0)
        pkg = entry.load_package()
        pkg.load_library()
        print(json.dumps(run_prefill_section(pkg, args.steps, args.warmup, args.prefill_seqs)))
        return
    if args.only_talker_step:
        import torch

        import __graft_entry__ as entry

        torch.cuda.set_device(0)
        pkg = entry.load_package()
        pkg.load_library()
        print(json.dumps({"talker_step": run_talker_step_section(pkg, args.steps),
                          "code_predictor": run_code_predictor_section(pkg, args.steps)}))
        return
    if args.only_code_predictor:
        import torch

        import __graft_entry__ as entry

        torch.cuda.set_device(0)
        pkg = entry.load_package()
        pkg.load_library()
        print(json.dumps(run_code_predictor_section(pkg, args.steps)))
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
