"""One NCCL rank of the split-across-GPUs decode check (launched by torchrun; see test_sharded_gpu.py)."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import __graft_entry__ as entry  # noqa: E402
import scenario  # noqa: E402
import sharded_helpers  # noqa: E402
from oracle import qm_oracle as oracle  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    qm = entry.load_package()
    qm.load_library()
    import importlib

    sh = importlib.import_module("qingming_qwen3_tts_b200.sharded")
    sc = scenario.DecodeScenario(seed=63, lengths=[8191] * 4)      # the long-context shape at reduced length
    exp = sc.expected()
    st = sharded_helpers.rank_local_state(sc, exp, sh, world, rank, include_new_token=False)
    tb = scenario._bf16_tensor
    eng = qm.TalkerAttention(layers=1, num_pages=st["num_pages"], max_positions=sc.max_pos)
    kview, vview = eng.pool_view(0)
    kview.copy_(tb(torch, st["kpool"]))
    vview.copy_(tb(torch, st["vpool"]))
    owner = rank == world - 1
    cache_pos = (sc.lengths - st["begins"]).astype(np.int32) if owner else np.full(sc.batch, -1, dtype=np.int32)
    table = torch.from_numpy(st["table"]).cuda()
    q_rot = eng.launch_qk_norm_rope_cache_m1_sliced(
        0, tb(torch, sc.q), tb(torch, sc.k), tb(torch, sc.v), tb(torch, sc.q_w), tb(torch, sc.k_w),
        torch.from_numpy(sc.lengths).cuda(), torch.from_numpy(cache_pos).cuda(), table)
    local_lens = st["local_lens"] + (1 if owner else 0)
    runner = sh.ShardedDecode()
    out = sh.sharded_decode_attention(eng, runner, 0, q_rot, torch.from_numpy(local_lens.astype(np.int32)).cuda(), table)
    torch.cuda.synchronize()
    assert eng.status() == 0
    bits = scenario._bits(out)
    m = oracle.error_metrics(oracle.bf16_to_f32(bits), exp["out_fp32"])
    assert m["max_abs"] <= 2e-2 and m["mean_rel"] <= 1e-2, m
    # every rank must hold the same bits
    mine = out.view(torch.int16).to(torch.int64).sum().reshape(1)
    sums = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(sums, mine)
    assert all(int(x) == int(sums[0]) for x in sums)
    # ---- the same step through the other exchange paths.  Every call gets different inputs (the streams' queries
    # rotated, all four streams having the same length) and every call is checked, so an exchange that did not
    # wait for its peers, or folded a stale slot, cannot pass.
    lens_dev = torch.from_numpy(local_lens.astype(np.int32)).cuda()
    variants = [torch.roll(q_rot, shifts=i, dims=0).contiguous() for i in range(4)]
    wanted = []
    for qv in variants:
        wanted.append(scenario._bits(sh.sharded_decode_attention(eng, runner, 0, qv, lens_dev, table)).copy())
    assert np.array_equal(wanted[0], bits)
    assert not np.array_equal(wanted[1], wanted[0])
    # a call with two of the four streams splits the keys over the CTAs differently, so it has its own reference
    first_two = (variants[2][:2].contiguous(), lens_dev[:2].contiguous(), table[:2].contiguous())
    wanted_two = scenario._bits(sh.sharded_decode_attention(eng, runner, 0, *first_two)).copy()

    def check(name, call):
        for i, qv in enumerate(variants):
            got = scenario._bits(call(qv, lens_dev, table))
            assert np.array_equal(got, wanted[i]), f"{name}: call {i} differs from all-gather + combine"
        # fewer rows in one call, then all rows again: the per-row call counters keep the ranks in step
        got = scenario._bits(call(*first_two))
        assert np.array_equal(got, wanted_two), f"{name}: two-stream call differs"
        got = scenario._bits(call(variants[3], lens_dev, table))
        assert np.array_equal(got, wanted[3]), f"{name}: call after a smaller one differs"

    # 1. one kernel over torch symmetric memory
    exchange = sh.PeerExchange(eng, rows_capacity=sc.batch * 16)
    check("peer exchange", lambda qv, ln, tb_: sh.sharded_decode_attention_peer(eng, exchange, 0, qv, ln, tb_))
    # the same exchange inside the split-KV kernel's own launch, mixed with the two-launch form on the same buffers
    check("fused exchange", lambda qv, ln, tb_: exchange.run_fused(0, qv, ln, tb_))
    check("peer exchange after fused", lambda qv, ln, tb_: sh.sharded_decode_attention_peer(eng, exchange, 0, qv, ln, tb_))
    # a rank that holds no keys of a stream still takes part: stream 1's keys all on rank 0
    lens_skewed = lens_dev.clone()
    if rank != 0:
        lens_skewed[1] = 0
    want_skewed = scenario._bits(sh.sharded_decode_attention(eng, runner, 0, variants[1], lens_skewed, table)).copy()
    got_skewed = scenario._bits(exchange.run_fused(0, variants[1], lens_skewed, table))
    assert np.array_equal(got_skewed, want_skewed), "fused exchange with an empty slice differs"
    # ... and replayed from a CUDA graph with new inputs each time (the call number is device state)
    static_q = variants[0].clone()
    out_graph = torch.empty_like(static_q)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sh.sharded_decode_attention_peer(eng, exchange, 0, static_q, lens_dev, table, out=out_graph)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sh.sharded_decode_attention_peer(eng, exchange, 0, static_q, lens_dev, table, out=out_graph)
    for i in (1, 2, 3, 0, 2):
        static_q.copy_(variants[i])
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(scenario._bits(out_graph), wanted[i]), f"graph replay with inputs {i} differs"
    # 2. the same kernel on buffers shared through CUDA IPC handles (the C++ host's route)
    ipc = sh.IpcExchange(eng, rows_capacity=sc.batch * 16)
    check("ipc exchange", lambda qv, ln, tb_: sh.sharded_decode_attention_peer(eng, ipc, 0, qv, ln, tb_))
    check("ipc fused exchange", lambda qv, ln, tb_: ipc.run_fused(0, qv, ln, tb_))
    # 3. the C entry point that does partial -> ncclAllGather -> combine on a communicator of its own
    nccl = sh.NcclSharded(eng, sc.batch)
    for i, qv in enumerate(variants):
        got = scenario._bits(nccl.run(0, qv, lens_dev, table))
        nccl.wait(deadline_ms=20000)
        assert np.array_equal(got, wanted[i]), f"qm_decode_attention_sharded: call {i} differs"
    torch.cuda.synchronize()
    assert eng.status() == 0
    dist.barrier()
    nccl.close()
    ipc.close()
    del exchange, graph
    eng.close()
    dist.barrier()
    if rank == 0:
        print("SHARDED_OK", m)
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        print("SHARDED_WORKER_FAILED rank", os.environ.get("RANK"), traceback.format_exc(), flush=True)
        raise
