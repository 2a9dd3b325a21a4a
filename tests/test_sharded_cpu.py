"""Host logic of the split-across-GPUs decode path, on CPU: two gloo ranks, the partial and combine steps done by
the oracle.  Checks the slice arithmetic, the all-gather layout and rank-order fold, and that a rank that never
joins is detected by the process-group timeout instead of hanging the others."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _load_sharded():
    import __graft_entry__ as entry

    entry.load_package()
    import importlib

    return importlib.import_module("qingming_qwen3_tts_b200.sharded")


def test_slice_bounds_partition_every_length():
    sh = _load_sharded()
    for world in (1, 2, 3, 4, 8):
        for length in (0, 1, 7, 64, 65, 1000, 65536, 65537):
            cuts = [sh.slice_bounds(length, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == length
            assert all(a[1] == b[0] for a, b in zip(cuts[:-1], cuts[1:]))
            sizes = [e - b for b, e in cuts]
            assert max(sizes) - min(sizes) <= 1
            if length:
                assert sh.owner_of(length - 1, length, world) == world - 1
                assert sh.owner_of(0, length, world) == min(r for r in range(world) if sizes[r])


def _worker(rank, world, port, result_dir, drop_rank):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    sh = _load_sharded()
    import scenario
    from oracle import qm_oracle as oracle

    sc = scenario.DecodeScenario(seed=77, lengths=[511, 130, 64])
    exp = sc.expected()
    if drop_rank == rank:
        # this rank leaves between steps without joining the collective
        os._exit(0)

    def partial_fn():
        out = np.zeros((sc.batch, 16, 130), dtype=np.float32)
        for s in range(sc.batch):
            length = int(sc.lengths[s]) + 1
            begin, end = sh.slice_bounds(length, world, rank)
            for h in range(16):
                m, l, o = oracle.attention_partial(exp["q_rot"][s, h], exp["key_caches"][s], exp["value_caches"][s],
                                                   h // 2, begin, end)
                out[s, h, 0], out[s, h, 1], out[s, h, 2:] = m, l, o
        return torch.from_numpy(out)

    def combine_fn(gathered):
        g = gathered.numpy()
        out = np.zeros((sc.batch, 16, 128), dtype=np.float32)
        for s in range(sc.batch):
            for h in range(16):
                out[s, h] = oracle.combine_partials(g[:, s, h, 0], g[:, s, h, 1], g[:, s, h, 2:])
        return out

    runner = sh.ShardedDecode()
    try:
        got = runner.run(partial_fn, combine_fn)
        ok = bool(np.allclose(got, exp["out_fp32"], atol=2e-5))
        Path(result_dir, f"rank{rank}.txt").write_text("ok" if ok else "mismatch")
    except Exception as exc:  # the other rank left: the collective must fail, not hang
        Path(result_dir, f"rank{rank}.txt").write_text("error:" + type(exc).__name__)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _free_port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_combine_to_full_attention(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), -1), nprocs=2, join=True)
    assert (tmp_path / "rank0.txt").read_text() == "ok"
    assert (tmp_path / "rank1.txt").read_text() == "ok"


def test_a_rank_that_leaves_is_detected_by_timeout(tmp_path):
    # rank 1 exits before the collective; rank 0 must come back with an error within the group timeout
    ctx = mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), 1), nprocs=2, join=False)
    import time

    deadline = time.time() + 90
    while not ctx.join(timeout=2):
        assert time.time() < deadline, "rank 0 is still waiting for the rank that left"
    text = (tmp_path / "rank0.txt").read_text()
    assert text.startswith("error:"), text
