"""The split-across-GPUs decode path on the GPU: partial states per slice, combine, and the sliced append.

One GPU is enough to exercise the kernels: the ranks' slices are processed one after the other on the same
device and their partials stacked as the all-gather would deliver them.  With two or more GPUs the same check
also runs as real NCCL ranks (one process per GPU)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario
import sharded_helpers

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL_MAX_ABS = 2e-2
TOL_MEAN_REL = 1e-2


def sharded_module():
    import importlib

    return importlib.import_module("qingming_qwen3_tts_b200.sharded")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_slices_processed_on_one_gpu_combine_to_full_attention(qm, world):
    import torch

    sh = sharded_module()
    sc = scenario.DecodeScenario(seed=61, lengths=[4000, 300, 2047, 6])
    exp = sc.expected()
    tb = scenario._bf16_tensor
    q_rot = tb(torch, exp["q_rot"])
    partials = []
    for rank in range(world):
        st = sharded_helpers.rank_local_state(sc, exp, sh, world, rank)
        eng = qm.TalkerAttention(layers=1, num_pages=st["num_pages"], max_positions=64)
        kview, vview = eng.pool_view(0)
        kview.copy_(tb(torch, st["kpool"]))
        vview.copy_(tb(torch, st["vpool"]))
        partials.append(eng.launch_attention_partial(0, q_rot, torch.from_numpy(st["local_lens"]).cuda(),
                                                     torch.from_numpy(st["table"]).cuda()).clone())
        torch.cuda.synchronize()
        assert eng.status() == 0
        eng.close()
    eng = qm.TalkerAttention(layers=1, num_pages=1, max_positions=64)
    out = eng.combine(torch.stack(partials))
    torch.cuda.synchronize()
    eng.close()
    m = oracle.error_metrics(oracle.bf16_to_f32(scenario._bits(out)), exp["out_fp32"])
    assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= TOL_MEAN_REL, m
    single = scenario.run_decode_on_gpu(qm, sc)["out"]
    m = oracle.error_metrics(oracle.bf16_to_f32(scenario._bits(out)), oracle.bf16_to_f32(single))
    assert m["max_abs"] <= 2.0 ** -7, m        # multi-rank result equals the single-GPU result to one bf16 ulp


def test_sliced_append_writes_only_on_the_owner(qm):
    import torch

    sh = sharded_module()
    world = 2
    sc = scenario.DecodeScenario(seed=62, lengths=[200, 129], random_weights=True)
    exp = sc.expected()
    tb = scenario._bf16_tensor
    for rank in range(world):
        st = sharded_helpers.rank_local_state(sc, exp, sh, world, rank, include_new_token=False)
        eng = qm.TalkerAttention(layers=1, num_pages=st["num_pages"], max_positions=sc.max_pos)
        kview, vview = eng.pool_view(0)
        kview.copy_(tb(torch, st["kpool"]))
        vview.copy_(tb(torch, st["vpool"]))
        owner = rank == world - 1
        cache_pos = (sc.lengths - st["begins"]).astype(np.int32) if owner else np.full(sc.batch, -1, dtype=np.int32)
        q_rot = eng.launch_qk_norm_rope_cache_m1_sliced(
            0, tb(torch, sc.q), tb(torch, sc.k), tb(torch, sc.v), tb(torch, sc.q_w), tb(torch, sc.k_w),
            torch.from_numpy(sc.lengths).cuda(), torch.from_numpy(cache_pos).cuda(), torch.from_numpy(st["table"]).cuda())
        torch.cuda.synchronize()
        assert eng.status() == 0
        d = np.abs(oracle.bf16_to_f32(scenario._bits(q_rot)) - oracle.bf16_to_f32(exp["q_rot"]))
        assert d.max() <= 2.0 ** -5 and (scenario._bits(q_rot) != exp["q_rot"]).mean() <= 1e-3
        kp, vp = scenario._bits(kview), scenario._bits(vview)
        if not owner:
            assert np.array_equal(kp, st["kpool"]) and np.array_equal(vp, st["vpool"])
        else:
            for s in range(sc.batch):
                slot = int(cache_pos[s])
                page = st["table"][s, slot // 64]
                assert np.array_equal(vp[page, :, slot % 64], sc.v[s])
                dk = np.abs(oracle.bf16_to_f32(kp[page, :, slot % 64]) - oracle.bf16_to_f32(exp["key_rows"][s]))
                assert dk.max() <= 2.0 ** -5
        eng.close()


def test_real_ranks_over_nccl_when_two_gpus_are_present(qm):
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "sharded_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-6000:] + proc.stderr[-1500:]
    assert "SHARDED_OK" in proc.stdout
