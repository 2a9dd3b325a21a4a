"""Failure detection on the GPU without faulting it: a device-side wait whose signal never comes must give up on
its own, report a status the host can read, and leave the context usable for the next call."""
import time

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu


def test_wait_without_signal_times_out_and_reports(qm):
    import torch

    eng = qm.TalkerAttention(layers=1, num_pages=2, max_positions=64)
    try:
        t0 = time.time()
        assert eng.lib.qm_selftest_wait_timeout(eng.pool, torch.cuda.current_stream().cuda_stream) == qm.QM_OK
        bits = eng.status()                       # synchronises the stream
        elapsed = time.time() - t0
        assert bits == qm.DEVSTAT_TIMEOUT, hex(bits)
        assert elapsed < 20.0, f"the bounded wait took {elapsed:.1f} s"
        assert eng.status() == 0                  # reading cleared it
    finally:
        eng.close()
    # the context is intact: a normal decode step still runs and is correct
    sc = scenario.DecodeScenario(seed=91, lengths=[70, 3])
    got = scenario.run_decode_on_gpu(qm, sc)
    m = oracle.error_metrics(oracle.bf16_to_f32(got["out"]), sc.expected()["out_fp32"])
    assert got["status"] == 0 and m["max_abs"] <= 2e-2 and m["mean_rel"] <= 1e-2
