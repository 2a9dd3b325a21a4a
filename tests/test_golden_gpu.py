"""The CUDA path against the reference kernels' own output bits (tests/golden/reference_kernels_golden.npz).

The fused append keeps the reference's rounding chain, reduction order and rsqrtf, so its bits must EQUAL the
reference kernel's.  Attention keeps scores in fp32 where the reference materialises bf16, so it is compared
under the stated bf16 tolerance.
"""
from pathlib import Path

import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario
from golden.make_reference_golden import DECODE_CASES, PREFILL_CASES

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_kernels_golden.npz")


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_decode_step_against_reference_kernel_bits(qm, name):
    seed, lengths, rw = DECODE_CASES[name]
    sc = scenario.DecodeScenario(seed=seed, lengths=lengths, random_weights=rw)
    got = scenario.run_decode_on_gpu(qm, sc)
    assert got["status"] == 0
    assert np.array_equal(got["q_rot"], GOLDEN[f"{name}_q_rot"]), "q_rot bits differ from the reference kernel"
    assert np.array_equal(got["key_pool_new_rows"], GOLDEN[f"{name}_key_rows"]), "appended K bits differ"
    m = oracle.error_metrics(oracle.bf16_to_f32(got["out"]), oracle.bf16_to_f32(GOLDEN[f"{name}_context"]))
    assert m["max_abs"] <= 2e-2 and m["mean_rel"] <= 1e-2, m


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_append_against_reference_kernel_bits(qm, name):
    seed, lengths, rw = PREFILL_CASES[name]
    ps = scenario.PrefillScenario(seed=seed, lengths=lengths, random_weights=rw)
    got = scenario.run_prefill_on_gpu(qm, ps, attention=False)
    assert got["status"] == 0
    assert np.array_equal(got["q_rot"], GOLDEN[f"{name}_q_rot"])
    for s in range(ps.batch):
        n = int(ps.lengths[s])
        gathered = oracle.gather_paged(got["key_pool"], ps.page_table[s], n, ps.max_cache)
        assert np.array_equal(gathered[:, :n], GOLDEN[f"{name}_key_cache_{s}"])
