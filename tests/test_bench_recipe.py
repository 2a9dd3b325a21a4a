"""The benchmark draws its inputs with the recipe of the parity tests (SplitMix64 -> Box-Muller -> bf16), written as
torch ops so that whole tensors are drawn in parallel.  It must produce the oracle generator's bits: on the CPU
exactly, on the GPU up to the rare element whose float64 logarithm or cosine rounds differently there."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import bench


def draws(device, seed, n):
    import torch

    return bench.recipe_normal_bf16(seed, (n,), device).view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("seed,n", [(1001, 100003), (7, 5), (3 * 1000 + 2, 1), (2 ** 63 + 12345, 4096)])
def test_recipe_matches_the_oracle_generator_on_cpu(seed, n):
    assert np.array_equal(draws("cpu", seed, n), oracle.normal_bf16(seed, (n,)))


def test_integer_draws_and_shuffle_match_the_oracle():
    assert np.array_equal(bench.splitmix64_ints(1099, 256, 4096, 64), oracle.uniform_int(1099, 256, 4096, 64))
    assert np.array_equal(bench.splitmix64_shuffle(2008, 631), oracle.shuffled_range(2008, 631))
    lengths = bench.workload_lengths()
    table, pages = bench.workload_page_table(lengths)
    used = np.concatenate([table[s, :(int(n) + 1 + 63) // 64] for s, n in enumerate(lengths)])
    assert sorted(used) == list(range(pages))            # every page belongs to exactly one stream


def test_both_arms_describe_the_same_workload():
    assert bench.workload_config(1) == bench.workload_config(1)
    assert set(bench.workload_config(8)) == {"workload", "streams_per_gpu", "kv_len", "q_heads", "kv_heads", "head_dim",
                                            "page_tokens", "layers_per_step", "parallelism", "l2"}


@pytest.mark.gpu
def test_recipe_on_the_gpu_matches_the_oracle_generator():
    n = 1 << 20
    got, want = draws("cuda", 1004, n), oracle.normal_bf16(1004, (n,))
    assert int((got != want).sum()) <= 2
