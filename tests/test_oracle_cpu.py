"""CPU checks of the oracle itself: known answers, internal consistency, and the reference's own host code."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

TOL_MAX_ABS = 2e-2      # bf16 tolerance stated for this path, against the fp32 oracle
TOL_MEAN_REL = 1e-2


def numpy_rne(x):
    bits = x.view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    quiet = ((bits >> 16) | 0x40).astype(np.uint16)
    return np.where(nan, quiet, rounded)


def test_bf16_conversion_all_patterns():
    # every bf16 pattern widened to f32 must convert back to itself (NaNs: quieted)
    all_bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    wide = oracle.bf16_to_f32(all_bits)
    back = oracle.f32_to_bf16(wide)
    is_nan = np.isnan(wide)
    assert np.array_equal(back[~is_nan], all_bits[~is_nan])
    assert np.array_equal(back[is_nan], all_bits[is_nan] | 0x40)


def test_bf16_rounding_matches_bit_formula():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(200000).astype(np.float32) * np.float32(37.0)
    ties = ((rng.integers(0, 1 << 16, 4096).astype(np.uint32) << 16) | 0x8000).view(np.float32)
    x = np.concatenate([x, ties, np.array([0.0, -0.0, np.inf, -np.inf, np.nan], dtype=np.float32)])
    assert np.array_equal(oracle.f32_to_bf16(x), numpy_rne(x))


def test_splitmix64_known_answers():
    # first outputs of SplitMix64 from state 0 (published test vector of the algorithm)
    import ctypes

    state = ctypes.c_uint64(0)
    lib = oracle.lib()
    lib.qmo_splitmix64.restype = ctypes.c_uint64
    got = [lib.qmo_splitmix64(ctypes.byref(state)) for _ in range(3)]
    assert got == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_normal_generator_statistics_and_determinism():
    a = oracle.normal_bf16(7, (1 << 16,))
    b = oracle.normal_bf16(7, (1 << 16,))
    assert np.array_equal(a, b)
    f = oracle.bf16_to_f32(a)
    assert abs(f.mean()) < 0.02 and abs(f.std() - 1.0) < 0.02


def test_rope_table_formula():
    cos, sin = oracle.make_rope(40, 3)
    i = np.arange(64, dtype=np.float64)
    inv = np.power(1.0e6, -2.0 * i / 128.0)
    pos = np.arange(3, 43, dtype=np.float64)[:, None]
    want_c = oracle.f32_to_bf16(np.cos(pos * inv).astype(np.float32))
    want_s = oracle.f32_to_bf16(np.sin(pos * inv).astype(np.float32))
    assert np.array_equal(cos[:, :64], want_c) and np.array_equal(cos[:, 64:], want_c)
    assert np.array_equal(sin[:, :64], want_s) and np.array_equal(sin[:, 64:], want_s)


@pytest.mark.skipif(not oracle.ref_available(), reason="reference harness not built on this machine")
def test_rope_table_matches_reference_host_function():
    # make_talker_rope is host code, so the reference's own function runs without a GPU
    want = oracle.ref_make_rope(700, 0)
    got = oracle.make_rope(700, 0)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    want = oracle.ref_make_rope(33, 8190)
    got = oracle.make_rope(33, 8190)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_rope_table_golden():
    g = np.load(scenario_path("rope_rows_golden.npz"))
    got = oracle.make_rope(int(g["rows"]), int(g["start"]))
    assert np.array_equal(got[0], g["cos"]) and np.array_equal(got[1], g["sin"])


def scenario_path(name):
    from pathlib import Path

    return Path(__file__).resolve().parent / "golden" / name


def test_norm_rope_unit_weight_preserves_norm():
    # RoPE is a rotation and RMSNorm makes the row RMS 1: the roped row keeps RMS ~ 1
    sc = scenario.DecodeScenario(seed=11, lengths=[5, 70])
    exp = sc.expected()
    rows = oracle.bf16_to_f32(exp["q_rot"]).reshape(-1, 128)
    rms = np.sqrt((rows.astype(np.float64) ** 2).mean(axis=1))
    assert np.all(np.abs(rms - 1.0) < 0.02)
    # V is appended raw
    assert np.array_equal(exp["value_rows"], sc.v)


def test_ref_mode_close_to_fp32_mode():
    sc = scenario.DecodeScenario(seed=0, lengths=[512])
    exp = sc.expected()
    m = oracle.error_metrics(oracle.bf16_to_f32(exp["out_ref"]), exp["out_fp32"])
    assert m["max_abs"] <= TOL_MAX_ABS and m["mean_rel"] <= 5 * TOL_MEAN_REL, m


def test_single_key_attention_returns_value_row():
    sc = scenario.DecodeScenario(seed=3, lengths=[0, 0])
    exp = sc.expected()
    for s in range(2):
        for h in range(16):
            assert np.array_equal(exp["out_ref"][s, h], sc.v[s, h // 2])
            assert np.allclose(exp["out_fp32"][s, h], oracle.bf16_to_f32(sc.v[s, h // 2]))


def test_partials_combine_to_full_attention():
    sc = scenario.DecodeScenario(seed=5, lengths=[300])
    exp = sc.expected()
    kc, vc = exp["key_caches"][0], exp["value_caches"][0]
    cuts = [0, 64, 65, 200, 301]
    for head in (0, 7, 15):
        parts = [oracle.attention_partial(exp["q_rot"][0, head], kc, vc, head // 2, a, b)
                 for a, b in zip(cuts[:-1], cuts[1:])]
        got = oracle.combine_partials([p[0] for p in parts], [p[1] for p in parts], np.stack([p[2] for p in parts]))
        assert np.allclose(got, exp["out_fp32"][0, head], atol=1e-5)
    # an empty slice contributes nothing
    m, l, o = oracle.attention_partial(exp["q_rot"][0, 0], kc, vc, 0, 10, 10)
    assert l == 0.0 and np.isneginf(m) and not o.any()


def test_paged_layout_roundtrip_is_bit_exact():
    sc = scenario.DecodeScenario(seed=9, lengths=[63, 64, 130])
    kp, vp = sc.pools()
    for s in range(sc.batch):
        n = int(sc.lengths[s])
        back = oracle.gather_paged(kp, sc.page_table[s], n, sc.max_cache)
        assert np.array_equal(back[:, :n], sc.key_caches[s][:, :n])
        # explicit index formula: element offset ((page*Hkv + h)*64 + slot)*128 + d
        flat = kp.reshape(-1)
        for t in (0, n // 2, n - 1):
            page = sc.page_table[s, t >> 6]
            for h in (0, 7):
                off = ((page * 8 + h) * 64 + (t & 63)) * 128
                assert np.array_equal(flat[off:off + 128], sc.key_caches[s][h, t])
    # pages are disjoint between streams
    used = sc.page_table[sc.page_table >= 0]
    assert len(set(used.tolist())) == len(used)


def test_prefill_rows_equal_decode_rows():
    # row i of causal prefill is decode attention over i + 1 keys
    ps = scenario.PrefillScenario(seed=2, lengths=[70])
    q_rot, kcs, vcs = ps.expected_append()
    out, mask = ps.expected_attention(mode="ref")
    assert mask.all()
    for i in (0, 1, 63, 64, 69):
        dec = oracle.decode_attention(q_rot[i:i + 1], kcs, vcs, [i + 1], mode="ref")
        assert np.array_equal(dec[0], out[i])


def test_prefill_append_equals_tokenwise_decode_append():
    ps = scenario.PrefillScenario(seed=4, lengths=[9], random_weights=True)
    q_rot, kcs, vcs = ps.expected_append()
    kc = np.zeros_like(kcs[0])
    vc = np.zeros_like(vcs[0])
    for t in range(9):
        qr = oracle.append(ps.q[t:t + 1], ps.k[t:t + 1], ps.v[t:t + 1], ps.q_w, ps.k_w, ps.cos[t:t + 1],
                           ps.sin[t:t + 1], t, kc, vc)
        assert np.array_equal(qr[0], q_rot[t])
    assert np.array_equal(kc, kcs[0]) and np.array_equal(vc, vcs[0])
