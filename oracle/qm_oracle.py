"""numpy front end of the CPU oracle (oracle/qm_oracle.c) and of the optional
reference-kernel harness (oracle/_ref/libqm_refkernels.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg, never by the library under test.

bf16 tensors are numpy uint16 arrays holding the raw bits.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int32, c_int64, c_uint16, c_uint64, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libqm_oracle.so"
REF_LIB = HERE / "_ref" / "libqm_refkernels.so"
D = 128
PAGE = 64

_lib = None
_ref = None


def build(reference_dir=None) -> None:
    """Compiles the C restatement and, when `reference_dir` (or the environment variable QM_REFERENCE_DIR) names a
    reference checkout, the harness around the reference's own kernels.  There is no default location."""
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    reference_dir = reference_dir or os.environ.get("QM_REFERENCE_DIR")
    if reference_dir and (Path(reference_dir) / "devices" / "rtx4090-24g" / "qwen3_tts_1_7b.cu").exists():
        subprocess.run(["make", "-C", str(HERE), "ref", f"REFERENCE_DIR={reference_dir}"], check=True, capture_output=True)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.qmo_f32_to_bf16.restype = c_uint16
        _lib.qmo_f32_to_bf16.argtypes = [c_float]
        _lib.qmo_bf16_to_f32.restype = c_float
        _lib.qmo_bf16_to_f32.argtypes = [c_uint16]
    return _lib


def _p(a):
    return a.ctypes.data_as(c_void_p) if a is not None else None


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16
    return a


# ------------------------------------------------------------------ helpers

def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().qmo_f32_to_bf16_array(_p(x), _p(out), c_int64(x.size))
    return out


def normal_bf16(seed: int, shape) -> np.ndarray:
    """N(0,1) bf16 tensor drawn in row-major order from SplitMix64(seed) by Box-Muller."""
    out = np.empty(shape, dtype=np.uint16)
    lib().qmo_fill_normal_bf16(c_uint64(seed), _p(out), c_int64(out.size))
    return out


def uniform_int(seed: int, lo: int, hi: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int32)
    lib().qmo_fill_uniform_int(c_uint64(seed), c_int32(lo), c_int32(hi), _p(out), c_int64(n))
    return out


def shuffled_range(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int32)
    lib().qmo_shuffled_range(c_uint64(seed), _p(out), c_int64(n))
    return out


def make_rope(rows: int, start: int = 0, theta: float = 1.0e6):
    cos = np.empty((rows, D), dtype=np.uint16)
    sin = np.empty((rows, D), dtype=np.uint16)
    lib().qmo_make_rope(c_int(rows), c_int(start), c_double(theta), _p(cos), _p(sin))
    return cos, sin


# ------------------------------------------------------------- path pieces

def append(q, k, v, q_w, k_w, cos_rows, sin_rows, first_pos, key_cache, value_cache, eps=1.0e-6):
    """Norm + RoPE + append of `tokens` consecutive positions of one sequence.

    q [tokens][Hq][128], k/v [tokens][Hkv][128]; cos_rows/sin_rows [tokens][128] for those positions;
    caches [Hkv][max_cache][128] updated in place.  Returns q_rot.
    """
    q, k, v = _u16(q), _u16(k), _u16(v)
    tokens, hq = q.shape[0], q.shape[1]
    hkv, max_cache = key_cache.shape[0], key_cache.shape[1]
    q_rot = np.empty_like(q)
    lib().qmo_append(_p(q), _p(k), _p(v), _p(_u16(q_w)), _p(_u16(k_w)), _p(_u16(cos_rows)), _p(_u16(sin_rows)),
                     c_float(eps), c_int(tokens), c_int(first_pos), c_int(hq), c_int(hkv), c_int(max_cache),
                     _p(q_rot), _p(key_cache), _p(value_cache))
    return q_rot


def decode_attention(q_rot, key_caches, value_caches, key_lens, mode="fp32"):
    """Batched decode attention.  q_rot [B][Hq][128]; caches: lists of [Hkv][max_cache][128] arrays.

    mode "ref" -> uint16 bf16 bits, "fp32" -> float32.
    """
    q_rot = _u16(q_rot)
    b, hq = q_rot.shape[0], q_rot.shape[1]
    hkv = key_caches[0].shape[0]
    kp = (c_void_p * b)(*[kc.ctypes.data for kc in key_caches])
    vp = (c_void_p * b)(*[vc.ctypes.data for vc in value_caches])
    maxc = np.array([kc.shape[1] for kc in key_caches], dtype=np.int32)
    lens = np.ascontiguousarray(key_lens, dtype=np.int32)
    out16 = np.empty((b, hq, D), dtype=np.uint16) if mode == "ref" else None
    out32 = np.empty((b, hq, D), dtype=np.float32) if mode != "ref" else None
    rc = lib().qmo_decode_attention_batch(_p(q_rot), kp, vp, _p(maxc), _p(lens), c_int(b), c_int(hq), c_int(hkv),
                                          c_int(0 if mode == "ref" else 1), _p(out16), _p(out32))
    assert rc == 0
    return out16 if mode == "ref" else out32


def prefill_attention(q_rot, key_cache, value_cache, seq, cache_before=0, rows=None, mode="fp32"):
    """Causal attention of one sequence over its cache.  rows=(begin,end) restricts the computed rows;
    the other rows of the result are left zero."""
    q_rot = _u16(q_rot)
    hq = q_rot.shape[1]
    hkv, max_cache = key_cache.shape[0], key_cache.shape[1]
    begin, end = rows if rows is not None else (0, seq)
    out16 = np.zeros((seq, hq, D), dtype=np.uint16) if mode == "ref" else None
    out32 = np.zeros((seq, hq, D), dtype=np.float32) if mode != "ref" else None
    rc = lib().qmo_prefill_attention(_p(q_rot), _p(key_cache), _p(value_cache), c_int(max_cache), c_int(seq),
                                     c_int(cache_before), c_int(hq), c_int(hkv), c_int(begin), c_int(end),
                                     c_int(0 if mode == "ref" else 1), _p(out16), _p(out32))
    assert rc == 0
    return out16 if mode == "ref" else out32


def attention_partial(q_row, key_cache, value_cache, kv_head, key_begin, key_end):
    m = c_float()
    l = c_float()
    o = np.empty(D, dtype=np.float32)
    lib().qmo_attention_partial(_p(_u16(q_row)), _p(key_cache), _p(value_cache), c_int(kv_head),
                                c_int(key_cache.shape[1]), c_int(key_begin), c_int(key_end), ctypes.byref(m),
                                ctypes.byref(l), _p(o))
    return m.value, l.value, o


def combine_partials(m, l, o):
    m = np.ascontiguousarray(m, dtype=np.float32)
    l = np.ascontiguousarray(l, dtype=np.float32)
    o = np.ascontiguousarray(o, dtype=np.float32)
    out = np.empty(D, dtype=np.float32)
    lib().qmo_combine_partials(_p(m), _p(l), _p(o), c_int(m.size), _p(out))
    return out


def gather_paged(pool, page_row, tokens, max_cache):
    """pool [pages][Hkv][64][128] -> contiguous [Hkv][max_cache][128] for one stream."""
    pool = _u16(pool)
    hkv = pool.shape[1]
    out = np.zeros((hkv, max_cache, D), dtype=np.uint16)
    row = np.ascontiguousarray(page_row, dtype=np.int32)
    lib().qmo_gather_paged(_p(pool), _p(row), c_int(tokens), c_int(hkv), c_int(PAGE), c_int(max_cache), _p(out))
    return out


def scatter_paged(cache, page_row, tokens, pool):
    cache = _u16(cache)
    row = np.ascontiguousarray(page_row, dtype=np.int32)
    lib().qmo_scatter_paged(_p(cache), _p(row), c_int(tokens), c_int(cache.shape[0]), c_int(PAGE),
                            c_int(cache.shape[1]), _p(pool))


# ------------------------------------------------------------ error metrics

def error_metrics(got_f32: np.ndarray, want_f32: np.ndarray) -> dict:
    """max-abs, aggregate relative (sum|a-b| / sum|b|) and element-wise mean relative error."""
    diff = np.abs(got_f32.astype(np.float64) - want_f32.astype(np.float64))
    return {
        "max_abs": float(diff.max()) if diff.size else 0.0,
        "mean_rel": float(diff.sum() / max(np.abs(want_f32).astype(np.float64).sum(), 1e-30)),
        "mean_rel_elementwise": float((diff / np.maximum(np.abs(want_f32), 1e-3)).mean()) if diff.size else 0.0,
    }


# ------------------------------------------- reference kernels (GPU, optional)

def ref_available() -> bool:
    return REF_LIB.exists()


def ref() -> ctypes.CDLL:
    """The reference's own CUDA kernels behind the harness; needs a GPU to call."""
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(str(REF_LIB))
    return _ref


def ref_decode_append(q, k, v, q_w, k_w, cos_row, sin_row, key_cache, value_cache, position):
    q, k, v = _u16(q), _u16(k), _u16(v)
    q_rot = np.empty_like(q)
    rc = ref().qmref_decode_append(_p(q), _p(k), _p(v), _p(_u16(q_w)), _p(_u16(k_w)), _p(_u16(cos_row)),
                                   _p(_u16(sin_row)), _p(q_rot), _p(key_cache), _p(value_cache), c_int(q.shape[0]),
                                   c_int(k.shape[0]), c_int(key_cache.shape[1]), c_int(position))
    assert rc == 0, rc
    return q_rot


def ref_prefill_append(q, k, v, q_w, k_w, cos_rows, sin_rows, key_cache, value_cache):
    q, k, v = _u16(q), _u16(k), _u16(v)
    q_rot = np.empty_like(q)
    rc = ref().qmref_prefill_append(_p(q), _p(k), _p(v), _p(_u16(q_w)), _p(_u16(k_w)), _p(_u16(cos_rows)),
                                    _p(_u16(sin_rows)), _p(q_rot), _p(key_cache), _p(value_cache), c_int(q.shape[0]),
                                    c_int(q.shape[1]), c_int(k.shape[1]), c_int(key_cache.shape[1]))
    assert rc == 0, rc
    return q_rot


def ref_attention(q_rot, key_cache, value_cache, query_length, cache_before, iterations=1):
    """Returns (context bits, mean ms per launch); context is None when the reference's launcher
    would need more than its 48 KB of dynamic shared memory."""
    q_rot = _u16(q_rot)
    hq = q_rot.shape[-2]
    out = np.empty_like(q_rot)
    ms = c_float()
    rc = ref().qmref_attention(_p(q_rot), _p(key_cache), _p(value_cache), _p(out), c_int(query_length),
                               c_int(cache_before), c_int(hq), c_int(key_cache.shape[0]), c_int(key_cache.shape[1]),
                               c_int(iterations), ctypes.byref(ms))
    if rc == -2:
        return None, None
    assert rc == 0, rc
    return out, ms.value


def ref_make_rope(rows, start=0):
    cos = np.empty((rows, D), dtype=np.uint16)
    sin = np.empty((rows, D), dtype=np.uint16)
    ref().qmref_make_rope(c_int(rows), c_int(start), _p(cos), _p(sin))
    return cos, sin


# ------------------------------------------------ rest of the talker layer

def scaled_normal_bf16(seed: int, shape, scale: float) -> np.ndarray:
    """bf16 tensor ~ N(0, scale^2): the seeded N(0,1) stream times `scale`, rounded once."""
    return f32_to_bf16(bf16_to_f32(normal_bf16(seed, shape)) * np.float32(scale))


def linear(x, w, bias=None, residual=None, mode="ref"):
    x, w = _u16(x), _u16(w)
    rows, k_dim = x.shape
    n_dim = w.shape[0]
    out = np.empty((rows, n_dim), dtype=np.uint16)
    lib().qmo_linear(_p(x), _p(w), _p(_u16(bias)) if bias is not None else None,
                     _p(_u16(residual)) if residual is not None else None, c_int(rows), c_int(n_dim), c_int(k_dim),
                     c_int(0 if mode == "ref" else 1), _p(out))
    return out


def rmsnorm(x, w, eps=1.0e-6):
    x = _u16(x)
    out = np.empty_like(x)
    lib().qmo_rmsnorm(_p(x), _p(_u16(w)), c_float(eps), c_int(x.shape[0]), c_int(x.shape[1]), _p(out))
    return out


def add_postnorm(hidden, attention, w, eps=1.0e-6):
    hidden, attention = _u16(hidden), _u16(attention)
    residual = np.empty_like(hidden)
    normalized = np.empty_like(hidden)
    lib().qmo_add_postnorm(_p(hidden), _p(attention), _p(_u16(w)), c_float(eps), c_int(hidden.shape[0]),
                           c_int(hidden.shape[1]), _p(residual), _p(normalized))
    return residual, normalized


def gate_up_swiglu(x, gate_w, up_w, mode="ref"):
    x, gate_w, up_w = _u16(x), _u16(gate_w), _u16(up_w)
    out = np.empty((x.shape[0], gate_w.shape[0]), dtype=np.uint16)
    lib().qmo_gate_up_swiglu(_p(x), _p(gate_w), _p(up_w), c_int(x.shape[0]), c_int(x.shape[1]), c_int(gate_w.shape[0]),
                             c_int(0 if mode == "ref" else 1), _p(out))
    return out


def ref_linear(x, w, bias=None, residual=None):
    x, w = _u16(x), _u16(w)
    out = np.empty((x.shape[0], w.shape[0]), dtype=np.uint16)
    rc = ref().qmref_linear_rows(_p(x), _p(w), _p(_u16(bias)) if bias is not None else None,
                                 _p(_u16(residual)) if residual is not None else None, _p(out), c_int(x.shape[0]),
                                 c_int(w.shape[0]), c_int(x.shape[1]))
    assert rc == 0, rc
    return out


def ref_rmsnorm(x, w):
    x = _u16(x)
    out = np.empty_like(x)
    rc = ref().qmref_rmsnorm_rows(_p(x), _p(_u16(w)), _p(out), c_int(x.shape[0]), c_int(x.shape[1]))
    assert rc == 0, rc
    return out


def ref_add_postnorm(hidden, attention, w):
    hidden, attention = _u16(hidden), _u16(attention)
    residual, normalized = np.empty_like(hidden), np.empty_like(hidden)
    rc = ref().qmref_add_postnorm_rows(_p(hidden), _p(attention), _p(_u16(w)), _p(residual), _p(normalized),
                                       c_int(hidden.shape[0]), c_int(hidden.shape[1]))
    assert rc == 0, rc
    return residual, normalized


def ref_gate_up_swiglu(x, gate_w, up_w):
    x, gate_w, up_w = _u16(x), _u16(gate_w), _u16(up_w)
    out = np.empty((x.shape[0], gate_w.shape[0]), dtype=np.uint16)
    rc = ref().qmref_gate_up_swiglu_rows(_p(x), _p(gate_w), _p(up_w), _p(out), c_int(x.shape[0]), c_int(x.shape[1]),
                                         c_int(gate_w.shape[0]))
    assert rc == 0, rc
    return out


def ref_linear_generic(x, w, bias=None, residual=None):
    """The reference's native_ops::linear_bf16 (+ code_predictor::launch_add) for all rows at once, on a GPU."""
    x, w = _u16(x), _u16(w)
    out = np.empty((x.shape[0], w.shape[0]), dtype=np.uint16)
    rc = ref().qmref_linear_generic(_p(x), _p(w), _p(_u16(bias)) if bias is not None else None,
                                    _p(_u16(residual)) if residual is not None else None, _p(out), c_int(x.shape[0]),
                                    c_int(w.shape[0]), c_int(x.shape[1]))
    assert rc == 0, rc
    return out


def ref_gate_up_swiglu_generic(x, gate_w, up_w):
    """The reference's two linear_bf16 calls and code_predictor::launch_swiglu for all rows at once, on a GPU."""
    x, gate_w, up_w = _u16(x), _u16(gate_w), _u16(up_w)
    out = np.empty((x.shape[0], gate_w.shape[0]), dtype=np.uint16)
    rc = ref().qmref_gate_up_swiglu_generic(_p(x), _p(gate_w), _p(up_w), _p(out), c_int(x.shape[0]), c_int(x.shape[1]),
                                            c_int(gate_w.shape[0]))
    assert rc == 0, rc
    return out


def final_head_sample(logits, history=None, generation_index=0, flags=0, eos_token=2150, reserved_begin=None, top_k=0,
                      temperature=0.9, rng_state=0):
    """One stream through the restated final-head chain.  Returns (code, processed scores, new rng state, history)."""
    logits = _u16(logits)
    vocab = logits.shape[0]
    hist = np.zeros(8192, dtype=np.int32) if history is None else np.ascontiguousarray(history, dtype=np.int32).copy()
    state = ctypes.c_uint64(int(rng_state))
    processed = np.empty(vocab, dtype=np.float32)
    fn = lib().qmo_final_head_sample
    fn.restype = c_int
    code = fn(_p(logits), c_int(vocab), _p(hist), c_int(hist.shape[0]), c_int(int(generation_index)), c_int(flags),
              c_int(eos_token), c_int(vocab - 1024 if reserved_begin is None else reserved_begin), c_int(top_k),
              ctypes.c_float(temperature), ctypes.byref(state), _p(processed))
    return int(code), processed, int(state.value), hist


def ref_final_head(logits, history=None, generation_index=0, flags=0, top_k=0, temperature=0.9, rng_state=0):
    """The reference's own final-head kernels (vocabulary 3072) on the GPU, one stream."""
    logits = _u16(logits)
    assert logits.shape[0] == 3072
    hist = np.zeros(8192, dtype=np.int32) if history is None else np.ascontiguousarray(history, dtype=np.int32).copy()
    state = ctypes.c_uint64(int(rng_state))
    processed = np.empty(3072, dtype=np.float32)
    code = ctypes.c_int32(0)
    rc = ref().qmref_final_head(_p(logits), _p(hist), c_int(int(generation_index)), c_int(int(generation_index)), c_int(flags),
                                c_int(top_k), ctypes.c_float(temperature), ctypes.byref(state), _p(processed),
                                ctypes.byref(code))
    assert rc == 0, rc
    return int(code.value), processed, int(state.value), hist


# -------------------------------- the reference's code-predictor kernels (GPU, optional; fixed predictor shapes)

def ref_predictor_qkv_m1(x, q_w, k_w, v_w):
    q = np.empty(q_w.shape[0], dtype=np.uint16)
    k = np.empty(k_w.shape[0], dtype=np.uint16)
    v = np.empty(v_w.shape[0], dtype=np.uint16)
    rc = ref().qmref_predictor_qkv_m1(_p(_u16(x)), _p(_u16(q_w)), _p(_u16(k_w)), _p(_u16(v_w)), _p(q), _p(k), _p(v))
    assert rc == 0, rc
    return q, k, v


def ref_predictor_qk_norm_rope_cache_m1(q, k, v, q_w, k_w, cos_row, sin_row, key_cache, value_cache, position):
    """Caches [8][16][128] are updated in place; returns q_rot [16][128]."""
    q = _u16(q)
    q_rot = np.empty_like(q)
    rc = ref().qmref_predictor_qk_norm_rope_cache_m1(_p(q), _p(_u16(k)), _p(_u16(v)), _p(_u16(q_w)), _p(_u16(k_w)),
                                                     _p(_u16(cos_row)), _p(_u16(sin_row)), _p(q_rot), _p(key_cache),
                                                     _p(value_cache), c_int(position))
    assert rc == 0, rc
    return q_rot


def ref_predictor_attention_m1(q_rot, key_cache, value_cache, key_length):
    q_rot = _u16(q_rot)
    out = np.empty_like(q_rot)
    rc = ref().qmref_predictor_attention_m1(_p(q_rot), _p(_u16(key_cache)), _p(_u16(value_cache)), _p(out), c_int(key_length))
    assert rc == 0, rc
    return out


def ref_predictor_linear_m1(x, w, residual=None):
    x, w = _u16(x), _u16(w)
    out = np.empty(w.shape[0], dtype=np.uint16)
    rc = ref().qmref_predictor_linear_m1(_p(x), _p(w), _p(_u16(residual)) if residual is not None else None, _p(out),
                                         c_int(w.shape[0]), c_int(w.shape[1]))
    assert rc == 0, rc
    return out


def ref_predictor_add_postnorm_m1(hidden, attention, w):
    hidden = _u16(hidden)
    residual, normalized = np.empty_like(hidden), np.empty_like(hidden)
    rc = ref().qmref_predictor_add_postnorm_m1(_p(hidden), _p(_u16(attention)), _p(_u16(w)), _p(residual), _p(normalized))
    assert rc == 0, rc
    return residual, normalized


def ref_predictor_gate_up_swiglu_m1(x, gate_w, up_w):
    out = np.empty(gate_w.shape[0], dtype=np.uint16)
    rc = ref().qmref_predictor_gate_up_swiglu_m1(_p(_u16(x)), _p(_u16(gate_w)), _p(_u16(up_w)), _p(out))
    assert rc == 0, rc
    return out
