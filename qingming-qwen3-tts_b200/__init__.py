"""B200-native talker attention path of the Qwen3-TTS engine.

This package holds the CUDA sources (``csrc/``), the build step and a thin
ctypes binding of the C ABI declared in ``include/qm_attention.h``.  The
binding exists for the tests and the benchmark: device memory and streams come
from PyTorch, every computation goes through the C entry points.  There is no
CPU path: if the shared library is missing or cannot be loaded, importing the
binding raises.

``TalkerAttention`` mirrors, method for method, the launcher surface of the
reference's ``NativeTalkerEngine`` for this path
(devices/rtx4090-24g/qwen3_tts_1_7b.cu):

    launch_qk_norm_rope_cache_m1   :17741    -> qm_decode_append_rope
    launch_attention               :17895    -> qm_decode_attention / qm_prefill_attention_varlen
    launch_rmsnorm x2 + launch_rope_rows x2 + scatter_prefill_cache
                                   :16763-16798 -> qm_prefill_append_rope_varlen
    reset_request                  :16607    -> qm_kv_pool_reset
    LayerCache                     :16419    -> qm_kv_pool_create
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_uint32, c_void_p

from ._build import LIB_PATH, build_library

QM_OK = 0
QM_EINVAL = -1
QM_ECAPACITY = -2
QM_ECUDA = -3
QM_ETIMEOUT = -4
QM_ENOMEM = -5
QM_EDEVICE = -6
QM_ENCCL = -7
IPC_HANDLE_BYTES = 64
QM_SAMPLE_REPETITION, QM_SAMPLE_SUPPRESS, QM_SAMPLE_RECORD = 1, 2, 4

DEVSTAT_BAD_PAGE = 1
DEVSTAT_BAD_POS = 2
DEVSTAT_TIMEOUT = 4

HEAD_DIM = 128
PAGE_TOKENS = 64
PARTIAL_STRIDE = HEAD_DIM + 2

# name -> (restype, argtypes); must list every symbol of include/qm_attention.h
ABI = {
    "qm_last_error_string": (c_char_p, []),
    "qm_validate_b200_device": (c_int32, [c_int32, POINTER(c_int32)]),
    "qm_kv_pool_create": (c_int32, [c_int32, c_int32, c_int32, POINTER(c_void_p)]),
    "qm_kv_pool_destroy": (c_int32, [c_void_p]),
    "qm_kv_pool_reset": (c_int32, [c_void_p, c_void_p]),
    "qm_kv_pool_key_ptr": (c_void_p, [c_void_p, c_int32]),
    "qm_kv_pool_value_ptr": (c_void_p, [c_void_p, c_int32]),
    "qm_kv_pool_num_pages": (c_int32, [c_void_p]),
    "qm_kv_pool_kv_heads": (c_int32, [c_void_p]),
    "qm_kv_pool_status": (c_int32, [c_void_p, c_void_p, POINTER(c_uint32)]),
    "qm_selftest_wait_timeout": (c_int32, [c_void_p, c_void_p]),
    "qm_rope_table_fill": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_double, c_void_p]),
    "qm_decode_append_rope": (c_int32, [c_void_p, c_int32] + [c_void_p] * 7 + [c_int32, c_void_p, c_void_p, c_int32,
                                                                           c_int32, c_int32, c_float, c_void_p, c_void_p]),
    "qm_decode_append_rope_sliced": (c_int32, [c_void_p, c_int32] + [c_void_p] * 7 + [c_int32, c_void_p, c_void_p, c_void_p,
                                                                                  c_int32, c_int32, c_int32, c_float, c_void_p,
                                                                                  c_void_p]),
    "qm_prefill_append_rope_varlen": (c_int32, [c_void_p, c_int32] + [c_void_p] * 7 +
                                      [c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                       c_float, c_void_p, c_void_p]),
    "qm_decode_workspace_bytes": (c_int64, [c_int32, c_int32]),
    "qm_decode_workspace_init": (c_int32, [c_void_p, c_int64, c_void_p]),
    "qm_decode_attention": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                      c_void_p, c_void_p, c_int64, c_void_p]),
    "qm_decode_step": (c_int32, [c_void_p, c_int32] + [c_void_p] * 7 + [c_int32, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                                                    c_float, c_void_p, c_void_p, c_int64, c_void_p]),
    "qm_decode_attention_static": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                             c_int32, c_void_p, c_void_p]),
    "qm_decode_attention_partial": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                              c_int32, c_void_p, c_void_p, c_int64, c_void_p]),
    "qm_attention_combine": (c_int32, [c_void_p, c_int32, c_int32, c_void_p, c_void_p]),
    "qm_rmsnorm": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_float, c_void_p]),
    "qm_add_postnorm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_float, c_void_p]),
    "qm_linear": (c_int32, [c_void_p] * 6 + [c_int32, c_int32, c_int32, c_void_p]),
    "qm_qkv_linear": (c_int32, [c_void_p] * 11 + [c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "qm_gate_up_swiglu": (c_int32, [c_void_p] * 5 + [c_int32, c_int32, c_int32, c_void_p]),
    "qm_linear_rows": (c_int32, [c_void_p] * 6 + [c_int32, c_int32, c_int32, c_void_p]),
    "qm_gate_up_swiglu_rows": (c_int32, [c_void_p] * 5 + [c_int32, c_int32, c_int32, c_void_p]),
    "qm_final_head_sample": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_int32, c_void_p, c_int32, c_int32,
                                       c_int32, c_int32, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "qm_embedding_gather": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "qm_exchange_buffer_bytes": (c_int64, [c_int32, c_int32]),
    "qm_attention_exchange_combine": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                                c_void_p, c_void_p]),
    "qm_decode_attention_exchange": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                               c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_int64, c_void_p]),
    "qm_exchange_decode_attention": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                               c_int32, c_void_p, c_void_p, c_int64, c_void_p]),
    "qm_exchange_create": (c_int32, [c_int32, c_int32, c_int32, POINTER(c_void_p)]),
    "qm_exchange_destroy": (c_int32, [c_void_p]),
    "qm_exchange_local_buffer": (c_void_p, [c_void_p]),
    "qm_exchange_ipc_handle": (c_int32, [c_void_p, c_void_p]),
    "qm_exchange_open_peers": (c_int32, [c_void_p, c_void_p]),
    "qm_exchange_set_peers": (c_int32, [c_void_p, c_void_p]),
    "qm_exchange_reset": (c_int32, [c_void_p, c_void_p]),
    "qm_exchange_combine": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_void_p]),
    "qm_decode_static_scratch_reset": (c_int32, [c_void_p, c_void_p]),
    "qm_decode_attention_sharded": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                              c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_void_p]),
    "qm_nccl_wait": (c_int32, [c_void_p, c_void_p, c_int32]),
    "qm_nccl_set_api": (c_int32, [c_void_p]),
    "qm_nccl_unique_id": (c_int32, [c_void_p]),
    "qm_nccl_comm_init_rank": (c_int32, [POINTER(c_void_p), c_int32, c_void_p, c_int32]),
    "qm_nccl_comm_destroy": (c_int32, [c_void_p]),
    "qm_prefill_attention_varlen": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                              c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
}

_lib = None


class QmError(RuntimeError):
    """Raised when a C entry point returns a non-zero status (the reference throws std::runtime_error)."""

    def __init__(self, code: int, text: str):
        super().__init__(f"qm status {code}: {text}")
        self.code = code


def load_library(path=None) -> ctypes.CDLL:
    """Loads libqm_attention_b200.so and declares every prototype.  Fails loudly when it is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    lib_path = str(path or os.environ.get("QM_ATTENTION_LIBRARY") or LIB_PATH)     # the variable selects another build of the library
    try:
        lib = ctypes.CDLL(lib_path)
    except OSError as exc:
        raise RuntimeError(
            f"cannot load {lib_path}: {exc}. Build it with __graft_entry__.build(); there is no CPU fallback."
        ) from exc
    for name, (restype, argtypes) in ABI.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _lib = lib
    return lib


def _check(code: int) -> None:
    if code != QM_OK:
        text = load_library().qm_last_error_string()
        raise QmError(code, text.decode() if text else "")


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


class TalkerAttention:
    """Owns a paged KV pool and a RoPE table on the current CUDA device and launches the attention path.

    Tensors are torch CUDA tensors: bf16 activations as torch.bfloat16, integer arrays as torch.int32.
    """

    def __init__(self, layers: int, num_pages: int, q_heads: int = 16, kv_heads: int = 8, max_positions: int = 8192,
                 theta: float = 1.0e6, epsilon: float = 1.0e-6):
        import torch

        self.lib = load_library()
        self.layers, self.num_pages = layers, num_pages
        self.q_heads, self.kv_heads = q_heads, kv_heads
        self.epsilon = epsilon
        self.max_positions = max_positions
        handle = c_void_p()
        _check(self.lib.qm_kv_pool_create(layers, num_pages, kv_heads, ctypes.byref(handle)))
        self.pool = handle
        self.rope_cos = torch.empty((max_positions, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
        self.rope_sin = torch.empty_like(self.rope_cos)
        _check(self.lib.qm_rope_table_fill(_ptr(self.rope_cos), _ptr(self.rope_sin), max_positions, 0, theta, _stream()))
        self._workspace = None

    def close(self) -> None:
        if getattr(self, "pool", None):
            self.lib.qm_kv_pool_destroy(self.pool)
            self.pool = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- cache object ------------------------------------------------------
    def max_cache(self, max_pages: int) -> int:
        """Tokens one stream can hold with `max_pages` page-table entries (the reference's max_cache())."""
        return max_pages * PAGE_TOKENS

    def reset_request(self) -> None:
        _check(self.lib.qm_kv_pool_reset(self.pool, _stream()))

    def status(self) -> int:
        bits = c_uint32()
        _check(self.lib.qm_kv_pool_status(self.pool, _stream(), ctypes.byref(bits)))
        return bits.value

    def pool_view(self, layer: int):
        """(K, V) torch views [num_pages][kv_heads][64][128] of one layer's pools (no copy)."""
        import torch

        shape = (self.num_pages, self.kv_heads, PAGE_TOKENS, HEAD_DIM)
        return tuple(_wrap_device_pointer(p, shape, torch.bfloat16)
                     for p in (self.lib.qm_kv_pool_key_ptr(self.pool, layer),
                               self.lib.qm_kv_pool_value_ptr(self.pool, layer)))

    # -- launchers ----------------------------------------------------------
    def launch_qk_norm_rope_cache_m1(self, layer, q, k, v, q_norm_weight, k_norm_weight, positions, page_table,
                                     q_rot=None):
        import torch

        batch = q.shape[0]
        if q_rot is None:
            q_rot = torch.empty_like(q)
        _check(self.lib.qm_decode_append_rope(
            self.pool, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_weight), _ptr(k_norm_weight),
            _ptr(self.rope_cos), _ptr(self.rope_sin), self.max_positions, _ptr(positions), _ptr(page_table),
            page_table.shape[1], batch, self.q_heads, self.epsilon, _ptr(q_rot), _stream()))
        return q_rot

    def launch_qk_norm_rope_cache_m1_sliced(self, layer, q, k, v, q_norm_weight, k_norm_weight, positions,
                                            cache_positions, page_table, q_rot=None):
        """Decode append when this pool holds a slice of each stream: RoPE row and cache slot given separately."""
        import torch

        batch = q.shape[0]
        if q_rot is None:
            q_rot = torch.empty_like(q)
        _check(self.lib.qm_decode_append_rope_sliced(
            self.pool, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_weight), _ptr(k_norm_weight),
            _ptr(self.rope_cos), _ptr(self.rope_sin), self.max_positions, _ptr(positions), _ptr(cache_positions),
            _ptr(page_table), page_table.shape[1], batch, self.q_heads, self.epsilon, _ptr(q_rot), _stream()))
        return q_rot

    def prefill_norm_rope_scatter(self, layer, q, k, v, q_norm_weight, k_norm_weight, cu_seqlens, page_table,
                                  start_positions=None, q_rot=None):
        import torch

        total = q.shape[0]
        batch = cu_seqlens.shape[0] - 1
        if q_rot is None:
            q_rot = torch.empty_like(q)
        _check(self.lib.qm_prefill_append_rope_varlen(
            self.pool, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_weight), _ptr(k_norm_weight),
            _ptr(self.rope_cos), _ptr(self.rope_sin), self.max_positions, _ptr(cu_seqlens), _ptr(start_positions),
            _ptr(page_table), page_table.shape[1], batch, total, self.q_heads, self.epsilon, _ptr(q_rot), _stream()))
        return q_rot

    def workspace(self, batch: int):
        import torch

        need = self.lib.qm_decode_workspace_bytes(batch, self.kv_heads)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
            _check(self.lib.qm_decode_workspace_init(_ptr(self._workspace), need, _stream()))
        return self._workspace

    def launch_attention(self, layer, q_rot, seq_lens, page_table, out=None):
        """Decode attention (query_length == 1): one query token per stream."""
        import torch

        batch = q_rot.shape[0]
        if out is None:
            out = torch.empty_like(q_rot)
        ws = self.workspace(batch)
        _check(self.lib.qm_decode_attention(self.pool, layer, _ptr(q_rot), _ptr(seq_lens), _ptr(page_table),
                                            page_table.shape[1], batch, self.q_heads, _ptr(out), _ptr(ws),
                                            ws.numel(), _stream()))
        return out

    def decode_step(self, layer, q, k, v, q_norm_weight, k_norm_weight, positions, page_table, out=None):
        """launch_qk_norm_rope_cache_m1 + launch_attention of one layer in a single launch."""
        import torch

        batch = q.shape[0]
        if out is None:
            out = torch.empty_like(q)
        ws = self.workspace(batch)
        _check(self.lib.qm_decode_step(
            self.pool, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_weight), _ptr(k_norm_weight), _ptr(self.rope_cos),
            _ptr(self.rope_sin), self.max_positions, _ptr(positions), _ptr(page_table), page_table.shape[1], batch,
            self.q_heads, self.epsilon, _ptr(out), _ptr(ws), ws.numel(), _stream()))
        return out

    # -- rest of the decoder layer (reference launcher names) ----------------
    def launch_rmsnorm(self, x, weight, out=None):
        import torch

        out = torch.empty_like(x) if out is None else out
        _check(self.lib.qm_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), x.shape[0], x.shape[1], self.epsilon, _stream()))
        return out

    def launch_add_postnorm_m1(self, hidden, attention, weight, residual=None, normalized=None):
        import torch

        residual = torch.empty_like(hidden) if residual is None else residual
        normalized = torch.empty_like(hidden) if normalized is None else normalized
        _check(self.lib.qm_add_postnorm(_ptr(hidden), _ptr(attention), _ptr(weight), _ptr(residual), _ptr(normalized),
                                        hidden.shape[0], hidden.shape[1], self.epsilon, _stream()))
        return residual, normalized

    def launch_linear_m1(self, x, weight, bias=None, residual=None, out=None):
        import torch

        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.qm_linear(self.pool, _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), _ptr(out), x.shape[0],
                                  weight.shape[0], weight.shape[1], _stream()))
        return out

    def launch_qkv_m1(self, x, q_weight, k_weight, v_weight, q_bias=None, k_bias=None, v_bias=None, out=None):
        """q, k, v projections in one launch; returns (q [rows][q_dim], k, v [rows][kv_dim])."""
        import torch

        rows = x.shape[0]
        if out is None:
            out = tuple(torch.empty((rows, w.shape[0]), dtype=torch.bfloat16, device="cuda")
                        for w in (q_weight, k_weight, v_weight))
        _check(self.lib.qm_qkv_linear(self.pool, _ptr(x), _ptr(q_weight), _ptr(q_bias), _ptr(k_weight), _ptr(k_bias),
                                      _ptr(v_weight), _ptr(v_bias), _ptr(out[0]), _ptr(out[1]), _ptr(out[2]), rows,
                                      x.shape[1], q_weight.shape[0], k_weight.shape[0], _stream()))
        return out

    def launch_gate_up_swiglu_m1(self, x, gate_weight, up_weight, out=None):
        import torch

        if out is None:
            out = torch.empty((x.shape[0], gate_weight.shape[0]), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.qm_gate_up_swiglu(self.pool, _ptr(x), _ptr(gate_weight), _ptr(up_weight), _ptr(out), x.shape[0],
                                          x.shape[1], gate_weight.shape[0], _stream()))
        return out

    def linear_generic(self, x, weight, bias=None, residual=None, out=None):
        """linear_generic of the reference's prefill loop (17.cu:16730-16860) for any number of token rows; with
        `residual`, the loop's launch_add is folded in."""
        import torch

        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.qm_linear_rows(self.pool, _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), _ptr(out), x.shape[0],
                                       weight.shape[0], weight.shape[1], _stream()))
        return out

    def gate_up_swiglu_rows(self, x, gate_weight, up_weight, out=None):
        """Gate and up projections plus swiglu_kernel (17.cu:8771) of the prefill loop, any number of rows."""
        import torch

        if out is None:
            out = torch.empty((x.shape[0], gate_weight.shape[0]), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.qm_gate_up_swiglu_rows(self.pool, _ptr(x), _ptr(gate_weight), _ptr(up_weight), _ptr(out),
                                               x.shape[0], x.shape[1], gate_weight.shape[0], _stream()))
        return out

    def final_head_sample(self, logits, generation_index=None, history=None, flags=0, eos_token=2150,
                          reserved_begin=None, top_k=0, temperature=0.9, rng_state=None, codes=None, processed=None):
        """NativeFinalHead::run_fast after the head projection (17.cu:14384-14560) for a batch of streams: cast,
        repetition penalty, token suppression, then argmax (top_k = 0) or top-k sampling; optionally records the
        code in the history.  rng_state is an int64 tensor holding each stream's SplitMix64 state."""
        import torch

        batch, vocab = logits.shape
        if codes is None:
            codes = torch.empty((batch,), dtype=torch.int32, device="cuda")
        if reserved_begin is None:
            reserved_begin = vocab - 1024
        capacity = history.shape[1] if history is not None else 0
        _check(self.lib.qm_final_head_sample(self.pool, _ptr(logits), batch, vocab, _ptr(history), capacity,
                                             _ptr(generation_index), flags, eos_token, reserved_begin, top_k,
                                             float(temperature), _ptr(rng_state), _ptr(codes), _ptr(processed), _stream()))
        return codes

    def embedding_gather(self, table, token_ids, out=None):
        """gather_embedding_kernel (17.cu:8875) for a batch: out[r] = table[token_ids[r]]."""
        import torch

        rows = token_ids.shape[0]
        if out is None:
            out = torch.empty((rows, table.shape[1]), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.qm_embedding_gather(self.pool, _ptr(table), _ptr(token_ids), rows, table.shape[0], table.shape[1],
                                            _ptr(out), _stream()))
        return out

    def launch_attention_static(self, layer, q_rot, seq_lens, page_table, out=None):
        """Decode attention through the entry point that uses the library's built-in scratch (no workspace)."""
        import torch

        batch = q_rot.shape[0]
        if out is None:
            out = torch.empty_like(q_rot)
        _check(self.lib.qm_decode_attention_static(self.pool, layer, _ptr(q_rot), _ptr(seq_lens), _ptr(page_table),
                                                   page_table.shape[1], batch, self.q_heads, _ptr(out), _stream()))
        return out

    def launch_attention_partial(self, layer, q_rot, seq_lens, page_table, partial=None):
        import torch

        batch = q_rot.shape[0]
        if partial is None:
            partial = torch.empty((batch, self.q_heads, PARTIAL_STRIDE), dtype=torch.float32, device="cuda")
        ws = self.workspace(batch)
        _check(self.lib.qm_decode_attention_partial(self.pool, layer, _ptr(q_rot), _ptr(seq_lens), _ptr(page_table),
                                                    page_table.shape[1], batch, self.q_heads, _ptr(partial),
                                                    _ptr(ws), ws.numel(), _stream()))
        return partial

    def combine(self, partials, out=None):
        """partials [parts][batch][q_heads][130] fp32 -> [batch][q_heads][128] bf16."""
        import torch

        parts, batch, heads = partials.shape[0], partials.shape[1], partials.shape[2]
        if out is None:
            out = torch.empty((batch, heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.qm_attention_combine(_ptr(partials), parts, batch * heads, _ptr(out), _stream()))
        return out

    def launch_attention_prefill(self, layer, q_rot, cu_seqlens, page_table, max_seqlen, start_positions=None,
                                 out=None):
        """Causal attention over packed varlen queries (query_length > 1)."""
        import torch

        total = q_rot.shape[0]
        batch = cu_seqlens.shape[0] - 1
        if out is None:
            out = torch.empty_like(q_rot)
        _check(self.lib.qm_prefill_attention_varlen(self.pool, layer, _ptr(q_rot), _ptr(cu_seqlens),
                                                    _ptr(start_positions), _ptr(page_table), page_table.shape[1],
                                                    batch, total, max_seqlen, self.q_heads, _ptr(out), _stream()))
        return out


def _wrap_device_pointer(ptr: int, shape, dtype):
    """A torch tensor aliasing device memory owned by the library (valid while the pool lives)."""
    import math

    import torch

    elems = math.prod(shape)

    class _Holder:
        pass

    holder = _Holder()
    holder.__cuda_array_interface__ = {
        "shape": (elems,),
        "typestr": "<i2",
        "data": (int(ptr), False),
        "version": 3,
    }
    flat = torch.as_tensor(holder, device="cuda")
    return flat.view(dtype).view(shape)
