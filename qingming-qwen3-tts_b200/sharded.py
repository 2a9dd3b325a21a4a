"""Decode attention for streams whose keys are split across the GPUs of one box.

Only very long contexts take this path (everything else shards by stream and needs no exchange).  Rank g holds
the contiguous token slice [g * L / G, (g + 1) * L / G) of every stream in its own pool; the new token's K/V row
is appended on the rank that owns its position.  Each rank runs the split-KV kernel over its slice and produces
the partial softmax state (m, l, o[128]) per (stream, query head); ONE all-gather of [B][Hq][130] fp32 per layer
(33 280 B per rank for 4 streams) brings every rank's partials into local memory, and the combine kernel folds
them in rank order, so every rank ends with the same bits.  K and V never cross NVLink.

The collective is torch.distributed (NCCL on GPUs; gloo in the CPU tests, where the partial and combine steps
are supplied by the caller).
"""
from __future__ import annotations


def slice_bounds(length: int, world: int, rank: int) -> tuple[int, int]:
    """Token range [begin, end) of a stream of `length` keys held by `rank` (contiguous, sizes differ by <= 1)."""
    begin = (length * rank) // world
    end = (length * (rank + 1)) // world
    return begin, end


def owner_of(position: int, length: int, world: int) -> int:
    """Rank whose slice contains `position` (0 <= position < length)."""
    for rank in range(world):
        begin, end = slice_bounds(length, world, rank)
        if begin <= position < end:
            return rank
    raise ValueError("position outside the stream")


class ShardedDecode:
    """partial_fn() -> local partials tensor [B][Hq][130]; combine_fn(gathered [G][B][Hq][130]) -> output."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._gathered = None

    def run(self, partial_fn, combine_fn):
        import torch

        partial = partial_fn().contiguous()
        # rank-major concatenation along dim 0 (the layout every backend accepts), viewed as [G][B][Hq][130]
        flat_shape = (self.world * partial.shape[0],) + tuple(partial.shape[1:])
        if self._gathered is None or tuple(self._gathered.shape) != flat_shape or self._gathered.device != partial.device:
            self._gathered = torch.empty(flat_shape, dtype=partial.dtype, device=partial.device)
        self.dist.all_gather_into_tensor(self._gathered, partial, group=self.group)
        return combine_fn(self._gathered.view((self.world,) + tuple(partial.shape)))


def sharded_decode_attention(engine, sharded: ShardedDecode, layer, q_rot, local_seq_lens, page_table, out=None):
    """One layer of decode attention over this rank's slice + exchange + combine, on the current CUDA stream.

    local_seq_lens[s] is the number of keys of stream s held in THIS rank's pool (0 is fine).
    """
    return sharded.run(
        lambda: engine.launch_attention_partial(layer, q_rot, local_seq_lens, page_table),
        lambda gathered: engine.combine(gathered, out=out),
    )


class PeerExchange:
    """Exchange + combine of the partials in one kernel over peer memory (qm_attention_exchange_combine) instead of
    an all-gather plus a combine kernel.  The exchange buffers are symmetric memory: every rank allocates one and
    maps the others' (torch.distributed._symmetric_memory over CUDA IPC / NVLink).  Call `run` at the same point on
    every rank, with the same number of rows."""

    def __init__(self, engine, rows_capacity: int, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.engine = engine
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.rows_capacity = rows_capacity
        nbytes = engine.lib.qm_exchange_buffer_bytes(self.world, rows_capacity)
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group.group_name)
        self.peer_ptrs = torch.tensor([int(p) for p in self.handle.buffer_ptrs], dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        dist.barrier(self.group)          # every buffer is zeroed and mapped before the first kernel touches it

    def run(self, partial, out=None):
        """partial [B][Hq][130] fp32 of this rank -> combined [B][Hq][128] bf16 (same bits on every rank)."""
        import torch

        from . import HEAD_DIM, _check, _ptr, _stream

        rows = partial.shape[0] * partial.shape[1]
        if out is None:
            out = torch.empty((partial.shape[0], partial.shape[1], HEAD_DIM), dtype=torch.bfloat16, device="cuda")
        _check(self.engine.lib.qm_attention_exchange_combine(
            self.engine.pool, _ptr(partial), _ptr(self.peer_ptrs), self.world, self.rank, rows, self.rows_capacity,
            _ptr(out), _stream()))
        return out


    def run_fused(self, layer, q_rot, local_seq_lens, page_table, out=None):
        """Split-KV kernel over this rank's slice with the exchange and the rank-order fold inside the same launch
        (qm_decode_attention_exchange)."""
        import torch

        from . import _check, _ptr, _stream

        batch = q_rot.shape[0]
        if out is None:
            out = torch.empty_like(q_rot)
        ws = self.engine.workspace(batch)
        _check(self.engine.lib.qm_decode_attention_exchange(
            self.engine.pool, layer, _ptr(q_rot), _ptr(local_seq_lens), _ptr(page_table), page_table.shape[1], batch,
            self.engine.q_heads, _ptr(out), _ptr(self.peer_ptrs), self.world, self.rank, self.rows_capacity, _ptr(ws),
            ws.numel(), _stream()))
        return out


class IpcExchange:
    """The same exchange on buffers the library allocates itself and shares through CUDA IPC handles
    (qm_exchange_create / qm_exchange_ipc_handle / qm_exchange_open_peers): what a C++ host with one process per GPU
    uses.  Here the 64-byte handles travel through torch.distributed's object all-gather."""

    def __init__(self, engine, rows_capacity: int, group=None):
        import ctypes

        import torch
        import torch.distributed as dist

        from . import IPC_HANDLE_BYTES, _check

        self.engine = engine
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        handle = ctypes.c_void_p()
        _check(engine.lib.qm_exchange_create(self.world, self.rank, rows_capacity, ctypes.byref(handle)))
        self.handle = handle
        mine = ctypes.create_string_buffer(IPC_HANDLE_BYTES)
        _check(engine.lib.qm_exchange_ipc_handle(self.handle, mine))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, bytes(mine.raw), group=self.group)
        packed = ctypes.create_string_buffer(b"".join(everyone), IPC_HANDLE_BYTES * self.world)
        _check(engine.lib.qm_exchange_open_peers(self.handle, packed))
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def run(self, partial, out=None):
        import torch

        from . import HEAD_DIM, _check, _ptr, _stream

        rows = partial.shape[0] * partial.shape[1]
        if out is None:
            out = torch.empty((partial.shape[0], partial.shape[1], HEAD_DIM), dtype=torch.bfloat16, device="cuda")
        _check(self.engine.lib.qm_exchange_combine(self.engine.pool, self.handle, _ptr(partial), rows, _ptr(out), _stream()))
        return out

    def run_fused(self, layer, q_rot, local_seq_lens, page_table, out=None):
        import torch

        from . import _check, _ptr, _stream

        batch = q_rot.shape[0]
        if out is None:
            out = torch.empty_like(q_rot)
        ws = self.engine.workspace(batch)
        _check(self.engine.lib.qm_exchange_decode_attention(
            self.engine.pool, self.handle, layer, _ptr(q_rot), _ptr(local_seq_lens), _ptr(page_table), page_table.shape[1],
            batch, self.engine.q_heads, _ptr(out), _ptr(ws), ws.numel(), _stream()))
        return out

    def close(self):
        if self.handle:
            self.engine.lib.qm_exchange_destroy(self.handle)
            self.handle = None


def sharded_decode_attention_peer(engine, exchange, layer, q_rot, local_seq_lens, page_table, out=None):
    """Split-KV kernel over this rank's slice, then the one-kernel peer-memory exchange + combine."""
    partial = engine.launch_attention_partial(layer, q_rot, local_seq_lens, page_table)
    return exchange.run(partial, out=out)


class NcclSharded:
    """qm_decode_attention_sharded on a communicator the library's own helpers create (ncclGetUniqueId on rank 0,
    passed to the others through torch.distributed, ncclCommInitRank on every rank): the path a C++ host takes,
    driven from Python for the tests and the benchmark."""

    def __init__(self, engine, batch: int, group=None):
        import ctypes

        import torch
        import torch.distributed as dist

        from . import PARTIAL_STRIDE, _check

        self.engine = engine
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        ident = ctypes.create_string_buffer(128)
        if self.rank == 0:
            _check(engine.lib.qm_nccl_unique_id(ident))
        box = [bytes(ident.raw)]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.group)
        ident = ctypes.create_string_buffer(box[0], 128)
        comm = ctypes.c_void_p()
        _check(engine.lib.qm_nccl_comm_init_rank(ctypes.byref(comm), self.world, ident, self.rank))
        self.comm = comm
        self.send = torch.empty((batch, engine.q_heads, PARTIAL_STRIDE), dtype=torch.float32, device="cuda")
        self.recv = torch.empty((self.world, batch, engine.q_heads, PARTIAL_STRIDE), dtype=torch.float32, device="cuda")

    def run(self, layer, q_rot, local_seq_lens, page_table, out=None):
        import torch

        from . import _check, _ptr, _stream

        batch = q_rot.shape[0]
        if out is None:
            out = torch.empty_like(q_rot)
        ws = self.engine.workspace(batch)
        _check(self.engine.lib.qm_decode_attention_sharded(
            self.engine.pool, layer, _ptr(q_rot), _ptr(local_seq_lens), _ptr(page_table), page_table.shape[1], batch,
            self.engine.q_heads, _ptr(out), _ptr(self.send), _ptr(self.recv), self.world, _ptr(ws), ws.numel(),
            self.comm, _stream()))
        return out

    def wait(self, deadline_ms=10000):
        from . import _check, _stream

        _check(self.engine.lib.qm_nccl_wait(self.comm, _stream(), deadline_ms))

    def close(self):
        if self.comm:
            self.engine.lib.qm_nccl_comm_destroy(self.comm)
            self.comm = None
