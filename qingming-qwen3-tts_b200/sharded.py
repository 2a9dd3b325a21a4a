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
