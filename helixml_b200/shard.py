"""Sharding of the state-space path over the GPUs of one node.

Every (batch row, channel) pair is an independent recurrence over time; B_t and C_t are shared by the
channels of one batch row only.  So the path shards with no exchange step:
  * by batch (model prefill): rank r gets a contiguous block of batch rows and a full weight replica;
  * by channel (wide scan): rank r gets a contiguous, tile-aligned block of channels of x/dt/z/A/D/conv
    and ALL of B and C; the only collective is an optional all-gather of y at the end.
The sequence axis is never split across GPUs (that would need a carry exchange)."""
from __future__ import annotations


def batch_shard(batch: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the batch rows of `rank`; the first `batch % world` ranks get one extra row."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of world {world}")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def channel_shard(d_inner: int, world: int, rank: int, align: int = 64) -> tuple[int, int]:
    """[start, stop) of the channels of `rank`, in units of `align` channels (one 128-byte bf16 tile), so that
    every shard's base pointer and row stride keep the 16-byte alignment the TMA path needs."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of world {world}")
    tiles = (d_inner + align - 1) // align
    t0, t1 = batch_shard(tiles, world, rank)
    return min(t0 * align, d_inner), min(t1 * align, d_inner)


def all_gather_channels(y_local, d_inner: int, world: int, align: int = 64):
    """All-gather of a channel-sharded y [B, L, D_r] into [B, L, D] over torch.distributed (NCCL on GPUs,
    gloo in the CPU tests).  Shards may be ragged, so each rank's slice is padded to the widest shard,
    gathered, and the padding cut off."""
    import torch
    import torch.distributed as dist
    widths = [channel_shard(d_inner, world, r, align) for r in range(world)]
    wmax = max(b - a for a, b in widths)
    pad = torch.zeros((*y_local.shape[:-1], wmax), dtype=y_local.dtype, device=y_local.device)
    pad[..., : y_local.shape[-1]] = y_local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[..., : b - a] for p, (a, b) in zip(parts, widths)], dim=-1)


def max_over_ranks(value: float, device=None) -> float:
    """The slowest rank's time: what a multi-GPU measurement reports."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
