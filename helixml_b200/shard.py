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


class PeerGather:
    """The all-gather of a channel-sharded y by peer stores (hx_allgather_y_push), one process per GPU.

    Every rank allocates the full [batch, seq_len, d_full] result with hx_alloc, exports it over CUDA IPC, and maps
    the peers' buffers; `push` then writes this rank's shard into all of them with one kernel.  The handles travel
    over torch.distributed's object all-gather (host side, set-up only).  Call `close` on every rank when done."""

    def __init__(self, batch: int, seq_len: int, d_full: int, dtype, world: int, rank: int):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import _lib as L
        self.batch, self.seq_len, self.d_full, self.world, self.rank, self.dtype = batch, seq_len, d_full, world, rank, dtype
        self.es = 2 if dtype == torch.bfloat16 else 4
        self.nbytes = batch * seq_len * d_full * self.es
        p = C.c_void_p()
        L.check(L.lib().hx_alloc(C.byref(p), self.nbytes))
        self.ptr = p.value
        handle = (C.c_ubyte * 64)()
        L.check(L.lib().hx_ipc_export(C.c_void_p(self.ptr), handle))
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle))
        self.dst = []
        for r in range(world):
            if r == rank:
                self.dst.append(self.ptr)
            else:
                q = C.c_void_p()
                buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                L.check(L.lib().hx_ipc_open(buf, C.byref(q)))
                self.dst.append(q.value)

    def push(self, y_local, col0: int, row_begin: int = 0, row_end: int | None = None, stream: int = 0, max_ctas_per_sm: int = 0):
        import ctypes as C
        from . import _lib as L
        if not y_local.is_contiguous():
            raise L.HxError(1, "push: the local shard must be dense [batch, seq_len, d_shard]")
        a = L.GatherArgs()
        a.world, a.rank = self.world, self.rank
        a.batch, a.seq_len, a.d_shard, a.d_full = self.batch, self.seq_len, y_local.shape[-1], self.d_full
        a.col0 = col0
        a.io_dtype = L.HX_BF16 if self.es == 2 else L.HX_F32
        a.y_local = y_local.data_ptr()
        for r in range(self.world):
            a.dst[r] = self.dst[r]
        a.row_begin, a.row_end = row_begin, self.batch if row_end is None else row_end
        a.max_ctas_per_sm = max_ctas_per_sm
        L.check(L.lib().hx_allgather_y_push(C.byref(a), C.c_void_p(stream)))

    def tensor(self):
        """This rank's full result as a torch tensor [batch, seq_len, d_full] over the same memory."""
        import torch

        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.nbytes // self.es,), "typestr": "<i2" if self.es == 2 else "<f4",
                                        "data": (self.ptr, False), "version": 3}
        t = torch.as_tensor(raw, device="cuda")
        if self.es == 2:
            t = t.view(torch.bfloat16)
        return t.view(self.batch, self.seq_len, self.d_full)

    def close(self):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import _lib as L
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()  # nobody closes a mapping a peer may still write through
        for r, q in enumerate(self.dst):
            if r != self.rank:
                L.check(L.lib().hx_ipc_close(C.c_void_p(q)))
        if self.world > 1:
            dist.barrier()  # every mapping is closed before the owners free
        L.check(L.lib().hx_free(C.c_void_p(self.ptr)))
        self.dst, self.ptr = [], None


def all_gather_channels(y_local, d_inner: int, world: int, align: int = 64):
    """All-gather of a channel-sharded y [B, L, D_r] into [B, L, D] over torch.distributed (gloo in the CPU tests,
    NCCL on GPUs): the host-side reference of the exchange, which PeerGather performs with peer stores.  Shards may
    be ragged, so each rank's slice is padded to the widest shard, gathered, and the padding cut off."""
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
