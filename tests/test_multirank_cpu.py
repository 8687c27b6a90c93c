"""World-size-2 (and 3) gloo tests, on CPU, of the multi-GPU host logic: the shard arithmetic, the
property the sharding rests on (shards computed alone equal the same rows/channels of the full problem,
checked with the CPU oracle standing in for the kernel), the ragged all-gather of y and the max-over-ranks
timing reduction."""
import os
import socket
import sys

import numpy as np
import pytest

from helixml_b200 import shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_arithmetic():
    for batch, world in [(32, 1), (32, 8), (7, 3), (2, 4)]:
        spans = [shard.batch_shard(batch, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == batch
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    for d, world in [(5120, 8), (1536, 4), (200, 3), (64, 2)]:
        spans = [shard.channel_shard(d, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == d
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(a % 64 == 0 for a, _ in spans)  # tile-aligned starts keep TMA alignment
    assert shard.channel_shard(5120, 8, 3) == (1920, 2560)
    with pytest.raises(ValueError):
        shard.batch_shard(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from helixml_b200 import shard as sh, synth
    from oracle import cbind
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cbind.set_num_threads(1)
    B, L, D, N = 4, 40, 200, 16
    inp = synth.scan_inputs(77, B, L, D, N, 4, bf16=False)
    kw = dict(D=inp["D"], z=inp["z"], conv_w=inp["conv_w"])
    full = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], **kw)
    if mode == "channels":
        a, b = sh.channel_shard(D, world, rank)
        y = cbind.selective_scan(inp["x"][:, :, a:b], inp["dt"][:, :, a:b], inp["A"][a:b], inp["B"], inp["C"],
                                 D=inp["D"][a:b], z=inp["z"][:, :, a:b], conv_w=inp["conv_w"][a:b])
        ok_local = np.array_equal(y, full[:, :, a:b])
        gathered = sh.all_gather_channels(torch.from_numpy(y), D, world).numpy()
        ok = ok_local and np.array_equal(gathered, full)
    else:
        a, b = sh.batch_shard(B, world, rank)
        y = cbind.selective_scan(inp["x"][a:b], inp["dt"][a:b], inp["A"], inp["B"][a:b], inp["C"][a:b],
                                 D=inp["D"], z=inp["z"][a:b], conv_w=inp["conv_w"])
        ok = np.array_equal(y, full[a:b])
    slowest = sh.max_over_ranks(10.0 + rank)
    ok = ok and slowest == 10.0 + world - 1
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "channels"), (2, "batch"), (3, "channels")])
def test_shards_are_independent_and_gather(world, mode):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=10) == 1
