"""world_size-2 gloo test (CPU) of the batch-sharding host logic: the shards' forward outputs
concatenate to the full result and the shared-operand gradient equals the all-reduced sum.  The
matmul itself is done by the CPU oracle here (the test is about the sharding / collective logic)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dfdx_b200.parallel import shard_range


def test_shard_range_partitions():
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from oracle import oracle
    from dfdx_b200.parallel import allreduce_shared_grads, gather_batch, shard_batch
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(6, 5, 4, generator=g, dtype=torch.float64)
    w = torch.randn(3, 4, generator=g, dtype=torch.float64)
    dy = torch.randn(6, 5, 3, generator=g, dtype=torch.float64)
    y_full, bwd_full = oracle.matmul(x, w.permute(1, 0))
    gx_full, gw_full = bwd_full(dy)
    xs, dys = shard_batch(x, world, rank), shard_batch(dy, world, rank)
    y, bwd = oracle.matmul(xs.contiguous(), w.permute(1, 0))
    gx, gw = bwd(dys.contiguous())
    gw = gw.contiguous()
    allreduce_shared_grads([gw])
    ok = torch.allclose(gw, gw_full, atol=1e-12)
    ok &= torch.allclose(gather_batch(y), y_full, atol=1e-12)
    ok &= torch.allclose(gather_batch(gx), gx_full, atol=1e-12)
    # one large matmul cut along the rows of its left operand (strong scaling of `MatMatKernel`): the shared
    # rhs's gradient is the all-reduced sum, through the overlapped reducer and a flat bucket of two gradients
    from dfdx_b200.parallel import FlatBucket, OverlappedReducer, shard_rows
    a = torch.randn(10, 4, generator=g, dtype=torch.float64)
    b = torch.randn(4, 3, generator=g, dtype=torch.float64)
    dc = torch.randn(10, 3, generator=g, dtype=torch.float64)
    c_full, bwd2 = oracle.matmul(a, b)
    ga_full, gb_full = bwd2(dc)
    a_r, dc_r = shard_rows(a, world, rank, align=4), shard_rows(dc, world, rank, align=4)
    c_r, bwd_r = oracle.matmul(a_r.contiguous(), b)
    ga_r, gb_r = bwd_r(dc_r.contiguous())
    bucket = FlatBucket([gb_r.shape, gw.shape], torch.float64, "cpu")
    bucket.views[0].copy_(gb_r)
    bucket.views[1].copy_(gw / world)             # already summed above: every rank holds the same values
    red = OverlappedReducer(None)
    red.start([bucket.flat])
    red.finish()
    ok &= torch.allclose(bucket.views[0], gb_full, atol=1e-12)
    ok &= torch.allclose(bucket.views[1], gw_full, atol=1e-12)
    rows = [shard_rows(torch.arange(10).view(10, 1), world, r, align=4).numel() for r in range(world)]
    ok &= sum(rows) == 10 and rows[0] % 4 == 0
    ok &= torch.allclose(c_r, shard_rows(c_full, world, rank, align=4), atol=1e-12)
    ok &= torch.allclose(ga_r, shard_rows(ga_full, world, rank, align=4), atol=1e-12)
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_sharded_matmul_gloo_world2():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}
