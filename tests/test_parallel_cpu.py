"""Tensor-parallel sharding logic on CPU: bit-identity of sharded quantisation, and a world_size-2 gloo
run of column-/row-parallel layers against the unsharded result (oracle stands in for the kernels)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import weight
from oracle import oracle


def test_sharded_quantisation_is_bit_identical():
    from mxfp4.parallel import shard_quantized
    w = weight(64, 512, 3, True)
    p, s = oracle.quantize(w)
    for world in (2, 4, 8):
        for rank in range(world):
            n = 64 // world
            ps, ss = shard_quantized(p, s, 0, world, rank)
            op, os_ = oracle.quantize(w[rank * n:(rank + 1) * n].contiguous())
            assert torch.equal(ps, op) and torch.equal(ss, os_)
            k = 512 // world
            ps, ss = shard_quantized(p, s, 1, world, rank)
            op, os_ = oracle.quantize(w[:, rank * k:(rank + 1) * k].contiguous())
            assert torch.equal(ps, op) and torch.equal(ss, os_)
    with pytest.raises(ValueError):
        shard_quantized(p, s, 1, 3, 0)
    with pytest.raises(ValueError):
        shard_quantized(p[:, :48], s[:, :3], 1, 2, 0)      # 96 columns: not whole blocks per rank


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        import conftest  # noqa: F401  (import paths)
        import fake_backend
        fake_backend.install()
        from mxfp4 import MXLinear
        from mxfp4.parallel import ColumnParallelMXLinear, RowParallelMXLinear
        torch.manual_seed(0)
        up = MXLinear(128, 256, bias=True)
        down = MXLinear(256, 128, bias=True)
        up.weight.data = weight(256, 128, 1, True).float()
        down.weight.data = weight(128, 256, 2, True).float()
        up.quantize(); down.quantize()
        x = torch.randn(6, 128, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
        full = down(torch.relu(up(x)))
        cp = ColumnParallelMXLinear.from_mxlinear(up)
        rp = RowParallelMXLinear.from_mxlinear(down)
        assert cp.packed_weight.shape == (128, 64) and rp.packed_weight.shape == (128, 64)
        h = cp(x)
        assert torch.equal(h, up(x)[:, rank * 128:(rank + 1) * 128])        # column shards are bit-identical
        y = rp(torch.relu(h))
        err = ((y.float() - full.float()).norm() / full.float().norm()).item()
        gathered = ColumnParallelMXLinear.from_mxlinear(up, gather_output=True)(x)
        ok = err < 0.1 and torch.equal(gathered, up(x))   # row-parallel: each shard re-quantises its own slice of the activations
        q.put((rank, ok, err))
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in res), res
