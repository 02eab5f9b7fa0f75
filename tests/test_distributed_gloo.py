"""CPU, world_size 2 over gloo: the sharding / reduction logic of aakaar_b200.distributed with the
numpy oracle injected as the per-rank compute (the CUDA backend needs a GPU per rank)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from util import uniform, normal, rel_fro
from oracle import matmul_oracle as mo
from aakaar_b200.distributed import shard_range, RowShardedMatmul, BatchShardedMatmul


class OracleBackend:
    """Same interface as CudaBackend, on numpy arrays and gloo."""
    sm_count = 148

    def __init__(self):
        self.limits = []

    def fwd(self, a, b, out=None):
        return mo.matmul_forward(a, b)

    def bwd(self, a, b, dc, need_da=True, need_db=True, da=None, db=None):
        ga, gb = mo.matmul_backward(a, b, dc)
        return (ga if need_da else None), (gb if need_db else None)

    def set_cta_limit(self, n):
        self.limits.append(n)

    def allreduce_start(self, x):
        t = torch.from_numpy(x)
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True), t

    def allreduce_wait(self, handle):
        handle[0].wait()


def test_shard_range_covers_everything():
    for total, world in ((8192, 8), (10, 3), (7, 8), (65536, 4)):
        spans = [shard_range(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and b - a >= d - c >= 0
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = 96, 40, 56
        a, b, dc = uniform((M, K), 1), uniform((K, N), 2), normal((M, N), 3)
        be = OracleBackend()
        sh = RowShardedMatmul(total_m=M, world=world, rank=rank, backend=be)
        lo, hi = sh.lo, sh.hi
        c_loc = sh.forward(np.ascontiguousarray(a[lo:hi]), b)
        da_loc, db = sh.backward(np.ascontiguousarray(a[lo:hi]), b, np.ascontiguousarray(dc[lo:hi]))
        assert be.limits == [148 - sh.comm_ctas, 0]      # CTA limit lowered during the overlap, then restored
        ref_c = mo.matmul_forward(a, b)
        ref_da, ref_db = mo.matmul_backward(a, b, dc)
        assert rel_fro(c_loc, ref_c[lo:hi]) < 1e-6
        assert rel_fro(da_loc, ref_da[lo:hi]) < 1e-6
        assert rel_fro(db, ref_db) < 1e-6                # full weight gradient on every rank

        nb = 6
        ab, bb = uniform((nb, 8, 12), 4), uniform((nb, 12, 10), 5)
        bs = BatchShardedMatmul(total_batch=nb, world=world, rank=rank, backend=be)
        cb = bs.forward(ab[bs.lo:bs.hi], bb[bs.lo:bs.hi])
        assert rel_fro(cb, mo.matmul_forward(ab, bb)[bs.lo:bs.hi]) < 1e-6
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_row_and_batch_sharding_world2(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
