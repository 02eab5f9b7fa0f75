"""GPU, 2 ranks (skipped with fewer than 2 GPUs): row-sharded product with the all-reduce of the
replicated weight's gradient (NCCL called by the library itself, akr_mg_*), and batch sharding, against
the single-process oracle. torch.distributed (gloo) only carries the rendezvous id."""
import os
import subprocess
import sys

import pytest

from util import ROOT

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import numpy as np
sys.path.insert(0, os.environ["AKR_ROOT"]); sys.path.insert(0, os.path.join(os.environ["AKR_ROOT"], "tests"))
import torch.distributed as dist
from util import uniform, normal, rel_fro, TOL_FP32, TOL_TF32
from oracle import matmul_oracle as mo
from aakaar_b200 import cabi
from aakaar_b200.distributed import RowShardedMatmul, BatchShardedMatmul, CudaBackend, NodeComm, exchange_via_torch_store
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
cabi.check(cabi.lib().akr_set_device(int(os.environ["LOCAL_RANK"])))
dist.init_process_group("gloo")
comm = NodeComm(rank, world, exchange_via_torch_store)
assert comm.reduce_scalar(float(rank + 1), "sum") == world * (world + 1) / 2
assert comm.reduce_scalar(float(rank), "max") == world - 1
M, K, N = 1536, 640, 896
a, b, dc = uniform((M, K), 1), uniform((K, N), 2), normal((M, N), 3)
ref_c = mo.matmul_forward(a, b, np.float64)
ref_da, ref_db = mo.matmul_backward(a, b, dc, np.float64)
for mode, tol in ((cabi.MODE_FP32, TOL_FP32), (cabi.MODE_TF32, TOL_TF32)):
    sh = RowShardedMatmul(total_m=M, world=world, rank=rank, backend=CudaBackend(mode=mode, comm=comm))
    A, B, DC = (cabi.DeviceArray.from_numpy(np.ascontiguousarray(x)) for x in (a[sh.lo:sh.hi], b, dc[sh.lo:sh.hi]))
    c = sh.forward(A, B)
    da, db = sh.backward(A, B, DC)
    cabi.synchronize()
    assert rel_fro(c.to_numpy(), ref_c[sh.lo:sh.hi]) < tol
    assert rel_fro(da.to_numpy(), ref_da[sh.lo:sh.hi]) < tol
    assert rel_fro(db.to_numpy(), ref_db) < tol, rel_fro(db.to_numpy(), ref_db)   # summed over ranks
nb = 10
ab, bb = uniform((nb, 64, 96), 4), uniform((nb, 96, 80), 5)
bs = BatchShardedMatmul(total_batch=nb, world=world, rank=rank, backend=CudaBackend(mode=cabi.MODE_FP32))
cb = bs.forward(cabi.DeviceArray.from_numpy(ab[bs.lo:bs.hi]), cabi.DeviceArray.from_numpy(bb[bs.lo:bs.hi]))
assert rel_fro(cb.to_numpy(), mo.matmul_forward(ab, bb, np.float64)[bs.lo:bs.hi]) < TOL_FP32
comm.barrier()
comm.close()
dist.barrier()
dist.destroy_process_group()
sys.stdout.write(f"RANK_OK {rank}\n"); sys.stdout.flush()
'''


def test_row_and_batch_sharding_two_gpus(tmp_path):
    from aakaar_b200 import cabi
    if cabi.lib().akr_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, AKR_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "RANK_OK 0" in res.stdout and "RANK_OK 1" in res.stdout
