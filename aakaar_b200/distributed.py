"""Sharding of the matmul path across the GPUs of one node (one process per GPU).

The reference has no multi-GPU support at all (docs/limitations.md:15); these helpers are new
surface. Two layouts cover the path:

* ``BatchShardedMatmul`` - independent batched products split along the batch dim. Each rank owns a
  contiguous batch range of A, B, C and all gradients. No collective.
* ``RowShardedMatmul`` - one large product split along M with B replicated. Forward and dA are
  local; every rank's dB = A_r^T . dC_r is a partial sum, so dB is all-reduced (NCCL over NVLink).
  The all-reduce is issued right after the dB GEMM and overlaps the dA GEMM, which then runs on a
  reduced number of CTAs so that the collective's kernels find free SMs.

Compute and communication are injected as small backends so that the partitioning / reduction
logic is testable on CPU ranks (gloo); the default backend is the CUDA library through its C ABI.
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_range(total: int, world: int, rank: int):
    """Contiguous [lo, hi) of `total` units for `rank`; the first `total % world` ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("shard_range: bad world / rank")
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class CudaBackend:
    """Local products on this rank's GPU through the C ABI; collectives through torch.distributed."""

    def __init__(self, mode=-1, group=None):
        from . import cabi
        self.cabi = cabi
        self.mode = mode
        self.group = group

    def fwd(self, a, b, out=None):
        return self.cabi.matmul_fwd(a, b, mode=self.mode, out=out)

    def bwd(self, a, b, dc, need_da=True, need_db=True, da=None, db=None):
        return self.cabi.matmul_bwd(a, b, dc, mode=self.mode, need_da=need_da, need_db=need_db, da=da, db=db)

    def set_cta_limit(self, n):
        self.cabi.check(self.cabi.lib().akr_set_gemm_cta_limit(int(n)))

    def allreduce_start(self, x):
        import torch
        import torch.distributed as dist
        t = torch.as_tensor(x, device="cuda")   # zero-copy alias of the library's buffer
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=True), t

    def allreduce_wait(self, handle):
        work, _t = handle
        work.wait()   # orders the collective before later work on the current (default) stream


@dataclass
class BatchShardedMatmul:
    """8192 independent [256x256] products split along batch: rank r owns batches [lo, hi)."""
    total_batch: int
    world: int
    rank: int
    backend: object = None

    def __post_init__(self):
        self.lo, self.hi = shard_range(self.total_batch, self.world, self.rank)
        if self.backend is None:
            self.backend = CudaBackend()

    @property
    def local_batch(self):
        return self.hi - self.lo

    def forward(self, a_local, b_local, out=None):
        return self.backend.fwd(a_local, b_local, out=out)

    def backward(self, a_local, b_local, dc_local, da=None, db=None):
        return self.backend.bwd(a_local, b_local, dc_local, da=da, db=db)


@dataclass
class RowShardedMatmul:
    """C = A @ B with A, C, dC, dA split along M and B replicated; dB summed over ranks."""
    total_m: int
    world: int
    rank: int
    backend: object = None
    overlap: bool = True
    # SMs left free for the collective while it overlaps the dA GEMM (AKR_B200_COMM_CTAS overrides, for tuning)
    comm_ctas: int = int(__import__("os").environ.get("AKR_B200_COMM_CTAS", "20"))

    def __post_init__(self):
        self.lo, self.hi = shard_range(self.total_m, self.world, self.rank)
        if self.backend is None:
            self.backend = CudaBackend()

    @property
    def local_m(self):
        return self.hi - self.lo

    def forward(self, a_local, b, out=None):
        return self.backend.fwd(a_local, b, out=out)

    def backward(self, a_local, b, dc_local, da=None, db=None):
        """Returns (dA_local, dB) where dB is the full weight gradient on every rank."""
        be = self.backend
        if self.world == 1:
            return be.bwd(a_local, b, dc_local, da=da, db=db)
        # 1. partial dB first, 2. start its all-reduce, 3. dA underneath it, 4. join.
        _, db = be.bwd(a_local, b, dc_local, need_da=False, need_db=True, db=db)
        handle = be.allreduce_start(db)
        if self.overlap:
            be.set_cta_limit(max(1, self._sm_count() - self.comm_ctas))
        try:
            da, _ = be.bwd(a_local, b, dc_local, need_da=True, need_db=False, da=da)
        finally:
            if self.overlap:
                be.set_cta_limit(0)
        be.allreduce_wait(handle)
        return da, db

    def _sm_count(self):
        return getattr(self.backend, "sm_count", 148)
