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
logic is testable on CPU ranks (gloo); the default backend is the CUDA library through its C ABI,
with the collective issued by the library itself (`NodeComm` over akr_mg_*).
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


def _ptr_count(x):
    """(device pointer, element count) of a float32 device array: a cabi.DeviceArray or anything that
    exports __cuda_array_interface__ (the pybind Tensor does). Must be contiguous."""
    if hasattr(x, "ptr") and hasattr(x, "size"):
        return int(x.ptr), int(x.size)
    cai = x.__cuda_array_interface__
    n = 1
    for d in cai["shape"]:
        n *= int(d)
    return int(cai["data"][0]), n


class NodeComm:
    """The ranks of one node joined through the library's own collective entry points (akr_mg_*: NCCL
    called from C++ behind the C ABI - no torch on this path).

    `exchange` carries the 128-byte rendezvous id from rank 0 to the others: a callable that takes the
    id (bytes) on rank 0 and None elsewhere and returns the id on every rank. Under a launcher that
    provides a key-value store or a CPU process group this is a one-line broadcast
    (see `exchange_via_torch_store`); a file or a socket works as well.
    """

    def __init__(self, rank, world, exchange):
        import ctypes as C
        from . import cabi
        self.cabi, self.rank, self.world = cabi, int(rank), int(world)
        lib = cabi.lib()
        buf = C.create_string_buffer(cabi.MG_UNIQUE_ID_BYTES)
        uid = None
        if self.rank == 0:
            cabi.check(lib.akr_mg_get_unique_id(buf))
            uid = bytes(buf.raw)
        uid = exchange(uid)
        if not isinstance(uid, (bytes, bytearray)) or len(uid) != cabi.MG_UNIQUE_ID_BYTES:
            raise ValueError("NodeComm: the exchange must return the 128-byte id on every rank")
        cabi.check(lib.akr_mg_init(self.rank, self.world, C.c_char_p(bytes(uid))))
        self.stream = cabi.Stream()   # collectives run here, beside the compute stream
        self._scratch = None

    def allreduce_sum_async(self, x, after=None):
        """In-place float32 sum of the device array `x` over all ranks on the communication stream, ordered
        after everything enqueued so far on the compute stream `after` (None = the legacy default stream).
        Returns the event to wait for."""
        cabi = self.cabi
        import ctypes as C
        ready = cabi.Event().record(after)
        self.stream.wait_event(ready)
        ptr, n = _ptr_count(x)
        cabi.check(cabi.lib().akr_mg_allreduce_sum(C.cast(ptr, C.POINTER(C.c_float)), n, self.stream.h))
        return cabi.Event().record(self.stream)

    def allreduce_sum_on(self, x, stream):
        """The same collective enqueued directly on `stream` (no overlap; for pipelines that order it themselves)."""
        import ctypes as C
        ptr, n = _ptr_count(x)
        self.cabi.check(self.cabi.lib().akr_mg_allreduce_sum(C.cast(ptr, C.POINTER(C.c_float)), n,
                                                             stream.h if stream is not None else None))

    def reduce_scalar(self, value, op="max"):
        """One double reduced over all ranks through the device (timings: the maximum over ranks)."""
        import ctypes as C
        import numpy as np
        cabi = self.cabi
        if self._scratch is None:
            self._scratch = cabi.DeviceArray((2,))      # 8 bytes: one float64
        host = np.array([value], dtype=np.float64)
        cabi.check(cabi.lib().akr_memcpy_h2d(self._scratch.ptr, host.ctypes.data, 8, None))
        cabi.check(cabi.lib().akr_mg_allreduce(self._scratch.ptr, 1, cabi.DTYPE_F64,
                                               cabi.MG_MAX if op == "max" else cabi.MG_SUM, None))
        cabi.check(cabi.lib().akr_memcpy_d2h(host.ctypes.data, self._scratch.ptr, 8, None))
        cabi.synchronize()
        return float(host[0])

    def barrier(self):
        self.cabi.synchronize()
        self.reduce_scalar(0.0, "sum")

    def close(self):
        self.cabi.check(self.cabi.lib().akr_mg_finalize())


def exchange_via_torch_store(uid):
    """Rendezvous-id broadcast over an initialised torch.distributed group (any backend, gloo included).
    torch is the launcher's plumbing here, not part of the compute or collective path."""
    import torch.distributed as dist
    box = [uid]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class CudaBackend:
    """Local products on this rank's GPU through the C ABI; the dB reduction through a NodeComm."""

    def __init__(self, mode=-1, comm=None):
        from . import cabi
        self.cabi = cabi
        self.mode = mode
        self.comm = comm

    def fwd(self, a, b, out=None):
        return self.cabi.matmul_fwd(a, b, mode=self.mode, out=out)

    def bwd(self, a, b, dc, need_da=True, need_db=True, da=None, db=None):
        return self.cabi.matmul_bwd(a, b, dc, mode=self.mode, need_da=need_da, need_db=need_db, da=da, db=db)

    def set_cta_limit(self, n):
        self.cabi.check(self.cabi.lib().akr_set_gemm_cta_limit(int(n)))

    def allreduce_start(self, x):
        if self.comm is None:
            raise RuntimeError("CudaBackend: a NodeComm is needed to sum a gradient over ranks")
        return self.comm.allreduce_sum_async(x)

    def allreduce_wait(self, handle):
        self.cabi.stream_wait_event(None, handle)   # later work on the compute stream sees the summed gradient


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
    # SMs left free for the collective while it overlaps the dA GEMM: 128 CTAs run the 1024 tiles of an
    # 8192 x 8192 output in exactly 8 rounds (any count from 129 to 146 needs 8 rounds as well)
    comm_ctas: int = 20

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
