"""ctypes binding of the C ABI (``include/akr_b200.h``) - the same entry points the pybind11
module calls, reachable without it. Used by the parity tests and the benchmark to drive the
library exactly as a foreign-language host would: raw device pointers, shapes and strides.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libakr_b200.so")

AKR_MAX_DIMS = 8
MODE_GLOBAL, MODE_FP32, MODE_TF32 = -1, 0, 1
OK, ERR_INVALID, ERR_RUNTIME, ERR_CUDA, ERR_NOGPU, ERR_ABORTED = 0, -1, -2, -3, -4, -5


class View(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("ndim", C.c_int32),
        ("dtype", C.c_int32),
        ("shape", C.c_int64 * AKR_MAX_DIMS),
        ("stride", C.c_int64 * AKR_MAX_DIMS),
    ]


class AkrError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[akr {code}] {msg}")
        self.code = code
        self.msg = msg


def load():
    if not os.path.exists(_LIB_PATH):
        raise ImportError(f"{_LIB_PATH} is not built: run `python -m aakaar_b200._build`")
    lib = C.CDLL(_LIB_PATH)
    lib.akr_last_error.restype = C.c_char_p
    lib.akr_launch_count.restype = C.c_int64
    vp, sz, fp = C.c_void_p, C.c_size_t, C.POINTER(C.c_float)
    V = C.POINTER(View)
    sigs = {
        "akr_alloc": [sz, C.POINTER(fp)],
        "akr_free": [fp, sz],
        "akr_host_alloc": [sz, C.POINTER(vp)],
        "akr_host_free": [vp],
        "akr_memcpy_h2d": [vp, vp, sz, vp],
        "akr_memcpy_d2h": [vp, vp, sz, vp],
        "akr_memcpy_d2d": [vp, vp, sz, vp],
        "akr_memset_zero": [vp, sz, vp],
        "akr_stream_synchronize": [vp],
        "akr_matmul_plan": [V, V, C.POINTER(C.c_int64), C.POINTER(C.c_int32)],
        "akr_matmul_fwd": [V, V, V, V, C.c_int, vp],
        "akr_matmul_bwd": [V, V, V, V, V, C.c_int, vp],
        "akr_matmul_a_bt": [V, V, V, C.c_int, vp],
        "akr_matmul_at_b": [V, V, V, C.c_int, vp],
        "akr_matmul_fwd_simt": [V, V, V, vp],
        "akr_matmul_fwd_typed": [V, V, V, vp],
        "akr_matmul_bwd_tanh": [V, V, V, V, V, C.c_int, vp],
        "akr_matmul_bwd_colsum": [V, V, V, V, V, fp, C.c_int, C.c_int, vp],
        "akr_mse_fwd_grad_colsum": [fp, fp, fp, fp, fp, C.c_int64, C.c_int64, vp],
        "akr_mse_fwd_grad": [fp, fp, fp, fp, sz, vp],
        "akr_matmul_fwd_axpby": [V, V, C.c_float, C.c_float, V, V, C.c_int, vp],
        "akr_matmul_at_b_noalloc": [V, V, V, vp],
        "akr_workspace_bytes": [C.POINTER(sz)],
        "akr_launch_count": [C.c_int],
        "akr_allocator_stats": [C.POINTER(C.c_int64), C.POINTER(C.c_int64)],
        "akr_contiguous": [V, fp, vp],
        "akr_add": [V, V, V, vp],
        "akr_sum_to": [V, V, vp],
        "akr_scale": [fp, C.c_float, fp, sz, vp],
        "akr_fill": [fp, C.c_float, sz, vp],
        "akr_tanh_fwd": [fp, fp, sz, vp],
        "akr_tanh_bwd": [fp, fp, fp, sz, vp],
        "akr_mse_fwd": [fp, fp, fp, sz, vp],
        "akr_mse_bwd": [fp, fp, fp, fp, sz, vp],
        "akr_sgd_step": [fp, fp, fp, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, sz, vp],
        "akr_sgd_step_multi": [C.c_int, C.POINTER(fp), C.POINTER(fp), C.POINTER(fp), C.POINTER(sz), C.POINTER(C.c_int),
                               C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int, vp],
        "akr_scatter": [fp, V, vp],
        "akr_im2col_3d": [fp, fp, vp, vp],
        "akr_col2im_3d": [fp, fp, vp, vp],
        "akr_set_tf32": [C.c_int],
        "akr_set_cudnn_tf32": [C.c_int],
        "akr_set_device": [C.c_int],
        "akr_set_gemm_cta_limit": [C.c_int],
        "akr_debug_configure": [C.c_int, C.c_uint],
        "akr_gemm_clock_read": [C.c_int] + [C.POINTER(C.c_double)] * 4,
        "akr_stream_create": [C.POINTER(vp)],
        "akr_stream_destroy": [vp],
        "akr_stream_wait_event": [vp, vp],
        "akr_event_create": [C.POINTER(vp)],
        "akr_event_record": [vp, vp],
        "akr_event_synchronize": [vp],
        "akr_event_elapsed_ms": [vp, vp, C.POINTER(C.c_float)],
        "akr_event_destroy": [vp],
        "akr_mg_get_unique_id": [vp],
        "akr_mg_init": [C.c_int, C.c_int, vp],
        "akr_mg_allreduce": [vp, sz, C.c_int, C.c_int, vp],
        "akr_mg_allreduce_sum": [fp, sz, vp],
        "akr_mg_world": [C.POINTER(C.c_int), C.POINTER(C.c_int)],
        "akr_mg_nccl_version": [C.POINTER(C.c_int)],
        "akr_mg_finalize": [],
    }
    for name, args in sigs.items():
        getattr(lib, name).argtypes = args
    lib.akr_set_tf32.restype = None
    lib.akr_set_cudnn_tf32.restype = None
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def check(rc):
    if rc != OK:
        raise AkrError(rc, lib().akr_last_error().decode())


class DeviceArray:
    """A device buffer from the library's caching allocator plus view metadata (element strides)."""

    def __init__(self, shape, strides=None, ptr=None, offset=0, base=None):
        self.shape = tuple(int(s) for s in shape)
        n = int(np.prod(self.shape)) if self.shape else 1
        if ptr is None:
            p = C.POINTER(C.c_float)()
            check(lib().akr_alloc(n, C.byref(p)))
            self._owned = (p, n)
            self.ptr = C.cast(p, C.c_void_p).value
        else:
            self._owned = None
            self.ptr = ptr + 4 * offset
        self.base = base
        if strides is None:
            strides, acc = [], 1
            for d in reversed(self.shape):
                strides.append(acc)
                acc *= d
            strides = tuple(reversed(strides))
        self.strides = tuple(int(s) for s in strides)
        self.size = n

    def __del__(self):
        if getattr(self, "_owned", None) is not None and _lib is not None:
            p, n = self._owned
            _lib.akr_free(p, n)
            self._owned = None

    @classmethod
    def from_numpy(cls, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        d = cls(arr.shape)
        check(lib().akr_memcpy_h2d(d.ptr, arr.ctypes.data, arr.nbytes, None))
        check(lib().akr_stream_synchronize(None))
        return d

    @property
    def __cuda_array_interface__(self):
        """Zero-copy export (e.g. ``torch.as_tensor(x, device="cuda")`` for a NCCL collective)."""
        return {"shape": self.shape, "typestr": "<f4", "data": (self.ptr, False), "version": 3,
                "strides": tuple(4 * s for s in self.strides)}

    def view(self):
        v = View()
        v.data = self.ptr
        v.ndim = len(self.shape)
        v.dtype = 0
        for i in range(AKR_MAX_DIMS):
            v.shape[i] = self.shape[i] if i < len(self.shape) else 1
            v.stride[i] = self.strides[i] if i < len(self.shape) else 0
        return v

    def transpose(self, d0, d1):
        sh, st = list(self.shape), list(self.strides)
        sh[d0], sh[d1] = sh[d1], sh[d0]
        st[d0], st[d1] = st[d1], st[d0]
        return DeviceArray(sh, st, ptr=self.ptr, base=self)

    def as_strided(self, shape, strides, offset=0):
        return DeviceArray(shape, strides, ptr=self.ptr, offset=offset, base=self)

    def to_numpy(self):
        """Downloads the underlying elements of a CONTIGUOUS array."""
        assert self._is_contiguous(), "to_numpy needs a contiguous array"
        out = np.empty(self.shape, dtype=np.float32)
        check(lib().akr_memcpy_d2h(out.ctypes.data, self.ptr, out.nbytes, None))
        check(lib().akr_synchronize())
        return out

    def _is_contiguous(self):
        acc = 1
        for d, s in zip(reversed(self.shape), reversed(self.strides)):
            if d != 1 and s != acc:
                return False
            acc *= d
        return True


class Stream:
    """A non-blocking CUDA stream owned by the library."""

    def __init__(self):
        self.h = C.c_void_p()
        check(lib().akr_stream_create(C.byref(self.h)))

    def wait_event(self, ev: "Event"):
        check(lib().akr_stream_wait_event(self.h, ev.h))

    def synchronize(self):
        check(lib().akr_stream_synchronize(self.h))

    def __del__(self):
        if _lib is not None and self.h:
            _lib.akr_stream_destroy(self.h)
            self.h = None


class Event:
    """CUDA event on the library's stream (NULL = legacy default stream)."""

    def __init__(self):
        self.h = C.c_void_p()
        check(lib().akr_event_create(C.byref(self.h)))

    def record(self, stream=None):
        check(lib().akr_event_record(self.h, stream.h if stream is not None else None))
        return self

    def synchronize(self):
        check(lib().akr_event_synchronize(self.h))

    def elapsed_ms(self, end: "Event") -> float:
        ms = C.c_float()
        check(lib().akr_event_elapsed_ms(self.h, end.h, C.byref(ms)))
        return float(ms.value)

    def __del__(self):
        if _lib is not None and self.h:
            _lib.akr_event_destroy(self.h)
            self.h = None


MG_UNIQUE_ID_BYTES = 128
MG_SUM, MG_MAX = 0, 1
DTYPE_F32, DTYPE_F64 = 0, 1


def stream_wait_event(stream, ev: "Event"):
    """Makes `stream` (a Stream, or None for the legacy default stream) wait for `ev`."""
    check(lib().akr_stream_wait_event(_sh(stream), ev.h))


def plan(a: DeviceArray, b: DeviceArray):
    shape = (C.c_int64 * (AKR_MAX_DIMS + 2))()
    nd = C.c_int32(0)
    va, vb = a.view(), b.view()
    check(lib().akr_matmul_plan(C.byref(va), C.byref(vb), shape, C.byref(nd)))
    return tuple(shape[i] for i in range(nd.value))


def _sh(stream):
    return stream.h if stream is not None else None


def matmul_fwd(a, b, bias=None, mode=MODE_GLOBAL, out=None, stream=None):
    c = out if out is not None else DeviceArray(plan(a, b))
    va, vb, vc = a.view(), b.view(), c.view()
    vbias = bias.view() if bias is not None else None
    check(lib().akr_matmul_fwd(C.byref(va), C.byref(vb), C.byref(vbias) if bias is not None else None,
                               C.byref(vc), mode, _sh(stream)))
    return c


def matmul_bwd(a, b, dc, mode=MODE_GLOBAL, need_da=True, need_db=True, da=None, db=None, stream=None):
    if need_da and da is None:
        da = DeviceArray(a.shape)
    if need_db and db is None:
        db = DeviceArray(b.shape)
    va, vb, vg = a.view(), b.view(), dc.view()
    vda = da.view() if need_da else None
    vdb = db.view() if need_db else None
    check(lib().akr_matmul_bwd(C.byref(va), C.byref(vb), C.byref(vg),
                               C.byref(vda) if need_da else None, C.byref(vdb) if need_db else None,
                               mode, _sh(stream)))
    return (da if need_da else None), (db if need_db else None)


def matmul_bwd_tanh(a_tanh, b, dc, mode=MODE_GLOBAL, need_dz=True, need_db=True, stream=None):
    """(dZ, dB) for C = tanh(Z) @ B given A = tanh(Z): dZ = (dC B^T) * (1 - A^2) in the GEMM epilogue."""
    dz = DeviceArray(a_tanh.shape) if need_dz else None
    db = DeviceArray(b.shape) if need_db else None
    va, vb, vg = a_tanh.view(), b.view(), dc.view()
    vdz = dz.view() if need_dz else None
    vdb = db.view() if need_db else None
    check(lib().akr_matmul_bwd_tanh(C.byref(va), C.byref(vb), C.byref(vg), C.byref(vdz) if need_dz else None,
                                    C.byref(vdb) if need_db else None, mode, _sh(stream)))
    return dz, db


def fptr(x: DeviceArray):
    """The array's base pointer typed as float* for the entry points that take raw pointers."""
    return C.cast(x.ptr, C.POINTER(C.c_float))


def matmul_bwd_colsum(a, b, dc, a_is_tanh=False, mode=MODE_GLOBAL, need_db=True, stream=None):
    """(dA or dZ, dB, column sums of the first): the backward of C = A @ B that hands the bias gradient of the
    Linear layer behind A along (``akr_matmul_bwd_colsum``)."""
    da = DeviceArray(a.shape)
    db = DeviceArray(b.shape) if need_db else None
    cs = DeviceArray((a.shape[-1],))
    va, vb, vg, vda = a.view(), b.view(), dc.view(), da.view()
    vdb = db.view() if need_db else None
    check(lib().akr_matmul_bwd_colsum(C.byref(va), C.byref(vb), C.byref(vg), C.byref(vda),
                                      C.byref(vdb) if need_db else None, fptr(cs), 1 if a_is_tanh else 0, mode,
                                      _sh(stream)))
    return da, db, cs


def matmul_axpby(a, b, alpha=1.0, beta=0.0, d=None, mode=MODE_GLOBAL, out=None, stream=None):
    """alpha * (a @ b) + beta * d in one launch."""
    c = out if out is not None else DeviceArray(plan(a, b))
    va, vb, vc = a.view(), b.view(), c.view()
    vd = d.view() if d is not None else None
    check(lib().akr_matmul_fwd_axpby(C.byref(va), C.byref(vb), alpha, beta, C.byref(vd) if d is not None else None,
                                     C.byref(vc), mode, _sh(stream)))
    return c


def matmul_simt(a, b):
    c = DeviceArray(plan(a, b))
    va, vb, vc = a.view(), b.view(), c.view()
    check(lib().akr_matmul_fwd_simt(C.byref(va), C.byref(vb), C.byref(vc), None))
    return c


_TYPED = {"float32": 0, "float64": 1, "int32": 2, "int64": 3}


def matmul_typed(a_np, b_np):
    """Forward-only product of two host arrays of one dtype (float32/float64/int32/int64) through
    ``akr_matmul_fwd_typed``; the arrays may be strided views (their base storage is uploaded as is)."""
    a_np, b_np = np.asarray(a_np), np.asarray(b_np)
    code = _TYPED[a_np.dtype.name]
    item = a_np.dtype.itemsize

    def upload(x):
        # the byte range the view touches is uploaded as it lies; the view keeps its own strides
        lo = sum(min(0, (d - 1) * st) for d, st in zip(x.shape, x.strides))
        hi = sum(max(0, (d - 1) * st) for d, st in zip(x.shape, x.strides)) + x.dtype.itemsize
        dev = DeviceArray(((hi - lo + 3) // 4,))
        check(lib().akr_memcpy_h2d(dev.ptr, x.ctypes.data + lo, hi - lo, None))
        v = View()
        v.data = dev.ptr - lo
        v.ndim, v.dtype = x.ndim, _TYPED[x.dtype.name]
        for i in range(AKR_MAX_DIMS):
            v.shape[i] = x.shape[i] if i < x.ndim else 1
            v.stride[i] = x.strides[i] // x.dtype.itemsize if i < x.ndim else 0
        return dev, v

    da, va = upload(a_np)
    db, vb = upload(b_np)
    shape = (C.c_int64 * (AKR_MAX_DIMS + 2))()
    nd = C.c_int32(0)
    check(lib().akr_matmul_plan(C.byref(va), C.byref(vb), shape, C.byref(nd)))
    out = np.empty(tuple(shape[i] for i in range(nd.value)), dtype=a_np.dtype)
    dc = DeviceArray(((max(out.nbytes, 4) + 3) // 4,))
    vc = View()
    vc.data, vc.ndim, vc.dtype = dc.ptr, out.ndim, code
    for i in range(AKR_MAX_DIMS):
        vc.shape[i] = out.shape[i] if i < out.ndim else 1
        vc.stride[i] = out.strides[i] // item if i < out.ndim else 0
    check(lib().akr_matmul_fwd_typed(C.byref(va), C.byref(vb), C.byref(vc), None))
    check(lib().akr_memcpy_d2h(out.ctypes.data, dc.ptr, out.nbytes, None))
    check(lib().akr_synchronize())
    return out


def h2d(dst: DeviceArray, src_np, stream=None, dst_offset_elems=0):
    """Asynchronous copy of a C-contiguous float32 numpy array (ideally page-locked) into `dst`."""
    check(lib().akr_memcpy_h2d(dst.ptr + 4 * dst_offset_elems, src_np.ctypes.data, src_np.nbytes, _sh(stream)))


def d2h(dst_np, src: DeviceArray, stream=None, src_offset_elems=0):
    check(lib().akr_memcpy_d2h(dst_np.ctypes.data, src.ptr + 4 * src_offset_elems, dst_np.nbytes, _sh(stream)))


def gemm_clock_read(ctas=148):
    """What the clock probe (akr_debug_configure(32768, 0)) recorded for the last GEMM launch: a dict with the SM
    clock in MHz (mean, min over the CTAs), the longest CTA in cycles and in microseconds. Synchronize first."""
    a, b, c, d = C.c_double(), C.c_double(), C.c_double(), C.c_double()
    check(lib().akr_gemm_clock_read(ctas, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
    return {"sm_mhz": a.value, "sm_mhz_min": b.value, "cycles": c.value, "us": d.value}


def synchronize():
    check(lib().akr_synchronize())
