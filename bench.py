#!/usr/bin/env python
"""Benchmark of the fp32 matmul hot path: forward + backward GEMMs at 8192^3 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is C = A @ B, dA = dC . B^T, dB = A^T . dC on fp32 operands of 8192 x 8192 per GPU
(3 * 2 * 8192^3 = 3.30 TFLOP). At N > 1 (launched by torch.distributed.run, one process per GPU) the
product is the row-sharded large GEMM: M = 8192 * N split along M, B replicated, dB all-reduced
over NCCL - weak scaling, at N = 8 exactly the M=65536, N=K=8192 workload.

The JSON line reports: `value` = whole-job TFLOP/s in TF32 mode with inputs resident in HBM;
`e2e` = the same metric through the Python API with pinned HOST buffers (H2D of A, B, dC and D2H of
C, dA, dB inside the timed region); `modes` = the fp32-accurate (3xTF32) mode beside TF32;
`roofline` = the dominant GEMM launch against the measured tensor peak; `cpu_baseline` = the
reference's own CPU path (OpenBLAS build under oracle/_ref) timed on this box's host cores.

`--impl reference` times only that CPU path (the reference has no sm_100 GPU build).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_SQ = 8192
FLOP_PER_STEP = 3 * 2 * N_SQ ** 3           # per GPU
WORKLOAD = "square GEMM fwd+dA+dB, M=N=K=8192 per GPU, fp32 operands N(0, 1/sqrt(K)), seeds 401/402/403"


def set_size(n):
    """--size: a smaller square problem for profiler captures (the benchmark itself is 8192)."""
    global N_SQ, FLOP_PER_STEP, WORKLOAD
    N_SQ = n
    FLOP_PER_STEP = 3 * 2 * n ** 3
    WORKLOAD = WORKLOAD.replace("8192", str(n))

# DRAM bytes moved by one launch of the dominant kernel (forward C = A.B at 8192^3, TF32 mode, 512 x 256 tiles on
# CTA pairs), from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum); see profiles/. None = not captured.
NCU_TRAFFIC_BYTES = 1891505408  # forward launch at 8192^3: 1 654 704 384 read + 236 801 024 written (dA and dB within 0.3 %)



class _StdoutToStderr:
    """Libraries (NCCL prints its version banner) must not write into the one-JSON-line stdout:
    while active, file descriptor 1 points at stderr."""

    def __enter__(self):
        sys.stdout.flush()
        self._saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self._saved, 1)
        os.close(self._saved)
        return False


def _init_ranks(rank, world):
    """Joins the ranks of the node. torch.distributed (gloo, CPU) is only the launcher's plumbing: it carries
    the 128-byte rendezvous id and small host-side sums. The collective of the data path - the dB all-reduce -
    and the barriers / max-over-ranks around the timed regions are the library's own (akr_mg_*: NCCL called
    from C++ behind the C ABI). Returns (dist, comm)."""
    import torch.distributed as dist
    from aakaar_b200.distributed import NodeComm, exchange_via_torch_store
    with _StdoutToStderr():
        dist.init_process_group("gloo")
        comm = NodeComm(rank, world, exchange_via_torch_store)
        comm.barrier()               # forces communicator set-up (and NCCL's banner) now
    return dist, comm

def normal(shape, seed, sigma):
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(sigma))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU in a background thread (NVML, read-only;
    falls back to polling nvidia-smi when the NVML binding is missing)."""
    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
               ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index):
        self.rows = []          # (timestamp, sm_mhz, max_sm_mhz, power_w, reasons bitmask)
        self.gpu_index = gpu_index
        self._stop = threading.Event()
        self.thread = None
        self.source = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self._stop.is_set():
                    try:
                        self.rows.append((time.time(), float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)),
                                          float(mx), pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0, int(get_reasons(h))))
                    except Exception:  # noqa: BLE001
                        pass
                    time.sleep(0.002)
            self.source = "nvml"
        except Exception:  # noqa: BLE001
            fields = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                      "clocks_event_reasons.sw_power_cap,clocks_event_reasons.sw_thermal_slowdown,"
                      "clocks_event_reasons.hw_thermal_slowdown")

            def loop():
                while not self._stop.is_set():
                    try:
                        out = subprocess.run(["nvidia-smi", f"--query-gpu={fields}", "--format=csv,noheader,nounits",
                                              "-i", str(self.gpu_index)], capture_output=True, text=True, timeout=5).stdout
                        r = [x.strip() for x in out.strip().split(",")]
                        mask = sum(bit for (name, bit), v in zip(self.REASONS, r[3:7]) if v.lower().startswith("active"))
                        self.rows.append((time.time(), float(r[0]), float(r[1]), float(r[2]), mask))
                    except Exception:  # noqa: BLE001
                        time.sleep(0.05)
            self.source = "nvidia-smi"
        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=5)

    def summary(self, t0, t1):
        rows = [r for r in self.rows if t0 <= r[0] <= t1]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": self.source}
        mask = 0
        for r in rows:
            mask |= r[4]
        return {"sm_mhz": statistics.median(r[1] for r in rows), "sm_min_mhz": min(r[1] for r in rows),
                "sm_max_mhz": max(r[2] for r in rows), "power_w_max": max(r[3] for r in rows),
                "reasons": sorted(name for name, bit in self.REASONS if mask & bit), "samples": len(rows),
                "source": self.source}


# ---------------------------------------------------------------------------------- reference (CPU) arm

def host_cores():
    """Host cores this process may run on (the affinity mask, not the machine's total)."""
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def load_reference_module():
    """Imports the reference's CPU build with OpenBLAS / OpenMP set to every core this process may use.
    A launcher such as torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; OpenBLAS reads
    that variable when it is loaded, so it is overridden BEFORE the import and set again through
    OpenBLAS's own API afterwards. Returns (module or None, threads OpenBLAS reports)."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not any(f.startswith("_C") and f.endswith(".so") for f in (os.listdir(ref_dir) if os.path.isdir(ref_dir) else [])):
        return None, None
    cores = host_cores()
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "GOTO_NUM_THREADS"):
        os.environ[var] = str(cores)
    sys.path.insert(0, ref_dir)
    import _C as ref  # the reference's own pybind11 module, CPU build
    threads = None
    try:
        import ctypes
        with open(os.path.join(ref_dir, "openblas_path.txt")) as f:
            blas = ctypes.CDLL(f.read().strip())     # already loaded by the import above: same handle
        blas.openblas_set_num_threads(int(cores))
        threads = int(blas.openblas_get_num_threads())
    except Exception:  # noqa: BLE001
        pass
    return ref, threads


def cpu_step(ref, a_np, b_np, dc_np):
    """One fwd+bwd of the reference's CPU path (or of the numpy oracle when the build is absent)."""
    t0 = time.perf_counter()
    if ref is not None:
        a = ref.from_numpy(a_np, "cpu", True)
        b = ref.from_numpy(b_np, "cpu", True)
        c = ref.cpu_matmul(a, b)
        c.backward(ref.from_numpy(dc_np, "cpu", False))
        _ = (a.grad.shape, b.grad.shape)
    else:
        from oracle import matmul_oracle as mo
        mo.matmul_forward(a_np, b_np)
        mo.matmul_backward(a_np, b_np, dc_np)
    return time.perf_counter() - t0


def cpu_inputs(m_rows):
    s = 1.0 / np.sqrt(N_SQ)
    return normal((m_rows, N_SQ), 401, s), normal((N_SQ, N_SQ), 402, s), normal((m_rows, N_SQ), 403, 1.0)


def pick_cpu_rows(ref, target_s):
    """Rows of the 8192-row problem one CPU step covers so that a step costs about `target_s`."""
    a, b, dc = cpu_inputs(128)
    cpu_step(ref, a, b, dc)
    t = cpu_step(ref, a, b, dc)
    rate = 3 * 2 * 128 * N_SQ * N_SQ / max(t, 1e-6)   # flop/s
    rows = int(target_s * rate / (3 * 2 * N_SQ * N_SQ))
    rows = max(128, min(N_SQ, (rows // 128) * 128))
    return rows


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    ref, blas_threads = load_reference_module()
    kind = "reference" if ref is not None else "port"
    cores = blas_threads or host_cores()
    total_steps = args.steps + args.warmup
    rows = pick_cpu_rows(ref, target_s=max(0.5, 150.0 / max(total_steps, 1)))
    a, b, dc = cpu_inputs(rows)
    for _ in range(args.warmup):
        cpu_step(ref, a, b, dc)
    times = [cpu_step(ref, a, b, dc) for _ in range(args.steps)]
    flop = 3 * 2 * rows * N_SQ * N_SQ
    t = sum(times) / len(times)
    val = flop / t / 1e12
    sample = f"{rows} of 8192 rows of A and dC against the full 8192x8192 B (fwd+dA+dB), every step"
    line = {
        "impl": "reference", "metric": "matmul fwd+bwd TFLOP/s at 8192^3", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "device": "host CPU", "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample,
                         "openblas_threads": blas_threads, "host_cores": host_cores()},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def cpu_baseline_child():
    """Bounded CPU sample, run in a child process so that OpenBLAS threads do not linger."""
    ref, blas_threads = load_reference_module()
    rows = pick_cpu_rows(ref, target_s=12.0)
    a, b, dc = cpu_inputs(rows)
    t = cpu_step(ref, a, b, dc)
    flop = 3 * 2 * rows * N_SQ * N_SQ
    print(json.dumps({"value": flop / t / 1e12, "unit": "TFLOP/s", "cores": blas_threads or host_cores(),
                      "openblas_threads": blas_threads, "host_cores": host_cores(),
                      "kind": "reference" if ref is not None else "port",
                      "sample": f"one fwd+dA+dB step on {rows} of 8192 rows of A and dC against the full B ({t:.1f} s)"}))


# ---------------------------------------------------------------------------------- batch-sharded config

def c5a_phase(cabi, lib, dist, rank, world, max_over_ranks, barrier, total=8192, steps=10, warmup=3):
    """8192 independent [256x256]@[256x256] products (fwd + dA + dB) split along the batch over the
    ranks, no collective: the strong-scaling row of the workload list. Returns per mode the whole-job
    time at `world` ranks, the time of the full batch on ONE GPU measured in the same run (rank 0 alone
    while the others wait) and their ratio. Inputs: a seeded 256-batch slab of uniform[-1,1) values
    repeated along the batch (the timing does not depend on the values), dC = ones."""
    import ctypes as C
    from aakaar_b200.distributed import shard_range, BatchShardedMatmul, CudaBackend
    peaks, _ = measured_peaks()
    slab_n = 256

    def filled(nb, seed):
        g = np.random.Generator(np.random.PCG64(seed))
        slab = g.random((slab_n, 256, 256), dtype=np.float32) * np.float32(2.0) - np.float32(1.0)
        dev = cabi.DeviceArray((nb, 256, 256))
        first = min(nb, slab_n)
        cabi.h2d(dev, slab[:first], None, 0)
        done = first
        while done < nb:            # repeat on the device
            n = min(done, nb - done)
            cabi.check(lib.akr_memcpy_d2d(dev.ptr + 4 * done * 65536, dev.ptr, 4 * n * 65536, None))
            done += n
        cabi.synchronize()
        return dev, slab

    def ones(nb):
        dev = cabi.DeviceArray((nb, 256, 256))
        cabi.check(lib.akr_fill(C.cast(dev.ptr, C.POINTER(C.c_float)), 1.0, nb * 65536, None))
        return dev

    def run(nb, sh_world, sh_rank, sync_ranks):
        A, a_slab = filled(nb, 501 + sh_rank)
        B, b_slab = filled(nb, 502 + 1000 * (sh_rank + 1))
        DC = ones(nb)
        Cd, DAd, DBd = (cabi.DeviceArray((nb, 256, 256)) for _ in range(3))
        res = {}
        for name, mode, tol in (("tf32", cabi.MODE_TF32, 2e-3), ("fp32_3xtf32", cabi.MODE_FP32, 1e-5)):
            sh = BatchShardedMatmul(total_batch=nb * sh_world, world=sh_world, rank=sh_rank, backend=CudaBackend(mode=mode))

            def step():
                sh.forward(A, B, out=Cd)
                sh.backward(A, B, DC, da=DAd, db=DBd)
            for _ in range(warmup):
                step()
            if sync_ranks:
                barrier()
            else:
                cabi.synchronize()
            e0, e1 = cabi.Event().record(), cabi.Event()
            for _ in range(steps):
                step()
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_ms(e1) / steps
            if sync_ranks:
                ms = max_over_ranks(ms)
            # one batch entry of each result against float64
            got = np.empty((3, 256, 256), np.float32)
            for j, dev in enumerate((Cd, DAd, DBd)):
                cabi.d2h(got[j], dev, None, (nb - 1) * 65536)
            cabi.synchronize()
            a64, b64 = a_slab[(nb - 1) % slab_n].astype(np.float64), b_slab[(nb - 1) % slab_n].astype(np.float64)
            one = np.ones((256, 256))
            refs = (a64 @ b64, one @ b64.T, a64.T @ one)
            err = max(float(np.linalg.norm(got[j] - r) / np.linalg.norm(r)) for j, r in enumerate(refs))
            if not err < tol:
                raise RuntimeError(f"bench.py: batch-sharded config, mode {name}: parity {err} > {tol}")
            res[name] = {"ms": ms, "rel_frobenius_err": err}
        return res

    lo, hi = shard_range(total, world, rank)
    sharded = run(hi - lo, world, rank, True)
    single = sharded
    if world > 1:
        barrier()
        single = run(total, 1, 0, False) if rank == 0 else None
        barrier()
    if rank != 0:
        return None
    bytes_step = 9 * total * 256 * 256 * 4      # whole job: 3 products x (2 operands + 1 result)
    out = {"workload": f"{total} independent [256x256]@[256x256] fp32 products, fwd + dA + dB, batch split over "
                       f"{world} rank(s), no collective", "scaling": "strong", "bound": "hbm",
           "algorithmic_bytes_per_step": bytes_step, "steps": steps, "warmup": warmup}
    for name in ("tf32", "fp32_3xtf32"):
        ms, ms1 = sharded[name]["ms"], single[name]["ms"]
        out[name] = {"ms": ms, "gbs": bytes_step / ms / 1e6, "frac_of_hbm": bytes_step / ms / 1e6 / (peaks["hbm_gbs"] * world),
                     "ms_1gpu_same_run": ms1, "speedup_vs_1gpu": ms1 / ms,
                     "rel_frobenius_err": sharded[name]["rel_frobenius_err"]}
    return out


# ---------------------------------------------------------------------------------- GPU arm

def run_gpu_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world > 1:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)
    n_gpus = world

    from aakaar_b200 import cabi
    import aakaar_b200 as ak
    from aakaar_b200 import _C
    from aakaar_b200.distributed import RowShardedMatmul, CudaBackend

    lib = cabi.lib()
    if lib.akr_device_count() <= 0:
        raise RuntimeError("bench.py: no CUDA device; the product path has no CPU fallback")
    cabi.check(lib.akr_set_device(local_rank))

    dist, comm = None, None
    if world > 1:
        dist, comm = _init_ranks(rank, world)

    def barrier():
        cabi.synchronize()
        if comm is not None:
            comm.barrier()

    def max_over_ranks(x):
        return x if comm is None else comm.reduce_scalar(x, "max")

    def finish():
        if comm is not None:
            comm.close()
        if dist is not None:
            dist.destroy_process_group()

    # ---- inputs: generated on the host into PINNED buffers (also the source of the e2e copies)
    s = 1.0 / np.sqrt(N_SQ)
    hA, hB, hDC = _C.pinned_empty([N_SQ, N_SQ]), _C.pinned_empty([N_SQ, N_SQ]), _C.pinned_empty([N_SQ, N_SQ])
    hA[...] = normal((N_SQ, N_SQ), 401 + 1000 * rank, s)
    hB[...] = normal((N_SQ, N_SQ), 402, s)
    hDC[...] = normal((N_SQ, N_SQ), 403 + 1000 * rank, 1.0)
    hC, hDA, hDB = _C.pinned_empty([N_SQ, N_SQ]), _C.pinned_empty([N_SQ, N_SQ]), _C.pinned_empty([N_SQ, N_SQ])

    A, B, DC = cabi.DeviceArray.from_numpy(hA), cabi.DeviceArray.from_numpy(hB), cabi.DeviceArray.from_numpy(hDC)
    Cd, DAd, DBd = cabi.DeviceArray((N_SQ, N_SQ)), cabi.DeviceArray((N_SQ, N_SQ)), cabi.DeviceArray((N_SQ, N_SQ))

    results = {}
    gpu_index = local_rank
    try:   # NVML / nvidia-smi count physical GPUs; CUDA_VISIBLE_DEVICES may remap them
        gpu_index = int(os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[local_rank])
    except (ValueError, IndexError):
        pass
    sampler = ClockSampler(gpu_index)
    if rank == 0:
        sampler.start()

    def device_phase(mode, steps, warmup):
        be = CudaBackend(mode=mode, comm=comm)
        sh = RowShardedMatmul(total_m=N_SQ * n_gpus, world=n_gpus, rank=rank, backend=be)
        ev = [[cabi.Event() for _ in range(4)] for _ in range(steps)]

        def step(i=None):
            if i is not None:
                ev[i][0].record()
            sh.forward(A, B, out=Cd)
            if i is not None:
                ev[i][1].record()
            if n_gpus == 1:
                be.bwd(A, B, DC, need_da=True, need_db=False, da=DAd)
                if i is not None:
                    ev[i][2].record()
                be.bwd(A, B, DC, need_da=False, need_db=True, db=DBd)
            else:
                sh.backward(A, B, DC, da=DAd, db=DBd)
                if i is not None:
                    ev[i][2].record()
            if i is not None:
                ev[i][3].record()

        for _ in range(warmup):
            step()
        barrier()
        lib.akr_launch_count(1)
        t_wall0 = time.time()
        e0, e1 = cabi.Event().record(), cabi.Event()
        for i in range(steps):
            step(i)
        e1.record()
        e1.synchronize()
        barrier()
        t_wall1 = time.time()
        launches = int(lib.akr_launch_count(0))
        ms = max_over_ranks(e0.elapsed_ms(e1)) / steps
        per = [[ev[i][j].elapsed_ms(ev[i][j + 1]) for j in range(3)] for i in range(steps)]
        kern_ms = [sum(p[j] for p in per) / steps for j in range(3)]
        return ms, kern_ms, launches, (t_wall0, t_wall1)

    # ---- parity of what the timed phases leave in the output buffers (outside every timed region):
    # sampled rows of C, dA and dB against float64 on the host. dB is the sum over ranks, so every
    # rank contributes A_r[:, rows]^T . dC_r and the references are summed with a small all-reduce.
    def parity_check(tol):
        cabi.synchronize()
        rows = np.array([3, N_SQ // 3 + 1, (2 * N_SQ) // 3 + 5, N_SQ - 1])
        a64 = np.asarray(hA)[rows].astype(np.float64)
        dc64 = np.asarray(hDC)[rows].astype(np.float64)
        b64 = np.asarray(hB).astype(np.float64)
        ref_c, ref_da = a64 @ b64, dc64 @ b64.T
        del b64
        ref_db = np.asarray(hA)[:, rows].astype(np.float64).T @ np.asarray(hDC).astype(np.float64)
        if dist is not None:
            import torch
            t = torch.from_numpy(np.ascontiguousarray(ref_db))
            dist.all_reduce(t)          # float64 on the host (gloo): the reference, not the path under test
            ref_db = t.numpy()
        got = np.empty((3, len(rows), N_SQ), np.float32)
        for j, dev in enumerate((Cd, DAd, DBd)):
            for i, r in enumerate(rows):
                cabi.d2h(got[j, i], dev, None, int(r) * N_SQ)
        cabi.synchronize()
        errs = [float(np.linalg.norm(got[j].astype(np.float64) - ref) / np.linalg.norm(ref))
                for j, ref in enumerate((ref_c, ref_da, ref_db))]
        worst = max_over_ranks(max(errs))
        return {"rel_frobenius": {"C": errs[0], "dA": errs[1], "dB_summed_over_ranks": errs[2]},
                "worst_over_ranks": worst, "tol": tol, "rows": [int(r) for r in rows], "ok": bool(worst < tol)}

    ms_tf32, kern_tf32, launches, wall = device_phase(cabi.MODE_TF32, args.steps, args.warmup)
    parity = {"tf32": parity_check(2e-3)} if not args.profile else {}
    if args.profile:
        # profiler capture: only the TF32 device phase (optionally the fp32-accurate one instead)
        if args.profile == "fp32":
            ms_tf32, kern_tf32, launches, wall = device_phase(cabi.MODE_FP32, args.steps, args.warmup)
        if rank == 0:
            sampler.stop()
            print(json.dumps({"profile_run": True, "size": N_SQ, "ms_per_step": ms_tf32, "kernel_ms": kern_tf32,
                              "gpu_launches": launches}), flush=True)
        finish()
        return 0
    steps32 = max(3, args.steps // 4)
    ms_fp32, kern_fp32, launches32, _ = device_phase(cabi.MODE_FP32, steps32, max(3, args.warmup))
    parity["fp32_3xtf32"] = parity_check(1e-5)
    if not all(p["ok"] for p in parity.values()):
        print(json.dumps({"parity": parity}), file=sys.stderr, flush=True)
        raise RuntimeError("bench.py: the timed path's results disagree with the float64 reference")

    # ---- measured TF32 ceiling: the forward kernel issuing its MMAs back to back with the TMA loads
    # switched off (operands are whatever shared memory holds; the result is not used).
    def mma_only_ms(reps=10):
        cabi.check(lib.akr_debug_configure(1, 0))
        try:
            for _ in range(3):
                cabi.matmul_fwd(A, B, mode=cabi.MODE_TF32, out=Cd)
            cabi.synchronize()
            e0, e1 = cabi.Event().record(), cabi.Event()
            for _ in range(reps):
                cabi.matmul_fwd(A, B, mode=cabi.MODE_TF32, out=Cd)
            e1.record()
            e1.synchronize()
            return e0.elapsed_ms(e1) / reps
        finally:
            cabi.check(lib.akr_debug_configure(0, 0))
    t_m0 = time.time()
    ms_mma_only = mma_only_ms()
    t_m1 = time.time()

    # ---- the SM clock and the cycle count inside the forward kernel under the same sustained load (clock probe of the
    #      library: per-CTA clock64 / %globaltimer): the duration of a power-capped product is cycles / clock, and the
    #      cycles can be set against those its MMAs alone need. Outside every timed region.
    def clock_probe(steps=12):
        cabi.check(lib.akr_debug_configure(32768, 0))
        try:
            for _ in range(steps):
                cabi.matmul_fwd(A, B, mode=cabi.MODE_TF32, out=Cd)
                cabi.matmul_bwd(A, B, DC, mode=cabi.MODE_TF32, need_db=False, da=DAd)
                cabi.matmul_bwd(A, B, DC, mode=cabi.MODE_TF32, need_da=False, db=DBd)
            cabi.matmul_fwd(A, B, mode=cabi.MODE_TF32, out=Cd)
            cabi.synchronize()
            r = cabi.gemm_clock_read(148)
        finally:
            cabi.check(lib.akr_debug_configure(0, 0))
        sms = 148
        mma_cycles = 2.0 * N_SQ * N_SQ * N_SQ / (sms * 4096.0)   # 128 x 256 x 8 per 128 cycles per SM
        return {"kernel": "fwd C=A.B", "sm_mhz": r["sm_mhz"], "sm_mhz_min": r["sm_mhz_min"], "kcycles": r["cycles"] / 1e3,
                "us": r["us"], "mma_kcycles_perfectly_balanced": mma_cycles / 1e3,
                "mma_cycle_share": mma_cycles / r["cycles"],
                "how": "clock64 and %globaltimer of thread 0 of every CTA between set-up and teardown "
                       "(akr_debug_configure(32768) / akr_gemm_clock_read), forward launch after 12 back-to-back steps"}
    in_kernel = clock_probe()

    c5a = c5a_phase(cabi, lib, dist, rank, n_gpus, max_over_ranks, barrier)

    # ---- end to end through the Python API, host buffers in, host buffers out
    def e2e_phase(steps, warmup):
        ak.set_tf32(True)
        sh = RowShardedMatmul(total_m=N_SQ * n_gpus, world=n_gpus, rank=rank,
                              backend=CudaBackend(mode=cabi.MODE_TF32, comm=comm))

        def step():
            a = _C.from_pinned(hA, True)
            b = _C.from_pinned(hB, True)
            dc = _C.from_pinned(hDC, False)
            c = ak.matmul(a, b)
            c.backward(dc)
            if n_gpus > 1:
                comm.allreduce_sum_on(b.grad, None)    # on the compute stream: this path runs one thing at a time
            c.copy_to_host(hC)
            a.grad.copy_to_host(hDA)
            b.grad.copy_to_host(hDB)
            ak.synchronize()

        for _ in range(warmup):
            step()
        barrier()
        e0, e1 = cabi.Event().record(), cabi.Event()
        for _ in range(steps):
            step()
        e1.record()
        e1.synchronize()
        barrier()
        ak.set_tf32(False)
        return max_over_ranks(e0.elapsed_ms(e1)) / steps

    # ---- end to end through the C ABI with three streams: H2D, compute and D2H overlap.
    # Row chunks of A / dC feed the forward and dA GEMMs as they arrive; dB is computed in row
    # panels once dC is complete, each panel's download overlapping the next panel's GEMM.
    def e2e_pipelined_phase(steps, warmup, nch=4):
        s_in, s_c, s_out = cabi.Stream(), cabi.Stream(), cabi.Stream()
        rows = N_SQ // nch
        mode = cabi.MODE_TF32
        # One GPU: two sets of device buffers, so that step i's downloads overlap step i+1's uploads
        # (PCIe is full duplex; within one step the dB download can only start when all uploads are in).
        nsets = 2
        sets = [(A, B, DC, Cd, DAd, DBd), tuple(cabi.DeviceArray((N_SQ, N_SQ)) for _ in range(6))]
        in_free = [None] * nsets    # event: the GEMMs that read this set's inputs have finished
        out_free = [None] * nsets   # event: this set's outputs have been downloaded

        def rowv(x, i):
            return x.as_strided((rows, N_SQ), (N_SQ, 1), offset=i * rows * N_SQ)

        def colv(x, j):
            return x.as_strided((N_SQ, rows), (N_SQ, 1), offset=j * rows)

        def step(k):
            A_, B_, DC_, C_, DA_, DB_ = sets[k % nsets]
            ev = lambda: cabi.Event()   # noqa: E731
            if in_free[k % nsets] is not None:
                s_in.wait_event(in_free[k % nsets])
            if out_free[k % nsets] is not None:
                s_c.wait_event(out_free[k % nsets])
            e_b = ev()
            cabi.h2d(B_, hB, s_in); e_b.record(s_in)
            e_a, e_dc = [], []
            for i in range(nch):
                cabi.h2d(A_, hA[i * rows:(i + 1) * rows], s_in, i * rows * N_SQ)
                e_a.append(ev().record(s_in))
            for i in range(nch):
                cabi.h2d(DC_, hDC[i * rows:(i + 1) * rows], s_in, i * rows * N_SQ)
                e_dc.append(ev().record(s_in))
            s_c.wait_event(e_b)
            for i in range(nch):                                   # forward, chunk by chunk
                s_c.wait_event(e_a[i])
                cabi.matmul_fwd(rowv(A_, i), B_, mode=mode, out=rowv(C_, i), stream=s_c)
                e = ev().record(s_c)
                s_out.wait_event(e)
                cabi.d2h(hC[i * rows:(i + 1) * rows], C_, s_out, i * rows * N_SQ)
            for i in range(nch):                                   # dA, chunk by chunk
                s_c.wait_event(e_dc[i])
                cabi.matmul_bwd(rowv(A_, i), B_, rowv(DC_, i), mode=mode, need_da=True, need_db=False,
                                da=rowv(DA_, i), stream=s_c)
                e = ev().record(s_c)
                s_out.wait_event(e)
                cabi.d2h(hDA[i * rows:(i + 1) * rows], DA_, s_out, i * rows * N_SQ)
            for j in range(nch):                                   # dB in row panels (k range j of A)
                cabi.matmul_bwd(colv(A_, j), rowv(B_, j), DC_, mode=mode, need_da=False, need_db=True,
                                db=rowv(DB_, j), stream=s_c)
                if comm is not None:                               # the panel's sum over ranks, in stream order
                    comm.allreduce_sum_on(rowv(DB_, j), s_c)
                e = ev().record(s_c)
                s_out.wait_event(e)
                cabi.d2h(hDB[j * rows:(j + 1) * rows], DB_, s_out, j * rows * N_SQ)
            in_free[k % nsets] = ev().record(s_c)
            out_free[k % nsets] = ev().record(s_out)
            if prev_done[0] is not None:
                prev_done[0].synchronize()     # at most two steps in flight: bounds the host's run-ahead
            prev_done[0] = out_free[k % nsets]

        prev_done = [None]
        for k in range(warmup):
            step(k)
        cabi.synchronize()
        s_out.synchronize()
        barrier()
        prev_done[0] = None
        t0 = time.perf_counter()
        for k in range(steps):
            step(warmup + k)
        s_out.synchronize()
        cabi.synchronize()
        t1 = time.perf_counter()
        barrier()
        return max_over_ranks((t1 - t0) * 1e3) / steps

    ms_e2e_api = e2e_phase(max(3, min(args.steps, 5)), 3)
    probe_rows = (5, N_SQ // 2 + 4, N_SQ - 1)
    snap = [np.array(h[r]) for h, r in zip((hC, hDA, hDB), probe_rows)]
    for h, r in zip((hC, hDA, hDB), probe_rows):
        h[r] = 0.0
    ms_e2e = e2e_pipelined_phase(max(3, min(args.steps, 10)), 3)
    # the overlapped path must deliver the same results as the sequential one
    e2e_dev = max(float(np.abs(np.array(h[r]) - s0).max() / (np.abs(s0).max() + 1e-30))
                  for h, r, s0 in zip((hC, hDA, hDB), probe_rows, snap))
    if not e2e_dev < 1e-5:
        raise RuntimeError(f"bench.py: overlapped end-to-end path disagrees with the sequential one ({e2e_dev})")
    if rank == 0:
        sampler.stop()

    if rank != 0:
        finish()
        return 0

    clocks = sampler.summary(*wall)
    if clocks["samples"] < 3:   # very short timed region: fall back to every sample of the run
        clocks = sampler.summary(0, float("inf"))
        clocks["note"] = "timed region shorter than the sampling period; samples cover the whole run"
    peaks, peak_src = measured_peaks()
    # Denominator: MEASURED_PEAKS.json holds no TF32 figure; dense TF32 is half of dense bf16. The burst
    # figure applies when the SM clock stayed at its maximum through the timed region, the sustained
    # (power-capped) one otherwise.
    at_max = (clocks.get("sm_mhz") or 0) >= 0.97 * (clocks.get("sm_max_mhz") or 1e9)
    peak_kind = "bf16_tflops" if at_max else "bf16_tflops_sustained"
    tf32_peak = peaks[peak_kind] / 2.0
    value = n_gpus * FLOP_PER_STEP / (ms_tf32 * 1e-3) / 1e12
    names = ["fwd C=A.B (K-major A, N-major B)", "dA=dC.B^T (K-major, K-major)", "dB=A^T.dC (M-major, N-major)"]
    if n_gpus > 1:
        names = names[:1] + ["dB + all-reduce + dA", "-"]
    dom = max(range(3), key=lambda j: kern_tf32[j]) if n_gpus == 1 else 0
    per_launch_flop = 2 * N_SQ ** 3
    achieved = per_launch_flop / (kern_tf32[dom] * 1e-3) / 1e12
    mma_clk = sampler.summary(t_m0, t_m1)
    mma_only_tf = per_launch_flop / (ms_mma_only * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": names[dom], "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                "frac": achieved / tf32_peak,
                "peak_source": f"MEASURED_PEAKS.json {peak_kind}/2 ({peak_src}; "
                               f"{'burst: median SM clock at maximum' if at_max else 'sustained: SM clock below maximum'}"
                               f" in the timed region); nominal dense TF32 1125",
                "frac_of_burst_div2": achieved / (peaks["bf16_tflops"] / 2.0),
                "frac_of_sustained_div2": achieved / (peaks["bf16_tflops_sustained"] / 2.0),
                "frac_of_nominal_1125": achieved / 1125.0,
                "peak_tf32_mma_only": {"tflops": mma_only_tf, "ms_per_launch": ms_mma_only,
                                       "sm_mhz": mma_clk.get("sm_mhz"), "frac": achieved / mma_only_tf,
                                       "how": "the forward kernel of this workload with its TMA loads switched off "
                                              "(tcgen05.mma kind::tf32 issued back to back), CUDA events, 10 launches"},
                "in_kernel": in_kernel,
                "traffic": NCU_TRAFFIC_BYTES, "traffic_over_algorithmic": NCU_TRAFFIC_BYTES / (3 * N_SQ * N_SQ * 4.0),
                "by_kernel": [{"kernel": names[j], "ms": kern_tf32[j],
                               "tflops": per_launch_flop / (kern_tf32[j] * 1e-3) / 1e12 if n_gpus == 1 else None}
                              for j in range(3)]
                + [{"kernel": "fp32-accurate (3xTF32) " + names[j], "ms": kern_fp32[j],
                    "tflops": per_launch_flop / (kern_fp32[j] * 1e-3) / 1e12,
                    "frac_of_peak_div3": per_launch_flop / (kern_fp32[j] * 1e-3) / 1e12 / (tf32_peak / 3.0)}
                   for j in range(3) if n_gpus == 1]}

    cpu = None
    if n_gpus == 1 and not args.no_cpu_baseline:
        try:
            out = subprocess.run([sys.executable, os.path.abspath(__file__), "--_cpu-child"], capture_output=True,
                                 text=True, timeout=600)
            cpu = json.loads(out.stdout.strip().splitlines()[-1])
        except Exception as exc:  # noqa: BLE001
            cpu = {"value": None, "unit": "TFLOP/s", "cores": host_cores(), "kind": "reference",
                   "sample": f"failed: {exc}"}

    bytes_each_way = 3 * N_SQ * N_SQ * 4
    line = {
        "metric": "matmul fwd+bwd TFLOP/s at 8192^3", "value": value, "unit": "TFLOP/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_tf32, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "tf32 products, f32 accumulate (f32 storage)",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "mode": "set_tf32(True)", "l2": "inputs (768 MB) larger than L2 (126 MB)",
                   "sharding": "none" if n_gpus == 1 else f"M = {N_SQ * n_gpus} split along M over {n_gpus} ranks, "
                                                          "B replicated, dB all-reduced (NCCL through akr_mg_allreduce_sum)"},
        "clocks": clocks,
        "e2e": {"value": n_gpus * FLOP_PER_STEP / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": ms_e2e, "h2d_bytes_per_step": bytes_each_way, "d2h_bytes_per_step": bytes_each_way,
                "path": "C ABI, pinned host buffers, copies and GEMMs overlapped on three streams, two device buffer sets so that a step's downloads overlap the next step's uploads (every step uploads its inputs and downloads its results; at N > 1 every dB panel is summed over the ranks before its download)",
                "python_api_sequential": {"ms_per_step": ms_e2e_api,
                                          "value": n_gpus * FLOP_PER_STEP / (ms_e2e_api * 1e-3) / 1e12}},
        "gpu_launches": launches,
        "roofline": roofline,
        "parity": parity,
        "c5a": c5a,
        "cpu_baseline": cpu,
        "modes": {
            "tf32": {"ms_per_step": ms_tf32, "tflops": value, "frac_of_peak": value / n_gpus / tf32_peak,
                     "frac_of_nominal_1125": value / n_gpus / 1125.0},
            "fp32_3xtf32": {"ms_per_step": ms_fp32, "steps": steps32,
                            "tflops": n_gpus * FLOP_PER_STEP / (ms_fp32 * 1e-3) / 1e12,
                            "frac_of_peak_div3": n_gpus * FLOP_PER_STEP / (ms_fp32 * 1e-3) / 1e12 / n_gpus / (tf32_peak / 3),
                            "kernel_ms": kern_fp32, "gpu_launches": launches32},
        },
    }
    print(json.dumps(line), flush=True)
    finish()
    return 0


# ---------------------------------------------------------------------------------- other configurations

def run_config(args):
    """Secondary workloads (parity-test configurations, not the headline line): `c3` the broadcast
    batched product with a transposed-view operand, `c5a` 8192 independent 256^3 products split
    along batch over the ranks, `c2` the Linear-tanh-Linear-MSE-SGD training step."""
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    from aakaar_b200 import cabi
    import aakaar_b200 as ak
    from aakaar_b200.distributed import shard_range
    lib = cabi.lib()
    cabi.check(lib.akr_set_device(local_rank))
    dist, comm = None, None
    if world > 1:
        dist, comm = _init_ranks(rank, world)
    peaks, peak_src = measured_peaks()

    def uniform(shape, seed):
        g = np.random.Generator(np.random.PCG64(seed))
        return (g.random(shape, dtype=np.float32) * np.float32(2.0) - np.float32(1.0))

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        cabi.synchronize()
        if comm is not None:
            comm.barrier()
        lib.akr_launch_count(1)
        e0, e1 = cabi.Event().record(), cabi.Event()
        for _ in range(steps):
            fn()
        e1.record()
        e1.synchronize()
        ms = e0.elapsed_ms(e1) / steps
        launches = int(lib.akr_launch_count(0))
        if comm is not None:
            ms = comm.reduce_scalar(ms, "max")
        return ms, launches

    out = {"config": args.config, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "data": "synthetic"}
    results = {}
    both_modes = [(n, m) for n, m in (("tf32", cabi.MODE_TF32), ("fp32_3xtf32", cabi.MODE_FP32))
                  if args.only_mode in ("", n.split("_")[0])]
    if args.config == "c3":
        base = cabi.DeviceArray.from_numpy(uniform((64, 8, 64, 512), 301))
        B = cabi.DeviceArray.from_numpy(uniform((1, 8, 64, 512), 302))
        A = base.transpose(2, 3)
        DC = cabi.DeviceArray.from_numpy(np.ones((64, 8, 512, 512), np.float32))
        Cd, DAd, DBd = cabi.DeviceArray((64, 8, 512, 512)), cabi.DeviceArray((64, 8, 512, 64)), cabi.DeviceArray((1, 8, 64, 512))
        bytes_step = 1731 * 2 ** 20           # each operand read once, each result written once (fwd + dA + dB)
        flop_step = 3 * 2 * 64 * 8 * 512 * 64 * 512
        for name, mode in both_modes:
            def step(mode=mode):
                cabi.matmul_fwd(A, B, mode=mode, out=Cd)
                cabi.matmul_bwd(A, B, DC, mode=mode, da=DAd, db=DBd)
            ms, launches = timed(step, args.steps, args.warmup)
            parts = {}
            for pname, fn in (() if args.only_mode else
                              (("fwd", lambda m=mode: cabi.matmul_fwd(A, B, mode=m, out=Cd)),
                               ("dA", lambda m=mode: cabi.matmul_bwd(A, B, DC, mode=m, need_db=False, da=DAd)),
                               ("dB", lambda m=mode: cabi.matmul_bwd(A, B, DC, mode=m, need_da=False, db=DBd)))):
                parts[pname] = timed(fn, args.steps, 2)[0]
            results[name] = {"ms_per_step": ms, "gbs": bytes_step / ms / 1e6, "tflops": flop_step / ms / 1e9,
                             "frac_of_hbm": bytes_step / ms / 1e6 / peaks["hbm_gbs"], "gpu_launches_per_step": launches / args.steps,
                             "kernel_ms": parts}
        out.update({"workload": "A [64,8,512,64] (transposed view) @ B [1,8,64,512], dC ones; fwd + dA + dB (dB summed over 64)",
                    "bound": "hbm", "algorithmic_bytes_per_step": bytes_step, "hbm_peak_gbs": peaks["hbm_gbs"],
                    "peak_source": peak_src, "scaling": "n/a"})
    elif args.config == "c5a":
        total = 8192
        lo, hi = shard_range(total, world, rank)
        nb = hi - lo
        g = np.random.Generator(np.random.PCG64(501 + rank))
        A = cabi.DeviceArray.from_numpy(g.random((nb, 256, 256), dtype=np.float32) * 2 - 1)
        B = cabi.DeviceArray.from_numpy(g.random((nb, 256, 256), dtype=np.float32) * 2 - 1)
        DC = cabi.DeviceArray.from_numpy(np.ones((nb, 256, 256), np.float32))
        Cd, DAd, DBd = cabi.DeviceArray((nb, 256, 256)), cabi.DeviceArray((nb, 256, 256)), cabi.DeviceArray((nb, 256, 256))
        bytes_step = 9 * total * 256 * 256 * 4     # whole job: 3 GEMMs x (2 operands + 1 result)
        flop_step = 3 * 2 * total * 256 ** 3
        for name, mode in both_modes:
            def step(mode=mode):
                cabi.matmul_fwd(A, B, mode=mode, out=Cd)
                cabi.matmul_bwd(A, B, DC, mode=mode, da=DAd, db=DBd)
            ms, launches = timed(step, args.steps, args.warmup)
            results[name] = {"ms_per_step": ms, "gbs": bytes_step / ms / 1e6, "tflops": flop_step / ms / 1e9,
                             "frac_of_hbm": bytes_step / ms / 1e6 / (peaks["hbm_gbs"] * world),
                             "gpu_launches_per_step": launches / args.steps}
        out.update({"workload": f"8192 independent [256x256]@[256x256] products, batch split over {world} rank(s), fwd + dA + dB",
                    "bound": "hbm", "algorithmic_bytes_per_step": bytes_step, "hbm_peak_gbs": peaks["hbm_gbs"],
                    "peak_source": peak_src, "scaling": "strong"})
    elif args.config == "conv2d":
        # caller of the path: 3x3 convolution, 64 -> 128 channels, 56 x 56 images, batch 32, as unfold + matmul
        Bn, Ci, Co, Hh, Ww, Kk = 32, 64, 128, 56, 56, 3
        xn = normal((Bn, Ci, Hh, Ww), 601, 1.0)
        wn = uniform((Co, Ci, Kk, Kk), 602) * np.float32(1.0 / np.sqrt(Ci * Kk * Kk))
        dyn = normal((Bn, Co, Hh, Ww), 603, 1.0)
        col_b = Bn * Ci * Kk * Kk * Hh * Ww * 4
        x_b, y_b, w_b = xn.nbytes, dyn.nbytes, wn.nbytes
        # unfold (x -> col), forward (col, W -> y), dW (dy, col -> dW), dcol (W, dy -> dcol), fold (dcol -> dx)
        bytes_step = (x_b + col_b) + (col_b + w_b + y_b) + (y_b + col_b + w_b) + (w_b + y_b + col_b) + (col_b + x_b)
        flop_step = 3 * 2 * Bn * Co * (Ci * Kk * Kk) * (Hh * Ww)
        for name, tf32 in (("tf32", True), ("fp32_3xtf32", False)):
            ak.set_tf32(tf32)
            x = ak.from_numpy(xn, "cuda", requires_grad=True)
            w = ak.from_numpy(wn, "cuda", requires_grad=True)
            dy = ak.from_numpy(dyn, "cuda")

            def step():
                x.zero_grad()
                w.zero_grad()
                ak.conv2d(x, w, padding=(1, 1)).backward(dy)
            ms, launches = timed(step, args.steps, args.warmup)
            results[name] = {"ms_per_step": ms, "gbs": bytes_step / ms / 1e6, "tflops": flop_step / ms / 1e9,
                             "frac_of_hbm": bytes_step / ms / 1e6 / peaks["hbm_gbs"],
                             "gpu_launches_per_step": launches / args.steps}
        ak.set_tf32(False)
        out.update({"workload": "conv2d 3x3 pad 1, x[32,64,56,56], w[128,64,3,3]: unfold + [1,128,576]@[32,576,3136], backward to x and w",
                    "bound": "hbm", "algorithmic_bytes_per_step": bytes_step, "flop_per_step": flop_step,
                    "bytes_note": "with the unfolded matrix materialised, as in the reference's fallback (9x the input)",
                    "hbm_peak_gbs": peaks["hbm_gbs"], "peak_source": peak_src, "scaling": "n/a"})
    else:  # c2
        xn = normal((4096, 1024), 201, 1.0)
        tn = normal((4096, 1024), 202, 1.0)
        flop_step = 5 * 2 * 4096 * 1024 * 4096
        # *_unfused: the tanh node's backward as its own elementwise pass (the reference's graph);
        # default: folded into the epilogue of the second layer's dA product
        for name, tf32, fused in [c for c in (("tf32", True, True), ("fp32_3xtf32", False, True),
                                              ("tf32_unfused", True, False), ("fp32_3xtf32_unfused", False, False))
                                  if not args.only_mode or (c[0] == {"tf32": "tf32", "fp32": "fp32_3xtf32"}[args.only_mode])]:
            ak.set_tf32(tf32)
            ak._C._set_backward_fusion(fused)
            np.random.seed(203)
            l1, l2 = ak.nn.Linear(1024, 4096), ak.nn.Linear(4096, 1024)
            x, t = ak.from_numpy(xn, "cuda"), ak.from_numpy(tn, "cuda")
            opt = ak.optim.SGD(l1.parameters() + l2.parameters(), lr=0.01)

            def step():
                opt.zero_grad()
                loss = ak.mse_loss(l2(l1(x).tanh()), t)
                loss.backward()
                opt.step()
            ms, launches = timed(step, args.steps, args.warmup)
            results[name] = {"ms_per_step": ms, "tflops": flop_step / ms / 1e9, "gpu_launches_per_step": launches / args.steps}
        ak._C._set_backward_fusion(True)
        ak.set_tf32(False)
        out.update({"workload": "MLP step: x[4096,1024] -> Linear 1024->4096 -> tanh -> Linear 4096->1024 -> MSE, backward, SGD",
                    "bound": "tensor", "flop_per_step": flop_step, "flop_note": "5 needed GEMMs (the reference runs 6)",
                    "scaling": "n/a"})
    out["results"] = results
    if rank == 0:
        print(json.dumps(out), flush=True)
    if comm is not None:
        comm.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", default="sq8192", choices=["sq8192", "c2", "c3", "c5a", "conv2d"],
                    help="sq8192 = the benchmark; c2 / c3 / c5a / conv2d = secondary configurations (own JSON format)")
    ap.add_argument("--size", type=int, default=8192, help="square size (profiling only; the benchmark is 8192)")
    ap.add_argument("--profile", default="", choices=["", "tf32", "fp32"],
                    help="profiler capture run: one device phase only, warm-up not forced to 3")
    ap.add_argument("--only-mode", default="", choices=["", "tf32", "fp32"],
                    help="secondary configurations: run one arithmetic mode only (profiler captures)")
    ap.add_argument("--_cpu-child", dest="cpu_child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if not args.profile:
        args.warmup = max(args.warmup, 3)
    if args.size != 8192:
        set_size(args.size)
    if args.cpu_child:
        cpu_baseline_child()
        return 0
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.config != "sq8192":
        return run_config(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
