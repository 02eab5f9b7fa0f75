/*
 * akr_b200.h - C ABI of the B200 (sm_100a) fp32 matmul path.
 *
 * This is the drop-in boundary for the matmul hot path of the Aakaar tensor library: plain
 * pointers and sizes, no C++ types, no PyTorch types. A maintainer of the reference binds these
 * entry points from src/bindings.cpp in place of the functions of src/matmul_kernel.cu; the
 * reference function each entry point stands in for is cited beside it (paths relative to the
 * reference checkout).
 *
 * Conventions
 *   - Every function returns AKR_OK (0) or a negative status; nothing throws across this boundary.
 *     akr_last_error() returns the message of the last failing call on the calling thread.
 *     AKR_ERR_INVALID corresponds to the reference's std::invalid_argument (Python ValueError),
 *     AKR_ERR_RUNTIME / AKR_ERR_CUDA to std::runtime_error (Python RuntimeError).
 *   - Tensors are described by akr_view: base pointer of the view, up to 8 dims, shape and
 *     strides in ELEMENTS (the reference's Tensor::shape / Tensor::strides, src/tensor.h:46-50).
 *     Views may be transposed, sliced or broadcast; operands are never required to be contiguous.
 *   - All device pointers belong to the current CUDA device of the calling thread.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, which is what
 *     the reference uses). Work is asynchronous to the host, as in the reference. Calls that need
 *     scratch memory share one per-device workspace, ordered by the stream: issue the calls of one
 *     device on one stream, or serialise streams yourself.
 *   - There is no CPU fallback: without a usable GPU every compute entry point fails with
 *     AKR_ERR_NOGPU.
 */
#ifndef AKR_B200_H
#define AKR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AKR_MAX_DIMS 8

/* Exported entry points keep default visibility; everything else in the library is hidden. */
#if defined(__GNUC__)
#define AKR_API __attribute__((visibility("default")))
#else
#define AKR_API
#endif

enum {
    AKR_OK = 0,
    AKR_ERR_INVALID = -1, /* bad shape / argument: the reference's std::invalid_argument */
    AKR_ERR_RUNTIME = -2, /* the reference's std::runtime_error */
    AKR_ERR_CUDA = -3,    /* a CUDA runtime / driver call failed */
    AKR_ERR_NOGPU = -4,   /* no CUDA device: this library has no CPU path */
    AKR_ERR_ABORTED = -5  /* a kernel gave up on a bounded wait (device status word set) */
};

/* src/dtype.h: FLOAT32, FLOAT64, INT32, INT64. Everything is float32 except akr_matmul_fwd_typed. */
enum { AKR_DTYPE_F32 = 0, AKR_DTYPE_F64 = 1, AKR_DTYPE_I32 = 2, AKR_DTYPE_I64 = 3 };

/* Arithmetic mode of one call. AKR_MODE_GLOBAL follows akr_set_tf32(). */
enum {
    AKR_MODE_GLOBAL = -1,
    AKR_MODE_FP32 = 0, /* 3xTF32 split products: fp32-level accuracy (set_tf32(False)) */
    AKR_MODE_TF32 = 1  /* single TF32 products (set_tf32(True)) */
};

typedef struct akr_view {
    void* data;    /* first element of the view (device memory) */
    int32_t ndim;  /* 0..AKR_MAX_DIMS */
    int32_t dtype; /* AKR_DTYPE_F32 */
    int64_t shape[AKR_MAX_DIMS];
    int64_t stride[AKR_MAX_DIMS]; /* in elements; may be 0 (broadcast) */
} akr_view;

/* ------------------------------------------------------------------ errors / info */
AKR_API const char* akr_last_error(void);
AKR_API int akr_version(void);
/* Number of visible CUDA devices (0 without a driver); never fails. Cf. _C.device_count. */
AKR_API int akr_device_count(void);
AKR_API int akr_set_device(int ordinal);

/* ------------------------------------------------------------------ global switches
 * set_tf32_enabled / get_tf32_enabled, src/matmul_kernel.cu:20-37 (default off = fp32-accurate).
 * The cuDNN flag lives in the same reference file (:24-27) and is read by the conv sources; it is
 * kept so that a replaced matmul_kernel.cu still exports it, and does nothing here. */
AKR_API void akr_set_tf32(int enabled);
AKR_API int akr_get_tf32(void);
AKR_API void akr_set_cudnn_tf32(int enabled);
AKR_API int akr_get_cudnn_tf32(void);
/* cuda_synchronize, src/matmul_kernel.cu:39-41. Also reports a kernel that aborted. */
AKR_API int akr_synchronize(void);

/* ------------------------------------------------------------------ memory
 * CachingAllocator, src/allocator.h:12-60: exact-size free lists keyed by element count, blocks
 * are returned to the driver only by akr_empty_cache(); hit / miss counters as _allocator_stats. */
AKR_API int akr_alloc(size_t nfloats, float** out);
AKR_API int akr_free(float* ptr, size_t nfloats);
AKR_API int akr_empty_cache(void);
AKR_API int akr_allocator_stats(int64_t* hits, int64_t* misses);
/* Pinned host staging (src/pinned_allocator.h) and copies (Tensor::to_device, src/tensor.h:418-465;
 * from_numpy, src/bindings.cpp:2399-2469; to_numpy, src/tensor.h:473-517). */
AKR_API int akr_host_alloc(size_t bytes, void** out);
AKR_API int akr_host_free(void* ptr);
AKR_API int akr_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
AKR_API int akr_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
AKR_API int akr_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
AKR_API int akr_memset_zero(void* dst, size_t bytes, void* stream);
AKR_API int akr_stream_synchronize(void* stream);

/* ------------------------------------------------------------------ matmul
 * Shape planning of plan_nd_matmul, src/matmul_kernel.cu:55-83: right-aligned broadcast of the
 * batch dims, inner-dimension check. Writes the result shape (batch dims + [M, N]).
 * Pure host code: works without a GPU. */
AKR_API int akr_matmul_plan(const akr_view* a, const akr_view* b, int64_t* out_shape, int32_t* out_ndim);

/* Forward: run_cublas_matmul, src/matmul_kernel.cu:111-143, for every broadcast batch index in ONE
 * launch, reading strided views in place. `c` must have the planned shape (any strides with a
 * unit-stride last dim). `bias` (optional, N values, shape [N] or [1, N]) is added to every row in
 * the epilogue: the `+ bias` of nn.Linear (aakaar/nn.py:14-15, broadcast add of
 * src/elementwise_kernel.cu:46-65). */
AKR_API int akr_matmul_fwd(const akr_view* a, const akr_view* b, const akr_view* bias_or_null, akr_view* c,
                   int mode, void* stream);

/* Backward of C = A @ B: the lambda of dispatch_matmul, src/bindings.cpp:1726-1759.
 *   dA = dC . B^T  and  dB = A^T . dC, each summed over the batch dims along which its operand was
 * broadcast (reduce_grad_to_shape, src/bindings.cpp:1467-1503 + sum_axis_kernel,
 * src/reduction_kernel.cu:10-26), without transposed copies or the unreduced intermediate.
 * da / db have the shapes of a / b; either may be NULL to skip that gradient. */
AKR_API int akr_matmul_bwd(const akr_view* a, const akr_view* b, const akr_view* dc, akr_view* da_or_null,
                   akr_view* db_or_null, int mode, void* stream);

/* Backward of C = A @ B where A = tanh(Z): returns the gradient with respect to Z,
 *   dZ = (dC . B^T) * (1 - A^2)   (tanh_backward_kernel, src/elementwise_kernel.cu:517-547, folded into the
 * epilogue of the dA product; A is read where it lies), and dB as akr_matmul_bwd. In the reference these are
 * the matmul node's backward followed by the tanh node's backward (src/bindings.cpp:777-806): one full pass
 * over the activation gradient less. dz has the shape of a; either output may be NULL. */
AKR_API int akr_matmul_bwd_tanh(const akr_view* a_tanh_out, const akr_view* b, const akr_view* dc,
                                akr_view* dz_or_null, akr_view* db_or_null, int mode, void* stream);

/* akr_matmul_bwd (a_is_tanh_output == 0) or akr_matmul_bwd_tanh (!= 0) that also returns the column sums of
 * the gradient it produces for A: da_colsum[k] = sum over all rows and batch entries of dA[.., k] (K floats).
 * When A is the output of a Linear layer, x W + b (aakaar/nn.py:14-15), these are that layer's bias gradient -
 * the reference's broadcast-add backward, src/bindings.cpp:1567-1571 -> reduce_grad_to_shape, :1467-1503 (a full
 * pass over dA in sum_axis_kernel, src/reduction_kernel.cu:10-26). In TF32 mode the sums are taken per 32-row
 * block in the GEMM's epilogue and added up by a small second kernel; no pass over dA. Other cases (fp32-accurate
 * mode, split contractions) fall back to that pass. Deterministic (no atomics). da must not be NULL. */
AKR_API int akr_matmul_bwd_colsum(const akr_view* a, const akr_view* b, const akr_view* dc, akr_view* da,
                                  akr_view* db_or_null, float* da_colsum, int a_is_tanh_output, int mode, void* stream);

/* C = alpha * (A @ B) + beta * D in one launch (D: an array of C's shape with any strides, may be NULL when
 * beta == 0). The two products of the Newton-Schulz iteration of the Muon optimizer
 * (aakaar/optim.py:533-542: `B = b * A + c * (A @ A)`, `X = a * X + X @ B`), which the reference runs as a
 * matmul plus two or three elementwise passes. D must not overlap C unless it is C itself. */
AKR_API int akr_matmul_fwd_axpby(const akr_view* a, const akr_view* b, float alpha, float beta,
                                 const akr_view* d_or_null, akr_view* c, int mode, void* stream);

/* 2-D products the reference exports separately:
 *   run_cublas_matmul_a_bt, src/matmul_kernel.cu:347-373: C(m,n) = A(m,k) . B(n,k)^T
 *   run_cublas_matmul_at_b, src/matmul_kernel.cu:378-402: C(m,n) = A(k,m)^T . B(k,n) */
AKR_API int akr_matmul_a_bt(const akr_view* a, const akr_view* b, akr_view* c, int mode, void* stream);
AKR_API int akr_matmul_at_b(const akr_view* a, const akr_view* b, akr_view* c, int mode, void* stream);

/* The weight-gradient product of akr_matmul_at_b, C(m,n) = A(k,m)^T . B(k,n), for callers that must
 * not allocate device memory when they call: a host whose own pool already owns all of HBM (a later
 * cudaMalloc would fail or eat into the pool), or a latency-critical loop that cannot absorb the
 * device-wide synchronisation cudaMalloc / cudaFree bring. It has no counterpart in the reference.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine. The scratch of the split
 *     contraction (partial tiles, tile counters, status word) is a fixed array inside the library:
 *     8 MiB of partial tiles and 4096 tile counters per GPU, held from library load until exit.
 *   - TF32 products only (AKR_MODE_TF32); both operands must be readable in place (16-byte aligned
 *     base, unit stride on one dim, the other stride a multiple of 4 elements). A product whose
 *     partial tiles would not fit, or an operand that would need a packed copy, is rejected with
 *     AKR_ERR_INVALID and a message naming the limit; use akr_matmul_at_b for those.
 *   - The first call on a device looks up the array's device address; make that call before any
 *     stream capture begins.
 *   - All calls on a device share the one array, which keeps the previous call's contents (what must
 *     start at zero is cleared on every call): two calls that overlap on the GPU, on different
 *     streams, race. Keep them on one stream or order them yourself.
 *   - The call itself never waits for the GPU and reads nothing back. A kernel that gave up on a
 *     bounded wait is reported, like those of every other entry point, by the next akr_synchronize()
 *     on that device (AKR_ERR_ABORTED). */
AKR_API int akr_matmul_at_b_noalloc(const akr_view* a, const akr_view* b, akr_view* c, void* stream);

/* Forward-only matmul of the reference's other dtypes, with the same broadcasting:
 *   run_cuda_matmul_f64, src/matmul_kernel.cu:151-191 (float64) and run_cuda_matmul_int_typed, :300-341
 *   (int32 / int64, 64-bit accumulation, wrap to the output type). No autograd in the reference either.
 * All three views must carry the same dtype (AKR_DTYPE_F64 / I32 / I64). Plain CUDA-core kernel. */
AKR_API int akr_matmul_fwd_typed(const akr_view* a, const akr_view* b, akr_view* c, void* stream);

/* Plain fp32 FMA matmul on CUDA cores with the same broadcasting (no tensor cores, no TF32).
 * A slow on-device cross-check for shapes where a host check takes too long; not used by the
 * product path. */
AKR_API int akr_matmul_fwd_simt(const akr_view* a, const akr_view* b, akr_view* c, void* stream);

/* Number of CTAs the persistent GEMM kernels may occupy (default and maximum: one per SM). A host
 * that overlaps a collective with a GEMM lowers it so that the collective's kernels find free SMs;
 * 0 restores the default. No counterpart in the reference (it has no multi-GPU path). */
AKR_API int akr_set_gemm_cta_limit(int ctas);

/* ------------------------------------------------------------------ multi-GPU
 * The path shards over the GPUs of one node, one process (or thread) per GPU: independent batched products
 * split along the batch need no exchange at all; a large product split along M with the weight B replicated
 * leaves every GPU a partial dB = A_r^T . dC_r, summed by ONE all-reduce. These entry points are that
 * exchange: NCCL (rings / trees / in-switch reduction over NVLink), loaded at run time from libnccl.so.2
 * (environment AKR_B200_NCCL_LIB names another file). No counterpart in the reference, which is single-GPU
 * (docs/limitations.md:15); its one replicated-weight reduction would be the sum_axis of
 * src/bindings.cpp:1467-1503 carried across devices.
 *   akr_mg_get_unique_id : rank 0 creates the 128-byte rendezvous id and hands it to the other ranks by any
 *                          means the host has (a file, a socket, a launcher's key-value store).
 *   akr_mg_init          : every rank, with its device current; collective (returns when all ranks called it).
 *   akr_mg_allreduce     : in-place reduction of `count` elements (AKR_DTYPE_F32 or AKR_DTYPE_F64) over all ranks,
 *                          enqueued on `stream`; AKR_MG_SUM or AKR_MG_MAX. Ranks must issue their collectives
 *                          in the same order.
 *   akr_mg_allreduce_sum : the float32 sum (the dB reduction).
 *   akr_mg_finalize      : waits for the device and destroys the communicator. */
#define AKR_MG_UNIQUE_ID_BYTES 128
enum { AKR_MG_SUM = 0, AKR_MG_MAX = 1 };
AKR_API int akr_mg_get_unique_id(void* id_out);
AKR_API int akr_mg_init(int rank, int world, const void* unique_id);
AKR_API int akr_mg_allreduce(void* data, size_t count, int dtype, int op, void* stream);
AKR_API int akr_mg_allreduce_sum(float* data, size_t n, void* stream);
AKR_API int akr_mg_world(int* rank, int* world);
AKR_API int akr_mg_nccl_version(int* version);
AKR_API int akr_mg_finalize(void);

/* Extra streams for hosts that overlap host<->device copies with the GEMMs (the reference issues
 * everything on the default stream; no counterpart there). Streams are non-blocking with respect to
 * the default stream; order them with events. */
AKR_API int akr_stream_create(void** stream);
AKR_API int akr_stream_destroy(void* stream);
AKR_API int akr_stream_wait_event(void* stream, void* event);

/* CUDA events for timing on the stream the work was issued on (the reference times with
 * synchronize() + host clocks, docs/concepts/hardware-and-cuda/performance.md:52-75). */
AKR_API int akr_event_create(void** event);
AKR_API int akr_event_record(void* event, void* stream);
AKR_API int akr_event_synchronize(void* event);
AKR_API int akr_event_elapsed_ms(void* start, void* end, float* ms);
AKR_API int akr_event_destroy(void* event);

/* Test and measurement hooks (no counterpart in the reference). Every wait inside the GEMM kernels is
 * bounded; a kernel whose wait runs out stops, frees its tensor memory and sets a status word that
 * akr_synchronize() reports as AKR_ERR_ABORTED, leaving the context usable. `wait_limit_ms` sets that
 * bound (0 = default, 4 s). Flags (or-ed):
 *    1  the GEMM kernels skip their TMA loads and multiply whatever shared memory holds: times the
 *       tcgen05.mma issue rate alone (the measured tensor-pipe ceiling a benchmark divides by); results invalid
 *   16  the load warp never signals its stages, so that every waiter gives up (failure-path test)
 *   32  fp32-accurate products run on the CTA-pair (cta_group::2) kernel wherever its tiles apply
 *       (by default contractions of at least 256 - at least 64 for aligned plain outputs - and enough 256 x 256 tiles to fill a quarter of the GPU)
 * 2048  TF32 products run on the CTA-pair kernel wherever it applies (by default a band of shapes)
 * 32768 clock probe: every CTA of a GEMM launch records the SM cycles and the nanoseconds it ran for
 *       (read with akr_gemm_clock_read)
 * akr_debug_configure(0, 0) restores normal operation. Further timing switches exist only in builds
 * compiled with -DAKR_B200_DIAG. */
AKR_API int akr_debug_configure(int flags, unsigned wait_limit_ms);

/* What the clock probe (flag 32768) recorded for the last GEMM launch of the current device, after a
 * synchronize: SM clock in MHz as cycles / nanoseconds per CTA (mean and minimum over the first `ctas`
 * CTAs of the grid), and the longest CTA in cycles and in microseconds. The clock is what a power-capped
 * product's duration depends on; the cycles can be set against those the MMAs alone need. Any pointer may
 * be null. No counterpart in the reference. */
AKR_API int akr_gemm_clock_read(int ctas, double* sm_mhz_mean, double* sm_mhz_min, double* cycles_max, double* us_max);

/* Bytes of scratch the library currently holds on this device (operand splits, split-K partials). */
AKR_API int akr_workspace_bytes(size_t* bytes);
/* Number of kernels launched by this library on this thread's device since the last reset. */
AKR_API int64_t akr_launch_count(int reset);

/* ------------------------------------------------------------------ support ops of the Linear step
 * Thin bandwidth-bound kernels so that nn.Linear training (Linear, tanh, MSE, SGD) runs end to end.
 *   contiguous    : strided gather, src/strided_copy_kernel.cu:13-41 (Tensor::contiguous)
 *   add           : same-shape or broadcast add, src/elementwise_kernel.cu:46-65
 *   sum_to        : reduce_grad_to_shape for a generic broadcast add (bias gradient)
 *   tanh fwd/bwd  : src/elementwise_kernel.cu:494-584
 *   mse fwd/bwd   : src/elementwise_kernel.cu:2253-2300
 *   sgd_step      : src/optim_kernels.cu:21-55 (plain / weight decay / momentum) */
AKR_API int akr_contiguous(const akr_view* src, float* dst, void* stream);
/* The adjoint of akr_contiguous: the dense, row-major `src` (dst's shape) is written through dst's strides. The
 * backward of Tensor.__getitem__ (src/bindings.cpp:2670-2727: the incoming gradient placed into a zero tensor
 * of the base's shape) and of copy_ into a view. */
AKR_API int akr_scatter(const float* src, akr_view* dst, void* stream);
AKR_API int akr_add(const akr_view* a, const akr_view* b, akr_view* out, void* stream);
/* out = a * b elementwise with the broadcasting of akr_add (mul_broadcast_kernel, src/elementwise_kernel.cu). */
AKR_API int akr_mul(const akr_view* a, const akr_view* b, akr_view* out, void* stream);
AKR_API int akr_sum_to(const akr_view* grad, akr_view* out, void* stream);
AKR_API int akr_scale(const float* x, float alpha, float* y, size_t n, void* stream);
AKR_API int akr_tanh_fwd(const float* x, float* y, size_t n, void* stream);
AKR_API int akr_tanh_bwd(const float* grad, const float* y, float* dx, size_t n, void* stream);
/* Sliding-window unfold and its adjoint: the im2col / col2im primitives in front of the matmul in the
 * reference's convolution fallback (aakaar/__init__.py:285-352; src/conv_kernel.cpp:15-60,
 * src/conv2d_kernel.cpp:7-70 and their .cu twins). x: contiguous (B, C, H, W); col: contiguous
 * (B, C*KH*KW, OH*OW), row (c, kh, kw), column (oh, ow), zero where the window leaves the input.
 * The 1-D forms are H = KH = OH = 1, SH = DH = 1, PH = 0. */
typedef struct akr_window {
    int64_t B, C, H, W;
    int32_t KH, KW, SH, SW, PH, PW, DH, DW;
    int64_t OH, OW;
} akr_window;
AKR_API int akr_im2col(const float* x, float* col, const akr_window* geom, void* stream);
AKR_API int akr_col2im(const float* grad_col, float* grad_x, const akr_window* geom, void* stream);
/* The 3-D forms (aakaar/__init__.py:354-363, 451-463; src/conv3d_kernel.cpp and its .cu twin): x contiguous
 * (B, C, D, H, W); col contiguous (B, C*KD*KH*KW, OD*OH*OW), row (c, kd, kh, kw), column (od, oh, ow). The fold
 * is also the forward pass of the transposed convolutions (aakaar/__init__.py:398-519), whose backward is the
 * unfold. */
typedef struct akr_window3d {
    int64_t B, C, D, H, W;
    int32_t KD, KH, KW, SD, SH, SW, PD, PH, PW, DD, DH, DW;
    int64_t OD, OH, OW;
} akr_window3d;
AKR_API int akr_im2col_3d(const float* x, float* col, const akr_window3d* geom, void* stream);
AKR_API int akr_col2im_3d(const float* grad_col, float* grad_x, const akr_window3d* geom, void* stream);

/* loss_out[0] = sum((pred - target)^2) / n; target == NULL gives the mean of squares of pred (the Frobenius
 * norm the Muon optimizer divides by, aakaar/optim.py:534). */
AKR_API int akr_mse_fwd(const float* pred, const float* target, float* loss_out, size_t n, void* stream);
/* The same, and in the same pass dpred = 2 (pred - target) / n: the gradient of the loss when the incoming
 * gradient is 1 (a loss at the root of backward()), which saves the backward pass over pred and target. */
AKR_API int akr_mse_fwd_grad(const float* pred, const float* target, float* loss_out, float* dpred, size_t n,
                             void* stream);
/* akr_mse_fwd_grad that also returns the column sums of dpred over a dense [rows][cols] layout (the bias gradient
 * of the Linear layer that produced pred), in the same pass. */
AKR_API int akr_mse_fwd_grad_colsum(const float* pred, const float* target, float* loss_out, float* dpred,
                                    float* dpred_colsum, int64_t rows, int64_t cols, void* stream);
AKR_API int akr_mse_bwd(const float* pred, const float* target, const float* grad_scalar, float* dpred,
                size_t n, void* stream);
AKR_API int akr_sgd_step(float* param, const float* grad, float* velocity_or_null, float lr, float momentum,
                 float weight_decay, float dampening, int nesterov, int has_momentum,
                 int velocity_initialized, size_t n, void* stream);
/* The same update for `count` parameter tensors in one launch (per 48 tensors): what SGD.step of the reference does
 * with one kernel per parameter (aakaar/optim.py:24-48 -> src/optim_kernels.cu:21-55). velocities may be NULL
 * without momentum; velocity_initialized[i] != 0 once tensor i has taken a step. */
AKR_API int akr_sgd_step_multi(int count, float* const* params, const float* const* grads, float* const* velocities,
                               const size_t* sizes, const int* velocity_initialized, float lr, float momentum,
                               float weight_decay, float dampening, int nesterov, int has_momentum, void* stream);
AKR_API int akr_fill(float* x, float value, size_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AKR_B200_H */
