// Bandwidth-bound helper kernels around the GEMM: operand packing, a plain-FMA
// reference matmul, and the elementwise / reduction ops of the Linear training step.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace akr {

constexpr int kMaxDims = 8;

// Source view of a pack: `nb` batch dims followed by a (rows, cols) matrix.
struct PackSrc {
    const float* ptr;
    int nb;
    int64_t bshape[kMaxDims];
    int64_t bstride[kMaxDims];
    int64_t rows, cols;
    int64_t row_stride, col_stride;
};

// Gathers `src` into a dense [batch][rows][ld] array (a view TMA cannot read in place). Padding columns
// [cols, ld) are zeroed.
cudaError_t launch_pack(const PackSrc& src, float* dst, int64_t ld, cudaStream_t s);

struct SimtGemm {
    const float *A, *B;
    float* C;
    int M, N, K;
    int nb;
    int64_t bshape[kMaxDims];
    int64_t a_bs[kMaxDims], b_bs[kMaxDims], c_bs[kMaxDims];
    int64_t a_rs, a_cs, b_rs, b_cs, c_rs, c_cs;
};
cudaError_t launch_simt_gemm(const SimtGemm& g, cudaStream_t s);
// Same product for dtype 1 = float64, 2 = int32, 3 = int64 (pointers reinterpreted, strides in elements).
cudaError_t launch_simt_gemm_typed(const SimtGemm& g, int dtype, cudaStream_t s);

struct StridedView {
    const float* ptr;
    int nd;
    int64_t shape[kMaxDims];
    int64_t stride[kMaxDims];
};
// dst (contiguous, shape = v.shape) = gather(v)
cudaError_t launch_gather(const StridedView& v, float* dst, cudaStream_t s);
// The adjoint: the view `dst` (its ptr is written) receives the dense, row-major `src` of the view's shape.
// Elements of a view with overlapping strides are written in an unspecified order.
cudaError_t launch_scatter(const float* src, const StridedView& dst, cudaStream_t s);
// out[i] = a[bcast(i)] + b[bcast(i)], out contiguous with shape `shape`
cudaError_t launch_add(const StridedView& a, const StridedView& b, float* out, int nd,
                       const int64_t* shape, cudaStream_t s, bool multiply = false);
// out (contiguous `out_shape`, same rank as g, dims of size 1 where reduced) = sum of g over reduced dims
cudaError_t launch_sum_to(const StridedView& g, const int64_t* out_shape, float* out, cudaStream_t s);
// Column sums of a dense [rows][cols] matrix (the bias gradient of a Linear layer): out[c] = sum_r g[r][c].
// `partials` must hold colsum_partial_floats(rows, cols) floats. Deterministic (no atomics).
size_t colsum_partial_floats(int64_t rows, int64_t cols);
cudaError_t launch_colsum(const float* g, int64_t rows, int64_t cols, float* out, float* partials, cudaStream_t s);

// In-place second-operand epilogue over a strided batched matrix, for products whose kernel has no such
// epilogue (the fp32-accurate mode): op 1: c += beta * x, op 2: c *= 1 - x^2. Batch dims as in StridedView.
struct EpiApply {
    float* c = nullptr;
    const float* x = nullptr;
    int nb = 0;
    int64_t bshape[kMaxDims] = {0}, c_bs[kMaxDims] = {0}, x_bs[kMaxDims] = {0};
    int64_t M = 0, N = 0, c_rs = 0, x_rs = 0, x_cs = 1;
    int op = 0;
    float beta = 0.f;
};
cudaError_t launch_epi_apply(const EpiApply& a, cudaStream_t s);

// Sliding-window unfold of a contiguous (B, C, [D,] H, W) array into (B, C*[KD*]KH*KW, [OD*]OH*OW) and its adjoint
// (gather form: every input element sums the window entries that read it). 1-D is H = KH = OH = 1.
struct WindowGeom {
    int64_t B = 0, C = 0, H = 0, W = 0;
    int KH = 1, KW = 1, SH = 1, SW = 1, PH = 0, PW = 0, DH = 1, DW = 1;
    int64_t OH = 0, OW = 0;
    // depth (3-D windows over a (B, C, D, H, W) array); all ones / zero padding for 1-D and 2-D
    int64_t D = 1;
    int KD = 1, SD = 1, PD = 0, DD = 1;
    int64_t OD = 1;
};
cudaError_t launch_im2col(const float* x, float* col, const WindowGeom& g, cudaStream_t s);
cudaError_t launch_col2im(const float* grad_col, float* grad_x, const WindowGeom& g, cudaStream_t s);

cudaError_t launch_scale(const float* x, float alpha, float* y, size_t n, cudaStream_t s);
cudaError_t launch_fill(float* x, float v, size_t n, cudaStream_t s);
cudaError_t launch_tanh_fwd(const float* x, float* y, size_t n, cudaStream_t s);
cudaError_t launch_tanh_bwd(const float* g, const float* y, float* dx, size_t n, cudaStream_t s);
// loss_out[0] = sum((p-t)^2)/n ; uses `partials` (>= 1024 floats) as scratch
cudaError_t launch_mse_fwd(const float* p, const float* t, float* loss_out, float* partials, size_t n,
                           cudaStream_t s, float* dp = nullptr);
cudaError_t launch_mse_bwd(const float* p, const float* t, const float* gscalar, float* dp, size_t n,
                           cudaStream_t s);
// Loss, its gradient dp = 2 (p - t) / n and the column sums of dp over a dense [rows][cols] layout in one pass
// (two launches, no atomics). cols must be a multiple of 4, all pointers 16-byte aligned; `scratch` holds
// mse_colsum_scratch_floats(rows, cols) floats.
size_t mse_colsum_scratch_floats(int64_t rows, int64_t cols);
cudaError_t launch_mse_fwd_colsum(const float* p, const float* t, float* loss_out, float* dp, float* colsum_out,
                                  int64_t rows, int64_t cols, float* scratch, cudaStream_t s);
// out[c] = sum over the `chunks` rows of a dense [chunks][cols] array (second stage of a column sum whose
// first stage another kernel produced, e.g. a GEMM epilogue).
cudaError_t launch_colsum_final(const float* partials, int chunks, int64_t cols, float* out, cudaStream_t s);
cudaError_t launch_sgd(float* p, const float* g, float* vel, float lr, float momentum, float wd,
                       float dampening, int nesterov, int has_momentum, int vel_init, size_t n,
                       cudaStream_t s);

// The same update for up to kSgdMultiMax tensors in one launch (chunk_start / total_chunks are filled in by the
// launcher).
constexpr int kSgdMultiMax = 48;
struct SgdMulti {
    int count = 0;
    float* param[kSgdMultiMax];
    const float* grad[kSgdMultiMax];
    float* vel[kSgdMultiMax];       // null without momentum
    size_t n[kSgdMultiMax];
    int vel_init[kSgdMultiMax];
    long long chunk_start[kSgdMultiMax];
    long long total_chunks = 0;
};
cudaError_t launch_sgd_multi(SgdMulti& m, float lr, float momentum, float wd, float dampening, int nesterov,
                             int has_momentum, cudaStream_t s);

}  // namespace akr
