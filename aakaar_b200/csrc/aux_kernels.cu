// Helper kernels around the GEMM (see aux_kernels.h). All are HBM-bound: grid-stride loops,
// coalesced along the unit-stride dim, grids sized in multiples of the SM count.
#include "aux_kernels.h"

#include <algorithm>
#include <cstdint>
#include <cstdlib>

namespace akr {

namespace {

constexpr int kThreads = 256;

// Every kernel of this file is launched with programmatic stream serialization and starts with dep_sync():
// it may be scheduled while the kernel before it in the stream drains, lets the kernel after it do the same,
// and touches global memory only once its predecessor has completed.
__device__ __forceinline__ void dep_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename K, typename... Args>
void launch_dep(K kernel, dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
#ifdef AKR_B200_DIAG
    static const bool off = std::getenv("AKR_B200_NO_PDL") != nullptr;  // A/B switch for measurements
#else
    constexpr bool off = false;
#endif
    cfg.numAttrs = off ? 0 : 1;
    cudaLaunchKernelEx(&cfg, kernel, args...);
}

int grid_for(size_t n, int per_thread = 4) {
    static int sms_dev[64] = {};  // per device: a process may drive several GPUs
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    int& sms = sms_dev[dev];
    if (sms == 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    size_t blocks = (n + (size_t)kThreads * per_thread - 1) / ((size_t)kThreads * per_thread);
    const size_t cap = (size_t)sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

struct PackArgs {
    const float* src;
    float* dst;
    int nb;
    int64_t bshape[kMaxDims];
    int64_t bstride[kMaxDims];
    int64_t rows, cols, ld;
    int64_t row_stride, col_stride;
    int64_t total;  // batch * rows * ld
};

__global__ void pack_kernel(const PackArgs a) {
    dep_sync();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += stride) {
        const int64_t c = i % a.ld;
        int64_t t = i / a.ld;
        const int64_t r = t % a.rows;
        t /= a.rows;
        float v = 0.f;
        if (c < a.cols) {
            int64_t off = r * a.row_stride + c * a.col_stride;
            for (int d = a.nb - 1; d >= 0; --d) {
                const int64_t idx = t % a.bshape[d];
                t /= a.bshape[d];
                off += idx * a.bstride[d];
            }
            v = __ldg(a.src + off);
        }
        a.dst[i] = v;
    }
}


constexpr int ST = 16;  // SIMT reference GEMM tile

__global__ void simt_gemm_kernel(const SimtGemm g) {
    dep_sync();
    __shared__ float As[ST][ST + 1];
    __shared__ float Bs[ST][ST + 1];
    int64_t t = blockIdx.z;
    int64_t ao = 0, bo = 0, co = 0;
    for (int d = g.nb - 1; d >= 0; --d) {
        const int64_t idx = t % g.bshape[d];
        t /= g.bshape[d];
        ao += idx * g.a_bs[d];
        bo += idx * g.b_bs[d];
        co += idx * g.c_bs[d];
    }
    const int row = blockIdx.y * ST + threadIdx.y;
    const int col = blockIdx.x * ST + threadIdx.x;
    float acc = 0.f;
    for (int k0 = 0; k0 < g.K; k0 += ST) {
        const int ka = k0 + threadIdx.x;
        const int kb = k0 + threadIdx.y;
        As[threadIdx.y][threadIdx.x] =
            (row < g.M && ka < g.K) ? g.A[ao + (int64_t)row * g.a_rs + (int64_t)ka * g.a_cs] : 0.f;
        Bs[threadIdx.y][threadIdx.x] =
            (kb < g.K && col < g.N) ? g.B[bo + (int64_t)kb * g.b_rs + (int64_t)col * g.b_cs] : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ST; ++k) acc = fmaf(As[threadIdx.y][k], Bs[k][threadIdx.x], acc);
        __syncthreads();
    }
    if (row < g.M && col < g.N) g.C[co + (int64_t)row * g.c_rs + (int64_t)col * g.c_cs] = acc;
}

// Typed forward-only matmul (float64, int32, int64) on CUDA cores: same tiling as above. Integer
// products accumulate in 64 bits and wrap to the output type, as the reference's integer kernel does
// (src/matmul_kernel.cu:219-341); float64 stands in for its cublasDgemm loop (:151-191).
template <typename T, typename Acc>
__global__ void simt_gemm_typed_kernel(const SimtGemm g) {
    dep_sync();
    __shared__ T As[ST][ST + 1];
    __shared__ T Bs[ST][ST + 1];
    const T* A = reinterpret_cast<const T*>(g.A);
    const T* B = reinterpret_cast<const T*>(g.B);
    T* C = reinterpret_cast<T*>(g.C);
    int64_t t = blockIdx.z;
    int64_t ao = 0, bo = 0, co = 0;
    for (int d = g.nb - 1; d >= 0; --d) {
        const int64_t idx = t % g.bshape[d];
        t /= g.bshape[d];
        ao += idx * g.a_bs[d];
        bo += idx * g.b_bs[d];
        co += idx * g.c_bs[d];
    }
    const int row = blockIdx.y * ST + threadIdx.y;
    const int col = blockIdx.x * ST + threadIdx.x;
    Acc acc = 0;
    for (int k0 = 0; k0 < g.K; k0 += ST) {
        const int ka = k0 + threadIdx.x;
        const int kb = k0 + threadIdx.y;
        As[threadIdx.y][threadIdx.x] =
            (row < g.M && ka < g.K) ? A[ao + (int64_t)row * g.a_rs + (int64_t)ka * g.a_cs] : T(0);
        Bs[threadIdx.y][threadIdx.x] =
            (kb < g.K && col < g.N) ? B[bo + (int64_t)kb * g.b_rs + (int64_t)col * g.b_cs] : T(0);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ST; ++k) acc += (Acc)As[threadIdx.y][k] * (Acc)Bs[k][threadIdx.x];
        __syncthreads();
    }
    if (row < g.M && col < g.N) C[co + (int64_t)row * g.c_rs + (int64_t)col * g.c_cs] = (T)acc;
}

struct GatherArgs {
    const float* src;
    float* dst;
    int nd;
    int64_t shape[kMaxDims];
    int64_t stride[kMaxDims];
    int64_t total;
};

__global__ void gather_kernel(const GatherArgs a) {
    dep_sync();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += stride) {
        int64_t t = i, off = 0;
        for (int d = a.nd - 1; d >= 0; --d) {
            const int64_t idx = t % a.shape[d];
            t /= a.shape[d];
            off += idx * a.stride[d];
        }
        a.dst[i] = __ldg(a.src + off);
    }
}

// The adjoint of the gather: dense source (the view's shape, row-major) written through the view's strides.
__global__ void scatter_kernel(const GatherArgs a, float* __restrict__ dst_base) {
    dep_sync();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += stride) {
        int64_t t = i, off = 0;
        for (int d = a.nd - 1; d >= 0; --d) {
            const int64_t idx = t % a.shape[d];
            t /= a.shape[d];
            off += idx * a.stride[d];
        }
        dst_base[off] = __ldg(a.src + i);
    }
}

struct AddArgs {
    const float *a, *b;
    float* out;
    int nd;
    int64_t shape[kMaxDims];
    int64_t as[kMaxDims], bs[kMaxDims];
    int64_t total;
};

template <bool MUL>
__global__ void add_kernel(const AddArgs p) {
    dep_sync();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
        int64_t t = i, ao = 0, bo = 0;
        for (int d = p.nd - 1; d >= 0; --d) {
            const int64_t idx = t % p.shape[d];
            t /= p.shape[d];
            ao += idx * p.as[d];
            bo += idx * p.bs[d];
        }
        p.out[i] = MUL ? __ldg(p.a + ao) * __ldg(p.b + bo) : __ldg(p.a + ao) + __ldg(p.b + bo);
    }
}

template <bool MUL>
__global__ void add_flat_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                float4* __restrict__ o, int64_t n4) {
    dep_sync();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 x = __ldg(a + i), y = __ldg(b + i);
        o[i] = MUL ? make_float4(x.x * y.x, x.y * y.y, x.z * y.z, x.w * y.w)
                   : make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
}

// Sum over reduced dims. One block per 32 kept-output elements x 8 reduction lanes.
struct SumArgs {
    const float* g;
    float* out;
    int nk;  // kept dims
    int nr;  // reduced dims
    int64_t kshape[kMaxDims], kstride[kMaxDims];
    int64_t rshape[kMaxDims], rstride[kMaxDims];
    int64_t nkept, nred;
};

__global__ void sum_to_kernel(const SumArgs a) {
    dep_sync();
    __shared__ float part[8][33];
    const int64_t o = (int64_t)blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    if (o < a.nkept) {
        int64_t t = o, base = 0;
        for (int d = a.nk - 1; d >= 0; --d) {
            const int64_t idx = t % a.kshape[d];
            t /= a.kshape[d];
            base += idx * a.kstride[d];
        }
        for (int64_t r = threadIdx.y; r < a.nred; r += 8) {
            int64_t tr = r, off = base;
            for (int d = a.nr - 1; d >= 0; --d) {
                const int64_t idx = tr % a.rshape[d];
                tr /= a.rshape[d];
                off += idx * a.rstride[d];
            }
            acc += __ldg(a.g + off);
        }
    }
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && o < a.nkept) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += part[j][threadIdx.x];
        a.out[o] = s;
    }
}

// Column sums, stage 1: block (x = 128-column strip, y = row chunk); each warp strides over the rows
// of its chunk reading 512 contiguous bytes per row, the 8 warps are combined in shared memory.
__global__ void colsum_partial_kernel(const float* __restrict__ g, int64_t rows, int64_t cols,
                                      int64_t rows_per_chunk, float* __restrict__ partials) {
    dep_sync();
    __shared__ float4 part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col = (int64_t)blockIdx.x * 128 + lane * 4;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t r1 = min(rows, r0 + rows_per_chunk);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col + 3 < cols && (cols & 3) == 0) {
#pragma unroll 8
        for (int64_t r = r0 + warp; r < r1; r += 8) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(g + r * cols + col));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    } else {
        for (int64_t r = r0 + warp; r < r1; r += 8) {
            const float* p = g + r * cols + col;
            if (col < cols) acc.x += p[0];
            if (col + 1 < cols) acc.y += p[1];
            if (col + 2 < cols) acc.z += p[2];
            if (col + 3 < cols) acc.w += p[3];
        }
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float4 s = part[0][lane];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            const float4 v = part[w][lane];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        float* dst = partials + (int64_t)blockIdx.y * cols + col;
        if (col < cols) dst[0] = s.x;
        if (col + 1 < cols) dst[1] = s.y;
        if (col + 2 < cols) dst[2] = s.z;
        if (col + 3 < cols) dst[3] = s.w;
    }
}
// stage 2: out[c] = sum over chunks, in chunk order
__global__ void colsum_final_kernel(const float* __restrict__ partials, int chunks, int64_t cols,
                                    float* __restrict__ out) {
    dep_sync();
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int k = 0; k < chunks; ++k) s += partials[(int64_t)k * cols + c];
    out[c] = s;
}

__global__ void scale_kernel(const float* __restrict__ x, float alpha, float* __restrict__ y, size_t n) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = x[i] * alpha;
}
__global__ void fill_kernel(float* __restrict__ x, float v, size_t n) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = v;
}
__global__ void tanh_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, size_t n) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = tanhf(x[i]);
}
// 16-byte variants for dense, aligned arrays whose length is a multiple of four.
__global__ void tanh_fwd_vec_kernel(const float4* __restrict__ x, float4* __restrict__ y, size_t n4) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = x[i];
        y[i] = make_float4(tanhf(v.x), tanhf(v.y), tanhf(v.z), tanhf(v.w));
    }
}
__global__ void tanh_bwd_vec_kernel(const float4* __restrict__ g, const float4* __restrict__ y,
                                    float4* __restrict__ dx, size_t n4) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 t = y[i], q = g[i];
        dx[i] = make_float4(q.x * (1.0f - t.x * t.x), q.y * (1.0f - t.y * t.y), q.z * (1.0f - t.z * t.z),
                            q.w * (1.0f - t.w * t.w));
    }
}
// Plain SGD (no momentum, optional weight decay), 16 bytes per thread and round.
__global__ void sgd_plain_vec_kernel(float4* __restrict__ p, const float4* __restrict__ grad, float lr, float wd,
                                     size_t n4) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 w = p[i];
        float4 g = grad[i];
        if (wd != 0.0f) {
            g.x += w.x * wd; g.y += w.y * wd; g.z += w.z * wd; g.w += w.w * wd;
        }
        w.x -= g.x * lr; w.y -= g.y * lr; w.z -= g.z * lr; w.w -= g.w * lr;
        p[i] = w;
    }
}
// The update of several parameter tensors in ONE launch (an optimizer step over a model's parameter list): the
// tensors are cut into chunks of 4096 elements, blocks stride over the chunks of all of them.
__global__ void sgd_multi_kernel(const SgdMulti m, float lr, float momentum, float wd, float dampening, int nesterov,
                                 int has_momentum) {
    dep_sync();
    constexpr int CHUNK = 4096;
    for (long long c = blockIdx.x; c < m.total_chunks; c += gridDim.x) {
        int t = 0;
        while (t + 1 < m.count && c >= m.chunk_start[t + 1]) ++t;
        const size_t n = m.n[t];
        const size_t base = (size_t)(c - m.chunk_start[t]) * CHUNK;
        float* __restrict__ p = m.param[t];
        const float* __restrict__ g = m.grad[t];
        float* __restrict__ v = m.vel[t];
        const int vel_init = m.vel_init[t];
        const size_t end = base + CHUNK < n ? base + CHUNK : n;
        const bool vec = (n & 3) == 0 && (((uintptr_t)p | (uintptr_t)g | (uintptr_t)v) & 15u) == 0;
        if (vec && !has_momentum) {
            for (size_t i = base / 4 + threadIdx.x; i < end / 4; i += blockDim.x) {
                float4 w = reinterpret_cast<float4*>(p)[i];
                float4 gg = reinterpret_cast<const float4*>(g)[i];
                if (wd != 0.0f) {
                    gg.x += w.x * wd; gg.y += w.y * wd; gg.z += w.z * wd; gg.w += w.w * wd;
                }
                w.x -= gg.x * lr; w.y -= gg.y * lr; w.z -= gg.z * lr; w.w -= gg.w * lr;
                reinterpret_cast<float4*>(p)[i] = w;
            }
        } else {
            for (size_t i = base + threadIdx.x; i < end; i += blockDim.x) {
                float gg = g[i];
                if (wd != 0.0f) gg += p[i] * wd;
                float update = gg;
                if (has_momentum) {
                    const float vv = vel_init ? (v[i] * momentum + gg * (1.0f - dampening)) : gg;
                    v[i] = vv;
                    update = nesterov ? (gg + vv * momentum) : vv;
                }
                p[i] = p[i] - update * lr;
            }
        }
    }
}
__global__ void tanh_bwd_kernel(const float* __restrict__ g, const float* __restrict__ y,
                                float* __restrict__ dx, size_t n) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float t = y[i];
        dx[i] = g[i] * (1.0f - t * t);
    }
}

__device__ __forceinline__ float block_sum(float v) {
    __shared__ float warp_part[kThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    if (threadIdx.x < kThreads / 32) s = warp_part[threadIdx.x];
    if (threadIdx.x < 32) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    }
    return s;  // valid in thread 0
}

// dp (optional): the gradient of the mean with respect to p, 2 (p - t) / n, written in the same pass.
__global__ void mse_partial_kernel(const float* __restrict__ p, const float* __restrict__ t,
                                   float* __restrict__ partials, float* __restrict__ dp, float two_over_n, size_t n) {
    dep_sync();
    float acc = 0.f;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float d = t ? p[i] - t[i] : p[i];
        acc = fmaf(d, d, acc);
        if (dp) dp[i] = d * two_over_n;
    }
    const float s = block_sum(acc);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
}
__global__ void mse_final_kernel(const float* __restrict__ partials, int count, float n,
                                 float* __restrict__ out) {
    dep_sync();
    float acc = 0.f;
    for (int i = threadIdx.x; i < count; i += blockDim.x) acc += partials[i];
    const float s = block_sum(acc);
    if (threadIdx.x == 0) out[0] = s / n;
}
// The same with the column sums of dp (the bias gradient of the Linear layer that produced p) taken in the same
// pass. Block (x = 128-column strip, y = row chunk), one float4 per thread and row; the eight warps of a block
// are combined in shared memory and write one partial row per chunk (deterministic: no atomics).
__global__ void mse_colsum_partial_kernel(const float* __restrict__ p, const float* __restrict__ t,
                                          float* __restrict__ loss_partials, float* __restrict__ dp,
                                          float* __restrict__ col_partials, float two_over_n, int64_t rows,
                                          int64_t cols, int64_t rows_per_chunk) {
    dep_sync();
    __shared__ float4 part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col = (int64_t)blockIdx.x * 128 + lane * 4;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t r1 = min(rows, r0 + rows_per_chunk);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float loss = 0.f;
    if (col < cols) {  // cols is a multiple of 4 (checked by the launcher)
#pragma unroll 4
        for (int64_t r = r0 + warp; r < r1; r += 8) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(p + r * cols + col));
            const float4 b = __ldcs(reinterpret_cast<const float4*>(t + r * cols + col));
            const float4 d = make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w);
            loss = fmaf(d.x, d.x, loss); loss = fmaf(d.y, d.y, loss); loss = fmaf(d.z, d.z, loss); loss = fmaf(d.w, d.w, loss);
            const float4 g = make_float4(d.x * two_over_n, d.y * two_over_n, d.z * two_over_n, d.w * two_over_n);
            *reinterpret_cast<float4*>(dp + r * cols + col) = g;
            acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
        }
    }
    part[warp][lane] = acc;
    const float s = block_sum(loss);   // contains the barrier that also orders `part`
    if (threadIdx.x == 0) loss_partials[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = s;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float4 c = part[0][lane];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            const float4 v = part[w][lane];
            c.x += v.x; c.y += v.y; c.z += v.z; c.w += v.w;
        }
        *reinterpret_cast<float4*>(col_partials + (int64_t)blockIdx.y * cols + col) = c;
    }
}
// stage 2 of the above: column sums in chunk order; block 0 also finishes the loss.
__global__ void mse_colsum_final_kernel(const float* __restrict__ loss_partials, int loss_count, float n,
                                        float* __restrict__ loss_out, const float* __restrict__ col_partials,
                                        int chunks, int64_t cols, float* __restrict__ colsum_out) {
    dep_sync();
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c < cols) {
        float s = 0.f;
        for (int k = 0; k < chunks; ++k) s += col_partials[(int64_t)k * cols + c];
        colsum_out[c] = s;
    }
    if (blockIdx.x == 0) {
        float acc = 0.f;
        for (int i = threadIdx.x; i < loss_count; i += blockDim.x) acc += loss_partials[i];
        const float s = block_sum(acc);
        if (threadIdx.x == 0) loss_out[0] = s / n;
    }
}
__global__ void mse_bwd_kernel(const float* __restrict__ p, const float* __restrict__ t,
                               const float* __restrict__ gscalar, float inv_n, float* __restrict__ dp,
                               size_t n) {
    dep_sync();
    const float scale = 2.0f * inv_n * (gscalar ? gscalar[0] : 1.0f);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dp[i] = (p[i] - t[i]) * scale;
}

__global__ void sgd_kernel(float* __restrict__ p, const float* __restrict__ grad, float* __restrict__ vel,
                           float lr, float momentum, float wd, float dampening, int nesterov,
                           int has_momentum, int vel_init, size_t n) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float g = grad[i];
        if (wd != 0.0f) g += p[i] * wd;
        float update;
        if (has_momentum) {
            const float v = vel_init ? (vel[i] * momentum + g * (1.0f - dampening)) : g;
            vel[i] = v;
            update = nesterov ? (g + v * momentum) : v;
        } else {
            update = g;
        }
        p[i] = p[i] - update * lr;
    }
}

}  // namespace

cudaError_t launch_pack(const PackSrc& src, float* dst, int64_t ld, cudaStream_t s) {
    int64_t batch = 1;
    for (int d = 0; d < src.nb; ++d) batch *= src.bshape[d];
    const int64_t total = batch * src.rows * ld;
    if (total == 0) return cudaSuccess;
    PackArgs a;
    a.src = src.ptr;
    a.dst = dst;
    a.nb = src.nb;
    for (int d = 0; d < kMaxDims; ++d) {
        a.bshape[d] = d < src.nb ? src.bshape[d] : 1;
        a.bstride[d] = d < src.nb ? src.bstride[d] : 0;
    }
    a.rows = src.rows;
    a.cols = src.cols;
    a.ld = ld;
    a.row_stride = src.row_stride;
    a.col_stride = src.col_stride;
    a.total = total;
    launch_dep(pack_kernel, grid_for((size_t)total, 2), kThreads, s, a);
    return cudaGetLastError();
}

cudaError_t launch_simt_gemm(const SimtGemm& g, cudaStream_t s) {
    int64_t batch = 1;
    for (int d = 0; d < g.nb; ++d) batch *= g.bshape[d];
    if (batch > 65535) return cudaErrorInvalidValue;
    dim3 grid((g.N + ST - 1) / ST, (g.M + ST - 1) / ST, (unsigned)batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    launch_dep(simt_gemm_kernel, grid, dim3(ST, ST), s, g);
    return cudaGetLastError();
}

cudaError_t launch_simt_gemm_typed(const SimtGemm& g, int dtype, cudaStream_t s) {
    int64_t batch = 1;
    for (int d = 0; d < g.nb; ++d) batch *= g.bshape[d];
    if (batch > 65535) return cudaErrorInvalidValue;
    dim3 grid((g.N + ST - 1) / ST, (g.M + ST - 1) / ST, (unsigned)batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    switch (dtype) {
        case 1: launch_dep(simt_gemm_typed_kernel<double, double>, grid, dim3(ST, ST), s, g); break;
        case 2: launch_dep(simt_gemm_typed_kernel<int, long long>, grid, dim3(ST, ST), s, g); break;
        case 3: launch_dep(simt_gemm_typed_kernel<long long, long long>, grid, dim3(ST, ST), s, g); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_gather(const StridedView& v, float* dst, cudaStream_t s) {
    GatherArgs a;
    a.src = v.ptr;
    a.dst = dst;
    a.nd = v.nd;
    a.total = 1;
    for (int d = 0; d < kMaxDims; ++d) {
        a.shape[d] = d < v.nd ? v.shape[d] : 1;
        a.stride[d] = d < v.nd ? v.stride[d] : 0;
        a.total *= a.shape[d];
    }
    if (a.total == 0) return cudaSuccess;
    launch_dep(gather_kernel, grid_for((size_t)a.total, 2), kThreads, s, a);
    return cudaGetLastError();
}

cudaError_t launch_scatter(const float* src, const StridedView& dst, cudaStream_t s) {
    GatherArgs a;
    a.src = src;
    a.dst = nullptr;
    a.nd = dst.nd;
    a.total = 1;
    for (int d = 0; d < kMaxDims; ++d) {
        a.shape[d] = d < dst.nd ? dst.shape[d] : 1;
        a.stride[d] = d < dst.nd ? dst.stride[d] : 0;
        a.total *= a.shape[d];
    }
    if (a.total == 0) return cudaSuccess;
    launch_dep(scatter_kernel, grid_for((size_t)a.total, 2), kThreads, s, a, const_cast<float*>(dst.ptr));
    return cudaGetLastError();
}

cudaError_t launch_add(const StridedView& a, const StridedView& b, float* out, int nd,
                       const int64_t* shape, cudaStream_t s, bool multiply) {
    AddArgs p;
    p.a = a.ptr;
    p.b = b.ptr;
    p.out = out;
    p.nd = nd;
    p.total = 1;
    bool flat = true;
    int64_t expect = 1;
    for (int d = kMaxDims - 1; d >= 0; --d) {
        if (d < nd) {
            p.shape[d] = shape[d];
            p.as[d] = a.stride[d];
            p.bs[d] = b.stride[d];
            if (shape[d] != 1 && (a.stride[d] != expect || b.stride[d] != expect)) flat = false;
            expect *= shape[d];
            p.total *= shape[d];
        } else {
            p.shape[d] = 1;
            p.as[d] = p.bs[d] = 0;
        }
    }
    if (p.total == 0) return cudaSuccess;
    if (flat && (p.total & 3) == 0 && (((uintptr_t)a.ptr | (uintptr_t)b.ptr | (uintptr_t)out) & 15u) == 0) {
        const float4 *a4 = reinterpret_cast<const float4*>(a.ptr), *b4 = reinterpret_cast<const float4*>(b.ptr);
        float4* o4 = reinterpret_cast<float4*>(out);
        if (multiply) launch_dep(add_flat_kernel<true>, grid_for((size_t)p.total / 4, 2), kThreads, s, a4, b4, o4, p.total / 4);
        else launch_dep(add_flat_kernel<false>, grid_for((size_t)p.total / 4, 2), kThreads, s, a4, b4, o4, p.total / 4);
        return cudaGetLastError();
    }
    if (multiply) launch_dep(add_kernel<true>, grid_for((size_t)p.total, 2), kThreads, s, p);
    else launch_dep(add_kernel<false>, grid_for((size_t)p.total, 2), kThreads, s, p);
    return cudaGetLastError();
}

cudaError_t launch_sum_to(const StridedView& g, const int64_t* out_shape, float* out, cudaStream_t s) {
    SumArgs a;
    a.g = g.ptr;
    a.out = out;
    a.nk = a.nr = 0;
    a.nkept = a.nred = 1;
    for (int d = 0; d < g.nd; ++d) {
        if (out_shape[d] == g.shape[d]) {
            if (g.shape[d] == 1) continue;
            a.kshape[a.nk] = g.shape[d];
            a.kstride[a.nk] = g.stride[d];
            a.nkept *= g.shape[d];
            ++a.nk;
        } else {
            a.rshape[a.nr] = g.shape[d];
            a.rstride[a.nr] = g.stride[d];
            a.nred *= g.shape[d];
            ++a.nr;
        }
    }
    if (a.nkept == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((a.nkept + 31) / 32);
    launch_dep(sum_to_kernel, blocks, dim3(32, 8), s, a);
    return cudaGetLastError();
}

static int colsum_chunks(int64_t rows, int64_t cols) {
    const int64_t strips = (cols + 127) / 128;
    int64_t chunks = (148 * 4 + strips - 1) / strips;       // about four blocks per SM in total
    chunks = std::min<int64_t>(chunks, (rows + 63) / 64);    // at least 64 rows per chunk
    return (int)std::max<int64_t>(1, std::min<int64_t>(chunks, 256));
}
size_t colsum_partial_floats(int64_t rows, int64_t cols) { return (size_t)colsum_chunks(rows, cols) * (size_t)cols; }

cudaError_t launch_colsum(const float* g, int64_t rows, int64_t cols, float* out, float* partials, cudaStream_t s) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    const int chunks = colsum_chunks(rows, cols);
    const int64_t rpc = (rows + chunks - 1) / chunks;
    dim3 grid((unsigned)((cols + 127) / 128), (unsigned)chunks);
    launch_dep(colsum_partial_kernel, grid, 256, s, g, rows, cols, rpc, partials);
    launch_dep(colsum_final_kernel, (unsigned)((cols + 255) / 256), 256, s, partials, chunks, cols, out);
    return cudaGetLastError();
}

cudaError_t launch_scale(const float* x, float alpha, float* y, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    launch_dep(scale_kernel, grid_for(n), kThreads, s, x, alpha, y, n);
    return cudaGetLastError();
}
cudaError_t launch_fill(float* x, float v, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    launch_dep(fill_kernel, grid_for(n), kThreads, s, x, v, n);
    return cudaGetLastError();
}
cudaError_t launch_tanh_fwd(const float* x, float* y, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    if ((n & 3) == 0 && (((uintptr_t)x | (uintptr_t)y) & 15u) == 0)
        launch_dep(tanh_fwd_vec_kernel, grid_for(n / 4, 2), kThreads, s, (const float4*)x, (float4*)y, n / 4);
    else
        launch_dep(tanh_fwd_kernel, grid_for(n), kThreads, s, x, y, n);
    return cudaGetLastError();
}
cudaError_t launch_tanh_bwd(const float* g, const float* y, float* dx, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    if ((n & 3) == 0 && (((uintptr_t)g | (uintptr_t)y | (uintptr_t)dx) & 15u) == 0)
        launch_dep(tanh_bwd_vec_kernel, grid_for(n / 4, 2), kThreads, s, (const float4*)g, (const float4*)y, (float4*)dx, n / 4);
    else
        launch_dep(tanh_bwd_kernel, grid_for(n), kThreads, s, g, y, dx, n);
    return cudaGetLastError();
}
cudaError_t launch_mse_fwd(const float* p, const float* t, float* loss_out, float* partials, size_t n,
                           cudaStream_t s, float* dp) {
    int blocks = grid_for(n);
    if (blocks > 1024) blocks = 1024;
    launch_dep(mse_partial_kernel, blocks, kThreads, s, p, t, partials, dp, 2.0f * (1.0f / (float)n), n);
    launch_dep(mse_final_kernel, 1, kThreads, s, partials, blocks, (float)n, loss_out);
    return cudaGetLastError();
}
size_t mse_colsum_scratch_floats(int64_t rows, int64_t cols) {
    const int chunks = colsum_chunks(rows, cols);
    const size_t strips = (size_t)((cols + 127) / 128);
    return (size_t)chunks * (size_t)cols + (size_t)chunks * strips + 64;
}
cudaError_t launch_mse_fwd_colsum(const float* p, const float* t, float* loss_out, float* dp, float* colsum_out,
                                  int64_t rows, int64_t cols, float* scratch, cudaStream_t s) {
    const int chunks = colsum_chunks(rows, cols);
    const int64_t rpc = (rows + chunks - 1) / chunks;
    const unsigned strips = (unsigned)((cols + 127) / 128);
    float* col_partials = scratch;
    float* loss_partials = scratch + (size_t)chunks * (size_t)cols;
    const double n = (double)rows * (double)cols;
    dim3 grid(strips, (unsigned)chunks);
    launch_dep(mse_colsum_partial_kernel, grid, 256, s, p, t, loss_partials, dp, col_partials, (float)(2.0 / n), rows, cols,
               rpc);
    launch_dep(mse_colsum_final_kernel, (unsigned)((cols + 255) / 256), 256, s, (const float*)loss_partials,
               (int)(chunks * strips), (float)n, loss_out, (const float*)col_partials, chunks, cols, colsum_out);
    return cudaGetLastError();
}
// out[c] = sum over `chunks` rows of a [chunks][cols] array of partial column sums, in row order.
cudaError_t launch_colsum_final(const float* partials, int chunks, int64_t cols, float* out, cudaStream_t s) {
    if (cols == 0) return cudaSuccess;
    launch_dep(colsum_final_kernel, (unsigned)((cols + 255) / 256), 256, s, partials, chunks, cols, out);
    return cudaGetLastError();
}
__global__ void epi_apply_kernel(EpiApply a, size_t total) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t n = (int64_t)(i % (size_t)a.N);
        size_t r = i / (size_t)a.N;
        const int64_t m = (int64_t)(r % (size_t)a.M);
        r /= (size_t)a.M;
        int64_t co = m * a.c_rs + n, xo = m * a.x_rs + n * a.x_cs;
        for (int d = a.nb - 1; d >= 0; --d) {
            const int64_t idx = (int64_t)(r % (size_t)a.bshape[d]);
            r /= (size_t)a.bshape[d];
            co += idx * a.c_bs[d];
            xo += idx * a.x_bs[d];
        }
        const float x = a.x[xo], c = a.c[co];
        a.c[co] = a.op == 1 ? fmaf(a.beta, x, c) : c * (1.f - x * x);
    }
}
// Both arrays dense and laid out alike: a flat, 16-byte vectorised pass.
__global__ void epi_apply_flat_kernel(float4* __restrict__ c, const float4* __restrict__ x, size_t n4, int op,
                                      float beta) {
    dep_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 v = c[i];
        const float4 a = x[i];
        if (op == 1) {
            v.x = fmaf(beta, a.x, v.x); v.y = fmaf(beta, a.y, v.y); v.z = fmaf(beta, a.z, v.z); v.w = fmaf(beta, a.w, v.w);
        } else {
            v.x *= 1.f - a.x * a.x; v.y *= 1.f - a.y * a.y; v.z *= 1.f - a.z * a.z; v.w *= 1.f - a.w * a.w;
        }
        c[i] = v;
    }
}
cudaError_t launch_epi_apply(const EpiApply& a, cudaStream_t s) {
    size_t total = (size_t)a.M * (size_t)a.N;
    for (int d = 0; d < a.nb; ++d) total *= (size_t)a.bshape[d];
    if (total == 0) return cudaSuccess;
    bool flat = a.x_cs == 1 && a.c_rs == a.N && a.x_rs == a.N && (total & 3) == 0 &&
                (reinterpret_cast<uintptr_t>(a.c) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 &&
                (const float*)a.c != a.x;
    int64_t dense = a.M * a.N;
    for (int d = a.nb - 1; d >= 0 && flat; --d) {
        flat = a.c_bs[d] == dense && a.x_bs[d] == dense;
        dense *= a.bshape[d];
    }
    if (flat) {
        launch_dep(epi_apply_flat_kernel, grid_for(total / 4), kThreads, s, (float4*)a.c, (const float4*)a.x, total / 4, a.op,
                                                                       a.beta);
        return cudaGetLastError();
    }
    launch_dep(epi_apply_kernel, grid_for(total), kThreads, s, a, total);
    return cudaGetLastError();
}

// Unfold: one block per (b, c, kh, kw) row of `col` (blockIdx.x), every thread four consecutive window
// positions at a time (one 16-byte store): 32-bit index arithmetic, coalesced writes, reads that hit L1 / L2
// (each input plane is read KH*KW times).
template <bool VEC>
__global__ void im2col_kernel(const float* __restrict__ x, float* __restrict__ col, WindowGeom g) {
    dep_sync();
    const unsigned row = blockIdx.x;  // ((b * C + c) * KH + kh) * KW + kw
    const int kw = (int)(row % (unsigned)g.KW);
    const unsigned r1 = row / (unsigned)g.KW;
    const int kh = (int)(r1 % (unsigned)g.KH);
    const unsigned plane = r1 / (unsigned)g.KH;  // b * C + c
    const int OW = (int)g.OW, OHW = (int)(g.OH * g.OW), H = (int)g.H, W = (int)g.W;
    const float* xp = x + (size_t)plane * H * W;
    float* cp = col + (size_t)row * OHW;
    const int h_off = kh * g.DH - g.PH, w_off = kw * g.DW - g.PW;
    constexpr int V = VEC ? 4 : 1;
    for (int o0 = (blockIdx.y * blockDim.x + threadIdx.x) * V; o0 < OHW; o0 += gridDim.y * blockDim.x * V) {
        float v[V];
        int oh = o0 / OW, ow = o0 - oh * OW;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const int h = oh * g.SH + h_off, w = ow * g.SW + w_off;
            v[e] = (h >= 0 && h < H && w >= 0 && w < W) ? __ldg(xp + h * W + w) : 0.f;
            if (++ow == OW) {
                ow = 0;
                ++oh;
            }
        }
        if (VEC) *reinterpret_cast<float4*>(cp + o0) = make_float4(v[0], v[V > 1 ? 1 : 0], v[V > 2 ? 2 : 0], v[V > 3 ? 3 : 0]);
        else cp[o0] = v[0];
    }
}
// Fold (adjoint): one block row per (b, c) plane, every thread four consecutive elements of a plane at a time;
// each sums, in (kh, kw) order, the window entries that read it.
// S1: both strides are 1 (no divisions on the way back from an input position to the windows that read it).
template <bool VEC, bool S1>
__global__ void col2im_kernel(const float* __restrict__ gc, float* __restrict__ gx, WindowGeom g) {
    dep_sync();
    const unsigned plane = blockIdx.x;  // b * C + c
    const int OW = (int)g.OW, OH = (int)g.OH, OHW = OH * OW, H = (int)g.H, W = (int)g.W;
    const float* base = gc + (size_t)plane * g.KH * g.KW * OHW;
    float* gp = gx + (size_t)plane * H * W;
    constexpr int V = VEC ? 4 : 1;
    for (int i0 = (blockIdx.y * blockDim.x + threadIdx.x) * V; i0 < H * W; i0 += gridDim.y * blockDim.x * V) {
        float acc[V];
        int hs[V], ws[V];
        {
            int h = i0 / W, w = i0 - h * W;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                acc[e] = 0.f;
                hs[e] = h;
                ws[e] = w;
                if (++w == W) {
                    w = 0;
                    ++h;
                }
            }
        }
        for (int kh = 0; kh < g.KH; ++kh) {
            int ohs[V];
#pragma unroll
            for (int e = 0; e < V; ++e) {  // window row that reads input row hs[e] through tap kh, or -1
                const int nh = hs[e] + g.PH - kh * g.DH;
                int oh = S1 ? nh : nh / g.SH;
                if (nh < 0 || oh >= OH || (!S1 && oh * g.SH != nh)) oh = -1;
                ohs[e] = oh;
            }
            for (int kw = 0; kw < g.KW; ++kw) {
                const float* tap = base + (size_t)(kh * g.KW + kw) * OHW;
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const int nw = ws[e] + g.PW - kw * g.DW;
                    const int ow = S1 ? nw : nw / g.SW;
                    if (ohs[e] < 0 || nw < 0 || ow >= OW || (!S1 && ow * g.SW != nw)) continue;
                    acc[e] += __ldg(tap + ohs[e] * OW + ow);
                }
            }
        }
        if (VEC) *reinterpret_cast<float4*>(gp + i0) = make_float4(acc[0], acc[V > 1 ? 1 : 0], acc[V > 2 ? 2 : 0], acc[V > 3 ? 3 : 0]);
        else gp[i0] = acc[0];
    }
}
// 3-D windows: the same two kernels with a depth index. One block per (b, c, kd, kh, kw) row of `col`, four
// consecutive (od, oh, ow) positions per thread and store.
template <bool VEC>
__global__ void im2col3d_kernel(const float* __restrict__ x, float* __restrict__ col, WindowGeom g) {
    dep_sync();
    const unsigned row = blockIdx.x;  // (((b * C + c) * KD + kd) * KH + kh) * KW + kw
    const int kw = (int)(row % (unsigned)g.KW);
    const unsigned r1 = row / (unsigned)g.KW;
    const int kh = (int)(r1 % (unsigned)g.KH);
    const unsigned r2 = r1 / (unsigned)g.KH;
    const int kd = (int)(r2 % (unsigned)g.KD);
    const unsigned plane = r2 / (unsigned)g.KD;  // b * C + c
    const int OW = (int)g.OW, OH = (int)g.OH, OHW = OH * OW, ODHW = (int)g.OD * OHW;
    const int D = (int)g.D, H = (int)g.H, W = (int)g.W;
    const float* xp = x + (size_t)plane * D * H * W;
    float* cp = col + (size_t)row * ODHW;
    const int d_off = kd * g.DD - g.PD, h_off = kh * g.DH - g.PH, w_off = kw * g.DW - g.PW;
    constexpr int V = VEC ? 4 : 1;
    for (int o0 = (blockIdx.y * blockDim.x + threadIdx.x) * V; o0 < ODHW; o0 += gridDim.y * blockDim.x * V) {
        float v[V];
        int od = o0 / OHW;
        int rem = o0 - od * OHW;
        int oh = rem / OW, ow = rem - oh * OW;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const int d = od * g.SD + d_off, h = oh * g.SH + h_off, w = ow * g.SW + w_off;
            v[e] = (d >= 0 && d < D && h >= 0 && h < H && w >= 0 && w < W) ? __ldg(xp + ((size_t)d * H + h) * W + w) : 0.f;
            if (++ow == OW) {
                ow = 0;
                if (++oh == OH) {
                    oh = 0;
                    ++od;
                }
            }
        }
        if (VEC) *reinterpret_cast<float4*>(cp + o0) = make_float4(v[0], v[V > 1 ? 1 : 0], v[V > 2 ? 2 : 0], v[V > 3 ? 3 : 0]);
        else cp[o0] = v[0];
    }
}
// Fold: one block row per (b, c) volume, one element per thread; each sums, in (kd, kh, kw) order, the window
// entries that read it.
__global__ void col2im3d_kernel(const float* __restrict__ gc, float* __restrict__ gx, WindowGeom g) {
    dep_sync();
    const unsigned plane = blockIdx.x;  // b * C + c
    const int OW = (int)g.OW, OH = (int)g.OH, OD = (int)g.OD, OHW = OH * OW;
    const int D = (int)g.D, H = (int)g.H, W = (int)g.W, HW = H * W;
    const size_t odhw = (size_t)OD * OHW;
    const float* base = gc + (size_t)plane * g.KD * g.KH * g.KW * odhw;
    float* gp = gx + (size_t)plane * D * HW;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < D * HW; i += gridDim.y * blockDim.x) {
        const int d = i / HW;
        const int r = i - d * HW;
        const int h = r / W, w = r - h * W;
        float acc = 0.f;
        for (int kd = 0; kd < g.KD; ++kd) {
            const int nd = d + g.PD - kd * g.DD;
            const int od = nd / g.SD;
            if (nd < 0 || od >= OD || od * g.SD != nd) continue;
            for (int kh = 0; kh < g.KH; ++kh) {
                const int nh = h + g.PH - kh * g.DH;
                const int oh = nh / g.SH;
                if (nh < 0 || oh >= OH || oh * g.SH != nh) continue;
                for (int kw = 0; kw < g.KW; ++kw) {
                    const int nw = w + g.PW - kw * g.DW;
                    const int ow = nw / g.SW;
                    if (nw < 0 || ow >= OW || ow * g.SW != nw) continue;
                    acc += __ldg(base + (size_t)((kd * g.KH + kh) * g.KW + kw) * odhw + (size_t)od * OHW + oh * OW + ow);
                }
            }
        }
        gp[i] = acc;
    }
}
static bool is_3d(const WindowGeom& g) { return g.D != 1 || g.KD != 1 || g.OD != 1 || g.PD != 0; }
static cudaError_t launch_im2col3d(const float* x, float* col, const WindowGeom& g, cudaStream_t s) {
    const size_t rows = (size_t)g.B * g.C * g.KD * g.KH * g.KW;
    const size_t odhw = (size_t)g.OD * g.OH * g.OW;
    if (rows == 0 || odhw == 0) return cudaSuccess;
    if (rows > 0x7fffffffull || odhw > 0x7fffffffull || (size_t)g.D * g.H * g.W > 0x7fffffffull) return cudaErrorInvalidValue;
    const bool vec = (odhw & 3) == 0 && (reinterpret_cast<uintptr_t>(col) & 15u) == 0;
    const size_t per_block = (size_t)kThreads * (vec ? 4 : 1) * 4;
    const unsigned gy = (unsigned)std::min<size_t>((odhw + per_block - 1) / per_block, 64);
    if (vec) launch_dep(im2col3d_kernel<true>, dim3((unsigned)rows, gy), kThreads, s, x, col, g);
    else launch_dep(im2col3d_kernel<false>, dim3((unsigned)rows, gy), kThreads, s, x, col, g);
    return cudaGetLastError();
}
static cudaError_t launch_col2im3d(const float* grad_col, float* grad_x, const WindowGeom& g, cudaStream_t s) {
    const size_t planes = (size_t)g.B * g.C;
    const size_t dhw = (size_t)g.D * g.H * g.W;
    if (planes == 0 || dhw == 0) return cudaSuccess;
    if (planes > 0x7fffffffull || dhw > 0x7fffffffull || (size_t)g.OD * g.OH * g.OW > 0x7fffffffull) return cudaErrorInvalidValue;
    const unsigned gy = (unsigned)std::min<size_t>((dhw + kThreads - 1) / kThreads, 256);
    launch_dep(col2im3d_kernel, dim3((unsigned)planes, gy), kThreads, s, grad_col, grad_x, g);
    return cudaGetLastError();
}

cudaError_t launch_im2col(const float* x, float* col, const WindowGeom& g, cudaStream_t s) {
    if (is_3d(g)) return launch_im2col3d(x, col, g, s);
    const size_t rows = (size_t)g.B * g.C * g.KH * g.KW;
    const size_t ohw = (size_t)g.OH * g.OW;
    if (rows == 0 || ohw == 0) return cudaSuccess;
    if (rows > 0x7fffffffull || ohw > 0x7fffffffull || (size_t)g.H * g.W > 0x7fffffffull) return cudaErrorInvalidValue;
    const bool vec = (ohw & 3) == 0 && (reinterpret_cast<uintptr_t>(col) & 15u) == 0;
    const size_t per_block = (size_t)kThreads * (vec ? 4 : 1) * 4;  // about four rounds per thread
    const unsigned gy = (unsigned)std::min<size_t>((ohw + per_block - 1) / per_block, 64);
    if (vec) launch_dep(im2col_kernel<true>, dim3((unsigned)rows, gy), kThreads, s, x, col, g);
    else launch_dep(im2col_kernel<false>, dim3((unsigned)rows, gy), kThreads, s, x, col, g);
    return cudaGetLastError();
}
cudaError_t launch_col2im(const float* grad_col, float* grad_x, const WindowGeom& g, cudaStream_t s) {
    if (is_3d(g)) return launch_col2im3d(grad_col, grad_x, g, s);
    const size_t planes = (size_t)g.B * g.C;
    const size_t hw = (size_t)g.H * g.W;
    if (planes == 0 || hw == 0) return cudaSuccess;
    if (planes > 0x7fffffffull || hw > 0x7fffffffull || (size_t)g.OH * g.OW > 0x7fffffffull) return cudaErrorInvalidValue;
    const bool vec = (hw & 3) == 0 && (reinterpret_cast<uintptr_t>(grad_x) & 15u) == 0;
    const size_t per_block = (size_t)kThreads * (vec ? 4 : 1);
    const unsigned gy = (unsigned)std::min<size_t>((hw + per_block - 1) / per_block, 64);
    const bool s1 = g.SH == 1 && g.SW == 1;
    const dim3 grid((unsigned)planes, gy);
    if (vec && s1) launch_dep(col2im_kernel<true, true>, grid, kThreads, s, grad_col, grad_x, g);
    else if (vec) launch_dep(col2im_kernel<true, false>, grid, kThreads, s, grad_col, grad_x, g);
    else if (s1) launch_dep(col2im_kernel<false, true>, grid, kThreads, s, grad_col, grad_x, g);
    else launch_dep(col2im_kernel<false, false>, grid, kThreads, s, grad_col, grad_x, g);
    return cudaGetLastError();
}

cudaError_t launch_mse_bwd(const float* p, const float* t, const float* gscalar, float* dp, size_t n,
                           cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    launch_dep(mse_bwd_kernel, grid_for(n), kThreads, s, p, t, gscalar, 1.0f / (float)n, dp, n);
    return cudaGetLastError();
}
cudaError_t launch_sgd(float* p, const float* g, float* vel, float lr, float momentum, float wd,
                       float dampening, int nesterov, int has_momentum, int vel_init, size_t n,
                       cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    if (!has_momentum && (n & 3) == 0 && (((uintptr_t)p | (uintptr_t)g) & 15u) == 0) {
        launch_dep(sgd_plain_vec_kernel, grid_for(n / 4, 2), kThreads, s, (float4*)p, (const float4*)g, lr, wd, n / 4);
        return cudaGetLastError();
    }
    launch_dep(sgd_kernel, grid_for(n), kThreads, s, p, g, vel, lr, momentum, wd, dampening, nesterov,
                                                 has_momentum, vel_init, n);
    return cudaGetLastError();
}

cudaError_t launch_sgd_multi(SgdMulti& m, float lr, float momentum, float wd, float dampening, int nesterov,
                             int has_momentum, cudaStream_t s) {
    long long chunks = 0;
    for (int t = 0; t < m.count; ++t) {
        m.chunk_start[t] = chunks;
        chunks += (long long)((m.n[t] + 4095) / 4096);
    }
    m.total_chunks = chunks;
    if (chunks == 0) return cudaSuccess;
    const long long cap = (long long)grid_for((size_t)chunks * 4096, 4);
    launch_dep(sgd_multi_kernel, (unsigned)(chunks < cap ? chunks : cap), kThreads, s, m, lr, momentum, wd, dampening,
               nesterov, has_momentum);
    return cudaGetLastError();
}

}  // namespace akr
