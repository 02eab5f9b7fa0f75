// fp32 GEMM for B200 (sm_100a): TMA-staged 128-byte-swizzled tiles, tcgen05.mma kind::tf32
// accumulating in tensor memory, persistent CTAs with warp-specialised roles.
//
//   warp 0 (one thread)  : TMA producer, fills a ring of STAGES shared-memory stages
//   warp 1               : MMA issuer (all lanes run the loop, one elected lane issues); owns the TMEM
//                          allocation (two accumulators, ping-pong)
//   warps 2..5 (2..9 for 256-wide tiles): epilogue, TMEM -> registers -> global
//                          (bias / accumulate / split-K sum / fp32 promotion of partial chains)
//
// Four kernels share these roles: gemm_tf32_kernel (one CTA per 128 x 64 / 128 / 256 tile, both modes, split
// contractions), gemm_tf32_duo_kernel (256 x 256 per CTA pair, TF32), gemm_tf32_quad_kernel (512 x 256 per CTA pair,
// TF32) and gemm_tf32_pair_kernel (256 x 256 per CTA pair, fp32-accurate); gemm_sm100_launch picks one per product
// (use_duo / use_quad / use_pairs). A fifth, gemm_tf32_big_kernel (256 x 256 per CTA, TF32), is what the 512 x 256 pair
// tiles grew out of and are measured against; it is compiled in diagnostic builds only.
// What the measurements behind those choices say: a stage should carry at least eight MMAs (handing a stage over costs
// more than filling it), a TMA row should be 128 bytes, the issuing thread must never stall for more than the four
// MMAs the tensor pipe queues, and waiting threads must neither read the clock nor poll without pause.
//
// Replaces the per-batch cublasSgemm loops of the reference (src/matmul_kernel.cu:111-143 forward,
// :347-402 the two backward products) and, through the `red` batch dim, the unreduced
// weight-gradient product plus sum_axis passes of src/bindings.cpp:1750-1758, 1467-1503.
//
// Operand layouts: each operand may be K-major or M/N-major in global memory; the tile is staged
// the way it lies and the UMMA descriptors carry the major-ness, so transposed views need no copy.
// TF32 mode issues one MMA per 8-deep k-slice; 3xTF32 mode issues three (lo*hi, hi*lo, hi*hi), the
// low parts derived in shared memory by two converter warps (the tensor core truncates fp32 operands to TF32, so the
// raw tile is the high part): fp32-level accuracy with operands still read in place.
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace akr {

namespace {

constexpr int BM = 128;        // rows of D per CTA tile (UMMA M, one TMEM lane per row)
constexpr int BK = 32;         // fp32 per k-block: 128 bytes, one swizzle row
constexpr int UMMA_K = 8;      // k per tcgen05.mma kind::tf32
constexpr int CHUNK = 32;      // M/N elements per 128-byte row of an MN-major tile
constexpr int GROUP_M = 16;    // tile rasterisation: m-tiles per group (L2 reuse of B panels)
constexpr uint64_t DEFAULT_WAIT_LIMIT_NS = 4000000000ull;  // a wait longer than this aborts the kernel

// Timing experiments (skip the MMAs, skip the stores, force or forbid a kernel variant ...) are compiled in
// only with -DAKR_B200_DIAG; the shipped build keeps the five documented hooks of GemmDesc::debug and none
// of the experiment branches in its main loops.
#ifdef AKR_B200_DIAG
#define AKR_DIAG(flags, bit) (((flags) & (bit)) != 0)
#else
#define AKR_DIAG(flags, bit) false
#endif

struct KernelParams {
    CUtensorMap tmA, tmB;
    CUtensorMap tmC;           // output map for the TMA-store epilogue (valid when c_tma != 0)
    int c_tma;                 // 1: epilogue stores through TMA (aligned output, no accumulate, no split)
    float* C;
    const float* bias;
    // Second epilogue operand, an array of the output's shape with its own strides (aux_op != 0):
    // 1: C = alpha * AB + beta * aux, 2: C = alpha * AB * (1 - aux^2) (tanh' of a saved tanh output).
    const float* aux;
    long long aux_ld, aux_cs, aux_bs0, aux_bs1;
    int aux_op, aux_vec;
    float alpha, beta;
    float* partials;
    int* counters;
    int* status;
    float* colpart;  // [o0 * o1 * ceil(M / 32)][N] column sums per 32-row block of the output, or null
    long long ldc, c_bs0, c_bs1;
    int M, N, K;
    int o0, o1, red, splits;
    // Batch coordinates of the tensor maps: slot j of an operand's map takes (i1, i0, r, 0)[sel[j]].
    int a_sel[3], b_sel[3];
    // 1: the M/N-major operand's map is folded to (32, K, MN/32, ...) so that ONE box fetches the
    // whole tile (a box per 32-column chunk costs the TMA unit a fixed overhead per box).
    int a_fold, b_fold;
    int accumulate, vec_ok;
    int mt, nt, nkb, total_tiles;
    int debug;  // bit 0 = skip the TMA loads (MMA-only timing: the measured tensor-pipe ceiling),
                // bit 4 = the producer never signals a stage (exercises the bounded-wait abort path)
    unsigned long long wait_limit_ns;
};

struct Tile {
    int split, batch, i0, i1, m0, n0;
};

__device__ __forceinline__ Tile decode_tile(int t, const KernelParams& p, int bn, int bm = BM, int group_m = GROUP_M) {
    Tile c;
    c.split = t % p.splits;
    t /= p.splits;
    const int per_batch = p.mt * p.nt;
    c.batch = t / per_batch;
    const int r = t - c.batch * per_batch;
    c.i0 = c.batch / p.o1;
    c.i1 = c.batch - c.i0 * p.o1;
    const int group_sz = group_m * p.nt;
    const int g = r / group_sz;
    const int first_m = g * group_m;
    const int gm = min(p.mt - first_m, group_m);
    const int in = r - g * group_sz;
    const int n_t = in / gm;
    const int m_t = first_m + (in - n_t * gm);
    c.m0 = m_t * bm;
    c.n0 = n_t * bn;
    return c;
}

// Clock probe (debug bit 15): thread 0 of every CTA records the SM cycles (clock64) and the nanoseconds (%globaltimer)
// it spent between the end of the kernel's set-up and its teardown. Their ratio is the SM clock the kernel really ran
// at - under the power cap that, not the cycle count, decides how long a large product takes - and the cycle count
// can be set against the cycles the MMAs alone need. One predicate per CTA when the probe is off.
__device__ unsigned long long g_clock_probe[2 * 256];
#define AKR_DIAG_CLK_BEGIN                                                        \
    unsigned long long diag_c0 = 0, diag_t0 = 0;                                  \
    if ((p.debug & 32768) && threadIdx.x == 0) {                                  \
        diag_c0 = clock64();                                                      \
        diag_t0 = ptx::globaltimer_ns();                                          \
    }
#define AKR_DIAG_CLK_END                                                          \
    if ((p.debug & 32768) && threadIdx.x == 0 && blockIdx.x < 256) {              \
        g_clock_probe[2 * blockIdx.x] = clock64() - diag_c0;                      \
        g_clock_probe[2 * blockIdx.x + 1] = ptx::globaltimer_ns() - diag_t0;      \
    }

// One load stage holds the raw fp32 tiles of A and B as TMA delivers them, in every mode. The
// fp32-accurate mode keeps the derived low parts in a second, shorter ring of the same tile size (LO
// slots): a low-part tile only lives from its conversion to the end of its MMAs, so shared memory goes
// to raw stages - bytes in flight from HBM - rather than to a low copy per stage.
template <int BN, int TERMS, int BKT>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BKT * 4;
    static constexpr int B_BYTES = BN * BKT * 4;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};
constexpr int BAR_BYTES = 512;  // mbarriers + TMEM slot + flags behind the tiles

// 128-column slabs of a tile (a narrower tile is one slab) and the columns of one slab.
__host__ __device__ constexpr int slabs_of(int bn) { return bn >= 128 ? bn / 128 : 1; }
__host__ __device__ constexpr int slab_cols(int bn) { return bn >= 128 ? 128 : bn; }

// Threads of one CTA: producer warp, MMA warp and one epilogue warp per (TMEM lane quarter,
// 128-column slab of the tile).
// plus, in the fp32-accurate mode, the converter warps that derive the low parts in shared memory: two beside the
// eight epilogue warps of a 256-column tile, six (four) beside the four epilogue warps of a 64- (128-) column one -
// on an HBM-bound shape with a 64-column output two converter warps took 1190 cycles per 24 KB k-block with loads,
// MMAs and stores all switched off, more than the 1040 cycles its bytes take from HBM (512 products of 512 x 64 x 512:
// 0.158 ms with two, 0.146 with four, 0.137 with six, 0.143 with eight; 16384 x 128 x 4096: 0.110 ms with two, 0.098
// with four. Eight beside a 128-column tile - fourteen warps - never finished and is not to be tried again: at launch
// 448 threads x 144 registers leave the register file no room for the hand-over of setmaxnreg).
template <int BN, int TERMS = 1>
__host__ __device__ constexpr int conv_warps() {
    return TERMS == 3 ? (BN <= 64 ? 6 : (BN == 128 ? 4 : 2)) : 0;
}
template <int BN, int TERMS = 1>
constexpr int num_threads() { return 64 + slabs_of(BN) * 128 + conv_warps<BN, TERMS>() * 32; }

// Bytes of shared memory each epilogue warp uses to turn "one row per lane" into coalesced stores.
constexpr int EPI_STAGE_BYTES = 32 * 128;

// Stores a 32 x 32 block of the output held one row per lane (lane l: row row0 + l, columns
// col0 .. col0+31). The block goes through a swizzled shared-memory tile so that every store
// instruction writes 4 rows x 128 contiguous bytes instead of 32 rows x 16 bytes: with one row per
// lane the LSU touches 32 cache lines per instruction, which capped the output rate of the
// write-heavy (short-K, batched) products well below what HBM takes.
// Must be called by all 32 lanes. Optionally adds a bias row vector and / or the previous contents.
struct Epi {
    const float* bias;   // row vector added to every row, or null
    const float* aux;    // element (row, col) of the tile's matrix at aux[row * aux_ld + col * aux_cs]
    long long aux_ld, aux_cs;
    int op;              // 0: none, 1: += beta * aux, 2: *= 1 - aux^2
    float alpha, beta;
    bool accumulate, aux_vec;
    // Column sums of the stored values (the bias gradient of the Linear layer that produced the operand this
    // output is the gradient of): row (row0 / 32) of this [row blocks][N] array receives the sums over the 32
    // rows of each block; a small second kernel adds the rows up. Null: not wanted.
    float* colpart;
};

__device__ __forceinline__ Epi plain_epi() {
    Epi e;
    e.bias = nullptr; e.aux = nullptr; e.aux_ld = 0; e.aux_cs = 1; e.op = 0; e.alpha = 1.f; e.beta = 0.f;
    e.accumulate = false; e.aux_vec = false;
    e.colpart = nullptr;
    return e;
}

// For the kernels without the second-operand path: scaling, bias and `C +=` only.
__device__ __forceinline__ Epi lean_epi(const KernelParams& p) {
    Epi e = plain_epi();
    e.bias = p.bias;
    e.alpha = p.alpha;
    e.accumulate = p.accumulate != 0;
    return e;
}

__device__ __forceinline__ Epi tile_epi(const KernelParams& p, const Tile& c) {
    Epi e;
    e.bias = p.bias;
    e.op = p.aux_op;
    e.aux = p.aux_op ? p.aux + c.i0 * p.aux_bs0 + c.i1 * p.aux_bs1 : nullptr;
    e.aux_ld = p.aux_ld; e.aux_cs = p.aux_cs;
    e.alpha = p.alpha; e.beta = p.beta;
    e.accumulate = p.accumulate != 0;
    e.aux_vec = p.aux_vec != 0;
    // rows of the partial array: batch-major, then 32-row blocks of the matrix
    e.colpart = p.colpart ? p.colpart + (size_t)c.batch * (size_t)((p.M + 31) / 32) * (size_t)p.N : nullptr;
    return e;
}

// value = op(alpha * product + previous contents + bias): one element of the epilogue.
__device__ __forceinline__ float epi_aux(float v, float a, const Epi& e) {
    return e.op == 1 ? fmaf(e.beta, a, v) : v * (1.f - a * a);
}

// AUX = false (the fp32-accurate kernels, which have no registers to spare next to their promotion
// accumulators): the second-operand path is compiled out; the host applies it in a separate pass.
template <bool AUX>
__device__ __forceinline__ void store_block_warp(float (&v)[32], float4* stage, float* out_base,
                                                 long long ld, int row0, int M, int col0, int N, bool vec,
                                                 const Epi& e, int lane) {
    if (e.alpha != 1.f) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= e.alpha;
    }
    if (e.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) v[j] += __ldg(e.bias + col0 + j);
    }
    // lane's row -> 8 chunks of 16 bytes, chunk index XOR (row & 7): conflict-free both ways
#pragma unroll
    for (int j = 0; j < 8; ++j)
        stage[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    __syncwarp();
    // Phase 2: this lane owns rows row0 + 4 i + (lane >> 3), four columns from `col`.
    const int c4 = lane & 7;
    const int col = col0 + 4 * c4;
    const int rsub = lane >> 3;
    const bool fast = vec && col + 3 < N;
    float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);  // this lane's four columns summed over its eight rows
    if (!AUX || (e.op == 0 && !e.accumulate)) {
        float4 x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {  // all eight reads in flight before the first global store
            const int r = 4 * i + rsub;
            x[i] = stage[r * 8 + (c4 ^ (r & 7))];
        }
        if (AUX && e.colpart != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (row0 + 4 * i + rsub < M) { cs.x += x[i].x; cs.y += x[i].y; cs.z += x[i].z; cs.w += x[i].w; }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int grow = row0 + 4 * i + rsub;
            if (grow < M && col < N) {
                float* dst = out_base + (long long)grow * ld + col;
                if (fast) {
                    if (!AUX && e.accumulate) {
                        const float4 o = *reinterpret_cast<const float4*>(dst);
                        x[i].x += o.x; x[i].y += o.y; x[i].z += o.z; x[i].w += o.w;
                    }
                    *reinterpret_cast<float4*>(dst) = x[i];
                } else {
                    const float el[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                        if (col + t < N) dst[t] = (!AUX && e.accumulate) ? dst[t] + el[t] : el[t];
                }
            }
        }
    } else {
        // With a second operand and / or `C +=`: four rows at a time, their global loads issued together
        // ahead of the first use (one load per row followed by its use and store would be eight serial
        // round trips per block).
        const bool aux_fast = e.op != 0 && fast && e.aux_vec;
        const bool acc_fast = e.accumulate && fast;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
            float4 a[4], o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int grow = row0 + 4 * (4 * h + i) + rsub;
                if (aux_fast && grow < M) a[i] = *reinterpret_cast<const float4*>(e.aux + (long long)grow * e.aux_ld + col);
                if (acc_fast && grow < M) o[i] = *reinterpret_cast<const float4*>(out_base + (long long)grow * ld + col);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = 4 * (4 * h + i) + rsub;
                const int grow = row0 + r;
                float4 x = stage[r * 8 + (c4 ^ (r & 7))];
                if (grow < M && col < N) {
                    float* dst = out_base + (long long)grow * ld + col;
                    if (fast) {
                        if (e.accumulate) {
                            x.x += o[i].x; x.y += o[i].y; x.z += o[i].z; x.w += o[i].w;
                        }
                        if (e.op != 0) {
                            if (!aux_fast) {
                                const float* ap = e.aux + (long long)grow * e.aux_ld + (long long)col * e.aux_cs;
                                a[i] = make_float4(ap[0], ap[e.aux_cs], ap[2 * e.aux_cs], ap[3 * e.aux_cs]);
                            }
                            x.x = epi_aux(x.x, a[i].x, e); x.y = epi_aux(x.y, a[i].y, e);
                            x.z = epi_aux(x.z, a[i].z, e); x.w = epi_aux(x.w, a[i].w, e);
                        }
                        cs.x += x.x; cs.y += x.y; cs.z += x.z; cs.w += x.w;
                        *reinterpret_cast<float4*>(dst) = x;
                    } else {
                        const float el[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            if (col + t < N) {
                                float val = e.accumulate ? dst[t] + el[t] : el[t];
                                if (e.op != 0)
                                    val = epi_aux(val, e.aux[(long long)grow * e.aux_ld + (long long)(col + t) * e.aux_cs], e);
                                dst[t] = val;
                                if (t == 0) cs.x += val;
                                else if (t == 1) cs.y += val;
                                else if (t == 2) cs.z += val;
                                else cs.w += val;
                            }
                    }
                }
            }
        }
    }
    if (AUX && e.colpart != nullptr) {
        // lanes c4, c4 + 8, c4 + 16, c4 + 24 hold the same four columns for different rows
        cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 8); cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 8);
        cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 8); cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 8);
        cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 16); cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 16);
        cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 16); cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 16);
        if (lane < 8 && row0 < M) {
            float* dst = e.colpart + (size_t)(row0 >> 5) * (size_t)N + col;
            if (col < N) dst[0] = cs.x;
            if (col + 1 < N) dst[1] = cs.y;
            if (col + 2 < N) dst[2] = cs.z;
            if (col + 3 < N) dst[3] = cs.w;
        }
    }
    __syncwarp();  // the tile is reused by the next block
}

// TMA-store variant: the four warps of one 128-column slab stage their 32-row bands into one
// [128 rows][128 bytes] tile (the same swizzle the tensor map declares) and one thread sends it as a
// single 16 KB box. The warps are free again as soon as the box has been read from shared memory;
// the write itself drains asynchronously, clipped at the matrix edge by the hardware.
// Must be called by all 128 threads of the slab (named barrier `bar_id`).
// BUFS == 2: the caller alternates between two staging tiles per slab, and the issuer only waits for
// the box BEFORE the one it just sent, so staging a block overlaps the TMA unit reading the previous one.
template <int BUFS = 1>
__device__ __forceinline__ void store_block_tma(float (&v)[32], float4* my_tile, uint32_t slab_tile_addr,
                                                const CUtensorMap* tmC, int col0, int row_base, int i1, int i0,
                                                int N, const float* bias, int lane, bool issuer, int bar_id) {
    if (bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) v[j] += __ldg(bias + col0 + j);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
        my_tile[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    ptx::fence_proxy_async_smem();
    ptx::named_barrier_sync(bar_id, 128);
    if (issuer) {
        ptx::tma_store_4d(tmC, slab_tile_addr, col0, row_base, i1, i0);
        ptx::bulk_commit_group();
        if (BUFS == 2) ptx::bulk_wait_read_1();
        else ptx::bulk_wait_read_all();
    }
    ptx::named_barrier_sync(bar_id, 128);  // the (other) tile may be overwritten
}

// The same block into a staging tile that nothing else will use (the idle load stages behind a CTA's last tile):
// no wait for the store to have read it, no second barrier; the issuing thread waits for all its stores at the end.
__device__ __forceinline__ void store_block_tma_once(float (&v)[32], float4* my_tile, uint32_t slab_tile_addr,
                                                     const CUtensorMap* tmC, int col0, int row_base, int i1, int i0,
                                                     int N, const float* bias, int lane, bool issuer, int bar_id) {
    if (bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) v[j] += __ldg(bias + col0 + j);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
        my_tile[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    ptx::fence_proxy_async_smem();
    ptx::named_barrier_sync(bar_id, 128);
    if (issuer) {
        ptx::tma_store_4d(tmC, slab_tile_addr, col0, row_base, i1, i0);
        ptx::bulk_commit_group();
    }
}

// Per-warp variant for write-heavy short contractions: every epilogue warp stages its own 32 x 32 block
// (4 KB, same swizzle) and its lane 0 sends it as a box of 32 rows; no barrier between warps at all. The
// caller alternates between two staging tiles per warp; the lane waits for the box before the one it just
// sent. Needs an output map encoded with 32-row boxes.
__device__ __forceinline__ void store_block_tma_warp(float (&v)[32], float4* my_tile, uint32_t my_tile_addr,
                                                     const CUtensorMap* tmC, int col0, int row0, int i1, int i0, int N,
                                                     const float* bias, int lane) {
    if (bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) v[j] += __ldg(bias + col0 + j);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
        my_tile[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        ptx::tma_store_4d(tmC, my_tile_addr, col0, row0, i1, i0);
        ptx::bulk_commit_group();
        ptx::bulk_wait_read_1();
    }
    __syncwarp();  // the other staging tile of this warp may be overwritten
}

// KC > 0: the tensor core only accumulates KC k-blocks at a time; the epilogue warps add those
// partial tiles into fp32 registers with round-to-nearest. The accumulator inside the tensor core
// truncates on every add, which over a long contraction costs more accuracy than the fp32-accurate
// mode may lose, so that mode keeps the in-core chains short. KC == 0: one chain per output tile.
// BKT: fp32 per k-block. 32 = one 128-byte swizzle row per K-major tile row; 16 = 64-byte rows
// (64-byte swizzle), used by the fp32-accurate mode to have four finer stages in flight instead of
// two coarse ones (its stages carry hi and lo parts and are twice as large per k).
// Staging tiles per slab of the general kernel: two when shared memory has room for them.
template <int BN, int TERMS, int STAGES, int BKT, int LO = 0>
struct EpiBufs {
    static constexpr int value =
        ((STAGES + LO) * SmemLayout<BN, TERMS, BKT>::STAGE_BYTES + 2 * slabs_of(BN) * 4 * EPI_STAGE_BYTES + 2048 <= 232448)
            ? 2
            : 1;
};
// Instantiations for short, write-heavy contractions (few stages, two staging sets): every epilogue warp sends
// its own 32-row boxes, without a barrier between warps.
template <int BN, int TERMS, int STAGES, int BKT, int LO>
struct WarpStore {
    static constexpr bool value = EpiBufs<BN, TERMS, STAGES, BKT, LO>::value == 2 && BN == 256 &&
                                  ((TERMS == 1 && STAGES == 3) || (TERMS == 3 && STAGES == 4));
};

// LO: slots of the low-part ring (fp32-accurate mode; 0 in TF32 mode).
template <int BN, int MAJA, int MAJB, int TERMS, int STAGES, int KC, int BKT, int LO>
__global__ void __launch_bounds__(num_threads<BN, TERMS>(), 1)
gemm_tf32_kernel(const __grid_constant__ KernelParams p) {
    using L = SmemLayout<BN, TERMS, BKT>;
    // A k-block deeper than 32 is held as sub-tiles of 32 (a K-major row of the swizzled layout is 128 bytes): BKT = 64
    // gives the narrow TF32 tiles stages of eight MMAs (handing a stage over costs more than filling it).
    constexpr int SUB = BKT > 32 ? 32 : BKT;
    constexpr int SUBS = BKT / SUB;
    static_assert(SUBS == 1 || TERMS == 1, "sub-tiles are a TF32-mode layout");
    constexpr int A_SUB_BYTES = BM * SUB * 4, B_SUB_BYTES = BN * SUB * 4;
    constexpr int SLABS = slabs_of(BN);
    constexpr int SLAB_W = slab_cols(BN);
    constexpr int EPI_WARPS = SLABS * 4;
    constexpr int CONV_WARPS = conv_warps<BN, TERMS>();
    constexpr int CHUNK_ITERS = KC > 0 ? KC : 0x7fffffff;
    constexpr int TMEM_COLS = 2 * BN;  // two accumulators
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM allocation must be a power of two");
    static_assert((TERMS == 3) == (LO > 0), "the low-part ring exists exactly in the fp32-accurate mode");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;

    // [stages][epilogue staging: one 16 KB tile per 128-column slab (two where they fit: the TMA-store
    // epilogue then alternates between them), 1024-byte aligned][barriers]
    // [raw stages][low-part slots][epilogue staging ...][barriers]
    constexpr int EPI_BUFS = EpiBufs<BN, TERMS, STAGES, BKT, LO>::value;
    constexpr int EPI_BYTES = EPI_BUFS * SLABS * 4 * EPI_STAGE_BYTES;
    constexpr int TILE_BYTES = (STAGES + LO) * L::STAGE_BYTES;
    constexpr int LO_BASE = STAGES * L::STAGE_BYTES;
    uint8_t* epi_stage_base = smem + TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TILE_BYTES + EPI_BYTES);
    const uint32_t bar_base = smem_base + TILE_BYTES + EPI_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    auto conv_bar = [&](int l) { return bar_base + 8u * (2 * STAGES + 4 + l); };          // low parts written
    auto lofree_bar = [&](int l) { return bar_base + 8u * (2 * STAGES + 4 + LO + l); };   // low-part slot reusable
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + 2 * LO);
    static_assert((2 * STAGES + 4 + 2 * LO) * 8 + 16 <= BAR_BYTES, "barrier area too small");
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = reinterpret_cast<int*>(tmem_slot + 2);

    // `warp` is the role index: 0 producer, 1 MMA, 2 .. 2+EPI_WARPS-1 epilogue, then the converters. The
    // fp32-accurate 256- and 128-wide instantiations have more than eight warps, capped at 168 registers each unless
    // the epilogue warps (128 promotion accumulators per thread) sit in warpgroups of their own and take registers
    // the other warpgroups give back: there the first EPI_WARPS hardware warps are the epilogue, the next two the
    // producer and the MMA warp, the rest the converters.
    constexpr bool REMAP = TERMS == 3 && BN >= 128;
    const int hw_warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform for the compiler too
    const int warp = !REMAP ? hw_warp
                            : (hw_warp < EPI_WARPS ? hw_warp + 2 : (hw_warp < EPI_WARPS + 2 ? hw_warp - EPI_WARPS : hw_warp));
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int l = 0; l < LO; ++l) {
            ptx::mbar_init(conv_bar(l), CONV_WARPS > 0 ? CONV_WARPS : 1);
            ptx::mbar_init(lofree_bar(l), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), EPI_WARPS);
        }
        *abort_flag = 0;
        *last_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc<TMEM_COLS>(ptx::smem_u32(tmem_slot));
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up done (shared memory, tensor memory, barriers only). Let the next kernel of the stream begin its own
    // set-up on SMs this grid leaves, and do not touch global memory before the previous kernel has finished.
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    AKR_DIAG_CLK_BEGIN

    const int total_iters = p.red * p.nkb;  // contraction steps of one output tile

    if (warp < 2 || warp >= 2 + EPI_WARPS) {
    if (REMAP) ptx::reg_dealloc<96>();
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const Tile c = decode_tile(t, p, BN);
                const int it0 = (int)((long long)total_iters * c.split / p.splits);
                const int it1 = (int)((long long)total_iters * (c.split + 1) / p.splits);
                for (int it = it0; it < it1; ++it) {
                    const int r = it / p.nkb;
                    const int k0 = (it - r * p.nkb) * BKT;
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fb = full_bar(stage);
                    if (p.debug & 16) continue;  // test hook: nothing ever arrives, every waiter must give up
                    if (p.debug & 1) {
                        ptx::mbar_arrive(fb);
                        ++issued;
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    ptx::mbar_arrive_expect_tx(fb, L::STAGE_BYTES);
                    const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
                    const uint32_t sb = sa + L::A_BYTES;
                    const int bcv[4] = {c.i1, c.i0, r, 0};
                    const int a0 = bcv[p.a_sel[0]], a1 = bcv[p.a_sel[1]], a2 = bcv[p.a_sel[2]];
                    const int b0 = bcv[p.b_sel[0]], b1 = bcv[p.b_sel[1]], b2 = bcv[p.b_sel[2]];
#pragma unroll
                    for (int sub = 0; sub < SUBS; ++sub) {
                        // (a sub-tile that starts at or behind K is filled with zeros by the copy and still counts its bytes)
                        const CUtensorMap* ma = &p.tmA;
                        const CUtensorMap* mb = &p.tmB;
                        const uint32_t da = sa + sub * A_SUB_BYTES;
                        const uint32_t db = sb + sub * B_SUB_BYTES;
                        const int ks = k0 + sub * SUB;
                        if (MAJA == 0) {
                            ptx::tma_load_5d(da, ma, fb, ks, c.m0, a0, a1, a2);
                        } else if (p.a_fold) {
                            ptx::tma_load_5d(da, ma, fb, 0, ks, c.m0 / CHUNK, a0, a1);
                        } else {
#pragma unroll
                            for (int ch = 0; ch < BM / CHUNK; ++ch)
                                ptx::tma_load_5d(da + ch * (SUB * 128), ma, fb, c.m0 + ch * CHUNK, ks,
                                                 a0, a1, a2);
                        }
                        if (MAJB == 0) {
                            ptx::tma_load_5d(db, mb, fb, ks, c.n0, b0, b1, b2);
                        } else if (p.b_fold) {
                            ptx::tma_load_5d(db, mb, fb, 0, ks, c.n0 / CHUNK, b0, b1);
                        } else {
#pragma unroll
                            for (int ch = 0; ch < BN / CHUNK; ++ch)
                                ptx::tma_load_5d(db + ch * (SUB * 128), mb, fb, c.n0 + ch * CHUNK, ks,
                                                 b0, b1, b2);
                        }
                    }
                    ++issued;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || *abort_flag) {
                // Gave up: let the copies still in flight land before the CTA tears down.
                int s = stage;
                uint32_t ph = phase;
                const int n = issued < STAGES ? (int)issued : STAGES;
                for (int i = 0; i < n; ++i) {
                    if (--s < 0) {
                        s = STAGES - 1;
                        ph ^= 1u;
                    }
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(full_bar(s), ph)) {
                        if (ptx::globaltimer_ns() - t0 > 200000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // All 32 lanes run the loop (waits included); one elected lane issues the MMAs and commits. With a single
        // lane inside a divergent branch every operand of every tcgen05.mma is moved into uniform registers one by
        // one: 87 cycles of issue per MMA, more than a 128 x 128 x 8 MMA takes to execute.
        {
            const uint32_t issuer = ptx::elect_one();
            constexpr uint32_t IDESC = ptx::idesc_tf32(BM, BN, MAJA, MAJB);
            int stage = 0;
            uint32_t phase = 0;
            int lo_slot = 0;        // low-part ring position (fp32-accurate mode)
            uint32_t lo_phase = 0;
            int handoff = 0;  // accumulator hand-offs so far (one per chunk of the contraction)
            bool ok = true;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const Tile c = decode_tile(t, p, BN);
                const int it0 = (int)((long long)total_iters * c.split / p.splits);
                const int it1 = (int)((long long)total_iters * (c.split + 1) / p.splits);
                for (int cs = it0, ce = it0; cs < it1 && ok; cs = ce) {
                    ce = (it1 - cs > CHUNK_ITERS) ? cs + CHUNK_ITERS : it1;
                    const int buf = handoff & 1;
                    const uint32_t acc_phase = (handoff >> 1) & 1u;
                    if (!ptx::mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    for (int it = cs; it < ce; ++it) {
                        // fp32-accurate mode: the stage is ready once the converter warps wrote its low parts
                        // (they waited for the raw tiles themselves)
                        if (!ptx::mbar_wait(TERMS == 3 ? conv_bar(lo_slot) : full_bar(stage), TERMS == 3 ? lo_phase : phase,
                                            abort_flag, p.wait_limit_ns)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
                        const uint32_t sb = sa + L::A_BYTES;
                        const uint32_t sa_lo = smem_base + LO_BASE + lo_slot * L::STAGE_BYTES;
                        const uint32_t sb_lo = sa_lo + L::A_BYTES;
#pragma unroll
                        for (int k8s = 0; k8s < BKT / UMMA_K; ++k8s) {
                            const int sub = k8s / (SUB / UMMA_K), k8 = k8s % (SUB / UMMA_K);
                            // K-major: step 32 bytes inside the 128-byte swizzle row.
                            // MN-major: step 8 k-rows (two 4-row swizzle groups, 8 * 128 bytes).
                            const uint32_t a_off = sub * A_SUB_BYTES + (MAJA == 0 ? k8 * 32 : k8 * 1024);
                            const uint32_t b_off = sub * B_SUB_BYTES + (MAJB == 0 ? k8 * 32 : k8 * 1024);
                            // K-major rows are SUB * 4 bytes (128- or 64-byte swizzle), 8 rows per group.
                            constexpr uint32_t K_LAY = SUB == 32 ? ptx::LAYOUT_SW128 : ptx::LAYOUT_SW64;
                            constexpr uint32_t K_SBO = 8 * SUB * 4;
                            const uint32_t a_lbo = MAJA == 0 ? 16 : SUB * 128;
                            const uint32_t b_lbo = MAJB == 0 ? 16 : SUB * 128;
                            const uint32_t a_sbo = MAJA == 0 ? K_SBO : 512;
                            const uint32_t b_sbo = MAJB == 0 ? K_SBO : 512;
                            constexpr uint32_t a_lay = MAJA == 0 ? K_LAY : ptx::LAYOUT_SW128_ATOM32B;
                            constexpr uint32_t b_lay = MAJB == 0 ? K_LAY : ptx::LAYOUT_SW128_ATOM32B;
                            const uint64_t da = ptx::smem_desc(sa + a_off, a_lbo, a_sbo, a_lay);
                            const uint64_t db = ptx::smem_desc(sb + b_off, b_lbo, b_sbo, b_lay);
                            const uint32_t first = (it == cs && k8s == 0) ? 0u : 1u;
                            if (AKR_DIAG(p.debug, 2)) {
                                if (k8s == 0 && it == cs) ptx::mma_tf32_ss_elected(issuer, d_tmem, da, db, IDESC, 0u);
                            } else if (TERMS == 3) {
                                const uint64_t da_lo = ptx::smem_desc(sa_lo + a_off, a_lbo, a_sbo, a_lay);
                                const uint64_t db_lo = ptx::smem_desc(sb_lo + b_off, b_lbo, b_sbo, b_lay);
                                ptx::mma_tf32_ss_elected(issuer, d_tmem, da_lo, db, IDESC, first);
                                ptx::mma_tf32_ss_elected(issuer, d_tmem, da, db_lo, IDESC, 1u);
                                ptx::mma_tf32_ss_elected(issuer, d_tmem, da, db, IDESC, 1u);
                            } else {
                                ptx::mma_tf32_ss_elected(issuer, d_tmem, da, db, IDESC, first);
                            }
                        }
                        ptx::mma_commit_elected(issuer, empty_bar(stage));  // stage reusable once these MMAs finish
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        if (TERMS == 3) {
                            ptx::mma_commit_elected(issuer, lofree_bar(lo_slot));  // and so is the low-part slot
                            if (++lo_slot == LO) {
                                lo_slot = 0;
                                lo_phase ^= 1u;
                            }
                        }
                    }
                    if (ok) ptx::mma_commit_elected(issuer, tfull_bar(buf));  // this chunk's accumulator is complete
                    ++handoff;
                }
            }
        }
    } else if (CONV_WARPS > 0 && warp >= 2 + EPI_WARPS) {
        // ------------------------------------------------------------ low-part converter (fp32 mode)
        // The tensor core truncates an fp32 operand to TF32, so the raw tile already acts as the high
        // part trunc(x). These warps write lo = x - trunc(x) (exact in fp32) beside it, at the same
        // offset, so the swizzled tile layout is preserved without knowing it.
        const int ct = (warp - 2 - EPI_WARPS) * 32 + lane;
        constexpr int RAW_BYTES = L::STAGE_BYTES;
        constexpr int LOS = LO > 0 ? LO : 1;
        int stage = 0, lo_slot = 0;
        uint32_t phase = 0, lo_phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
            const Tile c = decode_tile(t, p, BN);
            const int it0 = (int)((long long)total_iters * c.split / p.splits);
            const int it1 = (int)((long long)total_iters * (c.split + 1) / p.splits);
            for (int it = it0; it < it1; ++it) {
                // the raw tiles have landed, and the MMAs that read this low-part slot last have finished
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_warp(full_bar(stage), phase, abort_flag, p.wait_limit_ns)) ||
                    !__all_sync(0xffffffffu, ptx::mbar_wait_warp(lofree_bar(lo_slot), lo_phase ^ 1u, abort_flag, p.wait_limit_ns))) {
                    ok = false;
                    break;
                }
                const float4* src = reinterpret_cast<const float4*>(smem + stage * L::STAGE_BYTES);
                float4* dst = reinterpret_cast<float4*>(smem + LO_BASE + lo_slot * L::STAGE_BYTES);
                constexpr int PER_THREAD = RAW_BYTES / 16 / (CONV_WARPS > 0 ? CONV_WARPS * 32 : 1);
                constexpr int BATCH = PER_THREAD % 8 == 0 ? 8 : (PER_THREAD % 6 == 0 ? 6 : 4);  // loads in flight per thread
                static_assert(PER_THREAD % BATCH == 0 || CONV_WARPS == 0, "converter work must divide evenly");
#pragma unroll 1
                for (int b0 = 0; b0 < PER_THREAD; b0 += BATCH) {
                    float4 x[BATCH];
#pragma unroll
                    for (int u = 0; u < BATCH; ++u) x[u] = src[(b0 + u) * (CONV_WARPS * 32) + ct];
#pragma unroll
                    for (int u = 0; u < BATCH; ++u) {
                        x[u].x -= __uint_as_float(__float_as_uint(x[u].x) & 0xffffe000u);
                        x[u].y -= __uint_as_float(__float_as_uint(x[u].y) & 0xffffe000u);
                        x[u].z -= __uint_as_float(__float_as_uint(x[u].z) & 0xffffe000u);
                        x[u].w -= __uint_as_float(__float_as_uint(x[u].w) & 0xffffe000u);
                        dst[(b0 + u) * (CONV_WARPS * 32) + ct] = x[u];
                    }
                }
                ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(conv_bar(lo_slot));
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
                if (++lo_slot == LOS) {
                    lo_slot = 0;
                    lo_phase ^= 1u;
                }
            }
        }
    }
    } else {
        if (REMAP) ptx::reg_alloc<200>();
        // ------------------------------------------------------------ epilogue (roles 2 ..)
        const int q = hw_warp & 3;          // TMEM lane quarter this hardware warp may read
        const int slab = (warp - 2) >> 2;   // which 128-column slab of the tile
        const int nbatch = p.o0 * p.o1;
        const bool split_mode = p.splits > 1;
        float4* my_stage = reinterpret_cast<float4*>(epi_stage_base + (slab * 4 + q) * EPI_STAGE_BYTES);
        const uint32_t slab_tile_addr = smem_base + TILE_BYTES + slab * 4 * EPI_STAGE_BYTES;
        constexpr int EPI_ALT = SLABS * 4 * EPI_STAGE_BYTES;  // offset of the second set of staging tiles
        int epi_buf = 0;                                           // which set the next TMA-store block uses
        // three-stage instantiation (short, write-heavy contractions): every warp sends its own 32-row boxes
        constexpr bool WARP_STORE = WarpStore<BN, TERMS, STAGES, BKT, LO>::value;
        const uint32_t my_stage_addr = smem_base + TILE_BYTES + (slab * 4 + q) * EPI_STAGE_BYTES;
        const bool use_tma = p.c_tma != 0 && !split_mode;  // kernel-uniform
        int handoff = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
            const Tile c = decode_tile(t, p, BN);
            const int it0 = (int)((long long)total_iters * c.split / p.splits);
            const int it1 = (int)((long long)total_iters * (c.split + 1) / p.splits);
            const int row0 = c.m0 + q * 32;   // first row of this warp's 32-row band
            // Behind a CTA's last tile the load stages are idle (no later tile to prefetch, every MMA that read them
            // has completed once the accumulator is): each 32-column block of the tile gets a staging tile of its
            // own there, and the epilogue no longer waits block by block for a store to have read the one tile per
            // slab (7.7 of the 55 kilocycles of a 2048^3 product, one tile per CTA, were that chain).
            const bool ring_free = TERMS == 1 && !WARP_STORE && t + (int)gridDim.x >= p.total_tiles &&
                                   SLABS * (SLAB_W / 32) * 4 * EPI_STAGE_BYTES <= TILE_BYTES;
            float* out_base;
            long long out_ld;
            bool vec;
            if (split_mode) {
                out_base = p.partials + ((size_t)c.split * nbatch + c.batch) * (size_t)p.M * (size_t)p.N;
                out_ld = p.N;
                vec = (p.N & 3) == 0;
            } else {
                out_base = p.C + c.i0 * p.c_bs0 + c.i1 * p.c_bs1;
                out_ld = p.ldc;
                vec = p.vec_ok != 0;
            }
            const float* bias = split_mode ? nullptr : p.bias;
            const int slab_col0 = c.n0 + slab * 128;

            constexpr int ACC_N = KC > 0 ? SLAB_W : 1;  // fp32 promotion registers (unused without chains)
            float acc[ACC_N];
#pragma unroll
            for (int j = 0; j < ACC_N; ++j) acc[j] = 0.f;
            for (int cs = it0; cs < it1 && ok; cs = (it1 - cs > CHUNK_ITERS) ? cs + CHUNK_ITERS : it1) {
                const int buf = handoff & 1;
                const uint32_t acc_phase = (handoff >> 1) & 1u;
                bool got = __all_sync(0xffffffffu, ptx::mbar_wait_warp(tfull_bar(buf), acc_phase, abort_flag, p.wait_limit_ns));
                // the slab-wide TMA-store path synchronises the four warps of a slab: they must leave together
                if (use_tma && !WARP_STORE) got = ptx::named_barrier_and(2 + slab, 128, got);
                if (!got) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * BN + slab * 128;
#pragma unroll
                for (int ch = 0; ch < SLAB_W / 32; ++ch) {
                    const int col0 = slab_col0 + ch * 32;
                    if (col0 < p.N) {  // warp-uniform
                        __syncwarp();  // tcgen05.ld needs the whole warp converged
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(t_row + ch * 32, v);
                        ptx::tmem_ld_wait();
                        if (KC > 0) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) acc[ACC_N > 1 ? ch * 32 + j : 0] += __uint_as_float(v[j]);
                        } else {
                            float f[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                            if (AKR_DIAG(p.debug, 128)) {
                                // bit 7: timing experiment without the output stores
                            } else if (use_tma && WARP_STORE) {
                                store_block_tma_warp(f, my_stage + epi_buf * (EPI_ALT / 16), my_stage_addr + epi_buf * EPI_ALT,
                                                     &p.tmC, col0, row0, c.i1, c.i0, p.N, bias, lane);
                                epi_buf ^= 1;
                            } else if (use_tma && ring_free) {
                                // one staging tile of its own per 32-column block, in the load stages
                                const uint32_t off = (uint32_t)((slab * (SLAB_W / 32) + ch) * 4 * EPI_STAGE_BYTES);
                                store_block_tma_once(f, reinterpret_cast<float4*>(smem + off + q * EPI_STAGE_BYTES), smem_base + off,
                                                     &p.tmC, col0, c.m0, c.i1, c.i0, p.N, bias, lane, q == 0 && lane == 0, 2 + slab);
                            } else if (use_tma) {
                                store_block_tma<EPI_BUFS>(f, my_stage + epi_buf * (EPI_ALT / 16), slab_tile_addr + epi_buf * EPI_ALT,
                                                          &p.tmC, col0, c.m0, c.i1, c.i0, p.N, bias, lane,
                                                          q == 0 && lane == 0, 2 + slab);
                                if (EPI_BUFS == 2) epi_buf ^= 1;
                            } else {
                                store_block_warp<TERMS == 1>(f, my_stage, out_base, out_ld, row0, p.M, col0, p.N, vec,
                                                             split_mode ? plain_epi() : (TERMS == 1 ? tile_epi(p, c) : lean_epi(p)), lane);
                            }
                        }
                    }
                }
                // Accumulator drained: hand the TMEM buffer back to the MMA warp.
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
                ++handoff;
            }
            if (KC > 0 && ok) {
#pragma unroll
                for (int ch = 0; ch < SLAB_W / 32; ++ch) {
                    const int col0 = slab_col0 + ch * 32;
                    if (col0 < p.N) {
                        float f[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = acc[ACC_N > 1 ? ch * 32 + j : 0];
                        if (use_tma && WARP_STORE) {
                            store_block_tma_warp(f, my_stage + epi_buf * (EPI_ALT / 16), my_stage_addr + epi_buf * EPI_ALT,
                                                 &p.tmC, col0, row0, c.i1, c.i0, p.N, bias, lane);
                            epi_buf ^= 1;
                        } else if (use_tma) {
                            store_block_tma<EPI_BUFS>(f, my_stage + epi_buf * (EPI_ALT / 16), slab_tile_addr + epi_buf * EPI_ALT,
                                                      &p.tmC, col0, c.m0, c.i1, c.i0, p.N, bias, lane, q == 0 && lane == 0,
                                                      2 + slab);
                            if (EPI_BUFS == 2) epi_buf ^= 1;
                        } else {
                            store_block_warp<TERMS == 1>(f, my_stage, out_base, out_ld, row0, p.M, col0, p.N, vec,
                                                         split_mode ? plain_epi() : (TERMS == 1 ? tile_epi(p, c) : lean_epi(p)), lane);
                        }
                    }
                }
            }

            if (split_mode && ok && p.counters != nullptr) {
                // Single-launch variant (caller gave tile counters): the last CTA to finish this tile adds the
                // partials in split order (deterministic). Without counters a second kernel adds them up.
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                const int tile_id = (t / p.splits);
                if (threadIdx.x == 64) {
                    const int prev = atomicAdd(p.counters + tile_id, 1);
                    const int last = (prev == p.splits - 1) ? 1 : 0;
                    if (last) p.counters[tile_id] = 0;  // self-cleaning for the next launch
                    *last_flag = last;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                const int is_last = *last_flag;
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                if (is_last) {
                    // Lanes run along the columns (4 each) so that every load and store of the 32-row
                    // band is a contiguous 512-byte row segment.
                    __threadfence();
                    const size_t split_stride = (size_t)nbatch * p.M * p.N;
                    const float* pbase = p.partials + (size_t)c.batch * p.M * (size_t)p.N;
                    float* cbase = p.C + c.i0 * p.c_bs0 + c.i1 * p.c_bs1;
                    const int col = slab_col0 + lane * 4;
                    const bool pvec = (p.N & 3) == 0;
                    const bool cvec = p.vec_ok != 0;
                    // Four rows at a time, their loads issued together and the split loop unrolled: the sums
                    // of a row depend on each other, the loads do not (one row and one split at a time was
                    // a chain of dependent L2 round trips: 87 us for a 512 x 512 x 4096 product).
                    for (int r0 = 0; r0 < 32; r0 += 4) {
                        if (row0 + r0 >= p.M) break;
                        if (col >= p.N) continue;
                        const int nv = min(4, p.N - col);
                        float sum[4][4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int e = 0; e < 4; ++e) sum[u][e] = 0.f;
                        const float* prow = pbase + (size_t)(row0 + r0) * p.N + col;
                        if (pvec && nv == 4) {
#pragma unroll 4
                            for (int sp = 0; sp < p.splits; ++sp) {
                                float4 x[4];
#pragma unroll
                                for (int u = 0; u < 4; ++u)
                                    x[u] = (row0 + r0 + u < p.M)
                                               ? __ldcg(reinterpret_cast<const float4*>(prow + (size_t)sp * split_stride + (size_t)u * p.N))
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    sum[u][0] += x[u].x; sum[u][1] += x[u].y; sum[u][2] += x[u].z; sum[u][3] += x[u].w;
                                }
                            }
                        } else {
                            for (int sp = 0; sp < p.splits; ++sp)
#pragma unroll
                                for (int u = 0; u < 4; ++u)
                                    if (row0 + r0 + u < p.M)
                                        for (int e = 0; e < nv; ++e)
                                            sum[u][e] += __ldcg(prow + (size_t)sp * split_stride + (size_t)u * p.N + e);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int grow = row0 + r0 + u;
                            if (grow >= p.M) break;
                            float* dst = cbase + (long long)grow * p.ldc + col;
                            for (int e = 0; e < nv; ++e) {
                                float v = sum[u][e] * p.alpha;
                                if (p.bias != nullptr) v += __ldg(p.bias + col + e);
                                if (p.accumulate) v += dst[e];
                                if (TERMS == 1 && p.aux_op != 0) {
                                    const float a = p.aux[c.i0 * p.aux_bs0 + c.i1 * p.aux_bs1 + (long long)grow * p.aux_ld +
                                                          (long long)(col + e) * p.aux_cs];
                                    v = p.aux_op == 1 ? fmaf(p.beta, a, v) : v * (1.f - a * a);
                                }
                                sum[u][e] = v;
                            }
                            if (cvec && nv == 4) {
                                *reinterpret_cast<float4*>(dst) = make_float4(sum[u][0], sum[u][1], sum[u][2], sum[u][3]);
                            } else {
                                for (int e = 0; e < nv; ++e) dst[e] = sum[u][e];
                            }
                        }
                    }
                }
            }
        }
    }

    // the threads that issued bulk stores wait until the copies have read their shared-memory tiles before the CTA
    // winds down (the writes themselves complete with the grid; waiting for them here cost about 2 kilocycles per CTA)
    if (p.c_tma != 0 && warp >= 2 && warp < 2 + EPI_WARPS && lane == 0 &&
        (WarpStore<BN, TERMS, STAGES, BKT, LO>::value || (hw_warp & 3) == 0))
        ptx::bulk_wait_read_all();

    // ------------------------------------------------------------ teardown (all paths)
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc<TMEM_COLS>(tmem_base);
    }
    AKR_DIAG_CLK_END
    if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, 1);
}


// ---------------------------------------------------------------------------------- 256 x 256 tiles (diagnostic builds)
// The first TF32 kernel for large products, kept as the reference the 512 x 256 pair tiles are measured against:
// one CTA computes a 256 x 256 tile as two 128 x 256 accumulators
// that share the B tile in shared memory. Per flop it pulls one third fewer bytes from L2 than the
// 128 x 256 kernel above, whose speed is set by the L2 -> SM load rate rather than by the MMA pipe.
// Both accumulators fill all 512 TMEM columns, so a tile's MMAs may only start on an accumulator
// once the epilogue has drained it: one short stall per tile, amortised over a long contraction.
// No split-K and no fp32 promotion here; those stay with the general kernel.
// BKT = fp32 per k-block: 192 KB of load stages either way, as 3 x 64 KB (BKT = 32, the shipped form) or 6 x 32 KB
// (BKT = 16, diagnostic builds: twice as many stage hand-overs made 8192^3 16 % slower, 1.60 against 1.38 ms).
constexpr int BIG_BM = 256, BIG_BN = 256;  // (also the tile count the routing of the pair tiles is stated in)

#ifdef AKR_B200_DIAG
constexpr int BIG_RING_BYTES = 192 * 1024;
constexpr int BIG_THREADS = 64 + 256;
constexpr int BIG_SMEM = BIG_RING_BYTES + 1024 + 256 + 8 * EPI_STAGE_BYTES;

template <int MAJA, int MAJB, int BKT>
__global__ void __launch_bounds__(BIG_THREADS, 1)
gemm_tf32_big_kernel(const __grid_constant__ KernelParams p) {
    constexpr int BIG_A_BYTES = BIG_BM * BKT * 4, BIG_B_BYTES = BIG_BN * BKT * 4;
    constexpr int BIG_STAGE_BYTES = BIG_A_BYTES + BIG_B_BYTES;
    constexpr int BIG_STAGES = BIG_RING_BYTES / BIG_STAGE_BYTES;
    static_assert((2 * BIG_STAGES + 3) * 8 + 8 <= 256, "barrier area");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    constexpr int EPI_BYTES = 8 * EPI_STAGE_BYTES;  // staging (1024-byte aligned) before the barriers
    uint8_t* epi_stage_base = smem + BIG_STAGES * BIG_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BIG_STAGES * BIG_STAGE_BYTES + EPI_BYTES);
    const uint32_t bar_base = smem_base + BIG_STAGES * BIG_STAGE_BYTES + EPI_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (BIG_STAGES + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * BIG_STAGES);
    auto tempty_bar = [&](int h) { return bar_base + 8u * (2 * BIG_STAGES + 1 + h); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * BIG_STAGES + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform for the compiler too
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < BIG_STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(tfull_bar, 1);
        ptx::mbar_init(tempty_bar(0), 8);
        ptx::mbar_init(tempty_bar(1), 8);
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc<512>(ptx::smem_u32(tmem_slot));
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up done (shared memory, tensor memory, barriers only). Let the next kernel of the stream begin its own
    // set-up on SMs this grid leaves, and do not touch global memory before the previous kernel has finished.
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    AKR_DIAG_CLK_BEGIN
    const int total_iters = p.red * p.nkb;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const Tile c = decode_tile(t, p, BIG_BN, BIG_BM);
                for (int it = 0; it < total_iters; ++it) {
                    const int r = it / p.nkb;
                    const int k0 = (it - r * p.nkb) * BKT;
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fb = full_bar(stage);
                    if (p.debug & 16) continue;  // test hook: nothing ever arrives, every waiter must give up
                    if (p.debug & 1) {           // MMA-only timing: no loads, stale shared memory
                        ptx::mbar_arrive(fb);
                        ++issued;
                        if (++stage == BIG_STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    ptx::mbar_arrive_expect_tx(fb, BIG_STAGE_BYTES);
                    const uint32_t da = smem_base + stage * BIG_STAGE_BYTES;
                    const uint32_t db = da + BIG_A_BYTES;
                    const int bcv[4] = {c.i1, c.i0, r, 0};
                    const int a0 = bcv[p.a_sel[0]], a1 = bcv[p.a_sel[1]], a2 = bcv[p.a_sel[2]];
                    const int b0 = bcv[p.b_sel[0]], b1 = bcv[p.b_sel[1]], b2 = bcv[p.b_sel[2]];
                    if (MAJA == 0) {
                        ptx::tma_load_5d(da, &p.tmA, fb, k0, c.m0, a0, a1, a2);
                    } else if (p.a_fold) {
                        ptx::tma_load_5d(da, &p.tmA, fb, 0, k0, c.m0 / CHUNK, a0, a1);
                    } else {
#pragma unroll
                        for (int ch = 0; ch < BIG_BM / CHUNK; ++ch)
                            ptx::tma_load_5d(da + ch * (BKT * 128), &p.tmA, fb, c.m0 + ch * CHUNK, k0, a0, a1, a2);
                    }
                    if (MAJB == 0) {
                        ptx::tma_load_5d(db, &p.tmB, fb, k0, c.n0, b0, b1, b2);
                    } else if (p.b_fold) {
                        ptx::tma_load_5d(db, &p.tmB, fb, 0, k0, c.n0 / CHUNK, b0, b1);
                    } else {
#pragma unroll
                        for (int ch = 0; ch < BIG_BN / CHUNK; ++ch)
                            ptx::tma_load_5d(db + ch * (BKT * 128), &p.tmB, fb, c.n0 + ch * CHUNK, k0, b0, b1, b2);
                    }
                    ++issued;
                    if (++stage == BIG_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || *abort_flag) {
                // Gave up: let the copies still in flight land before the CTA tears down.
                int s = stage;
                uint32_t ph = phase;
                const int n = issued < BIG_STAGES ? (int)issued : BIG_STAGES;
                for (int i = 0; i < n; ++i) {
                    if (--s < 0) {
                        s = BIG_STAGES - 1;
                        ph ^= 1u;
                    }
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(full_bar(s), ph)) {
                        if (ptx::globaltimer_ns() - t0 > 200000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        {  // all 32 lanes run the loop, one elected lane issues (see the general kernel)
            const uint32_t issuer = ptx::elect_one();
            constexpr uint32_t IDESC = ptx::idesc_tf32(BM, BIG_BN, MAJA, MAJB);
            // K-major rows are BKT * 4 bytes (128- or 64-byte swizzle), 8 rows per group
            constexpr uint32_t K_LAY = BKT == 32 ? ptx::LAYOUT_SW128 : ptx::LAYOUT_SW64;
            constexpr uint32_t a_lay = MAJA == 0 ? K_LAY : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t b_lay = MAJB == 0 ? K_LAY : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t a_lbo = MAJA == 0 ? 16 : BKT * 128, b_lbo = MAJB == 0 ? 16 : BKT * 128;
            constexpr uint32_t a_sbo = MAJA == 0 ? 8 * BKT * 4 : 512, b_sbo = MAJB == 0 ? 8 * BKT * 4 : 512;
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++local) {
                const uint32_t tile_par = local & 1u;
                for (int it = 0; it < total_iters && ok; ++it) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = smem_base + stage * BIG_STAGE_BYTES;
                    const uint32_t sb = sa + BIG_A_BYTES;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (it == 0) {
                            // accumulator h must have been drained by the epilogue of the previous tile
                            if (!ptx::mbar_wait(tempty_bar(h), tile_par ^ 1u, abort_flag, p.wait_limit_ns)) {
                                ok = false;
                                break;
                            }
                            ptx::tc_fence_after();
                        }
                        // rows h*128.. of the A tile: 128 rows x 128 B (K-major) or 4 chunks x 4 KB
                        const uint32_t sa_h = sa + h * (BM * BKT * 4);
                        const uint32_t d_tmem = tmem_base + h * BIG_BN;
#pragma unroll
                        for (int k8 = 0; k8 < BKT / UMMA_K; ++k8) {
                            const uint32_t a_off = MAJA == 0 ? k8 * 32 : k8 * 1024;
                            const uint32_t b_off = MAJB == 0 ? k8 * 32 : k8 * 1024;
                            const uint64_t da = ptx::smem_desc(sa_h + a_off, a_lbo, a_sbo, a_lay);
                            const uint64_t db = ptx::smem_desc(sb + b_off, b_lbo, b_sbo, b_lay);
                            if (AKR_DIAG(p.debug, 2)) {  // timing experiment: loads and hand-shakes only
                                if (it == 0 && k8 == 0) ptx::mma_tf32_ss_elected(issuer, d_tmem, da, db, IDESC, 0u);
                                continue;
                            }
                            ptx::mma_tf32_ss_elected(issuer, d_tmem, da, db, IDESC, (it == 0 && k8 == 0) ? 0u : 1u);
                        }
                    }
                    if (!ok) break;
                    ptx::mma_commit_elected(issuer, empty_bar(stage));
                    if (++stage == BIG_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::mma_commit_elected(issuer, tfull_bar);  // both accumulators complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int slab = (warp - 2) >> 2;  // 128-column slab of the tile
        const bool vec = p.vec_ok != 0;
        const bool use_tma = p.c_tma != 0;
        float4* my_stage = reinterpret_cast<float4*>(epi_stage_base + (slab * 4 + q) * EPI_STAGE_BYTES);
        const uint32_t slab_tile_addr = smem_base + BIG_STAGES * BIG_STAGE_BYTES + slab * 4 * EPI_STAGE_BYTES;
        int local = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++local) {
            const Tile c = decode_tile(t, p, BIG_BN, BIG_BM);
            const Epi epi = tile_epi(p, c);
            const bool ring_free = t + (int)gridDim.x >= p.total_tiles;  // no later tile of this CTA is being prefetched
            bool got = __all_sync(0xffffffffu, ptx::mbar_wait_warp(tfull_bar, local & 1u, abort_flag, p.wait_limit_ns));
            if (use_tma) got = ptx::named_barrier_and(2 + slab, 128, got);  // a slab's four warps leave together
            if (!got) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const int slab_col0 = c.n0 + slab * 128;
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const int row0 = c.m0 + h * 128 + q * 32;
                float* out_base = p.C + c.i0 * p.c_bs0 + c.i1 * p.c_bs1;
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + h * BIG_BN + slab * 128;
                if (c.m0 + h * 128 < p.M) {  // warp-uniform: skip a half that lies below the matrix
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        const int col0 = slab_col0 + ch * 32;
                        if (col0 < p.N) {
                            __syncwarp();
                            uint32_t v[32];
                            ptx::tmem_ld_32x32(t_row + ch * 32, v);
                            ptx::tmem_ld_wait();
                            float f[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                            if (use_tma && ring_free && h * 4 + ch < 6) {
                                // behind the CTA's last tile the load stages are idle: six of a slab's eight blocks
                                // get a staging tile of their own there and are stored without waiting in between
                                const uint32_t off = (uint32_t)((slab * 6 + h * 4 + ch) * 4 * EPI_STAGE_BYTES);
                                store_block_tma_once(f, reinterpret_cast<float4*>(smem + off + q * EPI_STAGE_BYTES), smem_base + off,
                                                     &p.tmC, col0, c.m0 + h * 128, c.i1, c.i0, p.N, p.bias, lane,
                                                     q == 0 && lane == 0, 2 + slab);
                            } else if (use_tma)
                                store_block_tma(f, my_stage, slab_tile_addr, &p.tmC, col0, c.m0 + h * 128, c.i1, c.i0, p.N,
                                                p.bias, lane, q == 0 && lane == 0, 2 + slab);
                            else
                                store_block_warp<true>(f, my_stage, out_base, p.ldc, row0, p.M, col0, p.N, vec, epi, lane);
                        }
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tempty_bar(h));
            }
        }
    }

    if (p.c_tma != 0 && warp >= 2 && (warp & 3) == 0 && lane == 0) ptx::bulk_wait_read_all();
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc<512>(tmem_base);
    }
    AKR_DIAG_CLK_END
    if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, 1);
}
#endif  // AKR_B200_DIAG


// ---------------------------------------------------------------------------------- CTA pairs, fp32-accurate mode
// The 3xTF32 mode issues three MMAs per k-slice, each re-reading its operands from shared memory;
// with one CTA per tile that traffic (plus the low-part conversion) exceeds what shared memory
// delivers and bounds the mode. Here two CTAs of a cluster share one 256 x 256 tile through
// tcgen05.mma.cta_group::2: each holds 128 rows of A and 128 columns of B, so every MMA reads a
// third less per CTA, and each CTA loads (and converts) only its own share. No multicast copies.
//   leader = cluster rank 0: issues the MMAs and owns the barriers the pair synchronises on.
//   per CTA: warp 0 TMA producer (local barriers), warp 1 MMA (leader) + TMEM, warps 2..9 epilogue
//   with fp32 promotion of 64-deep chains, warps 10..11 low-part converters that also tell the leader
//   when this CTA's low parts are written (the peer with an arrive on the leader's barrier whose release is
//   CTA-scoped: its payload never crosses the cluster through memory - each CTA's tensor core reads its own
//   tiles, made visible to it by the converter's fence.proxy.async).
// 32-deep k-blocks (128-byte rows of the K-major tiles): with 16-deep ones the TMA unit moves twice as many rows per
// byte and every stage hand-over crosses the cluster twice as often (8192^3: 275 -> 287 TFLOP/s, 2048^3: 234 -> 256).
constexpr int PAIR_BM = 256, PAIR_BN = 256, PAIR_BK = 32, PAIR_KC = 64 / PAIR_BK;
constexpr int PAIR_A_BYTES = 128 * PAIR_BK * 4, PAIR_B_BYTES = 128 * PAIR_BK * 4;
constexpr int PAIR_RAW_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
// The tiles are laid out as PAIR_RAW_STAGES raw stages followed by LS low-part slots (32 KB each): a low-part tile
// only lives from its conversion to the end of its MMAs, but a slot's round trip crosses the cluster twice (the peer's
// "written" arrive, the leader's commit back). LS = 3 and one set of output staging tiles for long contractions;
// LS = 2 and two sets (staging a box overlaps the TMA unit reading the one before) for short ones, where the output
// is a large share of the bytes: 8192 products of 256^3 1.44 -> 1.37 ms, 8192^3 280 -> 275 TFLOP/s the other way.
constexpr int PAIR_RAW_STAGES = 96 / PAIR_BK;
constexpr int PAIR_SMEM_TILES = 7 * PAIR_RAW_BYTES;  // raw stages + low-part slots + staging sets, either way
constexpr int PAIR_BAR_BYTES = 512;  // 32 mbarriers + TMEM slot + flags
constexpr int PAIR_THREADS = 64 + 256 + 64;
constexpr int PAIR_EPI_WARPS = 8, PAIR_CONV_WARPS = 2;

template <int MAJA, int MAJB, int PAIR_LO_SLOTS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_tf32_pair_kernel(const __grid_constant__ KernelParams p) {
    constexpr int PAIR_EPI_SETS = PAIR_LO_SLOTS == 2 ? 2 : 1;
    static_assert((PAIR_RAW_STAGES + PAIR_LO_SLOTS) * PAIR_RAW_BYTES + PAIR_EPI_SETS * PAIR_EPI_WARPS * EPI_STAGE_BYTES == PAIR_SMEM_TILES,
                  "both layouts fill the same shared memory");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    constexpr int S = PAIR_RAW_STAGES;   // raw stages
    constexpr int LS = PAIR_LO_SLOTS;    // low-part slots
    constexpr int TILE_BYTES = (S + LS) * PAIR_RAW_BYTES;
    constexpr int LO_BASE = S * PAIR_RAW_BYTES;
    constexpr int stage_bytes = PAIR_RAW_BYTES;
    // [raw stages][low-part slots][staging: two slabs of 128 rows x 128 bytes, 1024-byte aligned][barriers]
    constexpr int STAGING_BYTES = PAIR_EPI_SETS * PAIR_EPI_WARPS * EPI_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TILE_BYTES + STAGING_BYTES);
    const uint32_t bar_base = smem_base + TILE_BYTES + STAGING_BYTES;
    auto landed_bar = [&](int s) { return bar_base + 8u * s; };            // local: this CTA's TMA tiles arrived (0..7)
    auto empty_bar = [&](int s) { return bar_base + 8u * (8 + s); };       // local: stage may be refilled (8..15)
    // leader: the low parts of both CTAs are written, per low-part slot (16..21)
    auto ready_bar = [&](int s) { return bar_base + 8u * (16 + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (22 + b); };      // local: accumulator chain done
    auto tempty_bar = [&](int b) { return bar_base + 8u * (24 + b); };     // leader: both epilogues drained
    auto lofree_bar = [&](int l) { return bar_base + 8u * (26 + l); };     // local: low-part slot may be rewritten (26..31)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* epi_stage_base = smem + TILE_BYTES;

    // Roles by hardware warp: 0..7 epilogue, 8 producer, 9 MMA, 10..11 converters, so that the two epilogue
    // warpgroups can take the registers the third one gives back. `warp` is the role index used below
    // (0 producer, 1 MMA, 2..9 epilogue, 10..11 converters).
    const int hw_warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform for the compiler too
    const int warp = hw_warp < 8 ? hw_warp + 2 : (hw_warp < 10 ? hw_warp - 8 : hw_warp);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 8; ++s) {
            ptx::mbar_init(landed_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        // the converter warps of both CTAs arrive here (the peer's directly on the leader's barrier)
        for (int s = 0; s < 6; ++s) ptx::mbar_init(ready_bar(s), 2 * PAIR_CONV_WARPS);
        for (int l = 0; l < LS; ++l) ptx::mbar_init(lofree_bar(l), 1);
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), 2 * PAIR_EPI_WARPS);
        }
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
        if (p.c_tma) ptx::prefetch_tensormap(&p.tmC);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair<512>(ptx::smem_u32(tmem_slot));
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up done (shared memory, tensor memory, barriers only). Let the next kernel of the stream begin its own
    // set-up on SMs this grid leaves, and do not touch global memory before the previous kernel has finished.
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    AKR_DIAG_CLK_BEGIN
    const int total_iters = p.red * p.nkb;
    // A split contraction gives every tile-split its share [first, first + count) of the (summed batch, k) steps.
    auto split_first = [&](int t) { return (int)((long long)total_iters * (t % p.splits) / p.splits); };
    auto split_count = [&](int t) {
        return (int)((long long)total_iters * (t % p.splits + 1) / p.splits) - (int)((long long)total_iters * (t % p.splits) / p.splits);
    };
    const int kc = (AKR_DIAG(p.debug, 64)) ? 0x3fffffff : PAIR_KC;  // bit 6: one chain per tile (timing experiment)

    // 128 promotion accumulators per epilogue thread do not fit the uniform 168 registers of a 12-warp CTA (they
    // spilled into the chain loop); the third warpgroup (producer, MMA, converters) needs far fewer and gives
    // them back first.
    if (hw_warp >= 8) {
    ptx::reg_dealloc<96>();
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (own tiles, local barriers)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs) {
                const Tile c = decode_tile(t, p, PAIR_BN, PAIR_BM);
                const int m_row0 = c.m0 + 128 * (int)rank;  // this CTA's rows of A
                const int n_col0 = c.n0 + 128 * (int)rank;  // this CTA's columns of B
                const int first = split_first(t), n_it = split_count(t);
                for (int it = 0; it < n_it; ++it) {
                    const int r = (first + it) / p.nkb;
                    const int k0 = (first + it - r * p.nkb) * PAIR_BK;
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fb = landed_bar(stage);
                    if (p.debug & 16) continue;  // test hook: nothing ever arrives, every waiter must give up
                    if (p.debug & 1) {           // timing experiment: no loads, stale shared memory
                        ptx::mbar_arrive(fb);
                        ++issued;
                        if (++stage == S) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    const uint32_t sa = smem_base + stage * stage_bytes;
                    const uint32_t sb = sa + PAIR_A_BYTES;
                    ptx::mbar_arrive_expect_tx(fb, PAIR_RAW_BYTES);
                    const int bcv[4] = {c.i1, c.i0, r, 0};
                    const int a0 = bcv[p.a_sel[0]], a1 = bcv[p.a_sel[1]], a2 = bcv[p.a_sel[2]];
                    const int b0 = bcv[p.b_sel[0]], b1 = bcv[p.b_sel[1]], b2 = bcv[p.b_sel[2]];
                    {
                        const CUtensorMap* ma = &p.tmA;
                        const CUtensorMap* mb = &p.tmB;
                        const uint32_t da = sa;
                        const uint32_t db = sb;
                        if (MAJA == 0) {
                            ptx::tma_load_5d(da, ma, fb, k0, m_row0, a0, a1, a2);
                        } else if (p.a_fold) {
                            ptx::tma_load_5d(da, ma, fb, 0, k0, m_row0 / CHUNK, a0, a1);
                        } else {
#pragma unroll
                            for (int ch = 0; ch < 128 / CHUNK; ++ch)
                                ptx::tma_load_5d(da + ch * (PAIR_BK * 128), ma, fb, m_row0 + ch * CHUNK, k0, a0, a1, a2);
                        }
                        if (MAJB == 0) {
                            ptx::tma_load_5d(db, mb, fb, k0, n_col0, b0, b1, b2);
                        } else if (p.b_fold) {
                            ptx::tma_load_5d(db, mb, fb, 0, k0, n_col0 / CHUNK, b0, b1);
                        } else {
#pragma unroll
                            for (int ch = 0; ch < 128 / CHUNK; ++ch)
                                ptx::tma_load_5d(db + ch * (PAIR_BK * 128), mb, fb, n_col0 + ch * CHUNK, k0, b0, b1, b2);
                        }
                    }
                    ++issued;
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || *abort_flag) {
                int s2 = stage;
                uint32_t ph = phase;
                const int n = issued < S ? (int)issued : S;
                for (int i = 0; i < n; ++i) {
                    if (--s2 < 0) {
                        s2 = S - 1;
                        ph ^= 1u;
                    }
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(landed_bar(s2), ph)) {
                        if (ptx::globaltimer_ns() - t0 > 200000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader) {  // all 32 lanes run the loop, one elected lane issues (see the general kernel)
            const uint32_t issuer = ptx::elect_one();
            constexpr uint32_t IDESC = ptx::idesc_tf32(PAIR_BM, PAIR_BN, MAJA, MAJB);
            constexpr uint32_t K_SBO = 8 * PAIR_BK * 4;
            constexpr uint32_t PAIR_K_LAY = PAIR_BK == 32 ? ptx::LAYOUT_SW128 : ptx::LAYOUT_SW64;
            constexpr uint32_t a_lay = MAJA == 0 ? PAIR_K_LAY : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t b_lay = MAJB == 0 ? PAIR_K_LAY : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t a_lbo = MAJA == 0 ? 16 : PAIR_BK * 128, b_lbo = MAJB == 0 ? 16 : PAIR_BK * 128;
            constexpr uint32_t a_sbo = MAJA == 0 ? K_SBO : 512, b_sbo = MAJB == 0 ? K_SBO : 512;
            int stage = 0, slot = 0;
            uint32_t phase = 0, slot_phase = 0;
            int handoff = 0;
            bool ok = true;
            for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs) {
                const int n_it = split_count(t);
                for (int cs = 0, ce = 0; cs < n_it && ok; cs = ce) {
                    ce = (n_it - cs > kc) ? cs + kc : n_it;
                    const int buf = handoff & 1;
                    const uint32_t acc_phase = (handoff >> 1) & 1u;
                    if (!ptx::mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * PAIR_BN;
                    for (int it = cs; it < ce; ++it) {
                        if (!ptx::mbar_wait(ready_bar(slot), slot_phase, abort_flag, p.wait_limit_ns)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t sa = smem_base + stage * stage_bytes;
                        const uint32_t sb = sa + PAIR_A_BYTES;
                        const uint32_t sa_lo = smem_base + LO_BASE + slot * PAIR_RAW_BYTES;
                        const uint32_t sb_lo = sa_lo + PAIR_A_BYTES;
#pragma unroll
                        for (int k8 = 0; k8 < PAIR_BK / UMMA_K; ++k8) {
                            const uint32_t a_off = MAJA == 0 ? k8 * 32 : k8 * 1024;
                            const uint32_t b_off = MAJB == 0 ? k8 * 32 : k8 * 1024;
                            const uint64_t da = ptx::smem_desc(sa + a_off, a_lbo, a_sbo, a_lay);
                            const uint64_t db = ptx::smem_desc(sb + b_off, b_lbo, b_sbo, b_lay);
                            const uint64_t da_lo = ptx::smem_desc(sa_lo + a_off, a_lbo, a_sbo, a_lay);
                            const uint64_t db_lo = ptx::smem_desc(sb_lo + b_off, b_lbo, b_sbo, b_lay);
                            const uint32_t first = (it == cs && k8 == 0) ? 0u : 1u;
                            if (AKR_DIAG(p.debug, 2)) {  // timing experiment: loads and hand-shakes only
                                if (first == 0u) ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db, IDESC, 0u);
                                continue;
                            }
                            ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da_lo, db, IDESC, first);
                            ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db_lo, IDESC, 1u);
                            ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db, IDESC, 1u);
                        }
                        // both CTAs may refill this stage once these MMAs have read it
                        ptx::mma_commit_pair_elected(issuer, empty_bar(stage));
                        if (++stage == S) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        ptx::mma_commit_pair_elected(issuer, lofree_bar(slot));  // and rewrite this low-part slot
                        if (++slot == LS) {
                            slot = 0;
                            slot_phase ^= 1u;
                        }
                    }
                    if (ok) {  // this chain's accumulator is complete in both CTAs' tensor memory
                        ptx::mma_commit_pair_elected(issuer, tfull_bar(buf));
                    }
                    ++handoff;
                }
            }
        }
    } else if (warp >= 2 + PAIR_EPI_WARPS) {
        // ------------------------------------------------------------ low-part converter
        const int ct = (warp - 2 - PAIR_EPI_WARPS) * 32 + lane;
        int stage = 0, slot = 0;
        uint32_t phase = 0, slot_phase = 0;
        bool ok = true;
        const uint32_t leader_ready0 = ptx::map_to_cta(ready_bar(0), 0);  // the leader's ready barriers, seen from here
        for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs) {
            const int n_it = split_count(t);
            for (int it = 0; it < n_it; ++it) {
                // the raw tiles have landed, and the MMAs that read this low-part slot last have finished
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_warp(landed_bar(stage), phase, abort_flag, p.wait_limit_ns)) ||
                    !__all_sync(0xffffffffu, ptx::mbar_wait_warp(lofree_bar(slot), slot_phase ^ 1u, abort_flag, p.wait_limit_ns))) {
                    ok = false;
                    break;
                }
                if (!AKR_DIAG(p.debug, 4)) {  // bit 2: hand-shakes only, stale low parts (timing experiment)
                    const float4* src = reinterpret_cast<const float4*>(smem + stage * PAIR_RAW_BYTES);
                    float4* dst = reinterpret_cast<float4*>(smem + LO_BASE + slot * PAIR_RAW_BYTES);
                    constexpr int PER_THREAD = PAIR_RAW_BYTES / 16 / (PAIR_CONV_WARPS * 32);
                    constexpr int BATCH = 8;
                    static_assert(PER_THREAD % BATCH == 0, "converter work must divide evenly");
#pragma unroll 1
                    for (int b0 = 0; b0 < PER_THREAD; b0 += BATCH) {
                        float4 x[BATCH];
#pragma unroll
                        for (int u = 0; u < BATCH; ++u) x[u] = src[(b0 + u) * (PAIR_CONV_WARPS * 32) + ct];
#pragma unroll
                        for (int u = 0; u < BATCH; ++u) {
                            x[u].x -= __uint_as_float(__float_as_uint(x[u].x) & 0xffffe000u);
                            x[u].y -= __uint_as_float(__float_as_uint(x[u].y) & 0xffffe000u);
                            x[u].z -= __uint_as_float(__float_as_uint(x[u].z) & 0xffffe000u);
                            x[u].w -= __uint_as_float(__float_as_uint(x[u].w) & 0xffffe000u);
                            dst[(b0 + u) * (PAIR_CONV_WARPS * 32) + ct] = x[u];
                        }
                    }
                    ptx::fence_proxy_async_smem();
                }
                __syncwarp();
                // both CTAs' converter warps arrive on the LEADER's barrier of this slot (a remote arrive for the peer)
                if (lane == 0) {
                    if (leader) ptx::mbar_arrive(ready_bar(slot));
                    else ptx::mbar_arrive_cluster(leader_ready0 + 8u * slot);
                }
                if (++stage == S) {
                    stage = 0;
                    phase ^= 1u;
                }
                if (++slot == LS) {
                    slot = 0;
                    slot_phase ^= 1u;
                }
            }
        }
    }
    } else {
        ptx::reg_alloc<200>();
        // ------------------------------------------------------------ epilogue (roles 2..9), fp32 promotion
        const int q = hw_warp & 3;  // TMEM lane quarter of this hardware warp
        const int slab = (warp - 2) >> 2;
        const bool split_mode = p.splits > 1;  // partial tiles to scratch, added up by the reduction kernel
        const bool vec = split_mode ? (p.N & 3) == 0 : p.vec_ok != 0;
        // Aligned plain outputs leave through TMA: the four warps of a slab stage a 128-row box of 32 columns and are
        // free again once the TMA unit has read it. With st.global the eight warps spent 9 of a tile's 22 kilocycles
        // in the stores (8192 products of 256^3: every SM writes its 128 KB at the same moment), longer than the two
        // chains the MMAs may run ahead of the promotion.
        const bool use_tma = p.c_tma != 0 && !split_mode;
        float4* my_stage = reinterpret_cast<float4*>(epi_stage_base + (warp - 2) * EPI_STAGE_BYTES);
        const uint32_t slab_tile_addr = smem_base + TILE_BYTES + slab * 4 * EPI_STAGE_BYTES;
        constexpr int EPI_ALT = PAIR_EPI_WARPS * EPI_STAGE_BYTES;  // offset of the second set of staging tiles
        int epi_buf = 0;
        int handoff = 0;
        bool ok = true;
#ifdef AKR_B200_DIAG
        long long diag_store = 0;
        const long long diag_e0 = clock64();
#endif
        for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs) {
            const Tile c = decode_tile(t, p, PAIR_BN, PAIR_BM);
            const int row_base = c.m0 + 128 * (int)rank;
            const int row0 = row_base + q * 32;
            const int slab_col0 = c.n0 + slab * 128;
            float* out_base = split_mode ? p.partials + ((size_t)c.split * (p.o0 * p.o1) + c.batch) * (size_t)p.M * (size_t)p.N
                                         : p.C + c.i0 * p.c_bs0 + c.i1 * p.c_bs1;
            const int n_it = split_count(t);
            float acc[128];
#pragma unroll
            for (int j = 0; j < 128; ++j) acc[j] = 0.f;
            for (int cs = 0; cs < n_it && ok; cs = (n_it - cs > kc) ? cs + kc : n_it) {
                const int buf = handoff & 1;
                const uint32_t acc_phase = (handoff >> 1) & 1u;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_warp(tfull_bar(buf), acc_phase, abort_flag, p.wait_limit_ns))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * PAIR_BN + slab * 128;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    if (slab_col0 + ch * 32 < p.N) {  // warp-uniform
                        __syncwarp();
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(t_row + ch * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[ch * 32 + j] += __uint_as_float(v[j]);
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(buf), 0));
                ++handoff;
            }
#ifdef AKR_B200_DIAG
            const long long diag_s0 = clock64();
#endif
            if (use_tma) ok = ptx::named_barrier_and(2 + slab, 128, ok);  // a slab's four warps store together or not at all
            if (ok && use_tma) {
                if (row_base < p.M) {  // CTA-uniform: the peer's half may lie below the matrix
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const int col0 = slab_col0 + ch * 32;
                        if (col0 < p.N) {  // slab-uniform
                            float f[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = acc[ch * 32 + j];
                            store_block_tma<PAIR_EPI_SETS>(f, my_stage + epi_buf * (EPI_ALT / 16), slab_tile_addr + epi_buf * EPI_ALT,
                                                           &p.tmC, col0, row_base, c.i1, c.i0, p.N, p.bias, lane,
                                                           q == 0 && lane == 0, 2 + slab);
                            if (PAIR_EPI_SETS == 2) epi_buf ^= 1;
                        }
                    }
                }
            } else if (ok) {
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const int col0 = slab_col0 + ch * 32;
                    if (col0 < p.N && !(AKR_DIAG(p.debug, 128) && acc[ch * 32] != 12345.f)) {  // bit 7: no stores (timing experiment)
                        float f[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = acc[ch * 32 + j];
                        store_block_warp<false>(f, my_stage, out_base, split_mode ? (long long)p.N : p.ldc, row0, p.M, col0, p.N, vec,
                                                split_mode ? plain_epi() : lean_epi(p), lane);
                    }
                }
            }
#ifdef AKR_B200_DIAG
            diag_store += clock64() - diag_s0;
#endif
        }
#ifdef AKR_B200_DIAG
        if (AKR_DIAG(p.debug, 262144) && hw_warp == 0 && lane == 0 && blockIdx.x < 256) {  // bit 18: cycles in the stores
            g_clock_probe[2 * blockIdx.x] = diag_store;
            g_clock_probe[2 * blockIdx.x + 1] = clock64() - diag_e0;
        }
#endif
    }

    // ------------------------------------------------------------ teardown (all paths)
    if (p.c_tma != 0 && hw_warp < 8 && (hw_warp & 3) == 0 && lane == 0) ptx::bulk_wait_read_all();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // no remote arrive or MMA of the pair is still in flight
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair<512>(tmem_base);
    }
    AKR_DIAG_CLK_END
    if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------- CTA pairs, TF32 mode
// One 256 x 256 tile per CTA pair (tcgen05.mma.cta_group::2, M = 256): each CTA holds 128 rows of A
// and 128 columns of B of every k-block, so per flop a CTA's shared memory takes half the TMA writes
// and two thirds of the MMA reads of a 128 x 256 tile on one CTA, and each CTA's tensor memory holds
// TWO 128 x 256 accumulators: the epilogue of a tile overlaps the MMAs of the next (the 256 x 256
// tile on one CTA fills all 512 columns and cannot do that).
//   both CTAs: warp 0 loads its own tiles, completion bytes counted on the LEADER's barrier
//   (cp.async.bulk.tensor ... .cta_group::2, one destination CTA per copy, no multicast);
//   leader: warp 1 issues the MMAs; tcgen05.commit signals "stage free" / "accumulator complete" to
//   both CTAs; warps 2..9 of each CTA drain its 128 rows.
// A stage holds a 64-deep k-block as two 32-deep sub-tiles per operand (a K-major row of the swizzled layout is 128
// bytes), so that a stage carries eight MMAs like the stages of the large-tile kernels: with 32-deep stages of four
// MMAs the main loop took 665 cycles per 512 of MMA work, and 601 with the loads switched off - the hand-over of a
// stage, not its bytes, was what it waited for.
constexpr int DUO_STAGES = 3, DUO_SUBS = 2;
constexpr int DUO_SUB_BYTES = 128 * BK * 4;                  // one operand, one 32-deep sub-tile: 16 KB
constexpr int DUO_A_BYTES = DUO_SUBS * DUO_SUB_BYTES, DUO_B_BYTES = DUO_SUBS * DUO_SUB_BYTES;
constexpr int DUO_STAGE_BYTES = DUO_A_BYTES + DUO_B_BYTES;   // 64 KB per CTA
constexpr int DUO_THREADS = 64 + 256;
constexpr int DUO_EPI_WARPS = 8;
constexpr int DUO_SMEM = DUO_STAGES * DUO_STAGE_BYTES + DUO_EPI_WARPS * EPI_STAGE_BYTES + 256 + 1024;

template <int MAJA, int MAJB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(DUO_THREADS, 1)
gemm_tf32_duo_kernel(const __grid_constant__ KernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    constexpr int SM = DUO_STAGES;
    constexpr int S = DUO_STAGES;
    // [3 stages][staging area][barriers]
    uint8_t* epi_stage_base = smem + DUO_STAGES * DUO_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM * DUO_STAGE_BYTES + DUO_EPI_WARPS * EPI_STAGE_BYTES);
    const uint32_t bar_base = smem_base + SM * DUO_STAGE_BYTES + DUO_EPI_WARPS * EPI_STAGE_BYTES;
    auto ready_bar = [&](int s) { return bar_base + 8u * s; };             // leader: both CTAs' tiles landed
    auto empty_bar = [&](int s) { return bar_base + 8u * (SM + s); };      // local: stage may be refilled
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * SM + b); };    // local: accumulator complete
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * SM + 2 + b); };  // leader: both CTAs drained it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SM + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform for the compiler too
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SM; ++s) {
            // the leader's expect-tx arrive, completed by both CTAs' bytes (MMA-only timing: one arrive per CTA instead,
            // so that the peer's producer still cannot be lapped)
            ptx::mbar_init(ready_bar(s), (p.debug & 1) ? 2 : 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), 2 * DUO_EPI_WARPS);
        }
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
        if (p.c_tma) ptx::prefetch_tensormap(&p.tmC);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair<512>(ptx::smem_u32(tmem_slot));
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up done (shared memory, tensor memory, barriers only). Let the next kernel of the stream begin its own
    // set-up on SMs this grid leaves, and do not touch global memory before the previous kernel has finished.
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    AKR_DIAG_CLK_BEGIN
    const int nkb2 = (p.nkb + DUO_SUBS - 1) / DUO_SUBS;  // 64-deep steps; the last may hold one sub-tile of zeros
    const int total_iters = p.red * nkb2;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (own tiles, leader's barrier)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs) {
                const Tile c = decode_tile(t, p, PAIR_BN, PAIR_BM);
                const int m_row0 = c.m0 + 128 * (int)rank;  // this CTA's rows of A
                const int n_col0 = c.n0 + 128 * (int)rank;  // this CTA's columns of B
                // a split contraction: this tile's share of the (summed batch, k) steps
                const int it0 = (int)((long long)total_iters * c.split / p.splits);
                const int it1 = (int)((long long)total_iters * (c.split + 1) / p.splits);
                for (int it = it0; it < it1; ++it) {
                    const int r = it / nkb2;
                    const int k00 = (it - r * nkb2) * (DUO_SUBS * BK);
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    if (p.debug & 16) continue;  // test hook: nothing ever arrives, every waiter must give up
                    const uint32_t lb = ptx::map_to_cta(ready_bar(stage), 0);
                    if (p.debug & 1) {  // timing experiment: no loads, stale shared memory
                        ptx::mbar_arrive_cluster(lb);
                        if (++stage == S) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    if (leader) ptx::mbar_arrive_expect_tx(ready_bar(stage), 2 * DUO_STAGE_BYTES);
                    const int bcv[4] = {c.i1, c.i0, r, 0};
                    const int a0 = bcv[p.a_sel[0]], a1 = bcv[p.a_sel[1]], a2 = bcv[p.a_sel[2]];
                    const int b0 = bcv[p.b_sel[0]], b1 = bcv[p.b_sel[1]], b2 = bcv[p.b_sel[2]];
#pragma unroll
                    for (int sub = 0; sub < DUO_SUBS; ++sub) {
                        // a sub-tile that starts at or behind K is filled with zeros by the copy and still counts its bytes
                        const int k0 = k00 + sub * BK;
                        const uint32_t da = smem_base + stage * DUO_STAGE_BYTES + sub * DUO_SUB_BYTES;
                        const uint32_t db = da + DUO_A_BYTES;
                        if (MAJA == 0) {
                            ptx::tma_load_5d_pair(da, &p.tmA, lb, k0, m_row0, a0, a1, a2);
                        } else if (p.a_fold) {
                            ptx::tma_load_5d_pair(da, &p.tmA, lb, 0, k0, m_row0 / CHUNK, a0, a1);
                        } else {
#pragma unroll
                            for (int ch = 0; ch < 128 / CHUNK; ++ch)
                                ptx::tma_load_5d_pair(da + ch * (BK * 128), &p.tmA, lb, m_row0 + ch * CHUNK, k0, a0, a1, a2);
                        }
                        if (MAJB == 0) {
                            ptx::tma_load_5d_pair(db, &p.tmB, lb, k0, n_col0, b0, b1, b2);
                        } else if (p.b_fold) {
                            ptx::tma_load_5d_pair(db, &p.tmB, lb, 0, k0, n_col0 / CHUNK, b0, b1);
                        } else {
#pragma unroll
                            for (int ch = 0; ch < 128 / CHUNK; ++ch)
                                ptx::tma_load_5d_pair(db + ch * (BK * 128), &p.tmB, lb, n_col0 + ch * CHUNK, k0, b0, b1, b2);
                        }
                    }
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || *abort_flag) {
                const uint64_t t0 = ptx::globaltimer_ns();  // let copies in flight land (they signal the leader)
                while (ptx::globaltimer_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader) {  // all 32 lanes run the loop, one elected lane issues (see the general kernel)
            const uint32_t issuer = ptx::elect_one();
            constexpr uint32_t IDESC = ptx::idesc_tf32(PAIR_BM, PAIR_BN, MAJA, MAJB);
            constexpr uint32_t a_lay = MAJA == 0 ? ptx::LAYOUT_SW128 : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t b_lay = MAJB == 0 ? ptx::LAYOUT_SW128 : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t a_lbo = MAJA == 0 ? 16 : BK * 128, b_lbo = MAJB == 0 ? 16 : BK * 128;
            constexpr uint32_t a_sbo = MAJA == 0 ? 1024 : 512, b_sbo = MAJB == 0 ? 1024 : 512;
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1u;
                if (!ptx::mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * PAIR_BN;
                const int split = t % p.splits;
                const int it0 = (int)((long long)total_iters * split / p.splits);
                const int it1 = (int)((long long)total_iters * (split + 1) / p.splits);
                for (int it = it0; it < it1; ++it) {
                    if (!ptx::mbar_wait(ready_bar(stage), phase, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k8s = 0; k8s < DUO_SUBS * (BK / UMMA_K); ++k8s) {
                        const int sub = k8s / (BK / UMMA_K), k8 = k8s % (BK / UMMA_K);
                        const uint32_t sa = smem_base + stage * DUO_STAGE_BYTES + sub * DUO_SUB_BYTES;
                        const uint32_t sb = sa + DUO_A_BYTES;
                        const uint32_t a_off = MAJA == 0 ? k8 * 32 : k8 * 1024;
                        const uint32_t b_off = MAJB == 0 ? k8 * 32 : k8 * 1024;
                        const uint64_t da = ptx::smem_desc(sa + a_off, a_lbo, a_sbo, a_lay);
                        const uint64_t db = ptx::smem_desc(sb + b_off, b_lbo, b_sbo, b_lay);
                        if (AKR_DIAG(p.debug, 2)) {  // timing experiment: loads and hand-shakes only
                            if (it == it0 && k8s == 0) ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db, IDESC, 0u);
                            continue;
                        }
                        ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db, IDESC, (it == it0 && k8s == 0) ? 0u : 1u);
                    }
                    ptx::mma_commit_pair_elected(issuer, empty_bar(stage));  // both CTAs may refill this stage
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::mma_commit_pair_elected(issuer, tfull_bar(buf));  // accumulator complete in both CTAs' tensor memory
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9): this CTA's 128 rows
        const int q = warp & 3;
        const int slab = (warp - 2) >> 2;
        const bool split_mode = p.splits > 1;  // partial tiles to scratch, added up by the reduction kernel
        const bool vec = split_mode ? (p.N & 3) == 0 : p.vec_ok != 0;
        const bool use_tma = p.c_tma != 0;
        float4* my_stage = reinterpret_cast<float4*>(epi_stage_base + (slab * 4 + q) * EPI_STAGE_BYTES);
        const uint32_t slab_tile_addr = smem_base + DUO_STAGES * DUO_STAGE_BYTES + slab * 4 * EPI_STAGE_BYTES;
        int local = 0;
        bool ok = true;
        for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs, ++local) {
            const Tile c = decode_tile(t, p, PAIR_BN, PAIR_BM);
            const Epi epi = split_mode ? plain_epi() : tile_epi(p, c);
            const bool ring_free = t + num_pairs >= p.total_tiles;  // no later tile of this pair is being prefetched
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1u;
            bool got = __all_sync(0xffffffffu, ptx::mbar_wait_warp(tfull_bar(buf), acc_phase, abort_flag, p.wait_limit_ns));
            if (use_tma) got = ptx::named_barrier_and(2 + slab, 128, got);  // a slab's four warps leave together
            if (!got) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const int row_base = c.m0 + 128 * (int)rank;
            const int row0 = row_base + q * 32;
            const int slab_col0 = c.n0 + slab * 128;
            float* out_base = split_mode ? p.partials + ((size_t)c.split * (p.o0 * p.o1) + c.batch) * (size_t)p.M * (size_t)p.N
                                         : p.C + c.i0 * p.c_bs0 + c.i1 * p.c_bs1;
            const long long out_ld = split_mode ? p.N : p.ldc;
            const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * PAIR_BN + slab * 128;
            if (row_base < p.M) {  // CTA-uniform: the peer's half may lie below the matrix
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    const int col0 = slab_col0 + ch * 32;
                    if (col0 < p.N) {
                        __syncwarp();
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(t_row + ch * 32, v);
                        ptx::tmem_ld_wait();
                        float f[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                        if (AKR_DIAG(p.debug, 128)) continue;  // timing experiment: no stores
                        if (use_tma && ring_free) {
                            // behind the pair's last tile the load stages are idle: a staging tile per block, no waits between
                            const uint32_t off = (uint32_t)((slab * 4 + ch) * 4 * EPI_STAGE_BYTES);
                            store_block_tma_once(f, reinterpret_cast<float4*>(smem + off + q * EPI_STAGE_BYTES), smem_base + off,
                                                 &p.tmC, col0, row_base, c.i1, c.i0, p.N, p.bias, lane, q == 0 && lane == 0, 2 + slab);
                        } else if (use_tma)
                            store_block_tma(f, my_stage, slab_tile_addr, &p.tmC, col0, row_base, c.i1, c.i0, p.N, p.bias,
                                            lane, q == 0 && lane == 0, 2 + slab);
                        else
                            store_block_warp<true>(f, my_stage, out_base, out_ld, row0, p.M, col0, p.N, vec, epi, lane);
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(buf), 0));
        }
    }

    // ------------------------------------------------------------ teardown (all paths)
    if (p.c_tma != 0 && warp >= 2 && (warp & 3) == 0 && lane == 0) ptx::bulk_wait_read_all();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // no remote arrive or MMA of the pair is still in flight
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair<512>(tmem_base);
    }
    AKR_DIAG_CLK_END
    if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------- 512 x 256 tiles on CTA pairs
// Large TF32 products are limited by the rate at which operand tiles reach shared memory, not by the
// MMA pipe. Here a CTA pair computes a 512 x 256 tile: each CTA holds 256 rows of A (two 128-row halves)
// and 128 columns of B per k-block, and the pair's MMAs (M = 256: one 128-row half from each CTA) fill
// both of its 128 x 256 accumulators from the same B tile. Per flop that is a quarter fewer bytes into
// shared memory than a 256 x 256 tile on one CTA (384 operand rows per k-block for 256 x 256 outputs
// instead of 512), and each MMA reads only half of B in each CTA. Like the single-CTA 256 x 256 kernel
// it fills all 512 TMEM columns: a tile's MMAs start on an accumulator once the epilogue has drained it.
//   both CTAs: warp 0 loads its own tiles, completion bytes counted on the LEADER's barrier
//   (cp.async.bulk.tensor ... .cta_group::2, one destination CTA per copy, no multicast);
//   leader: warp 1 issues the MMAs; tcgen05.commit signals both CTAs; warps 2..9 of each CTA drain its 256 rows.
constexpr int QUAD_BM = 512, QUAD_BN = 256;
constexpr int QUAD_RING_BYTES = 192 * 1024;  // 4 stages of 48 KB (32-deep k-blocks) or 8 of 24 KB (16-deep)
constexpr int QUAD_THREADS = 64 + 256;
constexpr int QUAD_EPI_WARPS = 8;
constexpr int QUAD_SMEM = QUAD_RING_BYTES + QUAD_EPI_WARPS * EPI_STAGE_BYTES + 256 + 1024;

template <int MAJA, int MAJB, int BKT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(QUAD_THREADS, 1)
gemm_tf32_quad_kernel(const __grid_constant__ KernelParams p) {
    constexpr int QUAD_A_BYTES = 256 * BKT * 4, QUAD_B_BYTES = 128 * BKT * 4;
    constexpr int QUAD_STAGE_BYTES = QUAD_A_BYTES + QUAD_B_BYTES;
    constexpr int QUAD_STAGES = QUAD_RING_BYTES / QUAD_STAGE_BYTES;
    static_assert((2 * QUAD_STAGES + 3) * 8 + 8 <= 256, "barrier area");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    constexpr int S = QUAD_STAGES;
    constexpr int EPI_BYTES = QUAD_EPI_WARPS * EPI_STAGE_BYTES;
    // [4 stages][staging area][barriers]
    uint8_t* epi_stage_base = smem + S * QUAD_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * QUAD_STAGE_BYTES + EPI_BYTES);
    const uint32_t bar_base = smem_base + S * QUAD_STAGE_BYTES + EPI_BYTES;
    auto ready_bar = [&](int s) { return bar_base + 8u * s; };                 // leader: both CTAs' tiles landed
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };           // local: stage may be refilled
    const uint32_t tfull_bar = bar_base + 8u * (2 * S);                        // local: both accumulators complete
    auto tempty_bar = [&](int h) { return bar_base + 8u * (2 * S + 1 + h); };  // leader: both CTAs drained half h
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform for the compiler too
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            // the leader's expect-tx arrive, completed by both CTAs' bytes (MMA-only timing: one arrive per CTA instead,
            // so that the peer's producer still cannot be lapped)
            ptx::mbar_init(ready_bar(s), (p.debug & 1) ? 2 : 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(tfull_bar, 1);
        ptx::mbar_init(tempty_bar(0), 2 * QUAD_EPI_WARPS);
        ptx::mbar_init(tempty_bar(1), 2 * QUAD_EPI_WARPS);
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&p.tmA);
        ptx::prefetch_tensormap(&p.tmB);
        if (p.c_tma) ptx::prefetch_tensormap(&p.tmC);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair<512>(ptx::smem_u32(tmem_slot));
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    AKR_DIAG_CLK_BEGIN
    const int total_iters = p.red * p.nkb;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (own tiles, leader's barrier)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs) {
                const Tile c = decode_tile(t, p, QUAD_BN, QUAD_BM, 8);
                const int m_row0 = c.m0 + 256 * (int)rank;  // this CTA's rows of A
                const int n_col0 = c.n0 + 128 * (int)rank;  // this CTA's columns of B
                for (int it = 0; it < total_iters; ++it) {
                    const int r = it / p.nkb;
                    const int k0 = (it - r * p.nkb) * BKT;
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    if (p.debug & 16) continue;  // test hook: nothing ever arrives, every waiter must give up
                    const uint32_t lb = ptx::map_to_cta(ready_bar(stage), 0);
                    if (p.debug & 1) {  // timing experiment: no loads, stale shared memory
                        ptx::mbar_arrive_cluster(lb);
                        if (++stage == S) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    if (leader) ptx::mbar_arrive_expect_tx(ready_bar(stage), 2 * QUAD_STAGE_BYTES);
                    const uint32_t da = smem_base + stage * QUAD_STAGE_BYTES;
                    const uint32_t db = da + QUAD_A_BYTES;
                    const int bcv[4] = {c.i1, c.i0, r, 0};
                    const int a0 = bcv[p.a_sel[0]], a1 = bcv[p.a_sel[1]], a2 = bcv[p.a_sel[2]];
                    const int b0 = bcv[p.b_sel[0]], b1 = bcv[p.b_sel[1]], b2 = bcv[p.b_sel[2]];
                    if (MAJA == 0) {
                        ptx::tma_load_5d_pair(da, &p.tmA, lb, k0, m_row0, a0, a1, a2);
                    } else if (p.a_fold) {
                        ptx::tma_load_5d_pair(da, &p.tmA, lb, 0, k0, m_row0 / CHUNK, a0, a1);
                    } else {
#pragma unroll
                        for (int ch = 0; ch < 256 / CHUNK; ++ch)
                            ptx::tma_load_5d_pair(da + ch * (BKT * 128), &p.tmA, lb, m_row0 + ch * CHUNK, k0, a0, a1, a2);
                    }
                    if (MAJB == 0) {
                        ptx::tma_load_5d_pair(db, &p.tmB, lb, k0, n_col0, b0, b1, b2);
                    } else if (p.b_fold) {
                        ptx::tma_load_5d_pair(db, &p.tmB, lb, 0, k0, n_col0 / CHUNK, b0, b1);
                    } else {
#pragma unroll
                        for (int ch = 0; ch < 128 / CHUNK; ++ch)
                            ptx::tma_load_5d_pair(db + ch * (BKT * 128), &p.tmB, lb, n_col0 + ch * CHUNK, k0, b0, b1, b2);
                    }
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || *abort_flag) {
                const uint64_t t0 = ptx::globaltimer_ns();  // let copies in flight land (they signal the leader)
                while (ptx::globaltimer_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader) {  // all 32 lanes run the loop, one elected lane issues (see the general kernel)
            const uint32_t issuer = ptx::elect_one();
            constexpr uint32_t IDESC = ptx::idesc_tf32(256, QUAD_BN, MAJA, MAJB);
            constexpr uint32_t K_LAY = BKT == 32 ? ptx::LAYOUT_SW128 : ptx::LAYOUT_SW64;
            constexpr uint32_t a_lay = MAJA == 0 ? K_LAY : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t b_lay = MAJB == 0 ? K_LAY : ptx::LAYOUT_SW128_ATOM32B;
            constexpr uint32_t a_lbo = MAJA == 0 ? 16 : BKT * 128, b_lbo = MAJB == 0 ? 16 : BKT * 128;
            constexpr uint32_t a_sbo = MAJA == 0 ? 8 * BKT * 4 : 512, b_sbo = MAJB == 0 ? 8 * BKT * 4 : 512;
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs, ++local) {
                const uint32_t tile_par = local & 1u;
                for (int it = 0; it < total_iters && ok; ++it) {
                    if (!ptx::mbar_wait(ready_bar(stage), phase, abort_flag, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = smem_base + stage * QUAD_STAGE_BYTES;
                    const uint32_t sb = sa + QUAD_A_BYTES;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (it == 0) {
                            // accumulator h must have been drained by both CTAs' epilogues of the previous tile
                            if (!ptx::mbar_wait(tempty_bar(h), tile_par ^ 1u, abort_flag, p.wait_limit_ns)) {
                                ok = false;
                                break;
                            }
                            ptx::tc_fence_after();
                        }
                        // rows h*128.. of each CTA's A tile: 128 rows x 128 B (K-major) or 4 chunks x 4 KB
                        const uint32_t sa_h = sa + h * (BM * BKT * 4);
                        const uint32_t d_tmem = tmem_base + h * QUAD_BN;
#pragma unroll
                        for (int k8 = 0; k8 < BKT / UMMA_K; ++k8) {
                            const uint32_t a_off = MAJA == 0 ? k8 * 32 : k8 * 1024;
                            const uint32_t b_off = MAJB == 0 ? k8 * 32 : k8 * 1024;
                            const uint64_t da = ptx::smem_desc(sa_h + a_off, a_lbo, a_sbo, a_lay);
                            const uint64_t db = ptx::smem_desc(sb + b_off, b_lbo, b_sbo, b_lay);
                            if (AKR_DIAG(p.debug, 2)) {  // timing experiment: loads and hand-shakes only
                                if (it == 0 && k8 == 0) ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db, IDESC, 0u);
                                continue;
                            }
                            ptx::mma_tf32_ss_pair_elected(issuer, d_tmem, da, db, IDESC, (it == 0 && k8 == 0) ? 0u : 1u);
                        }
                    }
                    if (!ok) break;
                    ptx::mma_commit_pair_elected(issuer, empty_bar(stage));  // both CTAs may refill this stage
                    if (++stage == S) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::mma_commit_pair_elected(issuer, tfull_bar);  // both accumulators complete in both CTAs' tensor memory
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9): this CTA's 256 rows
        const int q = warp & 3;
        const int slab = (warp - 2) >> 2;
        const bool vec = p.vec_ok != 0;
        const bool use_tma = p.c_tma != 0;
        float4* my_stage = reinterpret_cast<float4*>(epi_stage_base + (slab * 4 + q) * EPI_STAGE_BYTES);
        const uint32_t slab_tile_addr = smem_base + S * QUAD_STAGE_BYTES + slab * 4 * EPI_STAGE_BYTES;
        int local = 0;
        bool ok = true;
        for (int t = pair_id; t < p.total_tiles && ok; t += num_pairs, ++local) {
            const Tile c = decode_tile(t, p, QUAD_BN, QUAD_BM, 8);
            const Epi epi = tile_epi(p, c);
            const bool ring_free = t + num_pairs >= p.total_tiles;  // no later tile of this pair is being prefetched
            bool got = __all_sync(0xffffffffu, ptx::mbar_wait_warp(tfull_bar, local & 1u, abort_flag, p.wait_limit_ns));
            if (use_tma) got = ptx::named_barrier_and(2 + slab, 128, got);  // a slab's four warps leave together
            if (!got) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const int slab_col0 = c.n0 + slab * 128;
            float* out_base = p.C + c.i0 * p.c_bs0 + c.i1 * p.c_bs1;
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const int row_base = c.m0 + 256 * (int)rank + h * 128;
                const int row0 = row_base + q * 32;
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + h * QUAD_BN + slab * 128;
                if (row_base < p.M) {  // warp-uniform: skip a half that lies below the matrix
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        const int col0 = slab_col0 + ch * 32;
                        if (col0 < p.N) {
                            __syncwarp();
                            uint32_t v[32];
                            ptx::tmem_ld_32x32(t_row + ch * 32, v);
                            ptx::tmem_ld_wait();
                            float f[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                            if (use_tma && ring_free && h * 4 + ch < 6) {
                                // behind the pair's last tile the load stages are idle (see the single-CTA kernel)
                                const uint32_t off = (uint32_t)((slab * 6 + h * 4 + ch) * 4 * EPI_STAGE_BYTES);
                                store_block_tma_once(f, reinterpret_cast<float4*>(smem + off + q * EPI_STAGE_BYTES), smem_base + off,
                                                     &p.tmC, col0, row_base, c.i1, c.i0, p.N, p.bias, lane,
                                                     q == 0 && lane == 0, 2 + slab);
                            } else if (use_tma)
                                store_block_tma(f, my_stage, slab_tile_addr, &p.tmC, col0, row_base, c.i1, c.i0, p.N, p.bias,
                                                lane, q == 0 && lane == 0, 2 + slab);
                            else
                                store_block_warp<true>(f, my_stage, out_base, p.ldc, row0, p.M, col0, p.N, vec, epi, lane);
                        }
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(h), 0));
            }
        }
    }

    // ------------------------------------------------------------ teardown (all paths)
    if (p.c_tma != 0 && warp >= 2 && (warp & 3) == 0 && lane == 0) ptx::bulk_wait_read_all();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // no remote arrive or MMA of the pair is still in flight
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair<512>(tmem_base);
    }
    AKR_DIAG_CLK_END
    if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------- split-K reduction
// C = epilogue(sum over splits of the partial tiles), in split order (deterministic), by the whole GPU:
// one CTA adding up all partials of its tile alone is a chain of L2 round trips on a single SM
// (2.6 us per 128 KB partial), which capped the split count and left long-K, small-output products
// (weight gradients) several times slower than their loads.
struct SplitReduceParams {
    const float* partials;  // [splits][nbatch][M][N], dense
    float* C;
    const float* bias;
    const float* aux;
    long long ldc, c_bs0, c_bs1, aux_ld, aux_cs, aux_bs0, aux_bs1;
    int M, N, o1, nbatch, splits;
    int accumulate, aux_op;
    float alpha, beta;
};

template <bool VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const SplitReduceParams p) {
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();  // the partials come from the kernel before this one
    constexpr int W = VEC ? 4 : 1;
    const size_t ncol = (size_t)(p.N / W);
    const size_t total = (size_t)p.nbatch * p.M * ncol;
    const size_t split_stride = (size_t)p.nbatch * p.M * p.N;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int n = (int)(idx % ncol) * W;
        const size_t rm = idx / ncol;
        const int m = (int)(rm % (size_t)p.M);
        const int b = (int)(rm / (size_t)p.M);
        const float* src = p.partials + ((size_t)b * p.M + m) * p.N + n;
        float sum[W];
#pragma unroll
        for (int e = 0; e < W; ++e) sum[e] = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < p.splits; ++sp) {
            if (VEC) {
                const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * split_stride));
                sum[0] += x.x; sum[W > 1 ? 1 : 0] += x.y; sum[W > 2 ? 2 : 0] += x.z; sum[W > 3 ? 3 : 0] += x.w;
            } else {
                sum[0] += __ldcg(src + (size_t)sp * split_stride);
            }
        }
        const int i0 = b / p.o1, i1 = b - i0 * p.o1;
        float* dst = p.C + i0 * p.c_bs0 + i1 * p.c_bs1 + (long long)m * p.ldc + n;
#pragma unroll
        for (int e = 0; e < W; ++e) {
            float v = sum[e] * p.alpha;
            if (p.bias != nullptr) v += __ldg(p.bias + n + e);
            if (p.accumulate) v += dst[e];
            if (p.aux_op != 0) {
                const float a = p.aux[i0 * p.aux_bs0 + i1 * p.aux_bs1 + (long long)m * p.aux_ld + (long long)(n + e) * p.aux_cs];
                v = p.aux_op == 1 ? fmaf(p.beta, a, v) : v * (1.f - a * a);
            }
            sum[e] = v;
        }
        if (VEC) {
            *reinterpret_cast<float4*>(dst) = make_float4(sum[0], sum[W > 1 ? 1 : 0], sum[W > 2 ? 2 : 0], sum[W > 3 ? 3 : 0]);
        } else {
            dst[0] = sum[0];
        }
    }
}

// ---------------------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

void seterr(char* err, int errlen, const char* msg) {
    if (err && errlen > 0) {
        std::strncpy(err, msg, errlen - 1);
        err[errlen - 1] = 0;
    }
}

// How one operand is addressed by its tensor map.
struct MapPlan {
    bool fold = false;          // M/N-major operand fetched with one box per tile
    int sel[3] = {3, 3, 3};     // batch slot -> index into (i1, i0, r, 0)
    uint64_t ext[3] = {1, 1, 1};
    int64_t str[3] = {0, 0, 0};  // element strides of the batch slots
};

// Batch slots hold only the dims the operand really varies along; a folded map has two slots.
MapPlan plan_map(const GemmOperand& op, int mn, const int batch[3], bool allow_fold) {
    MapPlan mp;
    // kernel-side order of the candidates: i1 (o1), i0 (o0), r
    const int cand_idx[3] = {1, 0, 2};
    int n = 0;
    for (int j = 0; j < 3; ++j) {
        const int b = cand_idx[j];
        if (batch[b] > 1 && op.bs[b] != 0) {
            mp.sel[n] = j;
            mp.ext[n] = (uint64_t)batch[b];
            mp.str[n] = op.bs[b];
            ++n;
        }
    }
    mp.fold = allow_fold && op.mn_major && (mn % CHUNK == 0) && n <= 2;
    return mp;
}

bool make_map(CUtensorMap* out, const float* base, const GemmOperand& op, const MapPlan& mp, int mn,
              int k, int tile_mn, int bk) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    const uint64_t d0 = op.mn_major ? mn : k;
    const uint64_t d1 = op.mn_major ? k : mn;
    // Stride of a dim of extent 1 is never used for addressing; it only has to be well-formed.
    const uint64_t ld_b = (uint64_t)(d1 > 1 ? op.ld : ((d0 + 3) / 4) * 4) * 4;
    auto bstride = [&](int j) { return (uint64_t)(mp.ext[j] > 1 ? mp.str[j] * 4 : (int64_t)ld_b); };
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5];
    if (mp.fold) {
        // (32 contiguous, k rows, 32-column chunks, batch, batch)
        dims[0] = CHUNK; dims[1] = (cuuint64_t)k; dims[2] = (cuuint64_t)(mn / CHUNK);
        dims[3] = mp.ext[0]; dims[4] = mp.ext[1];
        strides[0] = ld_b; strides[1] = CHUNK * 4; strides[2] = bstride(0); strides[3] = bstride(1);
        box[0] = CHUNK; box[1] = (cuuint32_t)bk; box[2] = (cuuint32_t)(tile_mn / CHUNK); box[3] = 1; box[4] = 1;
    } else {
        // (unit-stride matrix dim, other matrix dim, batch, batch, batch)
        dims[0] = d0; dims[1] = d1; dims[2] = mp.ext[0]; dims[3] = mp.ext[1]; dims[4] = mp.ext[2];
        strides[0] = ld_b; strides[1] = bstride(0); strides[2] = bstride(1); strides[3] = bstride(2);
        box[0] = (cuuint32_t)(op.mn_major ? 32 : bk); box[1] = (cuuint32_t)(op.mn_major ? bk : tile_mn);
        box[2] = box[3] = box[4] = 1;
    }
    cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(base), dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     op.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                  : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool gemm_sm100_cta_limit_active();

// Per-device caches (function attributes, resident cluster counts, SM counts) are indexed by the current
// device: cudaFuncSetAttribute applies to the device that is current when it is called.
constexpr int kMaxDev = 64;
int cur_dev() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDev) d = 0;
    return d;
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor in
// the stream drains (its set-up overlaps that tail); it synchronises on the predecessor itself
// (grid_dep_wait) before its first access to global memory. Debug bit 12 launches normally.
bool g_pdl_off = false;
template <typename K>
void launch_pdl(K kern, int grid, int threads, int smem, cudaStream_t stream, const KernelParams& kp) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
#ifdef AKR_B200_DIAG
    static const bool env_off = std::getenv("AKR_B200_NO_PDL") != nullptr;  // A/B switch for measurements
#else
    constexpr bool env_off = false;
#endif
    // Not while a CTA limit is set: that is the phase in which a collective runs beside the GEMM, and there an
    // early-started GEMM measured 6 % slower (2 GPUs: 3.45-3.67 ms against 3.27-3.40 ms for dB + all-reduce + dA).
    cfg.numAttrs = (g_pdl_off || env_off || gemm_sm100_cta_limit_active()) ? 0 : 1;
    cudaLaunchKernelEx(&cfg, kern, kp);
}

template <int BN, int MAJA, int MAJB, int TERMS, int STAGES, int KC, int BKT, int LO>
int launch_variant(const KernelParams& kp, int grid, cudaStream_t stream, char* err, int errlen) {
    using L = SmemLayout<BN, TERMS, BKT>;
    constexpr int smem = (STAGES + LO) * L::STAGE_BYTES + 1024 + BAR_BYTES +
                         EpiBufs<BN, TERMS, STAGES, BKT, LO>::value * slabs_of(BN) * 4 * EPI_STAGE_BYTES;
    static_assert(smem <= 232448, "more shared memory than one CTA may have");
    auto kern = gemm_tf32_kernel<BN, MAJA, MAJB, TERMS, STAGES, KC, BKT, LO>;
    static bool attr_done_dev[kMaxDev] = {};  // per instantiation and device
    bool& attr_done = attr_done_dev[cur_dev()];
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            seterr(err, errlen, cudaGetErrorString(e));
            return -3;
        }
        attr_done = true;
    }
    launch_pdl(kern, grid, num_threads<BN, TERMS>(), smem, stream, kp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        seterr(err, errlen, cudaGetErrorString(e));
        return -3;
    }
    return 0;
}

template <int BN, int TERMS, int STAGES, int KC, int BKT, int LO = 0>
int launch_major(const GemmDesc& g, const KernelParams& kp, int grid, cudaStream_t s, char* err,
                 int errlen) {
    const int key = g.A.mn_major * 2 + g.B.mn_major;
    switch (key) {
        case 0: return launch_variant<BN, 0, 0, TERMS, STAGES, KC, BKT, LO>(kp, grid, s, err, errlen);
        case 1: return launch_variant<BN, 0, 1, TERMS, STAGES, KC, BKT, LO>(kp, grid, s, err, errlen);
        case 2: return launch_variant<BN, 1, 0, TERMS, STAGES, KC, BKT, LO>(kp, grid, s, err, errlen);
        default: return launch_variant<BN, 1, 1, TERMS, STAGES, KC, BKT, LO>(kp, grid, s, err, errlen);
    }
}

#ifdef AKR_B200_DIAG
template <int MAJA, int MAJB, int BKT>
int launch_big_variant(const KernelParams& kp, int grid, cudaStream_t stream, char* err, int errlen) {
    constexpr int smem = BIG_SMEM;
    auto kern = gemm_tf32_big_kernel<MAJA, MAJB, BKT>;
    static bool attr_done_dev[kMaxDev] = {};
    bool& attr_done = attr_done_dev[cur_dev()];
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            seterr(err, errlen, cudaGetErrorString(e));
            return -3;
        }
        attr_done = true;
    }
    launch_pdl(kern, grid, BIG_THREADS, smem, stream, kp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        seterr(err, errlen, cudaGetErrorString(e));
        return -3;
    }
    return 0;
}
#endif

// The three kernels on CTA pairs: the fp32-accurate one, TF32 with 256 x 256 tiles, TF32 with 512 x 256 tiles.
enum PairKind { PAIR_FP32 = 0, PAIR_DUO = 1, PAIR_QUAD = 2, PAIR_FP32_SHORT = 3 };
template <int KIND, int MAJA, int MAJB, int BKT = BK>
int launch_pair_variant(const KernelParams& kp, int grid, cudaStream_t stream, char* err, int errlen) {
    constexpr int smem = KIND == PAIR_QUAD ? QUAD_SMEM
                         : KIND == PAIR_DUO
                             ? DUO_SMEM
                             : PAIR_SMEM_TILES + 1024 + PAIR_BAR_BYTES;
    constexpr int threads = KIND == PAIR_QUAD ? QUAD_THREADS : (KIND == PAIR_DUO ? DUO_THREADS : PAIR_THREADS);
    auto kern = KIND == PAIR_QUAD ? gemm_tf32_quad_kernel<MAJA, MAJB, BKT>
                                  : (KIND == PAIR_DUO ? gemm_tf32_duo_kernel<MAJA, MAJB>
                                                      : gemm_tf32_pair_kernel<MAJA, MAJB, (KIND == PAIR_FP32_SHORT ? 2 : 3)>);
    static bool attr_done_dev[kMaxDev] = {};
    bool& attr_done = attr_done_dev[cur_dev()];
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            seterr(err, errlen, cudaGetErrorString(e));
            return -3;
        }
        attr_done = true;
    }
    // How many 2-CTA clusters can be resident at once (SM counts per GPC need not be even).
    static int max_pairs_dev[kMaxDev] = {};
    int& max_pairs = max_pairs_dev[cur_dev()];
    if (max_pairs == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 74);
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 64;
        }
        max_pairs = n;
#ifdef AKR_B200_DIAG
        if (std::getenv("AKR_B200_VERBOSE")) std::fprintf(stderr, "akr_b200: %d CTA pairs resident (%s kernel)\n", n, KIND == PAIR_QUAD ? "tf32 512x256 pair" : (KIND == PAIR_DUO ? "tf32 pair" : "fp32 pair"));
#endif
    }
    if (grid > 2 * max_pairs) grid = 2 * max_pairs;
    launch_pdl(kern, grid, threads, smem, stream, kp);  // cluster of 2 CTAs (compile-time cluster dims)
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        seterr(err, errlen, cudaGetErrorString(e));
        return -3;
    }
    return 0;
}

// An output every kernel can store through TMA boxes: 16-byte aligned rows, nothing added to or applied on the product.
bool plain_aligned_output(const GemmDesc& g) {
    const bool vec_ok = (reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.ldc & 3) == 0 && (g.o0 == 1 || (g.c_bs0 & 3) == 0) &&
                        (g.o1 == 1 || (g.c_bs1 & 3) == 0);
    return vec_ok && !g.accumulate && g.aux_op == 0 && g.alpha == 1.f && g.splits <= 1 && g.colpart == nullptr;
}

// CTA pairs serve the fp32-accurate mode wherever 256 x 256 tiles fill a good part of the machine and the
// contraction is long enough to amortise the pair's hand-shakes: each CTA reads only half of B per MMA and converts
// only its own share, which is what this shared-memory-bound mode needs (2560^3: 0.253 -> 0.183 ms, 4096 x 1024 x
// 4096: 0.185 -> 0.147 ms, 64 x (512 x 512 x 2048): 0.369 -> 0.312 ms against one CTA per 128 x 256 tile). Short
// contractions (below 256; below 64 when the output can leave through TMA) stay with the general kernel. Debug bit 5
// routes every eligible shape here.
bool use_pairs(const GemmDesc& g) {
    if (g.terms != 3 || g.M <= 128 || g.N <= 128 || AKR_DIAG(g.debug, 512)) return false;
    // split contractions too, when a reduction kernel adds the partial tiles up (no tile counters)
    if (g.splits > 1 && (g.counters != nullptr || AKR_DIAG(g.debug, 524288))) return false;
    const long long tiles = (long long)g.o0 * g.o1 * ((g.M + PAIR_BM - 1) / PAIR_BM) * ((g.N + PAIR_BN - 1) / PAIR_BN) *
                            (g.splits > 1 ? g.splits : 1);
    if (tiles * 4 < gemm_sm100_num_ctas()) return false;
    const long long iters = (long long)g.red * ((g.K + PAIR_BK - 1) / PAIR_BK);
    // Contractions of 256 and more (8 k-blocks): 8192 x 256^3 4.5 against 5.1 ms per fwd + dA + dB step, 1024 x 512 x 512 x
    // 256 2.0 against 2.1-2.4 ms; at 128 the two kernels were level while the pair kernel stored with st.global. With
    // its output leaving through TMA boxes it wins from a contraction of 64 on (512 x (512 x 512 x K), K = 64 / 96 /
    // 128 / 200: 0.135 -> 0.127, 0.184 -> 0.160, 0.222 -> 0.193, 0.318 -> 0.286 ms; 8192 x 8192 x 128: 0.108 -> 0.091).
    return iters >= 8 || (iters >= 2 && plain_aligned_output(g)) || (g.debug & 32);
}

// TF32 mode on CTA pairs (256 x 256 tiles, eight MMAs per 64-deep stage, the epilogue of a tile overlapping the next
// one's MMAs). Over many waves of long contractions the kernels whose tiles fill the tensor memory move fewer bytes per
// flop and win (8192^3: 1.35 against 1.48 ms, 4096^3: 0.186 against 0.197); everywhere else this one does:
//   contractions of 1024 .. 2047 at any tile count, longer ones when the 256 x 256 tiles do not fill the SMs
//   (2048^3: 0.0259 ms against 0.0315 on 128 x 256 tiles of single CTAs, 4096 x 1024 x 4096: 0.0514 against 0.0563);
//   contractions of 256 .. 1023 when the tiles keep every pair busy and the product is compute-bound
//   (3072 x 3072 x 512: 0.0176 against 0.0206 ms, 8192 x 8192 x 512: 0.113 against 0.133, 2048 x 2048 x 512 with its
//   64 tiles: 0.0130 against 0.0139).
// Debug bit 10 disables it (diagnostic builds), bit 11 prefers it wherever it is applicable.
bool use_duo(const GemmDesc& g) {
    if (g.terms != 1 || g.M <= 128 || g.N <= 128 || AKR_DIAG(g.debug, 1024)) return false;
    // split contractions too (each pair takes a share of the k-steps of a tile), when a reduction kernel adds the
    // partial tiles up; the single-launch form with tile counters stays with the one-CTA kernel
    if (g.splits > 1 && (g.counters != nullptr || AKR_DIAG(g.debug, 524288))) return false;
    const long long tiles = (long long)g.o0 * g.o1 * ((g.M + PAIR_BM - 1) / PAIR_BM) * ((g.N + PAIR_BN - 1) / PAIR_BN) *
                            (g.splits > 1 ? g.splits : 1);
    const long long iters = (long long)g.red * ((g.K + BK - 1) / BK);
    const int ctas = gemm_sm100_num_ctas();
    if (tiles * 16 < ctas) return false;  // from ten tiles on (1536^3, 36 tiles: 0.0240 -> 0.0202 ms; 1024^3, 16: 0.0162 -> 0.0157)
    if (g.debug & 2048) return true;
    if (iters >= 32) return tiles < ctas || iters < 64;
    // Short contractions only when the product is compute-bound: at 2 M N K / 4 (MK + KN + MN) below about 80 flop per
    // byte (batches of 256^3: 43) the three-stage kernel with its per-warp store boxes is the faster streamer
    // (8192 x 256^3: 0.93-0.98 ms per product against 1.01).
    const double flop_per_byte = 2.0 * g.M * g.N * g.K / (4.0 * ((double)g.M * g.K + (double)g.K * g.N + (double)g.M * g.N));
    return iters >= 8 && tiles * 4 >= ctas && flop_per_byte >= 80.0;
}

// 256 x 256 tiles pay off when they alone fill the machine and the contraction is long enough to
// amortise the accumulator hand-over between tiles.
bool use_big_tiles(const GemmDesc& g) {
    if (g.terms != 1 || g.splits > 1 || AKR_DIAG(g.debug, 8)) return false;
    const long long tiles = (long long)g.o0 * g.o1 * ((g.M + BIG_BM - 1) / BIG_BM) * ((g.N + BIG_BN - 1) / BIG_BN);
    const long long iters = (long long)g.red * ((g.K + BK - 1) / BK);
    return tiles >= gemm_sm100_num_ctas() && iters >= 32;
}

// 512 x 256 tiles on CTA pairs wherever 256 x 256 tiles on single CTAs would be chosen and the taller tiles
// still give every pair one: a quarter fewer operand bytes into shared memory per flop. Debug bit 13 keeps the
// single-CTA kernel (diagnostic builds).
bool use_quad(const GemmDesc& g) {
    if (!use_big_tiles(g) || AKR_DIAG(g.debug, 8192)) return false;
    const long long tiles = (long long)g.o0 * g.o1 * ((g.M + QUAD_BM - 1) / QUAD_BM) * ((g.N + QUAD_BN - 1) / QUAD_BN);
    return tiles * 2 >= gemm_sm100_num_ctas();
}

int pick_bn(const GemmDesc& g) {
    // Wide tiles when there is enough work to fill the machine with them, else narrow ones.
    if (g.N <= 64) return 64;
    if (g.N <= 128) return 128;
    // A split contraction was sized (gemm_sm100_pick_splits) for 256-wide tiles: keep them, so that
    // tiles x splits stays one balanced wave of CTAs.
    if (g.splits > 1) return 256;
    // Otherwise compare waves of CTAs: a 256-wide tile does twice the work of a 128-wide one, which in
    // turn moves more operand bytes per flop (modelled as a 15 % penalty).
    const long long rows = (long long)g.o0 * g.o1 * ((g.M + BM - 1) / BM);
    const long long t256 = rows * ((g.N + 255) / 256), t128 = rows * ((g.N + 127) / 128);
    const long long ctas = gemm_sm100_num_ctas();
    const double cost256 = 2.0 * (double)((t256 + ctas - 1) / ctas);
    const double cost128 = 1.15 * (double)((t128 + ctas - 1) / ctas);
    return cost256 <= cost128 ? 256 : 128;
}

}  // namespace

static int g_cta_limit = 0;
static double g_split_ratio = 0.0;  // tuning override (environment AKR_B200_SPLIT_RATIO), 0 = built-in
static int g_debug_flags = 0;
static unsigned long long g_wait_limit_ns = DEFAULT_WAIT_LIMIT_NS;

void gemm_sm100_debug_configure(int flags, unsigned wait_limit_ms) {
#ifdef AKR_B200_DIAG
    if (const char* r = std::getenv("AKR_B200_SPLIT_RATIO")) g_split_ratio = std::atof(r);
#endif
    g_debug_flags = flags;
    g_pdl_off = AKR_DIAG(flags, 4096);
    g_wait_limit_ns = wait_limit_ms ? (unsigned long long)wait_limit_ms * 1000000ull : DEFAULT_WAIT_LIMIT_NS;
}

void gemm_sm100_set_cta_limit(int ctas) { g_cta_limit = ctas > 0 ? ctas : 0; }
namespace {
bool gemm_sm100_cta_limit_active() { return g_cta_limit > 0; }
}  // namespace

int gemm_sm100_num_ctas() {
    static int sms_dev[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    int& sms = sms_dev[dev];
    if (sms == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        sms = v;
    }
    return (g_cta_limit > 0 && g_cta_limit < sms) ? g_cta_limit : sms;
}

bool gemm_sm100_operand_ok(const GemmOperand& op, int mn, int k, const int batch[3]) {
    if ((reinterpret_cast<uintptr_t>(op.ptr) & 15u) != 0) return false;
    const int other = op.mn_major ? k : mn;
    if (other > 1 && (op.ld <= 0 || (op.ld & 3) != 0)) return false;
    for (int i = 0; i < 3; ++i) {
        if (batch[i] > 1 && op.bs[i] != 0 && ((op.bs[i] & 3) != 0 || op.bs[i] < 0)) return false;
    }
    return true;
}

int gemm_sm100_pick_splits(const GemmDesc& g) {
    const int bn = g.N <= 64 ? 64 : (g.N <= 128 ? 128 : 256);
    const long long tiles = (long long)g.o0 * g.o1 * ((g.M + BM - 1) / BM) * ((g.N + bn - 1) / bn);
    const long long iters = (long long)g.red * ((g.K + BK - 1) / BK);
    const int ctas = gemm_sm100_num_ctas();
    // The fp32-accurate mode spends three times as long per k-block, so splitting pays for shorter contractions
    // there (measured: 1024^3 36.6 -> 25.3 us, 768^3 28.8 -> 19.6 us; TF32 mode gains nothing below 64 k-blocks).
    // (TF32 with very few tiles - at most a quarter of the SMs busy - splits from 32 k-blocks on, 8 left per split:
    // 768 x 768 x 1536 0.0217 -> 0.0159 ms, 512 x 512 x 1024 0.0161 -> 0.0128; with more tiles that costs: 1536 x 1536 x
    // 1024 0.0160 -> 0.0210.)
    const bool few = tiles * 4 <= ctas;
    const int min_iters = g.terms == 3 ? 16 : (few ? 32 : 64);
    const int min_per = g.terms == 3 ? 4 : (few ? 8 : 16);  // k-blocks (of 32) left to one split at least
    if (tiles * 2 > ctas || iters < min_iters) return 1;
    long long s = ctas / tiles;
    const long long max_by_work = iters / min_per;
    if (s > max_by_work) s = max_by_work;
    // (With tile counters, i.e. the single-launch variant, the last CTA of a tile adds up all its partials
    // alone, which costs about as much per partial as ten k-blocks: that caller should also cap the count
    // near sqrt(0.2 * iters).)
    if (g_split_ratio > 0.0) {
        const long long s_bal = (long long)(std::sqrt(g_split_ratio * (double)iters) + 0.5);
        if (s > s_bal) s = s_bal;
    }
    if (s > 64) s = 64;
    return s < 1 ? 1 : (int)s;
}

void gemm_sm100_split_scratch(const GemmDesc& g, size_t* partial_bytes, size_t* counter_count) {
    const int bn = pick_bn(g);
    const size_t tiles = (size_t)g.o0 * g.o1 * ((g.M + BM - 1) / BM) * ((g.N + bn - 1) / bn);
    *partial_bytes = g.splits > 1 ? (size_t)g.splits * g.o0 * g.o1 * g.M * g.N * sizeof(float) : 0;
    *counter_count = g.splits > 1 ? tiles : 0;
}

// Split contraction without tile counters: the partial tiles are added up by a second, GPU-wide kernel.
static int launch_split_reduce(const GemmDesc& g, const KernelParams& kp, cudaStream_t stream, char* err, int errlen) {
    SplitReduceParams rp;
    std::memset(&rp, 0, sizeof(rp));
    rp.partials = g.partials;
    rp.C = g.C;
    rp.bias = g.bias;
    rp.aux = g.aux_op ? g.aux : nullptr;
    rp.ldc = g.ldc; rp.c_bs0 = g.c_bs0; rp.c_bs1 = g.c_bs1;
    rp.aux_ld = g.aux_ld; rp.aux_cs = g.aux_cs; rp.aux_bs0 = g.aux_bs0; rp.aux_bs1 = g.aux_bs1;
    rp.M = g.M; rp.N = g.N; rp.o1 = g.o1; rp.nbatch = g.o0 * g.o1; rp.splits = kp.splits;
    rp.accumulate = g.accumulate; rp.aux_op = g.aux_op;
    rp.alpha = g.alpha; rp.beta = g.beta;
    const bool vec = kp.vec_ok && (g.N & 3) == 0;
    const size_t work = (size_t)rp.nbatch * g.M * (size_t)(vec ? g.N / 4 : g.N);
    size_t blocks = (work + 255) / 256;
    const size_t cap = (size_t)gemm_sm100_num_ctas() * 8;
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (g_pdl_off || gemm_sm100_cta_limit_active()) ? 0 : 1;
    if (vec) cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<true>, rp);
    else cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<false>, rp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        seterr(err, errlen, cudaGetErrorString(e));
        return -3;
    }
    return 0;
}

// What the clock probe recorded for the last GEMM launch of the current device: per-CTA cycles and nanoseconds.
int gemm_sm100_clock_read(int ctas, double* mhz_mean, double* mhz_min, double* cycles_max, double* us_max) {
    static unsigned long long h[2 * 256];
    if (ctas < 1) ctas = 1;
    if (ctas > 256) ctas = 256;
    if (cudaMemcpyFromSymbol(h, g_clock_probe, sizeof(h)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    double sum = 0, mn = 1e30, um = 0, cm = 0;
    int n = 0;
    for (int i = 0; i < ctas; ++i) {
        if (h[2 * i + 1] == 0) continue;
        const double mhz = 1e3 * (double)h[2 * i] / (double)h[2 * i + 1];
        sum += mhz;
        ++n;
        if (mhz < mn) mn = mhz;
        if ((double)h[2 * i + 1] * 1e-3 > um) um = (double)h[2 * i + 1] * 1e-3;
        if ((double)h[2 * i] > cm) cm = (double)h[2 * i];
    }
    if (n == 0) return -2;
    if (mhz_mean) *mhz_mean = sum / n;
    if (mhz_min) *mhz_min = mn;
    if (cycles_max) *cycles_max = cm;
    if (us_max) *us_max = um;
    return 0;
}

int gemm_sm100_launch(const GemmDesc& g, cudaStream_t stream, int* status_dev, char* err,
                      int errlen) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.o0 <= 0 || g.o1 <= 0 || g.red <= 0) {
        seterr(err, errlen, "gemm_sm100: empty problem");
        return -1;
    }
    const int batch[3] = {g.o0, g.o1, g.red};
    if (!gemm_sm100_operand_ok(g.A, g.M, g.K, batch) || !gemm_sm100_operand_ok(g.B, g.N, g.K, batch)) {
        seterr(err, errlen, "gemm_sm100: operand not readable by TMA (alignment / stride)");
        return -1;
    }
    if (g.aux_op != 0 && (!g.aux || g.terms != 1)) {
        seterr(err, errlen, "gemm_sm100: second epilogue operand missing, or requested in the fp32-accurate mode");
        return -1;
    }
    if (g.splits > 1 && !g.partials) {
        seterr(err, errlen, "gemm_sm100: split launch without scratch");
        return -1;
    }
    GemmDesc gd = g;
    gd.debug |= g_debug_flags;
    const bool duo = use_duo(gd);
    const bool quad = !duo && use_quad(gd);
    // (the 256 x 256 single-CTA kernel: wherever it would apply, the 512 x 256 pair tiles do too; diagnostic builds keep it)
    const bool big = AKR_DIAG(gd.debug, 8192) && !duo && !quad && use_big_tiles(gd);
    const bool pairs = duo || quad || use_pairs(gd);
    const int bn = big ? BIG_BN : (quad ? QUAD_BN : (pairs ? PAIR_BN : pick_bn(g)));
    const int bm = big ? BIG_BM : (quad ? QUAD_BM : (pairs ? PAIR_BM : BM));
    // 16-deep k-blocks: finer stages for the hi+lo mode. The large-tile TF32 kernels keep 32-deep ones: twice as
    // many stage hand-overs cost them 16 % at 8192^3 (debug bit 14 selects the finer ring in diagnostic builds).
    const bool fine = (big || quad) && AKR_DIAG(gd.debug, 16384);
    // fp32-accurate tiles of 64 and 128 columns take 32-deep k-blocks (128-byte rows): with 16-deep ones the TMA unit
    // moves twice as many rows per byte and the ring hands over twice as often (config 3's dA, N = 64: 0.216 -> 0.158
    // ms; 65536 x 128 x 1024: 0.138 -> 0.112 ms). 256-wide tiles have no room for 32-deep raw stages plus low-part slots.
    const bool fp32_wide_k = g.terms == 3 && !pairs && pick_bn(g) <= 128;
    // TF32 tiles of 128 columns take 64-deep k-blocks (two 32-deep sub-tiles per operand) from a contraction of 512:
    // their MMAs take 64 cycles, and a stage of four of them is over before it has been handed over (16384 x 128 x
    // 4096: 0.0545 -> 0.0534 ms; 4096 x 128 x 16384: 0.0609 -> 0.0593 ms). Shorter contractions want the extra stages
    // of the 32-deep ring, and 64-column tiles measured the same either way.
    const bool tf32_deep_k = g.terms == 1 && !pairs && !big && pick_bn(g) == 128 && g.K >= 512 && !AKR_DIAG(gd.debug, 2097152);
    const int bk = (g.terms == 3 && pairs) ? PAIR_BK : (tf32_deep_k ? 64 : (((g.terms == 3 && !fp32_wide_k) || fine) ? 16 : BK));

    KernelParams kp;
    std::memset(&kp, 0, sizeof(kp));
    MapPlan pa = plan_map(g.A, g.M, batch, !AKR_DIAG(g.debug, 4));
    MapPlan pb = plan_map(g.B, g.N, batch, !AKR_DIAG(g.debug, 4));
    const int box_k = bk > 32 ? 32 : bk;  // a deeper k-block is fetched as 32-deep sub-tiles
    auto build = [&](CUtensorMap* map, const GemmOperand& op, MapPlan& mp, int mn, int tile) {
        bool ok = make_map(map, op.ptr, op, mp, mn, g.K, tile, box_k);
        if (!ok && mp.fold) {  // the folded form is an optimisation: fall back to one box per chunk
            mp.fold = false;
            ok = make_map(map, op.ptr, op, mp, mn, g.K, tile, box_k);
        }
        return ok;
    };
    // rows of A / columns of B one TMA box brings: a CTA of a pair loads its own share of the pair's tile
    if (!build(&kp.tmA, g.A, pa, g.M, quad ? 256 : (pairs ? 128 : bm)) || !build(&kp.tmB, g.B, pb, g.N, pairs ? 128 : bn)) {
        seterr(err, errlen, "gemm_sm100: cuTensorMapEncodeTiled failed");
        return -2;
    }
    kp.a_fold = pa.fold ? 1 : 0;
    kp.b_fold = pb.fold ? 1 : 0;
    for (int i = 0; i < 3; ++i) {
        kp.a_sel[i] = pa.sel[i];
        kp.b_sel[i] = pb.sel[i];
    }
    kp.C = g.C;
    kp.bias = g.bias;
    kp.aux = g.aux_op ? g.aux : nullptr;
    kp.aux_op = g.aux_op;
    kp.aux_ld = g.aux_ld;
    kp.aux_cs = g.aux_cs;
    kp.aux_bs0 = g.aux_bs0;
    kp.aux_bs1 = g.aux_bs1;
    kp.aux_vec = (g.aux_op && g.aux_cs == 1 && (reinterpret_cast<uintptr_t>(g.aux) & 15u) == 0 && (g.aux_ld & 3) == 0 &&
                  (g.o0 == 1 || (g.aux_bs0 & 3) == 0) && (g.o1 == 1 || (g.aux_bs1 & 3) == 0))
                     ? 1
                     : 0;
    kp.alpha = g.alpha;
    kp.beta = g.beta;
    kp.partials = g.partials;
    kp.counters = g.counters;
    kp.colpart = g.colpart;
    kp.status = status_dev;
    kp.ldc = g.ldc;
    kp.c_bs0 = g.c_bs0;
    kp.c_bs1 = g.c_bs1;
    kp.M = g.M;
    kp.N = g.N;
    kp.K = g.K;
    kp.o0 = g.o0;
    kp.o1 = g.o1;
    kp.red = g.red;
    kp.splits = g.splits < 1 ? 1 : g.splits;
    kp.accumulate = g.accumulate;
    kp.vec_ok = ((reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.ldc & 3) == 0 &&
                 (g.o0 == 1 || (g.c_bs0 & 3) == 0) && (g.o1 == 1 || (g.c_bs1 & 3) == 0))
                    ? 1
                    : 0;
    // Output map for the TMA-store epilogue: (N, M, o1, o0), boxes of 32 columns x 128 rows.
    kp.c_tma = 0;
    if (g.colpart != nullptr && (g.terms != 1 || kp.splits != 1)) {
        seterr(err, errlen, "gemm_sm100: column sums of the output are produced by the TF32 kernels without a split contraction only");
        return -1;
    }
    if (kp.vec_ok && !g.accumulate && g.aux_op == 0 && g.alpha == 1.f && kp.splits == 1 && g.colpart == nullptr &&
        !AKR_DIAG(g.debug | g_debug_flags, 256)) {
        EncodeTiledFn enc = get_encode_fn();
        const uint64_t ldc_b = (uint64_t)(g.M > 1 ? g.ldc : ((g.N + 3) / 4) * 4) * 4;
        cuuint64_t dims[4] = {(cuuint64_t)g.N, (cuuint64_t)g.M, (cuuint64_t)g.o1, (cuuint64_t)g.o0};
        cuuint64_t strides[3] = {ldc_b, (cuuint64_t)(g.o1 > 1 ? g.c_bs1 * 4 : (long long)ldc_b),
                                 (cuuint64_t)(g.o0 > 1 ? g.c_bs0 * 4 : (long long)ldc_b)};
        // the three-stage instantiation for short contractions sends one box per warp (32 rows)
        const bool warp_boxes = !big && !pairs && bn == 256 && (long long)g.red * ((g.K + bk - 1) / bk) <= 8;
        cuuint32_t box[4] = {32u, warp_boxes ? 32u : 128u, 1u, 1u};
        cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
        if (enc && enc(&kp.tmC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, g.C, dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            kp.c_tma = 1;
    }
    kp.mt = (g.M + bm - 1) / bm;
    kp.nt = (g.N + bn - 1) / bn;
    kp.nkb = (g.K + bk - 1) / bk;
    const long long total = (long long)g.o0 * g.o1 * kp.mt * kp.nt * kp.splits;
    if (total > 0x7fffffffLL) {
        seterr(err, errlen, "gemm_sm100: too many tiles");
        return -1;
    }
    if ((long long)kp.red * kp.nkb < kp.splits) {
        seterr(err, errlen, "gemm_sm100: more splits than contraction steps");
        return -1;
    }
    kp.total_tiles = (int)total;
    kp.debug = g.debug | g_debug_flags;
    kp.wait_limit_ns = g_wait_limit_ns;
    const int ctas = gemm_sm100_num_ctas();
    const int grid = (int)(total < ctas ? total : ctas);

    if (pairs) {
        const int npairs = (int)std::min<long long>(total, ctas / 2);
        const int sel = g.A.mn_major * 2 + g.B.mn_major;
        if (quad) {
            switch (sel + (fine ? 4 : 0)) {
                case 0: return launch_pair_variant<PAIR_QUAD, 0, 0, 32>(kp, 2 * npairs, stream, err, errlen);
                case 1: return launch_pair_variant<PAIR_QUAD, 0, 1, 32>(kp, 2 * npairs, stream, err, errlen);
                case 2: return launch_pair_variant<PAIR_QUAD, 1, 0, 32>(kp, 2 * npairs, stream, err, errlen);
                case 3: return launch_pair_variant<PAIR_QUAD, 1, 1, 32>(kp, 2 * npairs, stream, err, errlen);
#ifdef AKR_B200_DIAG
                case 4: return launch_pair_variant<PAIR_QUAD, 0, 0, 16>(kp, 2 * npairs, stream, err, errlen);
                case 5: return launch_pair_variant<PAIR_QUAD, 0, 1, 16>(kp, 2 * npairs, stream, err, errlen);
                case 6: return launch_pair_variant<PAIR_QUAD, 1, 0, 16>(kp, 2 * npairs, stream, err, errlen);
                default: return launch_pair_variant<PAIR_QUAD, 1, 1, 16>(kp, 2 * npairs, stream, err, errlen);
#else
                default: return -1;
#endif
            }
        }
        if (duo) {
            int rcd;
            switch (sel) {
                case 0: rcd = launch_pair_variant<PAIR_DUO, 0, 0>(kp, 2 * npairs, stream, err, errlen); break;
                case 1: rcd = launch_pair_variant<PAIR_DUO, 0, 1>(kp, 2 * npairs, stream, err, errlen); break;
                case 2: rcd = launch_pair_variant<PAIR_DUO, 1, 0>(kp, 2 * npairs, stream, err, errlen); break;
                default: rcd = launch_pair_variant<PAIR_DUO, 1, 1>(kp, 2 * npairs, stream, err, errlen); break;
            }
            if (rcd != 0 || kp.splits == 1) return rcd;
            return launch_split_reduce(g, kp, stream, err, errlen);
        }
        int rcp;
        // contractions of at most 512 that store through TMA: two low-part slots, two sets of staging tiles
        const bool short_pair = kp.c_tma != 0 && (long long)kp.red * kp.nkb <= 16 && !AKR_DIAG(gd.debug, 4194304);
        if (short_pair) {
            switch (sel) {
                case 0: rcp = launch_pair_variant<PAIR_FP32_SHORT, 0, 0>(kp, 2 * npairs, stream, err, errlen); break;
                case 1: rcp = launch_pair_variant<PAIR_FP32_SHORT, 0, 1>(kp, 2 * npairs, stream, err, errlen); break;
                case 2: rcp = launch_pair_variant<PAIR_FP32_SHORT, 1, 0>(kp, 2 * npairs, stream, err, errlen); break;
                default: rcp = launch_pair_variant<PAIR_FP32_SHORT, 1, 1>(kp, 2 * npairs, stream, err, errlen); break;
            }
            return rcp;
        }
        switch (sel) {
            case 0: rcp = launch_pair_variant<PAIR_FP32, 0, 0>(kp, 2 * npairs, stream, err, errlen); break;
            case 1: rcp = launch_pair_variant<PAIR_FP32, 0, 1>(kp, 2 * npairs, stream, err, errlen); break;
            case 2: rcp = launch_pair_variant<PAIR_FP32, 1, 0>(kp, 2 * npairs, stream, err, errlen); break;
            default: rcp = launch_pair_variant<PAIR_FP32, 1, 1>(kp, 2 * npairs, stream, err, errlen); break;
        }
        if (rcp != 0 || kp.splits == 1) return rcp;
        return launch_split_reduce(g, kp, stream, err, errlen);
    }
#ifdef AKR_B200_DIAG
    if (big) {
        switch (g.A.mn_major * 2 + g.B.mn_major + (fine ? 4 : 0)) {
            case 0: return launch_big_variant<0, 0, 32>(kp, grid, stream, err, errlen);
            case 1: return launch_big_variant<0, 1, 32>(kp, grid, stream, err, errlen);
            case 2: return launch_big_variant<1, 0, 32>(kp, grid, stream, err, errlen);
            case 3: return launch_big_variant<1, 1, 32>(kp, grid, stream, err, errlen);
            case 4: return launch_big_variant<0, 0, 16>(kp, grid, stream, err, errlen);
            case 5: return launch_big_variant<0, 1, 16>(kp, grid, stream, err, errlen);
            case 6: return launch_big_variant<1, 0, 16>(kp, grid, stream, err, errlen);
            default: return launch_big_variant<1, 1, 16>(kp, grid, stream, err, errlen);
        }
    }
#endif
    // fp32-accurate mode: 16-deep k-blocks, chains of 4 of them (64 deep) inside the tensor core.
    int rc;
    if (g.terms == 3) {
        // raw stages (24 KB of 16-deep k-blocks for 256-wide tiles, 32 / 24 KB of 32-deep ones for 128- / 64-wide tiles)
        // in flight from HBM + a short ring of low-part tiles
        // A low-part slot is busy from its conversion until its MMAs have finished and the commit has arrived:
        // the narrower the tile, the shorter that work and the more slots it takes to cover the hand-over latency.
        const bool short_k = (long long)kp.red * kp.nkb <= 8 && kp.splits == 1;
        rc = bn == 256 ? (short_k ? launch_major<256, 3, 4, 4, 16, 2>(g, kp, grid, stream, err, errlen)
                                  : launch_major<256, 3, 5, 4, 16, 3>(g, kp, grid, stream, err, errlen))
             : bn == 128 ? launch_major<128, 3, 4, 2, 32, 2>(g, kp, grid, stream, err, errlen)
                         : launch_major<64, 3, 6, 2, 32, 2>(g, kp, grid, stream, err, errlen);
    } else if (bn == 64) {
        rc = launch_major<64, 1, 8, 0, 32>(g, kp, grid, stream, err, errlen);
    } else if (bn == 128 && tf32_deep_k) {
        rc = launch_major<128, 1, 3, 0, 64>(g, kp, grid, stream, err, errlen);
    } else {
        // Short contractions are write-heavy: three stages are plenty and leave room for a second set of
        // epilogue staging tiles.
        const bool short_k = (long long)kp.red * kp.nkb <= 8 && kp.splits == 1;
        rc = bn == 256 ? (short_k ? launch_major<256, 1, 3, 0, 32>(g, kp, grid, stream, err, errlen)
                                  : launch_major<256, 1, 4, 0, 32>(g, kp, grid, stream, err, errlen))
                       : launch_major<128, 1, 6, 0, 32>(g, kp, grid, stream, err, errlen);
    }
    if (rc != 0 || kp.splits == 1 || g.counters != nullptr) return rc;

    return launch_split_reduce(g, kp, stream, err, errlen);
}

}  // namespace akr
