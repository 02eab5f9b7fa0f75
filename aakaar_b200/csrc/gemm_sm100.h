// Host-side description of one batched fp32 GEMM for the sm_100a tcgen05 kernels.
//
//   D[o0, o1, m, n] = op( alpha * sum_r sum_k A[o0, o1, r, m, k] * B[o0, o1, r, k, n] (+ D) (+ bias[n]) )
//   op: identity, `+ beta * X[o0, o1, m, n]` or `* (1 - X[o0, o1, m, n]^2)` with a second array X
//
// o0/o1 are output batch dims, r is a batch dim that is summed away (the broadcast-batch
// reduction of a weight gradient). An operand that does not vary along a batch dim has
// stride 0 there. Either matrix dim of an operand may be the unit-stride one: the kernels read
// transposed views in place.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace akr {

struct GemmOperand {
    const float* ptr = nullptr;  // first element of the view
    int mn_major = 0;            // 1: the M (for A) / N (for B) index is unit stride; 0: K is
    int64_t ld = 0;              // element stride of the other matrix dim
    int64_t bs[3] = {0, 0, 0};   // element strides along o0, o1, r (0 = broadcast)
};

struct GemmDesc {
    int M = 0, N = 0, K = 0;
    int o0 = 1, o1 = 1, red = 1;  // batch extents
    GemmOperand A, B;
    float* C = nullptr;
    int64_t ldc = 0, c_bs0 = 0, c_bs1 = 0;
    const float* bias = nullptr;  // optional row vector of N values added to every row
    int accumulate = 0;           // 1: C += result
    float alpha = 1.f;            // scales the product
    // Second epilogue operand X (shape of the output, own strides; aux_cs is its column stride):
    // aux_op 1: result += beta * X; aux_op 2: result *= 1 - X^2 (gradient through a saved tanh output).
    const float* aux = nullptr;
    int aux_op = 0;
    float beta = 0.f;
    int64_t aux_ld = 0, aux_cs = 1, aux_bs0 = 0, aux_bs1 = 0;
    // Optional by-product: column sums of the stored output per 32-row block, `colpart` = [o0 * o1 * ceil(M / 32)][N]
    // floats (every entry is written). TF32 mode without a split contraction only.
    float* colpart = nullptr;
    int terms = 1;                // 1 = TF32, 3 = 3xTF32 (fp32-accurate; the low parts are derived in the kernel)
    // Split of the contraction across CTAs (weight gradients with few output tiles):
    // splits > 1 writes fp32 partials to `partials` ([splits][o0*o1][M][N]); they are added up in split
    // order (deterministic) by a second, GPU-wide kernel launched right behind the GEMM - or, when the
    // caller passes `counters` (one zeroed int per output tile, left at zero), inside the GEMM by the last
    // CTA to finish each tile: a single launch, slower for many splits.
    int splits = 1;
    float* partials = nullptr;
    int* counters = nullptr;
    int debug = 0;  // hooks: bit 0 skips the TMA loads (MMA-only timing, results invalid), bit 4 makes the load
                    // warp never signal (bounded-wait test), bit 5 routes fp32-accurate products through the CTA-pair
                    // kernel wherever its tiles apply, bit 11 prefers the TF32 256 x 256 CTA-pair kernel wherever it
                    // applies, bit 15 is the clock probe (gemm_sm100_clock_read).
                    // Builds with -DAKR_B200_DIAG add timing experiments: bit 1 skips the MMAs, bit 2 disables the
                    // folded one-box-per-tile maps, bit 3 the 256 x 256 tile kernel, bit 6 one chain per tile in the
                    // fp32 pair kernel, bit 7 skips the output stores, bit 8 disables the TMA-store epilogue, bit 9
                    // the fp32 CTA-pair kernel, bit 10 the TF32 CTA-pair kernel, bit 12 dependent launch, bit 13 the
                    // 512 x 256 pair tiles, bit 14 selects 16-deep k-blocks in the large-tile TF32 kernels.
};

// True when the operand can be read by TMA as it lies (16-byte aligned base, unit stride on one
// matrix dim, every other stride a multiple of 4 elements).
bool gemm_sm100_operand_ok(const GemmOperand& op, int mn, int k, const int batch[3]);

// Enqueue on `stream`. `status_dev` points at one device int that the kernel sets non-zero when a
// bounded wait ran out. Returns 0, or a negative akr status with the message in `err`.
int gemm_sm100_launch(const GemmDesc& g, cudaStream_t stream, int* status_dev, char* err,
                      int errlen);

// Number of CTAs the persistent kernels are launched with on the current device
// (the SM count, or the lower limit set below).
int gemm_sm100_num_ctas();
// Caps the persistent grid (0 = one CTA per SM).
void gemm_sm100_set_cta_limit(int ctas);
// Test hooks: extra GemmDesc::debug bits for every launch, and the bound of every in-kernel wait
// (0 = default, 4 s).
void gemm_sm100_debug_configure(int flags, unsigned wait_limit_ms);
// Clock probe (debug bit 15): SM clock (mean / min over the first `ctas` CTAs, MHz), longest CTA in cycles and in
// microseconds, of the last GEMM launch on the current device. -1: read failed, -2: nothing recorded.
int gemm_sm100_clock_read(int ctas, double* mhz_mean, double* mhz_min, double* cycles_max, double* us_max);

// Bytes of `partials` and number of `counters` entries a split launch needs.
void gemm_sm100_split_scratch(const GemmDesc& g, size_t* partial_bytes, size_t* counter_count);

// Picks a split factor for `g` (1 when the output already fills the GPU).
int gemm_sm100_pick_splits(const GemmDesc& g);

}  // namespace akr
