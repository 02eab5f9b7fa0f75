// Micro-benchmark of the tcgen05.mma kind::tf32 instruction stream on sm_100a, one CTA (or one CTA pair), no loads:
// the facts the GEMM kernels' issue loops are built on.
//   1. n MMAs of 128 x 256 x 8 (pair: 256 x 256 x 8 over two CTAs) issued back to back, one tcgen05.commit at the end:
//      cycles per MMA, and how far the issuing thread runs ahead of the pipe (issue time against total time).
//   2. The same with a commit after every G MMAs: what a commit costs the stream.
//   3. A ring: G MMAs, a commit, and before re-using a slot a wait for the commit S groups back (what a ring of S
//      load stages does to the issuer), loop state in registers only.
//   4. Ring 3 with a read of %globaltimer after the first failed poll of every wait (the first form of the kernels'
//      bounded waits). Alone it costs nothing; in the kernels it did, where some 300 waiting threads of the CTA read
//      the timer as well.
// Every wait is bounded by a poll count; a wait that gives up is reported. Built by aakaar_b200/_build.py into
// aakaar_b200/lib/mma_stream_bench; run it without arguments on a B200.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../sm100_ptx.cuh"
namespace ptx = akr::ptx;

namespace {

constexpr int kPollLimit = 2000000;
constexpr int A_BYTES = 128 * 32 * 4, B_BYTES = 256 * 32 * 4;  // one 32-deep k-block of a 128 x 256 tile

template <bool PAIR>
__device__ __forceinline__ void mma(uint32_t d, uint64_t da, uint64_t db, uint32_t acc) {
    if (PAIR) ptx::mma_tf32_ss_pair(d, da, db, ptx::idesc_tf32(256, 256, 0, 0), acc);
    else ptx::mma_tf32_ss(d, da, db, ptx::idesc_tf32(128, 256, 0, 0), acc);
}
template <bool PAIR>
__device__ __forceinline__ void commit(uint32_t bar) {
    if (PAIR) ptx::mma_commit_pair(bar);
    else ptx::mma_commit(bar);
}

struct State {
    uint32_t base, bar, tmem;
    uint32_t parity;  // bit b: parity of the next phase to wait for on barrier b
    bool failed;
};

// Bounded wait on barrier b; TIMER: read %globaltimer after the first failed poll, as the first build's waits did.
template <bool TIMER>
__device__ __forceinline__ void wait(State& st, int b) {
    const uint32_t addr = st.bar + 8 * b, par = (st.parity >> b) & 1u;
    bool got = ptx::mbar_test_wait(addr, par);
    if (!got && TIMER) (void)ptx::globaltimer_ns();
    for (int i = 0; i < kPollLimit && !got && !st.failed; ++i) got = ptx::mbar_test_wait(addr, par);
    if (!got) st.failed = true;
    st.parity ^= 1u << b;
}

template <bool PAIR>
__device__ __forceinline__ void issue(const State& st, int i) {
    const int k8 = i & 3;
    const uint64_t da = ptx::smem_desc(st.base + k8 * 32, 16, 1024, ptx::LAYOUT_SW128);
    const uint64_t db = ptx::smem_desc(st.base + A_BYTES + k8 * 32, 16, 1024, ptx::LAYOUT_SW128);
    mma<PAIR>(st.tmem + ((i >> 2) & 1) * 256, da, db, 1u);
}

// 512 MMAs as groups of G with a commit each; S > 0: wait for the commit S groups back before each group.
template <bool PAIR, int S, int G, bool TIMER>
__device__ long long run(State& st) {
    constexpr int groups = 512 / G;
    const long long t0 = clock64();
    int b = 1;
    for (int g = 0; g < groups; ++g) {
        if (S > 0 && g >= S) wait<TIMER>(st, b);
#pragma unroll
        for (int i = 0; i < G; ++i) issue<PAIR>(st, g * G + i);
        commit<PAIR>(st.bar + 8 * (S > 0 ? b : 1));
        if (S > 0 && ++b > S) b = 1;
    }
    if (S > 0) {
        for (int j = 0; j < S; ++j) {  // the last S commits, oldest first
            wait<false>(st, b);
            if (++b > S) b = 1;
        }
    } else {
        commit<PAIR>(st.bar);  // barrier 0: everything issued so far
        wait<false>(st, 0);
        if (groups & 1) st.parity ^= 2u;  // barrier 1 went through `groups` phases nobody waited for
    }
    return clock64() - t0;
}

template <bool PAIR>
__global__ void __launch_bounds__(64, 1) mma_stream(long long* out) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    State st;
    st.base = raw_addr + pad;
    st.bar = st.base + A_BYTES + B_BYTES;
    st.parity = 0;
    st.failed = false;
    float* f = reinterpret_cast<float*>(smem);
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x) f[i] = 1.0f + (i & 7) * 0.125f;
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + A_BYTES + B_BYTES + 128);
    const bool leader = !PAIR || ptx::cluster_ctarank() == 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) ptx::mbar_init(st.bar + 8 * i, 1);
        ptx::mbar_fence_init();
    }
    ptx::fence_proxy_async_smem();
    if (threadIdx.x >= 32) {
        if (PAIR) {
            ptx::tmem_alloc_pair<512>(ptx::smem_u32(slot));
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc<512>(ptx::smem_u32(slot));
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR) ptx::cluster_sync_all();
    ptx::tc_fence_after();
    st.tmem = *slot;
    if (threadIdx.x == 0 && leader) {
        int o = 0;
        (void)run<PAIR, 0, 512, false>(st);  // warm-up
        {                                    // 1. issue time and total time of 16 and of 512 MMAs
            const long long t0 = clock64();
            for (int i = 0; i < 16; ++i) issue<PAIR>(st, i);
            const long long t1 = clock64();
            commit<PAIR>(st.bar);
            wait<false>(st, 0);
            out[o++] = t1 - t0;
            out[o++] = clock64() - t0;
        }
        out[o++] = run<PAIR, 0, 512, false>(st);
        out[o++] = run<PAIR, 0, 32, false>(st);  // 2.
        out[o++] = run<PAIR, 0, 8, false>(st);
        out[o++] = run<PAIR, 0, 4, false>(st);
        out[o++] = run<PAIR, 3, 8, false>(st);  // 3.
        out[o++] = run<PAIR, 2, 8, false>(st);
        out[o++] = run<PAIR, 6, 4, false>(st);
        out[o++] = run<PAIR, 1, 8, false>(st);
        out[o++] = run<PAIR, 3, 8, true>(st);  // 4.
        out[o++] = run<PAIR, 6, 4, true>(st);
        out[31] = st.failed ? 1 : 0;
        if (st.failed) {  // let whatever is in flight finish before the tensor memory is given back
            const uint64_t t0 = ptx::globaltimer_ns();
            while (ptx::globaltimer_ns() - t0 < 2000000ull) {
            }
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR) ptx::cluster_sync_all();
    if (threadIdx.x >= 32) {
        ptx::tc_fence_after();
        if (PAIR) ptx::tmem_dealloc_pair<512>(st.tmem);
        else ptx::tmem_dealloc<512>(st.tmem);
    }
}

void report(const char* name, const long long* h) {
    std::printf("== %s%s\n", name, h[31] ? "  (A WAIT GAVE UP: numbers invalid)" : "");
    std::printf("16 MMAs: issued after %lld cycles, complete after %lld (16 x 128 = 2048)\n", h[0], h[1]);
    const char* rows[] = {"512 MMAs, one commit", "512 MMAs, commit every 32", "512 MMAs, commit every 8", "512 MMAs, commit every 4",
                          "ring of 3 slots x 8 MMAs", "ring of 2 slots x 8 MMAs", "ring of 6 slots x 4 MMAs", "ring of 1 slot x 8 MMAs (serialised)",
                          "ring of 3 x 8, clock read after a failed poll", "ring of 6 x 4, clock read after a failed poll"};
    for (int i = 0; i < 10; ++i) std::printf("%-48s %7lld cycles  (x%.3f of 512 x 128)\n", rows[i], h[2 + i], h[2 + i] / 65536.0);
}

}  // namespace

int main() {
    long long* d = nullptr;
    if (cudaMalloc(&d, 32 * sizeof(long long)) != cudaSuccess) {
        std::printf("no CUDA device\n");
        return 1;
    }
    const int smem = A_BYTES + B_BYTES + 1024 + 256;
    cudaFuncSetAttribute(mma_stream<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(mma_stream<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    long long h[32];
    for (int pair = 0; pair < 2; ++pair) {
        for (int it = 0; it < 2; ++it) {
            cudaMemset(d, 0, 32 * sizeof(long long));
            if (!pair) {
                mma_stream<false><<<1, 64, smem>>>(d);
            } else {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(2);
                cfg.blockDim = dim3(64);
                cfg.dynamicSmemBytes = smem;
                cudaLaunchAttribute attr;
                attr.id = cudaLaunchAttributeClusterDimension;
                attr.val.clusterDim.x = 2;
                attr.val.clusterDim.y = 1;
                attr.val.clusterDim.z = 1;
                cfg.attrs = &attr;
                cfg.numAttrs = 1;
                cudaLaunchKernelEx(&cfg, mma_stream<true>, d);
            }
            const cudaError_t e = cudaDeviceSynchronize();
            if (e != cudaSuccess) {
                std::printf("error: %s\n", cudaGetErrorString(e));
                return 1;
            }
        }
        cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
        report(pair ? "CTA pair, tcgen05.mma.cta_group::2 256 x 256 x 8" : "one CTA, tcgen05.mma.cta_group::1 128 x 256 x 8", h);
    }
    cudaFree(d);
    return 0;
}
