// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM kernels use:
// mbarriers, TMA tiled loads, tensor memory (TMEM) management, tcgen05 MMA / commit / load.
// Every wait is bounded: a wait that runs out records an abort flag instead of spinning forever.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace akr {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded waits. Both return false when the barrier did not flip within `limit_ns`, or when another role of this
// CTA already gave up (abort flag set); the caller then leaves its loop. Neither reads the clock before a few
// hundred polls have failed, and both pause between polls:
//  * %globaltimer is a shared resource. When every waiter read it after its first failed poll and again every 64
//    polls - some 300 threads of a CTA wait at any time, the epilogue warps for a whole tile - the one read of the
//    MMA issuer (normally a little ahead of its data) took hundreds of cycles, it woke up late every k-block and
//    the tensor pipe's short queue (about four MMAs) ran dry: 733 -> 575 kilocycles for two 256 x 256 x 8192 tiles
//    without those reads (524 is the MMA work itself). A single thread reading the timer that way loses nothing
//    (csrc/microbench/mma_stream.cu);
//  * a poll is a shared-memory access to the barrier word the TMA unit is counting bytes on. Polling without any
//    pause cost the CTA-pair TF32 kernel 7 % (its leader polls a barrier that both CTAs' copies complete on), and a
//    dozen warps polling that way cost the shared-memory-bound fp32-accurate kernels 6 %.
// mbar_wait: for the single threads on the critical path of the stage ring (MMA issuer, TMA producer): 100 ns pause.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        asm volatile("nanosleep.u32 100;" ::: "memory");
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0u) {
            if (*abort_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// mbar_wait_warp: for whole warps (epilogue warps waiting for an accumulator, converter warps waiting for a tile):
// the pause doubles from 32 to 256 ns, short against the microseconds such a wait lasts.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    uint32_t ns = 32;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        asm volatile("nanosleep.u32 %0;" ::"r"(ns) : "memory");
        if (mbar_try_wait(bar, parity)) return true;
        if (ns < 256) ns <<= 1;
        if ((++spins & 255u) == 0u) {
            if (*abort_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Non-suspending test of a barrier phase (micro-benchmarks).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while the kernel
// before it in the stream is still running; `grid_dep_wait` blocks until that kernel has completed
// and its writes are visible (a no-op for a normal launch). `grid_dep_launch` lets the NEXT kernel
// in the stream start being scheduled as this one's CTAs retire.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- register reallocation between warpgroups
// All four warps of a warpgroup (hardware warps 4g .. 4g+3) give registers back / take more. An SM
// sub-partition holds 16384 registers and hosts hardware warps w, w+4, w+8, ...: twelve warps at a uniform count
// are capped at 168 each; 2 x 208 + 96 per sub-partition fits exactly.
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// Rank-5 tiled load global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3), "r"(c4)
        : "memory");
}

// Rank-4 tiled store shared -> global (bulk async group). Rows / columns outside the tensor are clipped.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// The shared-memory source of every committed bulk store has been read (it may be overwritten).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All but the most recent bulk group of this thread have finished reading their shared-memory source.
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// Every committed bulk store of this thread has completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Named barrier over `nthreads` threads that also returns the AND of `pred` over all of them.
__device__ __forceinline__ bool named_barrier_and(int id, int nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %3, 0;\n\t"
        "barrier.cta.red.and.pred q, %1, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Generic-proxy writes to shared memory made visible to the async proxy (TMA / tcgen05 reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- TMEM
template <int NCOLS>
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem_addr) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     slot_smem_addr),
                 "r"(NCOLS)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05 MMA
// D[tmem] (+)= A[smem desc] * B[smem desc], TF32 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive once on `bar` when every MMA this thread issued before has finished.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// The same two instructions for a warp that runs its issue loop with all 32 lanes (uniform control flow, so
// that descriptors and addresses live in uniform registers): `leader` is nonzero in the one lane that issues.
// The lane is chosen once (elect_one) and must stay the same: a commit tracks the MMAs of the thread that executes it.
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t is_leader;
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, e;\n\t"
        "}\n"
        : "=r"(is_leader));
    return is_leader;
}
__device__ __forceinline__ void mma_tf32_ss_elected(uint32_t leader, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                    uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 e, %5, 0;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}
__device__ __forceinline__ void mma_commit_elected(uint32_t leader, uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "setp.ne.b32 e, %1, 0;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(bar), "r"(leader)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (sm_100 version bit set), 128-byte swizzle span.
//   K-major operand : layout 2 (16-byte swizzle atoms), lbo = 16 (unused by the swizzled form),
//                     sbo = byte stride between groups of 8 rows.
//   MN-major operand: 32-bit operands must use layout 1 (128-byte span, 32-byte swizzle atoms,
//                     pattern repeating every 4 k-rows); lbo = byte stride between 32-element
//                     (128 B) chunks along M/N, sbo = byte stride between groups of 4 k-rows.
constexpr uint32_t LAYOUT_SW128 = 2;
constexpr uint32_t LAYOUT_SW64 = 4;  // 64-byte swizzle span (K-major tiles with 64-byte rows)
constexpr uint32_t LAYOUT_SW128_ATOM32B = 1;
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;  // descriptor version for sm_100
    d |= static_cast<uint64_t>(layout) << 61;
    return d;
}

// Instruction descriptor for kind::tf32 with fp32 accumulation.
// a_mn / b_mn: 0 = operand is K-major in shared memory, 1 = M/N-major.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n, int a_mn, int b_mn) {
    return (1u << 4)                 // D format: F32
           | (2u << 7)               // A format: TF32
           | (2u << 10)              // B format: TF32
           | (uint32_t(a_mn) << 15)  // A major
           | (uint32_t(b_mn) << 16)  // B major
           | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

}  // namespace ptx
}  // namespace akr

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster share one MMA: the leader (cluster rank 0) issues it, each CTA supplies its
// 128 rows of A and its half of B from its own shared memory and receives its 128 rows of D in its
// own tensor memory. No multicast copies are used anywhere; each CTA loads its own tiles.
namespace akr {
namespace ptx {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of `local_addr` (a shared::cta address) in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// Rank-5 tiled load into THIS CTA's shared memory whose completion bytes are counted on an mbarrier
// given by a shared::cluster address, i.e. possibly the pair leader's barrier (no multicast: one
// destination, one CTA).
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(c4)
        : "memory");
}
// Arrive on an mbarrier given by its shared::cluster address (own or peer CTA). Release semantics at CTA scope
// (the instruction's default): what such a signal orders - tensor-memory reads finished, a CTA's own shared-memory
// tiles written for its own tensor core - never travels through memory to the other CTA. The same arrive with
// release at CLUSTER scope cost several microseconds per signal (measured: 2.6 against 1.6 ms on 8192 batched
// 256^3 products when the converter warps of a CTA pair signalled the leader that way).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem_addr) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr),
                 "r"(NCOLS)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the CTA pair (M = 256), issued by the leader CTA only.
__device__ __forceinline__ void mma_tf32_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The pair forms for an issuing warp that runs with all lanes (see mma_tf32_ss_elected).
__device__ __forceinline__ void mma_tf32_ss_pair_elected(uint32_t leader, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 e, %5, 0;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}
__device__ __forceinline__ void mma_commit_pair_elected(uint32_t leader, uint32_t bar) {
    const uint16_t both = 0x3;
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "setp.ne.b32 e, %2, 0;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
        "}\n"
        ::"r"(bar), "h"(both), "r"(leader)
        : "memory");
}
// When the pair MMAs issued so far have finished, arrive once on the mbarrier at shared-memory
// offset `bar` in BOTH CTAs of the pair (a barrier signal sent to the two CTAs, not a data copy).
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    const uint16_t both = 0x3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(both)
        : "memory");
}

}  // namespace ptx
}  // namespace akr
