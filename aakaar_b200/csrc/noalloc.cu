// akr_matmul_at_b_noalloc: the weight-gradient product C(m,n) = A(k,m)^T . B(k,n) for hosts that
// must not allocate device memory when they call into the library.
//
// Who that is: a host runtime that hands the whole of HBM to its own pool at start-up (any later
// cudaMalloc then fails, or eats into the pool's share), and latency-critical loops that cannot
// take the device-wide synchronisation cudaMalloc / cudaFree imply. The regular entry points grow a
// cached workspace with cudaMalloc the first time a shape needs scratch; this one never does. Its
// scratch - the fp32 partial tiles and per-tile counters of the split contraction - lives in
// file-scope device arrays of fixed size that every GPU loading the library holds until exit.
#include "../../include/akr_b200.h"

#include "gemm_sm100.h"

#include <cmath>
#include <cstdio>
#include <mutex>
#include <string>

namespace akr {
void set_last_error(const std::string& msg);  // defined beside akr_last_error()
std::mutex& device_launch_mutex(int dev);     // the lock every launching entry point of a device takes
}
using namespace akr;

namespace {

// Fixed scratch: 2 Mi floats (8 MiB) of partial tiles, 4096 tile counters, one status word.
constexpr size_t kPartialFloats = (size_t)2 << 20;
constexpr size_t kCounters = 4096;

static __device__ __align__(256) float g_partials[kPartialFloats];
static __device__ __align__(256) int g_counters[kCounters];
static __device__ __align__(256) int g_status[64];

// In host code the names above are host-side stand-ins, not device addresses. The device
// addresses are looked up once per device (with that device current) and cached here.
struct DeviceScratch {
    bool ready = false;
    float* partials = nullptr;
    int* counters = nullptr;
    int* status = nullptr;
};
constexpr int kMaxDevices = 64;
DeviceScratch g_scratch[kMaxDevices];
std::mutex g_mu;
int na_fail(int code, const std::string& msg) {
    akr::set_last_error(msg);  // read back by akr_last_error(), like every other entry point
    return code;
}

int setup_device(int dev, DeviceScratch** out) {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceScratch& s = g_scratch[dev];
    if (!s.ready) {
        cudaError_t e = cudaGetSymbolAddress((void**)&s.partials, g_partials);
        if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&s.counters, g_counters);
        if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&s.status, g_status);
        if (e != cudaSuccess)
            return na_fail(AKR_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        s.ready = true;
    }
    *out = &s;
    return AKR_OK;
}

}  // namespace

namespace akr {
// Called by akr_synchronize() after the device has gone idle: reports (and clears) the status word of this
// entry point's kernels on `dev`. Returns 1 when a kernel had given up on a bounded wait. Touches nothing on
// a device where the entry point was never called.
int noalloc_take_status(int dev) {
    if (dev < 0 || dev >= kMaxDevices) return 0;
    int* status = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch[dev].ready) return 0;
        status = g_scratch[dev].status;
    }
    int flag = 0;
    if (cudaMemcpy(&flag, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (flag != 0) cudaMemset(status, 0, sizeof(int));
    return flag != 0 ? 1 : 0;
}
}  // namespace akr

extern "C" {

AKR_API int akr_matmul_at_b_noalloc(const akr_view* a, const akr_view* b, akr_view* c, void* stream) {
    auto report = [](int rc) { return rc; };
    if (!a || !b || !c) return report(na_fail(AKR_ERR_INVALID, "matmul_at_b_noalloc: null view"));
    if (a->dtype != AKR_DTYPE_F32 || b->dtype != AKR_DTYPE_F32 || c->dtype != AKR_DTYPE_F32)
        return report(na_fail(AKR_ERR_RUNTIME, "matmul_at_b_noalloc: only float32 is supported"));
    if (a->ndim != 2 || b->ndim != 2 || c->ndim != 2)
        return report(na_fail(AKR_ERR_INVALID, "matmul_at_b_noalloc requires 2-D tensors"));
    for (int i = 0; i < 2; ++i)
        if (a->shape[i] <= 0 || b->shape[i] <= 0)
            return report(na_fail(AKR_ERR_INVALID, "Tensor dimensions must be positive"));
    if (a->shape[0] != b->shape[0])
        return report(na_fail(AKR_ERR_INVALID, "matmul_at_b: inner dimensions must match"));
    const int64_t K = a->shape[0], M = a->shape[1], N = b->shape[1];
    if (c->shape[0] != M || c->shape[1] != N)
        return report(na_fail(AKR_ERR_INVALID, "matmul_at_b_noalloc: output has the wrong shape"));
    if (N > 1 && c->stride[1] != 1)
        return report(na_fail(AKR_ERR_INVALID, "matmul_at_b_noalloc: output rows must be contiguous"));
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
        return report(na_fail(AKR_ERR_INVALID, "matmul_at_b_noalloc: dimension exceeds 2^31-1"));
    // Same refusals as the regular entry points make before they touch the GPU: a null pointer would be
    // encoded into a tensor map and fault on the device.
    if (!a->data) return report(na_fail(AKR_ERR_INVALID, "matmul_at_b a: null data pointer"));
    if (!b->data) return report(na_fail(AKR_ERR_INVALID, "matmul_at_b b: null data pointer"));
    if (!c->data) return report(na_fail(AKR_ERR_INVALID, "matmul_at_b output: null data pointer"));
    if (M > 1 && c->stride[0] < N)
        return report(na_fail(AKR_ERR_INVALID, "matmul_at_b_noalloc: output row stride is smaller than a row"));

    int ndev = 0, dev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        cudaGetLastError();
        return report(na_fail(AKR_ERR_NOGPU, "no CUDA device available: aakaar_b200 has no CPU path"));
    }
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return report(na_fail(AKR_ERR_CUDA, "matmul_at_b_noalloc: cannot identify the current device"));
    DeviceScratch* sc = nullptr;
    int rc = setup_device(dev, &sc);
    if (rc != AKR_OK) return report(rc);
    cudaStream_t st = (cudaStream_t)stream;

    // Operands are read in place through TMA; a layout that would need a packed copy needs scratch
    // of the operand's own size, which the fixed arrays do not provide.
    GemmDesc g;
    g.M = (int)M;
    g.N = (int)N;
    g.K = (int)K;
    auto as_operand = [](const akr_view* v, int64_t mn, int64_t k, GemmOperand* op) {
        // rows of the view run along k (stride[0]), columns along m/n (stride[1])
        const int64_t s_k = v->stride[0], s_mn = v->stride[1];
        op->ptr = (const float*)v->data;
        if ((mn == 1 || s_mn == 1) && (k == 1 || (s_k > 0 && (s_k & 3) == 0))) {
            op->mn_major = 1;
            op->ld = s_k;
            return true;
        }
        if ((k == 1 || s_k == 1) && (mn == 1 || (s_mn > 0 && (s_mn & 3) == 0))) {
            op->mn_major = 0;
            op->ld = s_mn;
            return true;
        }
        return false;
    };
    const int batch[3] = {1, 1, 1};
    if (!as_operand(a, M, K, &g.A) || !as_operand(b, N, K, &g.B) ||
        !gemm_sm100_operand_ok(g.A, g.M, g.K, batch) || !gemm_sm100_operand_ok(g.B, g.N, g.K, batch))
        return report(na_fail(AKR_ERR_INVALID,
                              "matmul_at_b_noalloc: operands must be readable in place (16-byte aligned base, unit "
                              "stride on one dim, the other stride a multiple of 4 elements); other layouts need a "
                              "packed copy, i.e. scratch this entry point does not have"));
    g.C = (float*)c->data;
    g.ldc = c->stride[0];
    g.terms = 1;  // TF32 products; the fp32-accurate mode needs split operands (scratch of operand size)
    g.splits = gemm_sm100_pick_splits(g);
    {
        // This entry point keeps the single-launch variant (tile counters, the last CTA of a tile adds up its
        // partials alone), whose reduction time grows with the split count: balance it against the
        // contraction left per split.
        const long long iters = (K + 31) / 32;
        const int s_bal = (int)(std::sqrt(0.2 * (double)iters) + 0.5);
        if (g.splits > s_bal) g.splits = s_bal < 1 ? 1 : s_bal;
    }
    size_t pbytes = 0, ncnt = 0;
    gemm_sm100_split_scratch(g, &pbytes, &ncnt);
    if (pbytes > kPartialFloats * sizeof(float) || ncnt > kCounters) {
        char msg[320];
        std::snprintf(msg, sizeof(msg),
                      "matmul_at_b_noalloc: this product needs %zu bytes of partial tiles and %zu tile counters; "
                      "the fixed scratch holds %zu bytes and %zu counters (use akr_matmul_at_b instead)",
                      pbytes, ncnt, kPartialFloats * sizeof(float), kCounters);
        return report(na_fail(AKR_ERR_INVALID, msg));
    }
    if (g.splits > 1) {
        g.partials = sc->partials;
        g.counters = sc->counters;
        // The counters must start at zero. A finished launch leaves them at zero, an aborted one may
        // not, so they are cleared on every call (a memset allocates nothing).
        cudaError_t e = cudaMemsetAsync(sc->counters, 0, ncnt * sizeof(int), st);
        if (e != cudaSuccess)
            return report(na_fail(AKR_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e)));
    }
    char err[256] = {0};
    std::lock_guard<std::mutex> launch_lock(akr::device_launch_mutex(dev));
    const int lrc = gemm_sm100_launch(g, st, sc->status, err, sizeof(err));
    if (lrc != 0) return report(na_fail(lrc == -1 ? AKR_ERR_INVALID : AKR_ERR_CUDA, err));
    return AKR_OK;
}

}  // extern "C"
