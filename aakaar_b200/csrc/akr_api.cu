// C ABI of the library (declared in include/akr_b200.h): shape planning with the reference's
// broadcasting rules, operand preparation (direct TMA views, packing, TF32 splitting), launch of
// the tcgen05 GEMM, the caching allocator and the support ops of the Linear training step.
#include "../../include/akr_b200.h"

#include "aux_kernels.h"
#include "gemm_sm100.h"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

using namespace akr;

namespace {

thread_local std::string g_err;
std::atomic<int> g_tf32{0};
std::atomic<int> g_cudnn_tf32{0};

int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    return fail(AKR_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

enum WsSlot { WS_A_PACK = 0, WS_B_PACK, WS_PARTIALS, WS_COUNTERS, WS_MISC, WS_COLPART, WS_COUNT };

struct Region {
    void* ptr = nullptr;
    size_t bytes = 0;
};

struct DeviceState {
    std::mutex mu;
    std::unordered_map<size_t, std::vector<float*>> free_blocks;
    int64_t hits = 0, misses = 0;
    Region ws[WS_COUNT];
    int* status = nullptr;
    int64_t launches = 0;
};

constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];

int current_device(int* dev) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return fail(AKR_ERR_NOGPU,
                    "no CUDA device available: aakaar_b200 runs on sm_100a GPUs only and has no CPU path");
    }
    e = cudaGetDevice(dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (*dev < 0 || *dev >= kMaxDevices) return fail(AKR_ERR_RUNTIME, "device ordinal out of range");
    return AKR_OK;
}

int get_state(DeviceState** out) {
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != AKR_OK) return rc;
    *out = &g_dev[dev];
    return AKR_OK;
}

// Scratch region that only grows. Growing frees the old block first (cudaFree waits for the
// device, so no kernel still reads it).
int ws_get(DeviceState* st, int slot, size_t bytes, void** out, bool zero_on_alloc = false) {
    Region& r = st->ws[slot];
    if (r.bytes < bytes) {
        if (r.ptr) cudaFree(r.ptr);
        r.ptr = nullptr;
        r.bytes = 0;
        size_t want = bytes + bytes / 8;
        want = (want + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);
        cudaError_t e = cudaMalloc(&r.ptr, want);
        if (e != cudaSuccess) {
            want = (bytes + 255) & ~(size_t)255;
            e = cudaMalloc(&r.ptr, want);
        }
        if (e != cudaSuccess) {
            r.ptr = nullptr;
            return cuda_fail(e, "workspace cudaMalloc");
        }
        r.bytes = want;
        if (zero_on_alloc) {
            e = cudaMemset(r.ptr, 0, want);
            if (e != cudaSuccess) return cuda_fail(e, "workspace cudaMemset");
        }
    }
    *out = r.ptr;
    return AKR_OK;
}

int status_word(DeviceState* st, int** out) {
    if (!st->status) {
        cudaError_t e = cudaMalloc(&st->status, 256);
        if (e != cudaSuccess) return cuda_fail(e, "status cudaMalloc");
        e = cudaMemset(st->status, 0, 256);
        if (e != cudaSuccess) return cuda_fail(e, "status cudaMemset");
    }
    *out = st->status;
    return AKR_OK;
}

int check_view(const akr_view* v, const char* name, int min_dims) {
    if (!v) return fail(AKR_ERR_INVALID, std::string(name) + ": null view");
    if (v->dtype != AKR_DTYPE_F32)
        return fail(AKR_ERR_RUNTIME, std::string(name) + ": only float32 is supported on the matmul path");
    if (v->ndim < min_dims) return fail(AKR_ERR_INVALID, "matmul requires tensors with at least 2 dimensions");
    if (v->ndim > AKR_MAX_DIMS) return fail(AKR_ERR_INVALID, std::string(name) + ": more than 8 dimensions");
    for (int i = 0; i < v->ndim; ++i)
        if (v->shape[i] <= 0) return fail(AKR_ERR_INVALID, "Tensor dimensions must be positive");
    if (!v->data) return fail(AKR_ERR_INVALID, std::string(name) + ": null data pointer");
    return AKR_OK;
}

struct Plan {
    int nb = 0;
    int64_t batch[AKR_MAX_DIMS];
    int64_t M = 0, K = 0, N = 0;
};

// plan_nd_matmul of the reference: right-aligned broadcast, same error texts.
int make_plan(const akr_view* a, const akr_view* b, Plan* p) {
    if (!a || !b) return fail(AKR_ERR_INVALID, "matmul: null view");
    if (a->ndim < 2 || b->ndim < 2)
        return fail(AKR_ERR_INVALID, "matmul requires tensors with at least 2 dimensions");
    if (a->ndim > AKR_MAX_DIMS || b->ndim > AKR_MAX_DIMS)
        return fail(AKR_ERR_INVALID, "matmul: more than 8 dimensions");
    p->M = a->shape[a->ndim - 2];
    p->K = a->shape[a->ndim - 1];
    const int64_t K2 = b->shape[b->ndim - 2];
    p->N = b->shape[b->ndim - 1];
    if (p->K != K2) return fail(AKR_ERR_INVALID, "Shape mismatch: inner dimensions must match for matmul");
    const int nba = a->ndim - 2, nbb = b->ndim - 2;
    p->nb = std::max(nba, nbb);
    for (int i = 0; i < p->nb; ++i) {
        const int64_t da = i < nba ? a->shape[nba - 1 - i] : 1;
        const int64_t db = i < nbb ? b->shape[nbb - 1 - i] : 1;
        if (da != db && da != 1 && db != 1)
            return fail(AKR_ERR_INVALID, "Batch dimensions are not broadcastable for matmul");
        p->batch[p->nb - 1 - i] = std::max(da, db);
    }
    return AKR_OK;
}

// Stride of `v` along broadcast batch dim i (of nb right-aligned dims); 0 when v is broadcast there.
int64_t batch_stride(const akr_view* v, int nb, int i) {
    const int nbv = v->ndim - 2;
    const int j = i - (nb - nbv);
    if (j < 0) return 0;
    return v->shape[j] == 1 ? 0 : v->stride[j];
}

struct Operand {
    const float* ptr = nullptr;
    int64_t s_mn = 0, s_k = 0;
    int64_t bs[AKR_MAX_DIMS] = {0};
};

struct Problem {
    int64_t M = 0, N = 0, K = 0;
    int nb = 0;
    int64_t bshape[AKR_MAX_DIMS];
    Operand A, B;
    float* C = nullptr;
    int64_t c_rs = 0;
    int64_t c_bs[AKR_MAX_DIMS] = {0};  // 0 on a dim of extent > 1: summed away
    const float* bias = nullptr;
    int mode = AKR_MODE_TF32;
    // epilogue: C = op(alpha * AB (+ bias)), op 1: + beta * X, op 2: * (1 - X^2); X has C's shape
    float alpha = 1.f, beta = 0.f;
    int aux_op = 0;
    const float* aux = nullptr;
    int64_t aux_rs = 0, aux_cs = 1;
    int64_t aux_bs[AKR_MAX_DIMS] = {0};
    // Optional by-product: colsum_out[n] = sum over all rows and batch entries of C[.., n] (N floats). Produced
    // by the GEMM's epilogue when the kernel can (colsum_done = true); otherwise the caller adds a separate pass.
    float* colsum_out = nullptr;
    mutable bool colsum_done = false;
};

struct Dim {
    int64_t e, a, b, c, x;  // extent; strides of A, B, C and the second epilogue operand
};

void collapse(std::vector<Dim>& d) {
    std::vector<Dim> out;
    for (const Dim& x : d) {
        if (!out.empty()) {
            Dim& p = out.back();
            if (p.a == x.a * x.e && p.b == x.b * x.e && p.c == x.c * x.e && p.x == x.x * x.e) {
                p.e *= x.e;
                p.a = x.a;
                p.b = x.b;
                p.c = x.c;
                p.x = x.x;
                continue;
            }
        }
        out.push_back(x);
    }
    d.swap(out);
}

struct Prepared {
    GemmOperand op;
    // strides along the collapsed (out dims..., red dims...) list
    std::vector<int64_t> bs;
};

// Decides how the GEMM kernel reads one operand: in place through TMA when its layout allows it,
// else from a packed copy.
int prepare_operand(DeviceState* st, const Operand& src, int64_t mn, int64_t k,
                    const std::vector<Dim>& dims, bool is_a, cudaStream_t stream, Prepared* out) {
    const size_t nd = dims.size();
    std::vector<int64_t> bs(nd);
    for (size_t i = 0; i < nd; ++i) bs[i] = is_a ? dims[i].a : dims[i].b;

    auto strides_ok = [&]() {
        for (size_t i = 0; i < nd; ++i)
            if (dims[i].e > 1 && bs[i] != 0 && (bs[i] < 0 || (bs[i] & 3) != 0)) return false;
        return (reinterpret_cast<uintptr_t>(src.ptr) & 15u) == 0;
    };
    const bool k_major_ok = (k == 1 || src.s_k == 1) && (mn == 1 || (src.s_mn > 0 && (src.s_mn & 3) == 0));
    const bool mn_major_ok = (mn == 1 || src.s_mn == 1) && (k == 1 || (src.s_k > 0 && (src.s_k & 3) == 0));

    if (strides_ok() && (k_major_ok || mn_major_ok)) {
        out->op.ptr = src.ptr;
        out->op.mn_major = k_major_ok ? 0 : 1;
        out->op.ld = k_major_ok ? src.s_mn : src.s_k;
        out->bs = bs;
        return AKR_OK;
    }

    // Packed copy: keep the operand's major-ness when it has a unit-stride matrix dim (coalesced
    // reads), else K-major. Batch dims the operand varies along become dense.
    const bool keep_mn = !(k == 1 || src.s_k == 1) && (mn == 1 || src.s_mn == 1);
    PackSrc ps;
    ps.ptr = src.ptr;
    ps.nb = 0;
    std::vector<int> varying;
    for (size_t i = 0; i < nd; ++i) {
        if (dims[i].e > 1 && bs[i] != 0) {
            ps.bshape[ps.nb] = dims[i].e;
            ps.bstride[ps.nb] = bs[i];
            ++ps.nb;
            varying.push_back((int)i);
        }
    }
    ps.rows = keep_mn ? k : mn;
    ps.cols = keep_mn ? mn : k;
    ps.row_stride = keep_mn ? src.s_k : src.s_mn;
    ps.col_stride = keep_mn ? src.s_mn : src.s_k;
    const int64_t ld = (ps.cols + 3) / 4 * 4;
    int64_t nbatch = 1;
    for (int i = 0; i < ps.nb; ++i) nbatch *= ps.bshape[i];
    const size_t bytes = (size_t)nbatch * ps.rows * ld * sizeof(float);
    void* packed = nullptr;
    int rc = ws_get(st, is_a ? WS_A_PACK : WS_B_PACK, bytes, &packed);
    if (rc != AKR_OK) return rc;
    cudaError_t e = launch_pack(ps, (float*)packed, ld, stream);
    if (e != cudaSuccess) return cuda_fail(e, "pack launch");
    st->launches++;
    out->op.ptr = (const float*)packed;
    out->op.mn_major = keep_mn ? 1 : 0;
    out->op.ld = ld;
    out->bs.assign(nd, 0);
    int64_t acc = ps.rows * ld;
    for (int j = (int)varying.size() - 1; j >= 0; --j) {
        out->bs[varying[j]] = acc;
        acc *= dims[varying[j]].e;
    }
    return AKR_OK;
}

int run_problem(const Problem& p, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = get_state(&st);
    if (rc != AKR_OK) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.K > 0x7fffffff)
        return fail(AKR_ERR_INVALID, "matmul: dimension exceeds 2^31-1");

    // Batch dims: drop extent 1, separate output dims from summed dims, merge neighbours.
    std::vector<Dim> outd, redd;
    for (int i = 0; i < p.nb; ++i) {
        if (p.bshape[i] == 1) continue;
        Dim d{p.bshape[i], p.A.bs[i], p.B.bs[i], p.c_bs[i], p.aux_op ? p.aux_bs[i] : 0};
        (d.c != 0 ? outd : redd).push_back(d);
    }
    collapse(outd);
    collapse(redd);
    std::vector<Dim> all = outd;
    all.insert(all.end(), redd.begin(), redd.end());
    for (const Dim& d : all)
        if (d.e > 0x7fffffff) return fail(AKR_ERR_INVALID, "matmul: batch extent exceeds 2^31-1");

    Prepared A, B;
    rc = prepare_operand(st, p.A, p.M, p.K, all, true, stream, &A);
    if (rc != AKR_OK) return rc;
    rc = prepare_operand(st, p.B, p.N, p.K, all, false, stream, &B);
    if (rc != AKR_OK) return rc;

    int* status = nullptr;
    rc = status_word(st, &status);
    if (rc != AKR_OK) return rc;

    const size_t no = outd.size(), nr = redd.size();
    // The kernel takes the two innermost output dims and the innermost summed dim; any further
    // dims are looped here (summed ones as accumulating launches).
    const size_t ko = std::min<size_t>(no, 2), kr = std::min<size_t>(nr, 1);
    // The fp32-accurate kernels have no second-operand epilogue: there the operand is applied by an
    // elementwise pass over the finished output (what the reference does in every mode).
    const bool aux_after = p.aux_op != 0 && p.mode == AKR_MODE_FP32;
    GemmDesc g;
    g.M = (int)p.M;
    g.N = (int)p.N;
    g.K = (int)p.K;
    g.A = A.op;
    g.B = B.op;
    g.ldc = p.c_rs;
    g.bias = p.bias;
    g.alpha = p.alpha;
    g.beta = p.beta;
    g.aux_op = aux_after ? 0 : p.aux_op;
    g.aux_ld = p.aux_rs;
    g.aux_cs = p.aux_cs;
    g.terms = p.mode == AKR_MODE_FP32 ? 3 : 1;
    g.o0 = g.o1 = g.red = 1;
    for (int i = 0; i < 3; ++i) g.A.bs[i] = g.B.bs[i] = 0;
    if (ko == 2) {
        g.o0 = (int)outd[no - 2].e;
        g.o1 = (int)outd[no - 1].e;
        g.A.bs[0] = A.bs[no - 2];
        g.A.bs[1] = A.bs[no - 1];
        g.B.bs[0] = B.bs[no - 2];
        g.B.bs[1] = B.bs[no - 1];
        g.c_bs0 = outd[no - 2].c;
        g.c_bs1 = outd[no - 1].c;
        g.aux_bs0 = outd[no - 2].x;
        g.aux_bs1 = outd[no - 1].x;
    } else if (ko == 1) {
        g.o1 = (int)outd[no - 1].e;
        g.A.bs[1] = A.bs[no - 1];
        g.B.bs[1] = B.bs[no - 1];
        g.c_bs1 = outd[no - 1].c;
        g.aux_bs1 = outd[no - 1].x;
    }
    if (kr == 1) {
        g.red = (int)redd[nr - 1].e;
        g.A.bs[2] = A.bs[no + nr - 1];
        g.B.bs[2] = B.bs[no + nr - 1];
    }
    g.splits = gemm_sm100_pick_splits(g);
    // Column sums in the epilogue: TF32 kernels, one launch (no host loop over leftover dims), no split.
    int colpart_rows = 0;
    if (p.colsum_out && p.mode == AKR_MODE_TF32 && g.splits == 1 && no <= 2 && nr == 0 && !aux_after) {
        colpart_rows = g.o0 * g.o1 * ((g.M + 31) / 32);
        void* cp = nullptr;
        rc = ws_get(st, WS_COLPART, (size_t)colpart_rows * (size_t)g.N * sizeof(float), &cp);
        if (rc != AKR_OK) return rc;
        g.colpart = (float*)cp;
    }
    if (g.splits > 1) {
        size_t pbytes = 0, ncnt = 0;
        gemm_sm100_split_scratch(g, &pbytes, &ncnt);
        void* pp = nullptr;
        rc = ws_get(st, WS_PARTIALS, pbytes, &pp);
        if (rc != AKR_OK) return rc;
        g.partials = (float*)pp;   // no tile counters: the partials are added up by the GPU-wide reduction kernel
        (void)ncnt;
    }

    // Host loops over the leftover dims.
    std::vector<int64_t> oidx(no > ko ? no - ko : 0, 0), ridx(nr > kr ? nr - kr : 0, 0);
    int64_t n_outer = 1, n_rouser = 1;
    for (size_t i = 0; i + ko < no; ++i) n_outer *= outd[i].e;
    for (size_t i = 0; i + kr < nr; ++i) n_rouser *= redd[i].e;
    char err[256] = {0};
    for (int64_t io = 0; io < n_outer; ++io) {
        int64_t t = io, ao = 0, bo = 0, co = 0, xo = 0;
        for (int i = (int)(no - ko) - 1; i >= 0; --i) {
            const int64_t idx = t % outd[i].e;
            t /= outd[i].e;
            ao += idx * A.bs[i];
            bo += idx * B.bs[i];
            co += idx * outd[i].c;
            xo += idx * outd[i].x;
        }
        for (int64_t ir = 0; ir < n_rouser; ++ir) {
            int64_t tr = ir, ar = 0, br = 0;
            for (int i = (int)(nr - kr) - 1; i >= 0; --i) {
                const int64_t idx = tr % redd[i].e;
                tr /= redd[i].e;
                ar += idx * A.bs[no + i];
                br += idx * B.bs[no + i];
            }
            GemmDesc gi = g;
            gi.A.ptr = g.A.ptr + ao + ar;
            gi.B.ptr = g.B.ptr + bo + br;
            gi.C = p.C + co;
            gi.accumulate = ir > 0 ? 1 : 0;
            // bias and the second epilogue operand apply once, to the complete sum: on the last launch
            const bool last = ir + 1 == n_rouser;
            if (!last) gi.bias = nullptr;
            gi.aux_op = last ? g.aux_op : 0;
            gi.aux = (last && p.aux && !aux_after) ? p.aux + xo : nullptr;
            const int lrc = gemm_sm100_launch(gi, stream, status, err, sizeof(err));
            if (lrc != 0) return fail(lrc == -1 ? AKR_ERR_INVALID : AKR_ERR_CUDA, err);
            st->launches += gi.splits > 1 ? 2 : 1;  // a split contraction is followed by its reduction kernel
        }
    }
    if (g.colpart) {
        cudaError_t e = launch_colsum_final(g.colpart, colpart_rows, g.N, p.colsum_out, stream);
        if (e != cudaSuccess) return cuda_fail(e, "column-sum launch");
        st->launches++;
        p.colsum_done = true;
    }
    if (aux_after) {
        EpiApply ea;
        ea.c = p.C;
        ea.x = p.aux;
        for (int i = 0; i < p.nb; ++i) {
            if (p.bshape[i] == 1 || p.c_bs[i] == 0) continue;  // extent 1, or summed away
            ea.bshape[ea.nb] = p.bshape[i];
            ea.c_bs[ea.nb] = p.c_bs[i];
            ea.x_bs[ea.nb] = p.aux_bs[i];
            ++ea.nb;
        }
        ea.M = p.M;
        ea.N = p.N;
        ea.c_rs = p.c_rs;
        ea.x_rs = p.aux_rs;
        ea.x_cs = p.aux_cs;
        ea.op = p.aux_op;
        ea.beta = p.beta;
        cudaError_t e = launch_epi_apply(ea, stream);
        if (e != cudaSuccess) return cuda_fail(e, "epilogue pass launch");
        st->launches++;
    }
    return AKR_OK;
}

int resolve_mode(int mode) {
    if (mode == AKR_MODE_GLOBAL) return g_tf32.load() ? AKR_MODE_TF32 : AKR_MODE_FP32;
    return mode == AKR_MODE_TF32 ? AKR_MODE_TF32 : AKR_MODE_FP32;
}

int check_out(const akr_view* c, int nd, const int64_t* shape, const char* name) {
    int rc = check_view(c, name, 0);
    if (rc != AKR_OK) return rc;
    if (c->ndim != nd) return fail(AKR_ERR_INVALID, std::string(name) + ": wrong number of dimensions");
    for (int i = 0; i < nd; ++i)
        if (c->shape[i] != shape[i]) return fail(AKR_ERR_INVALID, std::string(name) + ": wrong shape");
    if (nd >= 1 && c->shape[nd - 1] > 1 && c->stride[nd - 1] != 1)
        return fail(AKR_ERR_INVALID, std::string(name) + ": last dimension must have unit stride");
    return AKR_OK;
}

StridedView to_strided(const akr_view* v) {
    StridedView s;
    s.ptr = (const float*)v->data;
    s.nd = v->ndim;
    for (int i = 0; i < kMaxDims; ++i) {
        s.shape[i] = i < v->ndim ? v->shape[i] : 1;
        s.stride[i] = i < v->ndim ? v->stride[i] : 0;
    }
    return s;
}

int need_gpu(DeviceState** st) { return get_state(st); }

}  // namespace

namespace akr {
// Lets the library's other translation units record the message akr_last_error() returns.
void set_last_error(const std::string& msg) { g_err = msg; }
// The lock that serialises kernel launches (and the host-side state behind them) of one device.
std::mutex& device_launch_mutex(int dev) { return g_dev[dev >= 0 && dev < kMaxDevices ? dev : 0].mu; }
int noalloc_take_status(int dev);  // csrc/noalloc.cu
}  // namespace akr

extern "C" {

AKR_API const char* akr_last_error(void) { return g_err.c_str(); }
AKR_API int akr_version(void) { return 100; }

AKR_API int akr_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

AKR_API int akr_set_device(int ordinal) {
    cudaError_t e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    return AKR_OK;
}

AKR_API void akr_set_tf32(int enabled) { g_tf32.store(enabled ? 1 : 0); }
AKR_API int akr_get_tf32(void) { return g_tf32.load(); }
AKR_API void akr_set_cudnn_tf32(int enabled) { g_cudnn_tf32.store(enabled ? 1 : 0); }
AKR_API int akr_get_cudnn_tf32(void) { return g_cudnn_tf32.load(); }

AKR_API int akr_synchronize(void) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    bool aborted = false;
    if (st->status) {
        int flag = 0;
        e = cudaMemcpy(&flag, st->status, sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return cuda_fail(e, "status read");
        if (flag != 0) {
            cudaMemset(st->status, 0, sizeof(int));
            aborted = true;
        }
    }
    // kernels of the allocation-free entry point report through a status word of their own
    if (akr::noalloc_take_status((int)(st - g_dev)) != 0) aborted = true;
    if (aborted) return fail(AKR_ERR_ABORTED, "a GEMM kernel gave up on a bounded wait; its output is invalid");
    return AKR_OK;
}

AKR_API int akr_alloc(size_t nfloats, float** out) {
    if (!out) return fail(AKR_ERR_INVALID, "akr_alloc: null out");
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    auto it = st->free_blocks.find(nfloats);
    if (it != st->free_blocks.end() && !it->second.empty()) {
        *out = it->second.back();
        it->second.pop_back();
        st->hits++;
        return AKR_OK;
    }
    st->misses++;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, std::max<size_t>(nfloats, 1) * sizeof(float));
    if (e != cudaSuccess) {
        char msg[256];
        std::snprintf(msg, sizeof(msg),
                      "Aakaar CUDA allocation failed: %s (requested %zu bytes, cache had %lld hits / %lld "
                      "misses so far)",
                      cudaGetErrorString(e), nfloats * sizeof(float), (long long)st->hits,
                      (long long)st->misses);
        cudaGetLastError();
        return fail(AKR_ERR_RUNTIME, msg);
    }
    *out = (float*)p;
    return AKR_OK;
}

AKR_API int akr_free(float* ptr, size_t nfloats) {
    if (!ptr) return AKR_OK;
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    st->free_blocks[nfloats].push_back(ptr);
    return AKR_OK;
}

AKR_API int akr_empty_cache(void) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    for (auto& kv : st->free_blocks)
        for (float* p : kv.second) cudaFree(p);
    st->free_blocks.clear();
    for (int i = 0; i < WS_COUNT; ++i) {
        if (st->ws[i].ptr) cudaFree(st->ws[i].ptr);
        st->ws[i] = Region();
    }
    return AKR_OK;
}

AKR_API int akr_allocator_stats(int64_t* hits, int64_t* misses) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        dev = 0;
    }
    if (hits) *hits = g_dev[dev].hits;
    if (misses) *misses = g_dev[dev].misses;
    return AKR_OK;
}

AKR_API int akr_host_alloc(size_t bytes, void** out) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    cudaError_t e = cudaHostAlloc(out, std::max<size_t>(bytes, 1), cudaHostAllocDefault);
    if (e != cudaSuccess) return cuda_fail(e, "cudaHostAlloc");
    return AKR_OK;
}
AKR_API int akr_host_free(void* ptr) {
    if (!ptr) return AKR_OK;
    cudaError_t e = cudaFreeHost(ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFreeHost");
    return AKR_OK;
}

static int do_copy(void* dst, const void* src, size_t bytes, void* stream, cudaMemcpyKind kind) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    if (bytes == 0) return AKR_OK;
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync");
    return AKR_OK;
}
AKR_API int akr_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
    return do_copy(dst, src, bytes, stream, cudaMemcpyHostToDevice);
}
AKR_API int akr_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
    return do_copy(dst, src, bytes, stream, cudaMemcpyDeviceToHost);
}
AKR_API int akr_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
    return do_copy(dst, src, bytes, stream, cudaMemcpyDeviceToDevice);
}
AKR_API int akr_memset_zero(void* dst, size_t bytes, void* stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    cudaError_t e = cudaMemsetAsync(dst, 0, bytes, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync");
    return AKR_OK;
}
AKR_API int akr_stream_synchronize(void* stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    return AKR_OK;
}

AKR_API int akr_matmul_plan(const akr_view* a, const akr_view* b, int64_t* out_shape, int32_t* out_ndim) {
    Plan p;
    int rc = make_plan(a, b, &p);
    if (rc != AKR_OK) return rc;
    if (p.nb + 2 > AKR_MAX_DIMS) return fail(AKR_ERR_INVALID, "matmul: result has more than 8 dimensions");
    if (out_shape) {
        for (int i = 0; i < p.nb; ++i) out_shape[i] = p.batch[i];
        out_shape[p.nb] = p.M;
        out_shape[p.nb + 1] = p.N;
    }
    if (out_ndim) *out_ndim = p.nb + 2;
    return AKR_OK;
}

static int matmul_fwd_impl(const akr_view* a, const akr_view* b, const akr_view* bias, akr_view* c, float alpha,
                           float beta, const akr_view* d, int mode, void* stream) {
    Plan pl;
    int rc = make_plan(a, b, &pl);
    if (rc != AKR_OK) return rc;
    if ((rc = check_view(a, "matmul input a", 2)) != AKR_OK) return rc;
    if ((rc = check_view(b, "matmul input b", 2)) != AKR_OK) return rc;
    int64_t oshape[AKR_MAX_DIMS + 2];
    for (int i = 0; i < pl.nb; ++i) oshape[i] = pl.batch[i];
    oshape[pl.nb] = pl.M;
    oshape[pl.nb + 1] = pl.N;
    if ((rc = check_out(c, pl.nb + 2, oshape, "matmul output")) != AKR_OK) return rc;
    const float* bias_ptr = nullptr;
    if (bias) {
        if ((rc = check_view(bias, "matmul bias", 1)) != AKR_OK) return rc;
        bool ok = bias->shape[bias->ndim - 1] == pl.N && (pl.N == 1 || bias->stride[bias->ndim - 1] == 1);
        for (int i = 0; i + 1 < bias->ndim; ++i) ok = ok && bias->shape[i] == 1;
        if (!ok) return fail(AKR_ERR_INVALID, "matmul bias must be a contiguous row vector of N values");
        bias_ptr = (const float*)bias->data;
    }
    Problem p;
    p.M = pl.M;
    p.N = pl.N;
    p.K = pl.K;
    p.nb = pl.nb;
    for (int i = 0; i < pl.nb; ++i) {
        p.bshape[i] = pl.batch[i];
        p.A.bs[i] = batch_stride(a, pl.nb, i);
        p.B.bs[i] = batch_stride(b, pl.nb, i);
        p.c_bs[i] = c->stride[i];
        if (pl.batch[i] > 1 && c->stride[i] == 0)
            return fail(AKR_ERR_INVALID, "matmul output must not be a broadcast view");
    }
    p.A.ptr = (const float*)a->data;
    p.A.s_mn = a->stride[a->ndim - 2];
    p.A.s_k = a->stride[a->ndim - 1];
    p.B.ptr = (const float*)b->data;
    p.B.s_mn = b->stride[b->ndim - 1];
    p.B.s_k = b->stride[b->ndim - 2];
    p.C = (float*)c->data;
    p.c_rs = c->stride[c->ndim - 2];
    p.bias = bias_ptr;
    p.alpha = alpha;
    if (d) {
        if ((rc = check_view(d, "matmul addend", 2)) != AKR_OK) return rc;
        if (d->ndim != pl.nb + 2) return fail(AKR_ERR_INVALID, "matmul addend must have the shape of the output");
        for (int i = 0; i < pl.nb + 2; ++i)
            if (d->shape[i] != oshape[i]) return fail(AKR_ERR_INVALID, "matmul addend must have the shape of the output");
        p.aux_op = 1;
        p.beta = beta;
        p.aux = (const float*)d->data;
        p.aux_rs = d->stride[d->ndim - 2];
        p.aux_cs = d->stride[d->ndim - 1];
        for (int i = 0; i < pl.nb; ++i) p.aux_bs[i] = d->stride[i];
    }
    p.mode = resolve_mode(mode);
    return run_problem(p, (cudaStream_t)stream);
}

AKR_API int akr_matmul_fwd(const akr_view* a, const akr_view* b, const akr_view* bias, akr_view* c, int mode,
                   void* stream) {
    return matmul_fwd_impl(a, b, bias, c, 1.f, 0.f, nullptr, mode, stream);
}

AKR_API int akr_matmul_fwd_axpby(const akr_view* a, const akr_view* b, float alpha, float beta, const akr_view* d,
                                 akr_view* c, int mode, void* stream) {
    if (beta != 0.f && !d) return fail(AKR_ERR_INVALID, "matmul_fwd_axpby: beta != 0 needs an addend");
    return matmul_fwd_impl(a, b, nullptr, c, alpha, beta, beta != 0.f ? d : nullptr, mode, stream);
}

static int matmul_bwd_impl(const akr_view* a, const akr_view* b, const akr_view* dc, akr_view* da, akr_view* db,
                           bool a_is_tanh, int mode, void* stream, float* da_colsum = nullptr) {
    Plan pl;
    int rc = make_plan(a, b, &pl);
    if (rc != AKR_OK) return rc;
    if ((rc = check_view(a, "matmul input a", 2)) != AKR_OK) return rc;
    if ((rc = check_view(b, "matmul input b", 2)) != AKR_OK) return rc;
    int64_t oshape[AKR_MAX_DIMS + 2];
    for (int i = 0; i < pl.nb; ++i) oshape[i] = pl.batch[i];
    oshape[pl.nb] = pl.M;
    oshape[pl.nb + 1] = pl.N;
    if ((rc = check_view(dc, "matmul grad_output", 2)) != AKR_OK) return rc;
    if (dc->ndim != pl.nb + 2) return fail(AKR_ERR_INVALID, "matmul backward: grad_output has the wrong rank");
    for (int i = 0; i < pl.nb + 2; ++i)
        if (dc->shape[i] != oshape[i]) return fail(AKR_ERR_INVALID, "matmul backward: grad_output has the wrong shape");
    const int m = resolve_mode(mode);

    if (da) {
        if ((rc = check_out(da, a->ndim, a->shape, "matmul grad a")) != AKR_OK) return rc;
        Problem p;  // dA[m,k] = sum_n dC[m,n] * B[k,n]
        p.M = pl.M;
        p.N = pl.K;
        p.K = pl.N;
        p.nb = pl.nb;
        for (int i = 0; i < pl.nb; ++i) {
            p.bshape[i] = pl.batch[i];
            p.A.bs[i] = pl.batch[i] == 1 ? 0 : dc->stride[i];
            p.B.bs[i] = batch_stride(b, pl.nb, i);
            p.c_bs[i] = batch_stride(da, pl.nb, i);
        }
        p.A.ptr = (const float*)dc->data;
        p.A.s_mn = dc->stride[dc->ndim - 2];
        p.A.s_k = dc->stride[dc->ndim - 1];
        p.B.ptr = (const float*)b->data;
        p.B.s_mn = b->stride[b->ndim - 2];
        p.B.s_k = b->stride[b->ndim - 1];
        p.C = (float*)da->data;
        p.c_rs = da->stride[da->ndim - 2];
        p.mode = m;
        if (a_is_tanh) {  // gradient w.r.t. the tanh's input: (dC B^T) * (1 - A^2), A read where it lies
            p.aux_op = 2;
            p.aux = (const float*)a->data;
            p.aux_rs = a->stride[a->ndim - 2];
            p.aux_cs = a->stride[a->ndim - 1];
            for (int i = 0; i < pl.nb; ++i) p.aux_bs[i] = batch_stride(a, pl.nb, i);
        }
        p.colsum_out = da_colsum;
        if ((rc = run_problem(p, (cudaStream_t)stream)) != AKR_OK) return rc;
        if (da_colsum && !p.colsum_done) {
            // the kernel that ran has no column-sum epilogue (fp32-accurate mode, split contraction, ...): one
            // more pass over the finished gradient
            akr_view out;
            std::memset(&out, 0, sizeof(out));
            out.data = da_colsum;
            out.ndim = 1;
            out.dtype = AKR_DTYPE_F32;
            out.shape[0] = pl.K;
            out.stride[0] = 1;
            if ((rc = akr_sum_to(da, &out, stream)) != AKR_OK) return rc;
        }
    }
    if (db) {
        if ((rc = check_out(db, b->ndim, b->shape, "matmul grad b")) != AKR_OK) return rc;
        Problem p;  // dB[k,n] = sum_m A[m,k] * dC[m,n]
        p.M = pl.K;
        p.N = pl.N;
        p.K = pl.M;
        p.nb = pl.nb;
        for (int i = 0; i < pl.nb; ++i) {
            p.bshape[i] = pl.batch[i];
            p.A.bs[i] = batch_stride(a, pl.nb, i);
            p.B.bs[i] = pl.batch[i] == 1 ? 0 : dc->stride[i];
            p.c_bs[i] = batch_stride(db, pl.nb, i);
        }
        p.A.ptr = (const float*)a->data;
        p.A.s_mn = a->stride[a->ndim - 1];
        p.A.s_k = a->stride[a->ndim - 2];
        p.B.ptr = (const float*)dc->data;
        p.B.s_mn = dc->stride[dc->ndim - 1];
        p.B.s_k = dc->stride[dc->ndim - 2];
        p.C = (float*)db->data;
        p.c_rs = db->stride[db->ndim - 2];
        p.mode = m;
        if ((rc = run_problem(p, (cudaStream_t)stream)) != AKR_OK) return rc;
    }
    return AKR_OK;
}

AKR_API int akr_matmul_bwd(const akr_view* a, const akr_view* b, const akr_view* dc, akr_view* da, akr_view* db,
                   int mode, void* stream) {
    return matmul_bwd_impl(a, b, dc, da, db, false, mode, stream);
}

AKR_API int akr_matmul_bwd_tanh(const akr_view* a, const akr_view* b, const akr_view* dc, akr_view* dz, akr_view* db,
                                int mode, void* stream) {
    return matmul_bwd_impl(a, b, dc, dz, db, true, mode, stream);
}

AKR_API int akr_matmul_bwd_colsum(const akr_view* a, const akr_view* b, const akr_view* dc, akr_view* da,
                                  akr_view* db_or_null, float* da_colsum, int a_is_tanh_output, int mode, void* stream) {
    if (!da) return fail(AKR_ERR_INVALID, "matmul_bwd_colsum: the gradient whose column sums are wanted must be requested");
    if (!da_colsum) return fail(AKR_ERR_INVALID, "matmul_bwd_colsum: null column-sum buffer");
    return matmul_bwd_impl(a, b, dc, da, db_or_null, a_is_tanh_output != 0, mode, stream, da_colsum);
}

AKR_API int akr_matmul_a_bt(const akr_view* a, const akr_view* b, akr_view* c, int mode, void* stream) {
    int rc;
    if ((rc = check_view(a, "matmul_a_bt a", 2)) != AKR_OK) return rc;
    if ((rc = check_view(b, "matmul_a_bt b", 2)) != AKR_OK) return rc;
    if (a->ndim != 2 || b->ndim != 2) return fail(AKR_ERR_INVALID, "matmul_a_bt requires 2-D tensors");
    if (b->shape[1] != a->shape[1]) return fail(AKR_ERR_INVALID, "matmul_a_bt: inner dimensions must match");
    const int64_t oshape[2] = {a->shape[0], b->shape[0]};
    if ((rc = check_out(c, 2, oshape, "matmul_a_bt output")) != AKR_OK) return rc;
    Problem p;
    p.M = a->shape[0];
    p.N = b->shape[0];
    p.K = a->shape[1];
    p.A.ptr = (const float*)a->data;
    p.A.s_mn = a->stride[0];
    p.A.s_k = a->stride[1];
    p.B.ptr = (const float*)b->data;
    p.B.s_mn = b->stride[0];
    p.B.s_k = b->stride[1];
    p.C = (float*)c->data;
    p.c_rs = c->stride[0];
    p.mode = resolve_mode(mode);
    return run_problem(p, (cudaStream_t)stream);
}

AKR_API int akr_matmul_at_b(const akr_view* a, const akr_view* b, akr_view* c, int mode, void* stream) {
    int rc;
    if ((rc = check_view(a, "matmul_at_b a", 2)) != AKR_OK) return rc;
    if ((rc = check_view(b, "matmul_at_b b", 2)) != AKR_OK) return rc;
    if (a->ndim != 2 || b->ndim != 2) return fail(AKR_ERR_INVALID, "matmul_at_b requires 2-D tensors");
    if (b->shape[0] != a->shape[0]) return fail(AKR_ERR_INVALID, "matmul_at_b: inner dimensions must match");
    const int64_t oshape[2] = {a->shape[1], b->shape[1]};
    if ((rc = check_out(c, 2, oshape, "matmul_at_b output")) != AKR_OK) return rc;
    Problem p;
    p.M = a->shape[1];
    p.N = b->shape[1];
    p.K = a->shape[0];
    p.A.ptr = (const float*)a->data;
    p.A.s_mn = a->stride[1];
    p.A.s_k = a->stride[0];
    p.B.ptr = (const float*)b->data;
    p.B.s_mn = b->stride[1];
    p.B.s_k = b->stride[0];
    p.C = (float*)c->data;
    p.c_rs = c->stride[0];
    p.mode = resolve_mode(mode);
    return run_problem(p, (cudaStream_t)stream);
}

static int simt_forward(const akr_view* a, const akr_view* b, akr_view* c, int dtype, void* stream);

AKR_API int akr_matmul_fwd_typed(const akr_view* a, const akr_view* b, akr_view* c, void* stream) {
    if (!a || !b || !c) return fail(AKR_ERR_INVALID, "matmul: null view");
    const int dt = a->dtype;
    if (dt != AKR_DTYPE_F64 && dt != AKR_DTYPE_I32 && dt != AKR_DTYPE_I64)
        return fail(AKR_ERR_RUNTIME, "matmul_fwd_typed handles float64, int32 and int64 (use akr_matmul_fwd for float32)");
    if (b->dtype != dt || c->dtype != dt) return fail(AKR_ERR_RUNTIME, "matmul: operands must share one dtype");
    return simt_forward(a, b, c, dt, stream);
}

AKR_API int akr_matmul_fwd_simt(const akr_view* a, const akr_view* b, akr_view* c, void* stream) {
    return simt_forward(a, b, c, AKR_DTYPE_F32, stream);
}

static int simt_forward(const akr_view* a, const akr_view* b, akr_view* c, int dtype, void* stream) {
    Plan pl;
    int rc = make_plan(a, b, &pl);
    if (rc != AKR_OK) return rc;
    akr_view ta = *a, tb = *b, tc = *c;   // the shape checks below are dtype-agnostic
    ta.dtype = tb.dtype = tc.dtype = AKR_DTYPE_F32;
    if ((rc = check_view(&ta, "matmul input a", 2)) != AKR_OK) return rc;
    if ((rc = check_view(&tb, "matmul input b", 2)) != AKR_OK) return rc;
    int64_t oshape[AKR_MAX_DIMS + 2];
    for (int i = 0; i < pl.nb; ++i) oshape[i] = pl.batch[i];
    oshape[pl.nb] = pl.M;
    oshape[pl.nb + 1] = pl.N;
    if ((rc = check_out(&tc, pl.nb + 2, oshape, "matmul output")) != AKR_OK) return rc;
    DeviceState* st = nullptr;
    if ((rc = need_gpu(&st)) != AKR_OK) return rc;
    SimtGemm g;
    g.A = (const float*)a->data;
    g.B = (const float*)b->data;
    g.C = (float*)c->data;
    g.M = (int)pl.M;
    g.N = (int)pl.N;
    g.K = (int)pl.K;
    g.nb = pl.nb;
    for (int i = 0; i < kMaxDims; ++i) {
        g.bshape[i] = i < pl.nb ? pl.batch[i] : 1;
        g.a_bs[i] = i < pl.nb ? batch_stride(a, pl.nb, i) : 0;
        g.b_bs[i] = i < pl.nb ? batch_stride(b, pl.nb, i) : 0;
        g.c_bs[i] = i < pl.nb ? c->stride[i] : 0;
    }
    g.a_rs = a->stride[a->ndim - 2];
    g.a_cs = a->stride[a->ndim - 1];
    g.b_rs = b->stride[b->ndim - 2];
    g.b_cs = b->stride[b->ndim - 1];
    g.c_rs = c->stride[c->ndim - 2];
    g.c_cs = c->stride[c->ndim - 1];
    cudaError_t e = dtype == AKR_DTYPE_F32 ? launch_simt_gemm(g, (cudaStream_t)stream)
                                           : launch_simt_gemm_typed(g, dtype, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "simt matmul launch");
    st->launches++;
    return AKR_OK;
}

AKR_API int akr_debug_configure(int flags, unsigned wait_limit_ms) {
    gemm_sm100_debug_configure(flags, wait_limit_ms);
    return AKR_OK;
}

AKR_API int akr_gemm_clock_read(int ctas, double* sm_mhz_mean, double* sm_mhz_min, double* cycles_max, double* us_max) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    const int r = gemm_sm100_clock_read(ctas, sm_mhz_mean, sm_mhz_min, cycles_max, us_max);
    if (r == -2) return fail(AKR_ERR_INVALID, "akr_gemm_clock_read: no launch recorded (akr_debug_configure(32768, 0) first)");
    if (r != 0) return fail(AKR_ERR_CUDA, "akr_gemm_clock_read: cannot read the probe");
    return AKR_OK;
}

AKR_API int akr_set_gemm_cta_limit(int ctas) {
    gemm_sm100_set_cta_limit(ctas);
    return AKR_OK;
}

AKR_API int akr_stream_create(void** stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    cudaStream_t s;
    cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamCreateWithFlags");
    *stream = (void*)s;
    return AKR_OK;
}
AKR_API int akr_stream_destroy(void* stream) {
    cudaError_t e = cudaStreamDestroy((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamDestroy");
    return AKR_OK;
}
AKR_API int akr_stream_wait_event(void* stream, void* event) {
    cudaError_t e = cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
    return AKR_OK;
}

AKR_API int akr_event_create(void** event) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    cudaEvent_t ev;
    cudaError_t e = cudaEventCreate(&ev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
    *event = (void*)ev;
    return AKR_OK;
}
AKR_API int akr_event_record(void* event, void* stream) {
    cudaError_t e = cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
    return AKR_OK;
}
AKR_API int akr_event_synchronize(void* event) {
    cudaError_t e = cudaEventSynchronize((cudaEvent_t)event);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventSynchronize");
    return AKR_OK;
}
AKR_API int akr_event_elapsed_ms(void* start, void* end, float* ms) {
    cudaError_t e = cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventElapsedTime");
    return AKR_OK;
}
AKR_API int akr_event_destroy(void* event) {
    cudaError_t e = cudaEventDestroy((cudaEvent_t)event);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventDestroy");
    return AKR_OK;
}

AKR_API int akr_workspace_bytes(size_t* bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        dev = 0;
    }
    size_t total = 0;
    for (int i = 0; i < WS_COUNT; ++i) total += g_dev[dev].ws[i].bytes;
    if (bytes) *bytes = total;
    return AKR_OK;
}

AKR_API int64_t akr_launch_count(int reset) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        dev = 0;
    }
    const int64_t n = g_dev[dev].launches;
    if (reset) g_dev[dev].launches = 0;
    return n;
}

// ------------------------------------------------------------------ support ops

#define AKR_LAUNCH(expr, what)                          \
    do {                                                \
        DeviceState* st_ = nullptr;                     \
        int rc_ = need_gpu(&st_);                       \
        if (rc_ != AKR_OK) return rc_;                  \
        cudaError_t e_ = (expr);                        \
        if (e_ != cudaSuccess) return cuda_fail(e_, what); \
        st_->launches++;                                \
        return AKR_OK;                                  \
    } while (0)

AKR_API int akr_contiguous(const akr_view* src, float* dst, void* stream) {
    int rc = check_view(src, "contiguous", 0);
    if (rc != AKR_OK) return rc;
    AKR_LAUNCH(launch_gather(to_strided(src), dst, (cudaStream_t)stream), "gather launch");
}

AKR_API int akr_scatter(const float* src, akr_view* dst, void* stream) {
    int rc = check_view(dst, "scatter destination", 0);
    if (rc != AKR_OK) return rc;
    if (!src) return fail(AKR_ERR_INVALID, "scatter: null source");
    for (int i = 0; i < dst->ndim; ++i)
        if (dst->shape[i] > 1 && dst->stride[i] == 0) return fail(AKR_ERR_INVALID, "scatter: destination must not be a broadcast view");
    AKR_LAUNCH(launch_scatter(src, to_strided(dst), (cudaStream_t)stream), "scatter launch");
}

static int binary_op(const akr_view* a, const akr_view* b, akr_view* out, void* stream, bool multiply);
AKR_API int akr_add(const akr_view* a, const akr_view* b, akr_view* out, void* stream) {
    return binary_op(a, b, out, stream, false);
}
AKR_API int akr_mul(const akr_view* a, const akr_view* b, akr_view* out, void* stream) {
    return binary_op(a, b, out, stream, true);
}
static int binary_op(const akr_view* a, const akr_view* b, akr_view* out, void* stream, bool multiply) {
    int rc;
    if ((rc = check_view(a, "add a", 0)) != AKR_OK) return rc;
    if ((rc = check_view(b, "add b", 0)) != AKR_OK) return rc;
    if ((rc = check_view(out, "add out", 0)) != AKR_OK) return rc;
    const int nd = out->ndim;
    if (a->ndim > nd || b->ndim > nd) return fail(AKR_ERR_INVALID, "add: output rank too small");
    StridedView sa, sb;
    sa.ptr = (const float*)a->data;
    sb.ptr = (const float*)b->data;
    sa.nd = sb.nd = nd;
    int64_t expect = 1;
    for (int i = nd - 1; i >= 0; --i) {
        const int ia = i - (nd - a->ndim), ib = i - (nd - b->ndim);
        const int64_t da = ia >= 0 ? a->shape[ia] : 1, dbb = ib >= 0 ? b->shape[ib] : 1;
        if ((da != out->shape[i] && da != 1) || (dbb != out->shape[i] && dbb != 1))
            return fail(AKR_ERR_INVALID, "add: shapes are not broadcastable");
        sa.shape[i] = sb.shape[i] = out->shape[i];
        sa.stride[i] = (ia >= 0 && da != 1) ? a->stride[ia] : 0;
        sb.stride[i] = (ib >= 0 && dbb != 1) ? b->stride[ib] : 0;
        if (out->shape[i] != 1 && out->stride[i] != expect) return fail(AKR_ERR_INVALID, "add: output must be contiguous");
        expect *= out->shape[i];
    }
    AKR_LAUNCH(launch_add(sa, sb, (float*)out->data, nd, out->shape, (cudaStream_t)stream, multiply), "add launch");
}

AKR_API int akr_sum_to(const akr_view* grad, akr_view* out, void* stream) {
    int rc;
    if ((rc = check_view(grad, "sum_to grad", 0)) != AKR_OK) return rc;
    if ((rc = check_view(out, "sum_to out", 0)) != AKR_OK) return rc;
    if (out->ndim > grad->ndim) return fail(AKR_ERR_RUNTIME, "reduce_grad_to_shape: gradient has fewer dims than its target shape");
    int64_t oshape[AKR_MAX_DIMS];
    const int off = grad->ndim - out->ndim;
    for (int i = 0; i < grad->ndim; ++i) {
        oshape[i] = i < off ? 1 : out->shape[i - off];
        if (oshape[i] != grad->shape[i] && oshape[i] != 1)
            return fail(AKR_ERR_RUNTIME, "reduce_grad_to_shape: reduced gradient shape does not match target shape");
    }
    // Bias-gradient shape: a dense gradient summed over its leading dims only -> column sums.
    int lead = 0;
    while (lead < grad->ndim && oshape[lead] == 1) ++lead;
    bool colsum = lead > 0;
    int64_t expect = 1, rows = 1, cols = 1;
    for (int i = grad->ndim - 1; i >= 0 && colsum; --i) {
        if (grad->shape[i] != 1 && grad->stride[i] != expect) colsum = false;
        expect *= grad->shape[i];
        if (i >= lead) {
            if (oshape[i] != grad->shape[i]) colsum = false;
            cols *= grad->shape[i];
        } else {
            rows *= grad->shape[i];
        }
    }
    if (colsum && rows > 1 && cols >= 32) {
        DeviceState* st = nullptr;
        if ((rc = need_gpu(&st)) != AKR_OK) return rc;
        void* partials = nullptr;
        {
            std::lock_guard<std::mutex> lock(st->mu);
            if ((rc = ws_get(st, WS_MISC, std::max<size_t>(colsum_partial_floats(rows, cols), 4096) * sizeof(float),
                             &partials)) != AKR_OK)
                return rc;
        }
        cudaError_t e = launch_colsum((const float*)grad->data, rows, cols, (float*)out->data, (float*)partials,
                                      (cudaStream_t)stream);
        if (e != cudaSuccess) return cuda_fail(e, "column-sum launch");
        st->launches += 2;
        return AKR_OK;
    }
    AKR_LAUNCH(launch_sum_to(to_strided(grad), oshape, (float*)out->data, (cudaStream_t)stream), "sum_to launch");
}

AKR_API int akr_scale(const float* x, float alpha, float* y, size_t n, void* stream) {
    AKR_LAUNCH(launch_scale(x, alpha, y, n, (cudaStream_t)stream), "scale launch");
}
AKR_API int akr_fill(float* x, float value, size_t n, void* stream) {
    AKR_LAUNCH(launch_fill(x, value, n, (cudaStream_t)stream), "fill launch");
}
AKR_API int akr_tanh_fwd(const float* x, float* y, size_t n, void* stream) {
    AKR_LAUNCH(launch_tanh_fwd(x, y, n, (cudaStream_t)stream), "tanh launch");
}
AKR_API int akr_tanh_bwd(const float* grad, const float* y, float* dx, size_t n, void* stream) {
    AKR_LAUNCH(launch_tanh_bwd(grad, y, dx, n, (cudaStream_t)stream), "tanh backward launch");
}
static int window_geom(const akr_window* w, WindowGeom* g) {
    if (!w) return fail(AKR_ERR_INVALID, "im2col: null geometry");
    if (w->B <= 0 || w->C <= 0 || w->H <= 0 || w->W <= 0 || w->KH <= 0 || w->KW <= 0 || w->SH <= 0 || w->SW <= 0 ||
        w->DH <= 0 || w->DW <= 0 || w->PH < 0 || w->PW < 0 || w->OH <= 0 || w->OW <= 0)
        return fail(AKR_ERR_INVALID, "im2col: sizes, strides and dilations must be positive, padding non-negative");
    g->B = w->B; g->C = w->C; g->H = w->H; g->W = w->W;
    g->KH = w->KH; g->KW = w->KW; g->SH = w->SH; g->SW = w->SW;
    g->PH = w->PH; g->PW = w->PW; g->DH = w->DH; g->DW = w->DW;
    g->OH = w->OH; g->OW = w->OW;
    return AKR_OK;
}
AKR_API int akr_im2col(const float* x, float* col, const akr_window* geom, void* stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    WindowGeom g;
    if ((rc = window_geom(geom, &g)) != AKR_OK) return rc;
    if (!x || !col) return fail(AKR_ERR_INVALID, "im2col: null data pointer");
    cudaError_t e = launch_im2col(x, col, g, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "im2col launch");
    st->launches++;
    return AKR_OK;
}
AKR_API int akr_col2im(const float* grad_col, float* grad_x, const akr_window* geom, void* stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    WindowGeom g;
    if ((rc = window_geom(geom, &g)) != AKR_OK) return rc;
    if (!grad_col || !grad_x) return fail(AKR_ERR_INVALID, "col2im: null data pointer");
    cudaError_t e = launch_col2im(grad_col, grad_x, g, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "col2im launch");
    st->launches++;
    return AKR_OK;
}

static int window_geom_3d(const akr_window3d* w, WindowGeom* g) {
    if (!w) return fail(AKR_ERR_INVALID, "im2col_3d: null geometry");
    if (w->B <= 0 || w->C <= 0 || w->D <= 0 || w->H <= 0 || w->W <= 0 || w->KD <= 0 || w->KH <= 0 || w->KW <= 0 ||
        w->SD <= 0 || w->SH <= 0 || w->SW <= 0 || w->DD <= 0 || w->DH <= 0 || w->DW <= 0 || w->PD < 0 || w->PH < 0 ||
        w->PW < 0 || w->OD <= 0 || w->OH <= 0 || w->OW <= 0)
        return fail(AKR_ERR_INVALID, "im2col_3d: sizes, strides and dilations must be positive, padding non-negative");
    g->B = w->B; g->C = w->C; g->D = w->D; g->H = w->H; g->W = w->W;
    g->KD = w->KD; g->KH = w->KH; g->KW = w->KW; g->SD = w->SD; g->SH = w->SH; g->SW = w->SW;
    g->PD = w->PD; g->PH = w->PH; g->PW = w->PW; g->DD = w->DD; g->DH = w->DH; g->DW = w->DW;
    g->OD = w->OD; g->OH = w->OH; g->OW = w->OW;
    return AKR_OK;
}
AKR_API int akr_im2col_3d(const float* x, float* col, const akr_window3d* geom, void* stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    WindowGeom g;
    if ((rc = window_geom_3d(geom, &g)) != AKR_OK) return rc;
    if (!x || !col) return fail(AKR_ERR_INVALID, "im2col_3d: null data pointer");
    cudaError_t e = launch_im2col(x, col, g, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "im2col_3d launch");
    st->launches++;
    return AKR_OK;
}
AKR_API int akr_col2im_3d(const float* grad_col, float* grad_x, const akr_window3d* geom, void* stream) {
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    WindowGeom g;
    if ((rc = window_geom_3d(geom, &g)) != AKR_OK) return rc;
    if (!grad_col || !grad_x) return fail(AKR_ERR_INVALID, "col2im_3d: null data pointer");
    cudaError_t e = launch_col2im(grad_col, grad_x, g, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "col2im_3d launch");
    st->launches++;
    return AKR_OK;
}

static int mse_forward(const float* pred, const float* target, float* loss_out, float* dpred, size_t n, void* stream);
AKR_API int akr_mse_fwd_grad_colsum(const float* pred, const float* target, float* loss_out, float* dpred,
                                    float* dpred_colsum, int64_t rows, int64_t cols, void* stream) {
    if (!pred || !target || !loss_out || !dpred || !dpred_colsum)
        return fail(AKR_ERR_INVALID, "mse_fwd_grad_colsum: null pointer");
    if (rows <= 0 || cols <= 0) return fail(AKR_ERR_RUNTIME, "MSELoss: cannot reduce an empty tensor");
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    const bool aligned = ((reinterpret_cast<uintptr_t>(pred) | reinterpret_cast<uintptr_t>(target) |
                           reinterpret_cast<uintptr_t>(dpred) | reinterpret_cast<uintptr_t>(dpred_colsum)) & 15u) == 0;
    if ((cols & 3) != 0 || !aligned) {
        // odd widths: the plain loss + gradient pass, then a column sum of the gradient
        if ((rc = mse_forward(pred, target, loss_out, dpred, (size_t)rows * (size_t)cols, stream)) != AKR_OK) return rc;
        akr_view g, out;
        std::memset(&g, 0, sizeof(g));
        std::memset(&out, 0, sizeof(out));
        g.data = dpred; g.ndim = 2; g.dtype = AKR_DTYPE_F32;
        g.shape[0] = rows; g.shape[1] = cols; g.stride[0] = cols; g.stride[1] = 1;
        out.data = dpred_colsum; out.ndim = 1; out.dtype = AKR_DTYPE_F32; out.shape[0] = cols; out.stride[0] = 1;
        return akr_sum_to(&g, &out, stream);
    }
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(st->mu);
        if ((rc = ws_get(st, WS_MISC, std::max<size_t>(mse_colsum_scratch_floats(rows, cols), 4096) * sizeof(float),
                         &scratch)) != AKR_OK)
            return rc;
    }
    cudaError_t e = launch_mse_fwd_colsum(pred, target, loss_out, dpred, dpred_colsum, rows, cols, (float*)scratch,
                                          (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "mse launch");
    st->launches += 2;
    return AKR_OK;
}
AKR_API int akr_mse_fwd(const float* pred, const float* target, float* loss_out, size_t n, void* stream) {
    return mse_forward(pred, target, loss_out, nullptr, n, stream);
}
AKR_API int akr_mse_fwd_grad(const float* pred, const float* target, float* loss_out, float* dpred, size_t n,
                             void* stream) {
    if (!dpred) return fail(AKR_ERR_INVALID, "mse_fwd_grad: null gradient buffer");
    return mse_forward(pred, target, loss_out, dpred, n, stream);
}
static int mse_forward(const float* pred, const float* target, float* loss_out, float* dpred, size_t n, void* stream) {
    if (n == 0) return fail(AKR_ERR_RUNTIME, "MSELoss: cannot reduce an empty tensor");
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    void* partials = nullptr;
    {
        std::lock_guard<std::mutex> lock(st->mu);
        if ((rc = ws_get(st, WS_MISC, 4096 * sizeof(float), &partials)) != AKR_OK) return rc;
    }
    cudaError_t e = launch_mse_fwd(pred, target, loss_out, (float*)partials, n, (cudaStream_t)stream, dpred);
    if (e != cudaSuccess) return cuda_fail(e, "mse launch");
    st->launches += 2;
    return AKR_OK;
}
AKR_API int akr_mse_bwd(const float* pred, const float* target, const float* grad_scalar, float* dpred, size_t n,
                void* stream) {
    AKR_LAUNCH(launch_mse_bwd(pred, target, grad_scalar, dpred, n, (cudaStream_t)stream), "mse backward launch");
}
AKR_API int akr_sgd_step(float* param, const float* grad, float* velocity, float lr, float momentum,
                 float weight_decay, float dampening, int nesterov, int has_momentum,
                 int velocity_initialized, size_t n, void* stream) {
    if (has_momentum && !velocity) return fail(AKR_ERR_INVALID, "sgd_step: momentum needs a velocity buffer");
    AKR_LAUNCH(launch_sgd(param, grad, velocity, lr, momentum, weight_decay, dampening, nesterov,
                          has_momentum, velocity_initialized, n, (cudaStream_t)stream),
               "sgd launch");
}

AKR_API int akr_sgd_step_multi(int count, float* const* params, const float* const* grads, float* const* velocities,
                               const size_t* sizes, const int* velocity_initialized, float lr, float momentum,
                               float weight_decay, float dampening, int nesterov, int has_momentum, void* stream) {
    if (count < 0 || (count > 0 && (!params || !grads || !sizes)))
        return fail(AKR_ERR_INVALID, "sgd_step_multi: null argument");
    if (has_momentum && !velocities) return fail(AKR_ERR_INVALID, "sgd_step_multi: momentum needs velocity buffers");
    DeviceState* st = nullptr;
    int rc = need_gpu(&st);
    if (rc != AKR_OK) return rc;
    for (int first = 0; first < count; first += kSgdMultiMax) {   // 48 tensors per launch
        SgdMulti m;
        m.count = std::min(kSgdMultiMax, count - first);
        for (int i = 0; i < m.count; ++i) {
            const int j = first + i;
            if (!params[j] || !grads[j] || (has_momentum && !velocities[j]))
                return fail(AKR_ERR_INVALID, "sgd_step_multi: null tensor");
            m.param[i] = params[j];
            m.grad[i] = grads[j];
            m.vel[i] = has_momentum ? velocities[j] : nullptr;
            m.n[i] = sizes[j];
            m.vel_init[i] = velocity_initialized ? velocity_initialized[j] : 0;
        }
        cudaError_t e = launch_sgd_multi(m, lr, momentum, weight_decay, dampening, nesterov, has_momentum,
                                         (cudaStream_t)stream);
        if (e != cudaSuccess) return cuda_fail(e, "sgd launch");
        st->launches++;
    }
    return AKR_OK;
}

}  // extern "C"
