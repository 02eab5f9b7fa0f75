// akr_mg_*: the one collective of the sharded matmul path - the sum of a replicated weight's gradient over
// the GPUs of a node - behind the C ABI, so that a host written in any language gets the multi-GPU path
// without PyTorch. The collective itself is NCCL's ring / tree / in-switch reduction over NVLink; NCCL is
// loaded at run time (dlopen), so the library keeps no link-time dependency on it and single-GPU users
// never load it. No counterpart in the reference, which is single-GPU (docs/limitations.md:15).
#include "../../include/akr_b200.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>  // types and prototypes only

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace akr {
void set_last_error(const std::string& msg);  // defined beside akr_last_error()
}

namespace {

struct NcclApi {
    void* handle = nullptr;
    decltype(&ncclGetUniqueId) get_unique_id = nullptr;
    decltype(&ncclCommInitRank) comm_init_rank = nullptr;
    decltype(&ncclAllReduce) all_reduce = nullptr;
    decltype(&ncclCommDestroy) comm_destroy = nullptr;
    decltype(&ncclGetErrorString) error_string = nullptr;
    decltype(&ncclGetVersion) get_version = nullptr;
    std::string why;  // why loading failed
};

NcclApi g_api;
std::once_flag g_api_once;

template <typename F>
bool bind(void* h, const char* name, F* out, std::string* why) {
    *out = reinterpret_cast<F>(dlsym(h, name));
    if (*out) return true;
    *why = std::string("symbol ") + name + " not found in the NCCL library";
    return false;
}

const NcclApi& api() {
    std::call_once(g_api_once, [] {
        const char* path = std::getenv("AKR_B200_NCCL_LIB");  // explicit library file; default: the loader's search
        const char* names[] = {path, "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            g_api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (g_api.handle) break;
        }
        if (!g_api.handle) {
            g_api.why = "cannot load libnccl.so.2 (set AKR_B200_NCCL_LIB to its path)";
            return;
        }
        void* h = g_api.handle;
        const bool ok = bind(h, "ncclGetUniqueId", &g_api.get_unique_id, &g_api.why) &&
                        bind(h, "ncclCommInitRank", &g_api.comm_init_rank, &g_api.why) &&
                        bind(h, "ncclAllReduce", &g_api.all_reduce, &g_api.why) &&
                        bind(h, "ncclCommDestroy", &g_api.comm_destroy, &g_api.why) &&
                        bind(h, "ncclGetErrorString", &g_api.error_string, &g_api.why) &&
                        bind(h, "ncclGetVersion", &g_api.get_version, &g_api.why);
        if (!ok) g_api.handle = nullptr;
    });
    return g_api;
}

struct Comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};
constexpr int kMaxDevices = 64;
Comm g_comm[kMaxDevices];
std::mutex g_mu;

int mg_fail(int code, const std::string& msg) {
    akr::set_last_error(msg);
    return code;
}

int nccl_fail(ncclResult_t r, const char* what) {
    const NcclApi& a = api();
    return mg_fail(AKR_ERR_RUNTIME, std::string(what) + ": " + (a.error_string ? a.error_string(r) : "NCCL error"));
}

int current_device(int* dev) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return mg_fail(AKR_ERR_NOGPU, "no CUDA device available: aakaar_b200 has no CPU path");
    }
    if (cudaGetDevice(dev) != cudaSuccess || *dev < 0 || *dev >= kMaxDevices)
        return mg_fail(AKR_ERR_CUDA, "cannot identify the current device");
    return AKR_OK;
}

int need_api() {
    const NcclApi& a = api();
    if (!a.handle) return mg_fail(AKR_ERR_RUNTIME, "akr_mg: " + a.why);
    return AKR_OK;
}

}  // namespace

extern "C" {

AKR_API int akr_mg_get_unique_id(void* id_out) {
    if (!id_out) return mg_fail(AKR_ERR_INVALID, "akr_mg_get_unique_id: null buffer");
    int rc = need_api();
    if (rc != AKR_OK) return rc;
    static_assert(sizeof(ncclUniqueId) == AKR_MG_UNIQUE_ID_BYTES, "unique id size");
    ncclUniqueId id;
    ncclResult_t r = api().get_unique_id(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    std::memcpy(id_out, &id, sizeof(id));
    return AKR_OK;
}

AKR_API int akr_mg_init(int rank, int world, const void* unique_id) {
    if (world < 1 || rank < 0 || rank >= world) return mg_fail(AKR_ERR_INVALID, "akr_mg_init: bad rank / world");
    if (!unique_id) return mg_fail(AKR_ERR_INVALID, "akr_mg_init: null unique id");
    int rc = need_api();
    if (rc != AKR_OK) return rc;
    int dev = 0;
    if ((rc = current_device(&dev)) != AKR_OK) return rc;
    std::lock_guard<std::mutex> lock(g_mu);
    Comm& c = g_comm[dev];
    if (c.comm) return mg_fail(AKR_ERR_INVALID, "akr_mg_init: this device already has a communicator (akr_mg_finalize first)");
    ncclUniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    ncclResult_t r = api().comm_init_rank(&c.comm, world, id, rank);
    if (r != ncclSuccess) {
        c.comm = nullptr;
        return nccl_fail(r, "ncclCommInitRank");
    }
    c.rank = rank;
    c.world = world;
    return AKR_OK;
}

AKR_API int akr_mg_allreduce(void* data, size_t count, int dtype, int op, void* stream) {
    if (count == 0) return AKR_OK;
    if (!data) return mg_fail(AKR_ERR_INVALID, "akr_mg_allreduce: null data pointer");
    ncclDataType_t dt;
    if (dtype == AKR_DTYPE_F32) dt = ncclFloat32;
    else if (dtype == AKR_DTYPE_F64) dt = ncclFloat64;
    else return mg_fail(AKR_ERR_INVALID, "akr_mg_allreduce: dtype must be AKR_DTYPE_F32 or AKR_DTYPE_F64");
    ncclRedOp_t ro;
    if (op == AKR_MG_SUM) ro = ncclSum;
    else if (op == AKR_MG_MAX) ro = ncclMax;
    else return mg_fail(AKR_ERR_INVALID, "akr_mg_allreduce: op must be AKR_MG_SUM or AKR_MG_MAX");
    int rc = need_api();
    if (rc != AKR_OK) return rc;
    int dev = 0;
    if ((rc = current_device(&dev)) != AKR_OK) return rc;
    ncclComm_t comm;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        comm = g_comm[dev].comm;
    }
    if (!comm) return mg_fail(AKR_ERR_INVALID, "akr_mg_allreduce: no communicator on this device (akr_mg_init first)");
    ncclResult_t r = api().all_reduce(data, data, count, dt, ro, comm, (cudaStream_t)stream);
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
    return AKR_OK;
}

AKR_API int akr_mg_allreduce_sum(float* data, size_t n, void* stream) {
    return akr_mg_allreduce(data, n, AKR_DTYPE_F32, AKR_MG_SUM, stream);
}

AKR_API int akr_mg_world(int* rank, int* world) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        dev = 0;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    if (rank) *rank = g_comm[dev].comm ? g_comm[dev].rank : 0;
    if (world) *world = g_comm[dev].comm ? g_comm[dev].world : 1;
    return AKR_OK;
}

AKR_API int akr_mg_nccl_version(int* version) {
    int rc = need_api();
    if (rc != AKR_OK) return rc;
    int v = 0;
    ncclResult_t r = api().get_version(&v);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetVersion");
    if (version) *version = v;
    return AKR_OK;
}

AKR_API int akr_mg_finalize(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return AKR_OK;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    Comm& c = g_comm[dev];
    if (c.comm && api().handle) {
        cudaDeviceSynchronize();  // no collective of this communicator is still in flight
        api().comm_destroy(c.comm);
    }
    c = Comm();
    return AKR_OK;
}

}  // extern "C"
