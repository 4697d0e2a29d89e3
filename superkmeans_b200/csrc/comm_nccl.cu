// See comm_nccl.h.  The declarations below restate the public NCCL C API (nccl.h) for the few calls used.
#include "comm_nccl.h"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

namespace skmb {

namespace {

struct UniqueId {
    char internal[kNcclUniqueIdBytes];
};
using Comm = void*;
enum { kNcclSuccess = 0 };
enum { kNcclUint32 = 3, kNcclFloat32 = 7, kNcclFloat64 = 8 };   // ncclDataType_t
enum { kNcclSum = 0 };                                          // ncclRedOp_t

struct Api {
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(Comm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    const char* (*GetLastError)(Comm) = nullptr;
    void* handle = nullptr;
};

Api g_api;
std::mutex g_api_mu;

template <class F>
void resolve(F& fn, void* handle, const char* name, bool required = true) {
    fn = reinterpret_cast<F>(dlsym(handle, name));
    if (!fn && required) throw std::runtime_error(std::string("NCCL entry point not found: ") + name);
}

const Api& api(const char* library_path) {
    std::lock_guard<std::mutex> lock(g_api_mu);
    if (g_api.handle) return g_api;
    const char* env = std::getenv("SKM_NCCL_LIB");
    const char* candidates[] = {library_path, env, "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    std::string tried;
    for (const char* c : candidates) {
        if (!c || !*c) continue;
        h = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
        tried += std::string(" ") + c;
    }
    if (!h) throw std::runtime_error("cannot open NCCL (tried:" + tried + "); set SKM_NCCL_LIB to the path of libnccl.so.2");
    Api a;
    a.handle = h;
    resolve(a.GetUniqueId, h, "ncclGetUniqueId");
    resolve(a.CommInitRank, h, "ncclCommInitRank");
    resolve(a.CommDestroy, h, "ncclCommDestroy");
    resolve(a.AllReduce, h, "ncclAllReduce");
    resolve(a.GroupStart, h, "ncclGroupStart");
    resolve(a.GroupEnd, h, "ncclGroupEnd");
    resolve(a.GetErrorString, h, "ncclGetErrorString");
    resolve(a.GetLastError, h, "ncclGetLastError", false);
    g_api = a;
    return g_api;
}

void check(const Api& a, int rc, const char* what, Comm comm = nullptr) {
    if (rc == kNcclSuccess) return;
    std::string msg = std::string(what) + ": " + a.GetErrorString(rc);
    if (a.GetLastError) {
        const char* last = a.GetLastError(comm);
        if (last && *last) msg += std::string(" (") + last + ")";
    }
    throw std::runtime_error(msg);
}

} // namespace

void NcclComm::unique_id(uint8_t out[kNcclUniqueIdBytes], const char* library_path) {
    const Api& a = api(library_path);
    UniqueId id;
    check(a, a.GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out, id.internal, kNcclUniqueIdBytes);
}

NcclComm* NcclComm::create(const uint8_t id_bytes[kNcclUniqueIdBytes], int rank, int world, int device, const char* library_path) {
    if (world <= 0 || rank < 0 || rank >= world) throw std::invalid_argument("rank / world out of range");
    const Api& a = api(library_path);
    UniqueId id;
    std::memcpy(id.internal, id_bytes, kNcclUniqueIdBytes);
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("cannot select the CUDA device of the communicator");
    Comm c = nullptr;
    const int rc = a.CommInitRank(&c, world, id, rank);
    cudaSetDevice(prev);
    check(a, rc, "ncclCommInitRank");
    NcclComm* out = new NcclComm();
    out->comm_ = c;
    out->owned_ = true;
    out->rank_ = rank;
    out->world_ = world;
    return out;
}

NcclComm* NcclComm::wrap(void* nccl_comm, int rank, int world) {
    if (!nccl_comm) throw std::invalid_argument("communicator must not be NULL");
    api(nullptr);
    NcclComm* out = new NcclComm();
    out->comm_ = nccl_comm;
    out->owned_ = false;
    out->rank_ = rank;
    out->world_ = world;
    return out;
}

NcclComm::~NcclComm() {
    if (owned_ && comm_ && g_api.CommDestroy) g_api.CommDestroy(comm_);
}

void NcclComm::allreduce_group(float* f32, size_t n_f32, uint32_t* u32, size_t n_u32, double* f64, size_t n_f64, cudaStream_t stream) {
    const Api& a = api(nullptr);
    check(a, a.GroupStart(), "ncclGroupStart", comm_);
    int rc = kNcclSuccess;
    if (n_f32 && rc == kNcclSuccess) rc = a.AllReduce(f32, f32, n_f32, kNcclFloat32, kNcclSum, comm_, stream);
    if (n_u32 && rc == kNcclSuccess) rc = a.AllReduce(u32, u32, n_u32, kNcclUint32, kNcclSum, comm_, stream);
    if (n_f64 && rc == kNcclSuccess) rc = a.AllReduce(f64, f64, n_f64, kNcclFloat64, kNcclSum, comm_, stream);
    const int rc_end = a.GroupEnd();
    check(a, rc, "ncclAllReduce", comm_);
    check(a, rc_end, "ncclGroupEnd", comm_);
}

} // namespace skmb
