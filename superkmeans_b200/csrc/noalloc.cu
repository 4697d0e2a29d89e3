// Exact nearest-centroid assignment for callers that must not allocate device memory.
//
// Who that is: code that runs inside a host program which took all of the GPU's memory for its own pool when
// it started (a database or a serving process does that so that nothing else can fail it later), where a
// cudaMalloc either fails or has to be negotiated with that pool; and code on a latency-critical path,
// because cudaMalloc and cudaFree synchronise the whole device and stall every other stream of the process.
// The regular operator allocates its inputs' norms, the candidate pairs handed from the tensor-core pass to
// the fp32 refinement and a status word on every call; here those live in one file-scope device array of
// fixed size that every GPU which loads the library holds until the process exits.
//
// Consequences of sharing one array:
//   * sizes are bounded (kMaxRows, kMaxCentroids); larger requests are refused, not truncated;
//   * the array keeps what the last call left in it: the status word is cleared at the start of every call,
//     everything else is written before it is read;
//   * two calls whose kernels overlap on the same GPU (different streams, different host threads) write the
//     same scratch and race.  Callers serialise them.
//
// The device address of the array is looked up once per device, on the first call for that device, with
// that device current.  That first call should be made before any stream capture begins.
#include <mutex>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels_tc.cuh"
#include "noalloc.h"

namespace skmb {
namespace noalloc {

constexpr size_t kMaxRows = 262144;     // SKM_NOALLOC_MAX_ROWS
constexpr size_t kMaxCentroids = 65536; // SKM_NOALLOC_MAX_CENTROIDS
constexpr int kMaxDevices = 64;

struct Scratch {
    uint2 pairs[kMaxRows];          // two best candidates per row (tensor-core pass -> fp32 refinement)
    float row_norms[kMaxRows];      // squared norms of the rows
    float centroid_norms[kMaxCentroids];
    int status;                     // set by a kernel whose bounded wait ran out; must be 0 on entry
};

// In host code this name is only a handle for the runtime's symbol calls, never an address to hand to a kernel.
static __device__ __align__(256) unsigned char g_scratch[sizeof(Scratch)];

namespace {

std::mutex g_mutex;
Scratch* g_device_ptr[kMaxDevices] = {nullptr};

// Device address of g_scratch on `device`, which must be the current device.
Scratch* scratch_of_current_device(int device) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_device_ptr[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess) throw CudaError(std::string("cudaGetSymbolAddress(scratch) failed: ") + cudaGetErrorString(e));
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255) != 0) throw CudaError("the static scratch array has no usable device address");
        g_device_ptr[device] = static_cast<Scratch*>(p);
    }
    return g_device_ptr[device];
}

struct DeviceScope {
    int previous = -1;
    explicit DeviceScope(int device) {
        SKM_CUDA(cudaGetDevice(&previous));
        if (previous != device) SKM_CUDA(cudaSetDevice(device));
        else previous = -1;
    }
    ~DeviceScope() {
        if (previous >= 0) cudaSetDevice(previous);
    }
};

} // namespace

// x_dev [n][d], y_dev [k][d], out_knn_dev [n], out_dist_dev [n]: device memory of `device`.  Returns after the
// results are in the output arrays (the stream is synchronised to read the status word).
void find_nearest(int device, const float* x_dev, const float* y_dev, size_t n, size_t k, size_t d, uint32_t* out_knn_dev, float* out_dist_dev, cudaStream_t stream) {
    if (n > kMaxRows) throw std::invalid_argument("the allocation-free operator takes at most " + std::to_string(kMaxRows) + " rows per call, got " + std::to_string(n));
    if (k > kMaxCentroids) throw std::invalid_argument("the allocation-free operator takes at most " + std::to_string(kMaxCentroids) + " centroids, got " + std::to_string(k));
    if (k == 0 || d == 0) throw std::invalid_argument("n_centroids and dimensionality must be positive");
    if (n == 0) return;
    if (!x_dev || !y_dev || !out_knn_dev || !out_dist_dev) throw std::invalid_argument("inputs and outputs must not be NULL");
    int n_devices = 0;
    SKM_CUDA(cudaGetDeviceCount(&n_devices));
    if (device < 0) SKM_CUDA(cudaGetDevice(&device));
    if (device >= n_devices || device >= kMaxDevices) throw std::invalid_argument("no such CUDA device: " + std::to_string(device));

    DeviceScope scope(device);
    Scratch* s = scratch_of_current_device(device);
    SKM_CUDA(cudaMemsetAsync(&s->status, 0, sizeof(int), stream));
    launch_row_sqnorms(x_dev, n, d, d, s->row_norms, stream);
    launch_row_sqnorms(y_dev, k, d, d, s->centroid_norms, stream);
    if (tc::eligible(x_dev, d, y_dev, d)) {
        tc::launch_assign_full_flagged(x_dev, y_dev, n, k, d, s->row_norms, s->centroid_norms, out_knn_dev, out_dist_dev, s->pairs, &s->status, stream);
    } else {
        // Rows that TMA cannot address (pitch or base not a multiple of 16 bytes): fp32 SIMT kernel, which needs the norms only.
        launch_assign_full(x_dev, y_dev, n, k, d, s->row_norms, s->centroid_norms, out_knn_dev, out_dist_dev, nullptr, stream);
    }
    int status = 0;
    SKM_CUDA(cudaMemcpyAsync(&status, &s->status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    SKM_CUDA(cudaStreamSynchronize(stream));
    if (status != 0) throw CudaError("a tensor-core kernel gave up waiting on a barrier (code " + std::to_string(status) + ")");
}

} // namespace noalloc
} // namespace skmb
