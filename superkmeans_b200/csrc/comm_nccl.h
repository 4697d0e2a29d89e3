// Sum across the shards of a multi-GPU training run through NCCL, without a build-time dependency on it: the library
// is opened at run time (libnccl.so.2, as shipped with NCCL itself or bundled with PyTorch) and only the handful of entry
// points used here are resolved.  One NcclComm per process and GPU.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace skmb {

constexpr size_t kNcclUniqueIdBytes = 128;   // sizeof(ncclUniqueId)

class NcclComm {
  public:
    // Opens NCCL (throws std::runtime_error when it cannot be found; `library_path` overrides the search) and writes a
    // new unique id, which one rank creates and every rank of the run must receive before create().
    static void unique_id(uint8_t out[kNcclUniqueIdBytes], const char* library_path = nullptr);
    // Collective over all `world` ranks: ncclCommInitRank on `device`.
    static NcclComm* create(const uint8_t id[kNcclUniqueIdBytes], int rank, int world, int device, const char* library_path = nullptr);
    // Wraps a communicator the caller already owns (an ncclComm_t); destroy() then leaves it alone.
    static NcclComm* wrap(void* nccl_comm, int rank, int world);
    ~NcclComm();

    int rank() const { return rank_; }
    int world() const { return world_; }
    // In-place sums, enqueued on `stream` as one NCCL group (one launch): float sums, uint32 counts, double scalars.
    // Any of the three may be empty.  Throws std::runtime_error with NCCL's message on failure.
    void allreduce_group(float* f32, size_t n_f32, uint32_t* u32, size_t n_u32, double* f64, size_t n_f64, cudaStream_t stream);

  private:
    NcclComm() = default;
    void* comm_ = nullptr;
    bool owned_ = false;
    int rank_ = 0, world_ = 1;
};

} // namespace skmb
