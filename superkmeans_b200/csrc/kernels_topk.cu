// k nearest rows of Y for every row of Q, and the recall figure built on it.
//
// Used only by training with query vectors (SuperKMeans::GetGTAssignmentsAndDistances / ComputeRecall,
// superkmeans.h:1010-1087, on top of BatchComputer::FindKNearestNeighbors, batch_computers.h:191-274): once
// per Train for the ground truth (the objective_k nearest training points of every query) and once per
// iteration for the centroids a search would visit (the nearest ann_explore_fraction of the centroids).
//
// Y is walked in slabs of kSlab rows.  For a slab the dot products Q * Y_slab^T go to scratch with the
// fp32 tile GEMM; topk_merge_kernel (one CTA per query) turns them into distances
// ||q||^2 + ||y||^2 - 2 q.y, keeps those below the query's current k-th best in a shared-memory buffer
// and, whenever the buffer fills, sorts it (bitonic, 64-bit keys {ordered distance, index}) and keeps the
// best k.  Equal distances are ordered by index, as std::partial_sort on (distance, index) pairs does.
#include <cfloat>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "device_utils.cuh"

namespace skmb {

namespace {

constexpr int kTopkThreads = 256;
constexpr int kTopkBuf = 2048;   // keys held in shared memory; k <= kTopkMaxK leaves room for new candidates
constexpr size_t kSlab = 16384;

__device__ __forceinline__ unsigned long long make_key(float dist, uint32_t idx) {
    return (static_cast<unsigned long long>(float_to_ordered(dist)) << 32) | static_cast<unsigned long long>(idx);
}

// Ascending bitonic sort of buf[0 .. kTopkBuf) by all threads of the CTA.
__device__ void bitonic_sort(unsigned long long* buf) {
    for (int size = 2; size <= kTopkBuf; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = threadIdx.x; t < kTopkBuf / 2; t += kTopkThreads) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool up = ((lo & size) == 0);
                const unsigned long long a = buf[lo], b = buf[hi];
                if ((a > b) == up) {
                    buf[lo] = b;
                    buf[hi] = a;
                }
            }
        }
    }
    __syncthreads();
}

// dots: n_q x slab_ld dot products of this slab (columns [0, slab_n) valid, global indices col0 + c).
// state: n_q x k keys carried from slab to slab, ascending, ~0 = empty.
__global__ void __launch_bounds__(kTopkThreads) topk_merge_kernel(const float* __restrict__ dots, size_t slab_ld, size_t slab_n, size_t col0, const float* __restrict__ norms_q,
                                                                  const float* __restrict__ norms_y, uint32_t k, unsigned long long* __restrict__ state) {
    __shared__ unsigned long long buf[kTopkBuf];
    __shared__ uint32_t count;
    __shared__ unsigned long long tau;
    const size_t q = blockIdx.x;
    const float nq = norms_q[q];
    unsigned long long* st = state + q * k;
    for (int i = threadIdx.x; i < kTopkBuf; i += kTopkThreads) buf[i] = (i < static_cast<int>(k)) ? st[i] : ~0ull;
    if (threadIdx.x == 0) {
        count = k;
        tau = st[k - 1];
    }
    __syncthreads();
    const float* __restrict__ row = dots + q * slab_ld;
    for (size_t c0 = 0; c0 < slab_n; c0 += kTopkThreads) {
        const size_t c = c0 + threadIdx.x;
        if (c < slab_n) {
            const float dist = fmaf(-2.0f, row[c], nq) + norms_y[col0 + c];
            const unsigned long long key = make_key(dist, static_cast<uint32_t>(col0 + c));
            if (key < tau) {
                const uint32_t pos = atomicAdd(&count, 1u);
                buf[pos] = key;   // pos < k + kTopkThreads * rounds, bounded by the flush below
            }
        }
        __syncthreads();
        // one more round adds at most kTopkThreads keys: flush while that still fits
        if (count + kTopkThreads > kTopkBuf) {
            bitonic_sort(buf);
            for (int i = k + threadIdx.x; i < kTopkBuf; i += kTopkThreads) buf[i] = ~0ull;
            if (threadIdx.x == 0) {
                count = k;
                tau = buf[k - 1];
            }
            __syncthreads();
        }
    }
    bitonic_sort(buf);
    for (int i = threadIdx.x; i < static_cast<int>(k); i += kTopkThreads) st[i] = buf[i];
}

__global__ void topk_init_kernel(unsigned long long* state, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) state[i] = ~0ull;
}

// keys -> indices and distances (clamped at zero as FindKNearestNeighbors stores them; empty slots: index
// 0xFFFFFFFF, distance FLT_MAX)
__global__ void topk_finish_kernel(const unsigned long long* __restrict__ state, size_t n, uint32_t* __restrict__ idx, float* __restrict__ dist) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long key = state[i];
    if (key == ~0ull) {
        idx[i] = 0xFFFFFFFFu;
        if (dist) dist[i] = FLT_MAX;
    } else {
        idx[i] = static_cast<uint32_t>(key & 0xFFFFFFFFull);
        if (dist) dist[i] = fmaxf(0.0f, ordered_to_float(static_cast<uint32_t>(key >> 32)));
    }
}

// found[q] = number of the query's ground-truth points whose current cluster is among the clusters the query
// would visit (superkmeans.h:1063-1086).
__global__ void __launch_bounds__(128) recall_count_kernel(const uint32_t* __restrict__ gt, uint32_t objective_k, const uint32_t* __restrict__ promising, uint32_t n_explore,
                                                           const uint32_t* __restrict__ assignments, size_t n_assignments, uint32_t* __restrict__ found) {
    __shared__ uint32_t total;
    const size_t q = blockIdx.x;
    if (threadIdx.x == 0) total = 0;
    __syncthreads();
    uint32_t mine = 0;
    for (uint32_t j = threadIdx.x; j < objective_k; j += blockDim.x) {
        const uint32_t g = gt[q * objective_k + j];
        if (g >= n_assignments) continue;
        const uint32_t a = assignments[g];
        bool hit = false;
        for (uint32_t t = 0; t < n_explore && !hit; ++t) hit = promising[q * n_explore + t] == a;
        mine += hit ? 1u : 0u;
    }
    if (mine) atomicAdd(&total, mine);
    __syncthreads();
    if (threadIdx.x == 0) found[q] = total;
}

} // namespace

size_t topk_scratch_floats(size_t n_q) { return n_q * kSlab; }
size_t topk_max_k() { return kTopkBuf - 2 * kTopkThreads; }

void launch_topk_nn(const float* q, const float* y, size_t n_q, size_t n_y, size_t d, const float* norms_q, const float* norms_y, uint32_t k, uint32_t* out_idx,
                    float* out_dist, float* dots_scratch, unsigned long long* state, cudaStream_t stream) {
    if (n_q == 0 || k == 0) return;
    if (k > topk_max_k()) throw std::runtime_error("nearest-neighbour lists longer than " + std::to_string(topk_max_k()) + " entries are not supported");
    const size_t n_state = n_q * k;
    topk_init_kernel<<<static_cast<unsigned>((n_state + 255) / 256), 256, 0, stream>>>(state, n_state);
    SKM_LAUNCH_CHECK();
    for (size_t c0 = 0; c0 < n_y; c0 += kSlab) {
        const size_t cn = std::min(kSlab, n_y - c0);
        launch_gemm_nt(q, d, y + c0 * d, d, dots_scratch, kSlab, n_q, cn, d, stream);
        topk_merge_kernel<<<static_cast<unsigned>(n_q), kTopkThreads, 0, stream>>>(dots_scratch, kSlab, cn, c0, norms_q, norms_y, k, state);
        SKM_LAUNCH_CHECK();
    }
    topk_finish_kernel<<<static_cast<unsigned>((n_state + 255) / 256), 256, 0, stream>>>(state, n_state, out_idx, out_dist);
    SKM_LAUNCH_CHECK();
}

void launch_recall_count(const uint32_t* gt, uint32_t objective_k, const uint32_t* promising, uint32_t n_explore, const uint32_t* assignments, size_t n_assignments,
                         size_t n_q, uint32_t* found, cudaStream_t stream) {
    if (n_q == 0) return;
    recall_count_kernel<<<static_cast<unsigned>(n_q), 128, 0, stream>>>(gt, objective_k, promising, n_explore, assignments, n_assignments, found);
    SKM_LAUNCH_CHECK();
}

} // namespace skmb
