// CUDA kernels of the k-means hot path (sm_100a) and their launchers.
//
//   rotation / un-rotation      gemm_nt_kernel              (reference: adsampling.h:191-215, :273-298)
//   row norms                   row_sqnorms_kernel          (superkmeans.h:1147-1171)
//   exact assignment            assign_full_kernel          (batch_computers.h:104-171)
//   pruned assignment           assign_pruned_kernel        (batch_computers.h:297-409, pdxearch.h:118-327)
//   centroid update             radix sort + segmented sum  (superkmeans.h:729-765, :973-981)
//   consolidation               scale / split ops / pdxify / shift (superkmeans.h:936-998, layout.h:155-232)
#include "common.cuh"
#include "device_utils.cuh"
#include "gemm_simt.cuh"
#include "kernels_tc.cuh"

#include <atomic>
#include <cfloat>
#include <cstdlib>
#include <chrono>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace skmb {

// Number of kernels this library has launched in the process (reported by skm_kernel_launches).
static std::atomic<unsigned long long> g_kernel_launches{0};
unsigned long long kernel_launch_count() { return g_kernel_launches.load(); }
void note_kernel_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }
static std::atomic<unsigned long long> g_device_allocs{0};
unsigned long long device_alloc_count() { return g_device_allocs.load(std::memory_order_relaxed); }
void note_device_alloc() { g_device_allocs.fetch_add(1, std::memory_order_relaxed); }

// ---- device memory with an optional cache of large blocks (see common.cuh)
namespace {
struct CachedBlock {
    void* p;
    size_t bytes;
    int device;
};
std::mutex g_cache_mu;
std::vector<CachedBlock> g_cache;
std::unordered_map<void*, size_t> g_block_bytes;   // true size of every live block that was allocated through the cache path
bool g_cache_on = false;
constexpr size_t kCacheMinBytes = size_t{64} << 10;

// Sizes are rounded up to one of eight steps per power of two, so that requests that differ a little from call to call
// (buffers sized by a count that the data decide) land on the same block sizes and find each other in the cache.
size_t cache_bucket(size_t bytes) {
    size_t p2 = size_t{1} << 16;
    while (p2 * 2 <= bytes) p2 *= 2;
    const size_t step = p2 / 8;
    return (bytes + step - 1) / step * step;
}
thread_local double g_alloc_ms = 0.0;

struct AllocClock {
    std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
    ~AllocClock() { g_alloc_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count(); }
};

void drop_cache_locked() {
    int cur = 0;
    cudaGetDevice(&cur);
    for (auto& b : g_cache) {
        cudaSetDevice(b.device);
        cudaFree(b.p);
    }
    g_cache.clear();
    cudaSetDevice(cur);
}
} // namespace

void* device_alloc(size_t bytes) {
    AllocClock clock;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const bool cached_path = g_cache_on && bytes >= kCacheMinBytes;
    if (cached_path) {
        bytes = cache_bucket(bytes);
        std::lock_guard<std::mutex> lock(g_cache_mu);
        size_t best = g_cache.size();
        for (size_t i = 0; i < g_cache.size(); ++i) {
            const CachedBlock& b = g_cache[i];
            if (b.device == device && b.bytes >= bytes && b.bytes <= bytes + bytes / 4 && (best == g_cache.size() || b.bytes < g_cache[best].bytes)) best = i;
        }
        if (best != g_cache.size()) {
            void* p = g_cache[best].p;
            g_block_bytes[p] = g_cache[best].bytes;
            g_cache.erase(g_cache.begin() + static_cast<long>(best));
            return p;
        }
    }
    note_device_alloc();
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaErrorMemoryAllocation) {
        // what the cache holds may be exactly what is missing
        cudaGetLastError();
        {
            std::lock_guard<std::mutex> lock(g_cache_mu);
            drop_cache_locked();
        }
        e = cudaMalloc(&p, bytes);
    }
    cuda_check(e, "cudaMalloc", __FILE__, __LINE__);
    if (cached_path) {
        std::lock_guard<std::mutex> lock(g_cache_mu);
        g_block_bytes[p] = bytes;
    }
    return p;
}

void device_free(void* p, size_t bytes) {
    if (!p) return;
    AllocClock clock;
    {
        std::lock_guard<std::mutex> lock(g_cache_mu);
        const auto it = g_block_bytes.find(p);
        if (it != g_block_bytes.end()) {
            bytes = it->second;   // the block's true (rounded-up) size
            g_block_bytes.erase(it);
        }
    }
    if (g_cache_on && bytes >= kCacheMinBytes) {
        int device = 0;
        if (cudaGetDevice(&device) == cudaSuccess) {
            std::lock_guard<std::mutex> lock(g_cache_mu);
            g_cache.push_back(CachedBlock{p, bytes, device});
            return;
        }
    }
    cudaFree(p);
}

void set_workspace_cache(bool on) {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    g_cache_on = on;
    if (!on) drop_cache_locked();
}
bool workspace_cache_enabled() { return g_cache_on; }
void release_cached_memory() {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    drop_cache_locked();
}
size_t cached_memory_bytes() {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    size_t total = 0;
    for (const auto& b : g_cache) total += b.bytes;
    return total;
}
double alloc_free_ms() { return g_alloc_ms; }

// =================================================================================================
// Row squared norms over the first `upto` columns: one warp per row.
// =================================================================================================
__global__ void __launch_bounds__(256) row_sqnorms_kernel(const float* __restrict__ x, size_t n, size_t ld, size_t upto, float* __restrict__ out) {
    const size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= n) return;
    const int lane = threadIdx.x & 31;
    const float* p = x + row * ld;
    float acc = 0.f;
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const size_t upto4 = vec ? (upto & ~size_t{3}) : 0;
    for (size_t j = static_cast<size_t>(lane) * 4; j < upto4; j += 128) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p + j));
        acc = fmaf(v.x, v.x, acc);
        acc = fmaf(v.y, v.y, acc);
        acc = fmaf(v.z, v.z, acc);
        acc = fmaf(v.w, v.w, acc);
    }
    for (size_t j = upto4 + lane; j < upto; j += 32) {
        const float v = __ldg(p + j);
        acc = fmaf(v, v, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc;
}

void launch_row_sqnorms(const float* x, size_t n, size_t ld, size_t upto, float* out, cudaStream_t stream) {
    if (n == 0) return;
    const unsigned grid = static_cast<unsigned>((n + 7) / 8);
    row_sqnorms_kernel<<<grid, 256, 0, stream>>>(x, n, ld, upto, out);
    SKM_LAUNCH_CHECK();
}

// =================================================================================================
// NT GEMM with a plain store epilogue (rotation, un-rotation).
// =================================================================================================
__global__ void __launch_bounds__(256, 2) gemm_nt_kernel(
    const float* __restrict__ a, size_t lda, const float* __restrict__ b, size_t ldb, float* __restrict__ out, size_t ldo, size_t n, size_t n_out, size_t k_dim
) {
    __shared__ GemmSmem smem;
    const size_t row0 = static_cast<size_t>(blockIdx.x) * kTileM;
    const size_t col0 = static_cast<size_t>(blockIdx.y) * kTileN;
    const int m_valid = static_cast<int>(min(static_cast<size_t>(kTileM), n - row0));
    const int n_valid = static_cast<int>(min(static_cast<size_t>(kTileN), n_out - col0));
    float acc[8][8];
    gemm_tile_nt(a + row0 * lda, lda, m_valid, b + col0 * ldb, ldb, n_valid, static_cast<int>(k_dim), smem, acc);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const bool vec = (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = tile_row_of(ty, i);
        if (r >= m_valid) continue;
        float* orow = out + (row0 + r) * ldo + col0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = tile_col_of(tx, h * 4);
            if (vec && c + 3 < n_valid) {
                *reinterpret_cast<float4*>(orow + c) = make_float4(acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c + j < n_valid) orow[c + j] = acc[i][h * 4 + j];
            }
        }
    }
}

void launch_gemm_nt(const float* a, size_t lda, const float* b, size_t ldb, float* out, size_t ldo, size_t n, size_t n_out, size_t k_dim, cudaStream_t stream) {
    if (n == 0 || n_out == 0) return;
    // Tensor cores when TMA can address both operands: the rotation kernel cuts the accumulation into four chains summed
    // in fp32 registers, which keeps the result at the accuracy of this file's fp32 kernel (a single chain in tensor
    // memory would be ~1e-5 off, and rotated rows feed every later distance).
    if (tc::eligible(a, lda, b, ldb) && k_dim >= 32) {
        tc::launch_rotate(a, lda, b, ldb, out, ldo, n, n_out, k_dim, nullptr, stream);
        return;
    }
    // The point dimension is on grid.x (limit 2^31-1); output columns on grid.y.
    dim3 grid(static_cast<unsigned>((n + kTileM - 1) / kTileM), static_cast<unsigned>((n_out + kTileN - 1) / kTileN));
    gemm_nt_kernel<<<grid, 256, 0, stream>>>(a, lda, b, ldb, out, ldo, n, n_out, k_dim);
    SKM_LAUNCH_CHECK();
}

__global__ void transpose_square_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n) {
    __shared__ float t[32][33];
    const size_t bx = static_cast<size_t>(blockIdx.x) * 32, by = static_cast<size_t>(blockIdx.y) * 32;
    for (int r = threadIdx.y; r < 32; r += 8) {
        const size_t i = by + r, j = bx + threadIdx.x;
        if (i < n && j < n) t[r][threadIdx.x] = in[i * n + j];
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += 8) {
        const size_t i = bx + r, j = by + threadIdx.x;
        if (i < n && j < n) out[i * n + j] = t[threadIdx.x][r];
    }
}

void launch_transpose_square(const float* in, float* out, size_t n, cudaStream_t stream) {
    dim3 grid(static_cast<unsigned>((n + 31) / 32), static_cast<unsigned>((n + 31) / 32));
    transpose_square_kernel<<<grid, dim3(32, 8), 0, stream>>>(in, out, n);
    SKM_LAUNCH_CHECK();
}

// =================================================================================================
// Exact assignment.  One CTA owns 128 points and walks all centroid tiles; distances never leave
// registers.  Tie rules of the reference: first minimum inside a batch of 1024 centroids, a later
// batch wins only with a strictly smaller distance than the stored (clamped at 0) one.
// =================================================================================================
__global__ void __launch_bounds__(256, 2) assign_full_kernel(
    const float* __restrict__ x, const float* __restrict__ y, size_t n, size_t k, size_t d, const float* __restrict__ norms_x, const float* __restrict__ norms_y,
    uint32_t* __restrict__ out_knn, float* __restrict__ out_dist
) {
    __shared__ GemmSmem smem;
    const size_t row0 = static_cast<size_t>(blockIdx.x) * kTileM;
    const int m_valid = static_cast<int>(min(static_cast<size_t>(kTileM), n - row0));
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    __shared__ float s_nx[kTileM], s_best[kTileM];
    __shared__ uint32_t s_bidx[kTileM];
    if (threadIdx.x < kTileM) {
        s_nx[threadIdx.x] = (static_cast<int>(threadIdx.x) < m_valid) ? norms_x[row0 + threadIdx.x] : 0.f;
        s_best[threadIdx.x] = FLT_MAX;
        s_bidx[threadIdx.x] = 0;
    }
    float bmin[8];
    uint32_t bminidx[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        bmin[i] = FLT_MAX;
        bminidx[i] = 0;
    }
    __syncthreads();
    float acc[8][8];
    for (size_t col0 = 0; col0 < k; col0 += kTileN) {
        const int n_valid = static_cast<int>(min(static_cast<size_t>(kTileN), k - col0));
        gemm_tile_nt(x + row0 * d, d, m_valid, y + col0 * d, d, n_valid, static_cast<int>(d), smem, acc);
        float nyr[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = tile_col_of(tx, j);
            nyr[j] = (c < n_valid) ? __ldg(norms_y + col0 + c) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float nxv = s_nx[tile_row_of(ty, i)];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = tile_col_of(tx, j);
                if (c < n_valid) {
                    const float dist = fmaf(-2.0f, acc[i][j], nxv) + nyr[j];
                    if (dist < bmin[i]) {
                        bmin[i] = dist;
                        bminidx[i] = static_cast<uint32_t>(col0 + c);
                    }
                }
            }
        }
        const bool batch_end = ((col0 + kTileN) % kChunk == 0) || (col0 + kTileN >= k);
        if (batch_end) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float v = bmin[i];
                uint32_t vi = bminidx[i];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                    const uint32_t oi = __shfl_xor_sync(0xffffffffu, vi, o);
                    if (ov < v || (ov == v && oi < vi)) {
                        v = ov;
                        vi = oi;
                    }
                }
                if (tx == 0) {
                    const int r = tile_row_of(ty, i);
                    if (v < s_best[r]) {
                        s_best[r] = fmaxf(0.0f, v);
                        s_bidx[r] = vi;
                    }
                }
                bmin[i] = FLT_MAX;
                bminidx[i] = 0;
            }
        }
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < m_valid) {
        out_knn[row0 + threadIdx.x] = s_bidx[threadIdx.x];
        out_dist[row0 + threadIdx.x] = s_best[threadIdx.x];
    }
}

void launch_assign_full(const float* x, const float* y, size_t n, size_t k, size_t d, const float* norms_x, const float* norms_y, uint32_t* out_knn, float* out_dist, uint2* top2_scratch, cudaStream_t stream, float* y_split) {
    if (n == 0) return;
    if (top2_scratch && tc::eligible(x, d, y, d)) {
        tc::launch_assign_full(x, y, n, k, d, norms_x, norms_y, out_knn, out_dist, top2_scratch, stream, y_split);
        return;
    }
    const unsigned grid = static_cast<unsigned>((n + kTileM - 1) / kTileM);
    assign_full_kernel<<<grid, 256, 0, stream>>>(x, y, n, k, d, norms_x, norms_y, out_knn, out_dist);
    SKM_LAUNCH_CHECK();
}

// =================================================================================================
// Pruned assignment.
//
// A persistent CTA takes tiles of 128 points.  For every chunk of 1024 centroids it
//   1. computes the partial dot products over the first d' dimensions, 128 centroids at a time,
//      and turns them into partial distances ||x||'^2 + ||c||'^2 - 2 x.c;
//   2. keeps only (point, centroid) pairs whose partial distance is below best * ratio[d'] (the
//      ADSampling test); survivors go to a per-CTA candidate list in global scratch;
//   3. walks the survivors, eight lanes per pair: adds the horizontal dimensions 64 at a time from
//      the PDX-blocked centroid copy, re-testing against best * ratio[dims seen] after each block,
//      then the remaining vertical dimensions [d', vertical_d) from the auxiliary row-major copy,
//      and finally competes for the per-point minimum of the chunk;
//   4. lowers `best` of each point before the next chunk.
// `best` is constant inside a chunk, so pairs are independent of each other.  The pair formed with
// the point's previous centroid is held back until the survivor count of the chunk is known: when
// it is the only survivor the chunk is skipped for that point, as the reference does.
// =================================================================================================
constexpr int kListCap = kTileM * kChunk;

struct PrunedRowState {
    float thr[kTileM];
    float best[kTileM];
    uint32_t bestidx[kTileM];
    uint32_t prev[kTileM];
    float nxs[kTileM];
    uint32_t cnt[kTileM];
    uint32_t npc[kTileM];
    float prev_pd[kTileM];
    uint32_t prev_flag[kTileM];
    unsigned long long chunk_key[kTileM];
    uint32_t active[kTileM];
    uint32_t list_count;
};

template <bool VEC>
__device__ __forceinline__ void pruned_process_pair(
    const PrunedParams& p, PrunedRowState& st, size_t row0, int r, uint32_t cl, float pd, size_t chunk, size_t c0, size_t cs, int gl, uint32_t gmask
) {
    const size_t c = c0 + cl;
    const float b = st.best[r];
    const float* __restrict__ q = p.x + (row0 + r) * p.d;
    uint32_t dims = p.partial_d;
    bool alive = true;
    const size_t n_hblocks = p.horizontal_d / kHBlock;
    const float* __restrict__ blk = p.y_pdx + chunk * kChunk * p.d + static_cast<size_t>(p.vertical_d) * cs + static_cast<size_t>(cl) * kHBlock;
    for (size_t hb = 0; hb < n_hblocks; ++hb) {
        const float* __restrict__ cp = blk + hb * cs * kHBlock + gl * 8;
        const float* __restrict__ qp = q + p.vertical_d + hb * kHBlock + gl * 8;
        float s = 0.f;
        if (VEC) {
            const float4 c0v = __ldg(reinterpret_cast<const float4*>(cp));
            const float4 c1v = __ldg(reinterpret_cast<const float4*>(cp + 4));
            const float4 q0v = __ldg(reinterpret_cast<const float4*>(qp));
            const float4 q1v = __ldg(reinterpret_cast<const float4*>(qp + 4));
            float t;
            t = q0v.x - c0v.x; s = fmaf(t, t, s);
            t = q0v.y - c0v.y; s = fmaf(t, t, s);
            t = q0v.z - c0v.z; s = fmaf(t, t, s);
            t = q0v.w - c0v.w; s = fmaf(t, t, s);
            t = q1v.x - c1v.x; s = fmaf(t, t, s);
            t = q1v.y - c1v.y; s = fmaf(t, t, s);
            t = q1v.z - c1v.z; s = fmaf(t, t, s);
            t = q1v.w - c1v.w; s = fmaf(t, t, s);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float t = __ldg(qp + e) - __ldg(cp + e);
                s = fmaf(t, t, s);
            }
        }
        s += __shfl_xor_sync(gmask, s, 4);
        s += __shfl_xor_sync(gmask, s, 2);
        s += __shfl_xor_sync(gmask, s, 1);
        pd += s;
        dims += kHBlock;
        if (!(pd < b * __ldg(p.ratios + dims))) {
            alive = false;
            break;
        }
    }
    if (alive && p.partial_d < p.vertical_d) {
        const float* __restrict__ cp = p.y_aux + c * p.vertical_d + p.partial_d;
        const float* __restrict__ qp = q + p.partial_d;
        const uint32_t len = p.vertical_d - p.partial_d;
        float s = 0.f;
        for (uint32_t e = gl; e < len; e += 8) {
            const float t = __ldg(qp + e) - __ldg(cp + e);
            s = fmaf(t, t, s);
        }
        s += __shfl_xor_sync(gmask, s, 4);
        s += __shfl_xor_sync(gmask, s, 2);
        s += __shfl_xor_sync(gmask, s, 1);
        pd += s;
        if (!(pd < b)) alive = false;  // ratio[d] == 1
    }
    if (alive && gl == 0) {
        const unsigned long long key = (static_cast<unsigned long long>(float_to_ordered(pd)) << 32) | static_cast<unsigned long long>(c);
        atomicMin(&st.chunk_key[r], key);
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256, 2) assign_pruned_kernel(const PrunedParams p) {
    __shared__ GemmSmem smem;
    __shared__ PrunedRowState st;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = tid >> 3, gl = tid & 7;
    const uint32_t gmask = 0xFFu << ((lane >> 3) * 8);
    uint2* __restrict__ list = p.scratch + static_cast<size_t>(blockIdx.x) * kListCap;
    const size_t n_tiles = (p.n + kTileM - 1) / kTileM;
    const size_t n_chunks = (p.k + kChunk - 1) / kChunk;
    const float ratio_first = __ldg(p.ratios + p.partial_d);

    for (size_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const size_t row0 = tile * kTileM;
        const int m_valid = static_cast<int>(min(static_cast<size_t>(kTileM), p.n - row0));

        // Exact distance to the previous centroid gives the first threshold (batch_computers.h:372-377).
        // When the caller has computed it already (p.best_in) it is taken from there; rows flagged in
        // p.skip belong to the dense kernel and are left untouched here.
        if (p.best_in) {
            if (tid < kTileM) {
                const bool active = tid < m_valid && !(p.skip && p.skip[row0 + tid]);
                st.best[tid] = active ? p.best_in[row0 + tid] : -1.0f;   // negative: no partial distance passes
                st.bestidx[tid] = active ? p.knn[row0 + tid] : 0u;
                st.prev[tid] = active ? p.knn[row0 + tid] : 0xFFFFFFFFu;
                st.nxs[tid] = (tid < m_valid) ? p.norms_x[row0 + tid] : 0.f;
                st.npc[tid] = 0;
                st.active[tid] = active ? 1u : 0u;
            }
        } else
        for (int r = warp; r < kTileM; r += 8) {
            if (lane == 0) st.active[r] = (r < m_valid) ? 1u : 0u;
            if (r < m_valid) {
                const uint32_t pa = p.knn[row0 + r];
                const float* __restrict__ xr = p.x + (row0 + r) * p.d;
                const float* __restrict__ yr = p.y + static_cast<size_t>(pa) * p.d;
                float s = 0.f;
                if (VEC) {
                    for (size_t j = static_cast<size_t>(lane) * 4; j < p.d; j += 128) {
                        const float4 a = __ldg(reinterpret_cast<const float4*>(xr + j));
                        const float4 b = __ldg(reinterpret_cast<const float4*>(yr + j));
                        float t;
                        t = a.x - b.x; s = fmaf(t, t, s);
                        t = a.y - b.y; s = fmaf(t, t, s);
                        t = a.z - b.z; s = fmaf(t, t, s);
                        t = a.w - b.w; s = fmaf(t, t, s);
                    }
                } else {
                    for (size_t j = lane; j < p.d; j += 32) {
                        const float t = __ldg(xr + j) - __ldg(yr + j);
                        s = fmaf(t, t, s);
                    }
                }
                s = warp_sum(s);
                if (lane == 0) {
                    st.best[r] = s;
                    st.bestidx[r] = pa;
                    st.prev[r] = pa;
                    st.nxs[r] = p.norms_x[row0 + r];
                    st.npc[r] = 0;
                }
            } else if (lane == 0) {
                st.best[r] = 0.f;
                st.bestidx[r] = 0;
                st.prev[r] = 0xFFFFFFFFu;
                st.nxs[r] = 0.f;
                st.npc[r] = 0;
            }
        }
        __syncthreads();

        for (size_t chunk = 0; chunk < n_chunks; ++chunk) {
            const size_t c0 = chunk * kChunk;
            const size_t cs = min(static_cast<size_t>(kChunk), p.k - c0);
            if (tid < kTileM) {
                st.thr[tid] = st.best[tid] * ratio_first;
                st.cnt[tid] = 0;
                st.prev_flag[tid] = 0;
                st.chunk_key[tid] = ~0ull;
            }
            if (tid == 0) st.list_count = 0;
            __syncthreads();

            float acc[8][8];
            for (size_t sub0 = 0; sub0 < cs; sub0 += kTileN) {
                const int n_valid = static_cast<int>(min(static_cast<size_t>(kTileN), cs - sub0));
                gemm_tile_nt(p.x + row0 * p.d, p.d, m_valid, p.y + (c0 + sub0) * p.d, p.d, n_valid, static_cast<int>(p.partial_d), smem, acc);
                float nyr[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = tile_col_of(tx, j);
                    nyr[j] = (c < n_valid) ? __ldg(p.norms_y + c0 + sub0 + c) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = tile_row_of(ty, i);
                    if (r >= m_valid) continue;
                    const float t = st.thr[r];
                    const float nxv = st.nxs[r];
                    const uint32_t pv = st.prev[r];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int c = tile_col_of(tx, j);
                        if (c < n_valid) {
                            const float pd = fmaf(-2.0f, acc[i][j], nxv) + nyr[j];
                            if (pd < t) {
                                atomicAdd(&st.cnt[r], 1u);
                                const uint32_t cl = static_cast<uint32_t>(sub0) + c;
                                if (static_cast<size_t>(pv) == c0 + cl) {
                                    st.prev_pd[r] = pd;
                                    st.prev_flag[r] = 1;
                                } else {
                                    const uint32_t pos = atomicAdd(&st.list_count, 1u);
                                    list[pos] = make_uint2((static_cast<uint32_t>(r) << 16) | cl, __float_as_uint(pd));
                                }
                            }
                        }
                    }
                }
            }
            __syncthreads();

            const uint32_t total = st.list_count;
            for (uint32_t e = g; e < total; e += 32) {
                const uint2 ent = list[e];
                pruned_process_pair<VEC>(p, st, row0, static_cast<int>(ent.x >> 16), ent.x & 0xFFFFu, __uint_as_float(ent.y), chunk, c0, cs, gl, gmask);
            }
            for (int r = g; r < kTileM; r += 32) {
                if (r < m_valid && st.prev_flag[r] && st.cnt[r] != 1u) {
                    pruned_process_pair<VEC>(p, st, row0, r, st.prev[r] - static_cast<uint32_t>(c0), st.prev_pd[r], chunk, c0, cs, gl, gmask);
                }
            }
            __syncthreads();
            if (tid < kTileM) {
                st.npc[tid] += st.cnt[tid];
                const unsigned long long key = st.chunk_key[tid];
                if (key != ~0ull) {
                    st.best[tid] = ordered_to_float(static_cast<uint32_t>(key >> 32));
                    st.bestidx[tid] = static_cast<uint32_t>(key & 0xFFFFFFFFull);
                }
            }
            __syncthreads();
        }
        if (tid < m_valid && st.active[tid]) {
            p.knn[row0 + tid] = st.bestidx[tid];
            p.dist[row0 + tid] = st.best[tid];
            p.not_pruned[row0 + tid] = st.npc[tid];
        }
        __syncthreads();
    }
}

int pruned_grid_size(int device) {
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    return sms * 2;
}

size_t pruned_scratch_elems(int grid) { return static_cast<size_t>(grid) * kListCap; }

void launch_assign_pruned(const PrunedParams& p, int grid, cudaStream_t stream) {
    if (p.n == 0) return;
    const size_t n_tiles = (p.n + kTileM - 1) / kTileM;
    const int g = static_cast<int>(min(static_cast<size_t>(grid), n_tiles));
    const bool vec = (p.d % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.y_pdx) & 15) == 0);
    if (vec) {
        assign_pruned_kernel<true><<<g, 256, 0, stream>>>(p);
    } else {
        assign_pruned_kernel<false><<<g, 256, 0, stream>>>(p);
    }
    SKM_LAUNCH_CHECK();
}

// =================================================================================================
// Centroid update: stable LSD radix sort of point ids by assignment, then a segmented row sum in
// sorted order.  Everything is order-deterministic, so the same input gives bit-identical sums.
// =================================================================================================
constexpr int kSortUnit = 2048;  // elements handled by one warp

size_t update_sort_units(size_t n) { return (n + kSortUnit - 1) / kSortUnit; }
size_t update_tiles(size_t n) { return (n + kUpdateTile - 1) / kUpdateTile; }

__global__ void __launch_bounds__(256) sort_hist_kernel(const uint32_t* __restrict__ keys, size_t n, int shift, uint32_t* __restrict__ table, size_t n_units) {
    __shared__ uint32_t h[8][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = lane; i < 256; i += 32) h[warp][i] = 0;
    __syncwarp();
    const size_t unit = static_cast<size_t>(blockIdx.x) * 8 + warp;
    if (unit < n_units) {
        const size_t base = unit * kSortUnit;
        for (int s = 0; s < kSortUnit / 32; ++s) {
            const size_t idx = base + static_cast<size_t>(s) * 32 + lane;
            if (idx < n) atomicAdd(&h[warp][(keys[idx] >> shift) & 255u], 1u);
        }
        __syncwarp();
        for (int i = lane; i < 256; i += 32) table[static_cast<size_t>(i) * n_units + unit] = h[warp][i];
    }
}

// Exclusive scan of a uint32 array: (1) per-block scan of 2048 elements + block totals,
// (2) scan of the totals by one block, (3) add block offsets.
__global__ void __launch_bounds__(1024) scan_block_kernel(uint32_t* __restrict__ data, size_t n, uint32_t* __restrict__ totals) {
    __shared__ uint32_t ws[32];
    const size_t base = static_cast<size_t>(blockIdx.x) * 2048;
    const size_t i0 = base + static_cast<size_t>(threadIdx.x) * 2;
    const uint32_t a = (i0 < n) ? data[i0] : 0u;
    const uint32_t b = (i0 + 1 < n) ? data[i0 + 1] : 0u;
    uint32_t v = a + b;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) ws[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = ws[lane];
        uint32_t winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        ws[lane] = winc - w;
        if (lane == 31 && totals) totals[blockIdx.x] = winc;
    }
    __syncthreads();
    const uint32_t excl = ws[warp] + inc - v;
    if (i0 < n) data[i0] = excl;
    if (i0 + 1 < n) data[i0 + 1] = excl + a;
}

__global__ void __launch_bounds__(1024) scan_totals_kernel(uint32_t* __restrict__ totals, size_t m) {
    __shared__ uint32_t ws[32];
    __shared__ uint32_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (size_t base = 0; base < m; base += 1024) {
        const size_t i = base + threadIdx.x;
        const uint32_t v = (i < m) ? totals[i] : 0u;
        uint32_t inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) ws[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const uint32_t w = ws[lane];
            uint32_t winc = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
                if (lane >= o) winc += t;
            }
            ws[lane] = winc - w;
        }
        __syncthreads();
        const uint32_t c = carry;
        if (i < m) totals[i] = c + ws[warp] + inc - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry = c + ws[warp] + inc;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(1024) scan_add_kernel(uint32_t* __restrict__ data, size_t n, const uint32_t* __restrict__ totals) {
    const size_t base = static_cast<size_t>(blockIdx.x) * 2048;
    const uint32_t off = totals[blockIdx.x];
    const size_t i0 = base + static_cast<size_t>(threadIdx.x) * 2;
    if (i0 < n) data[i0] += off;
    if (i0 + 1 < n) data[i0 + 1] += off;
}

void exclusive_scan_u32(uint32_t* data, size_t n, uint32_t* totals_tmp, cudaStream_t stream) {
    if (n == 0) return;
    const size_t blocks = (n + 2047) / 2048;
    scan_block_kernel<<<static_cast<unsigned>(blocks), 1024, 0, stream>>>(data, n, totals_tmp);
    SKM_LAUNCH_CHECK();
    if (blocks > 1) {
        scan_totals_kernel<<<1, 1024, 0, stream>>>(totals_tmp, blocks);
        SKM_LAUNCH_CHECK();
        scan_add_kernel<<<static_cast<unsigned>(blocks), 1024, 0, stream>>>(data, n, totals_tmp);
        SKM_LAUNCH_CHECK();
    }
}

// Stable scatter: each warp re-reads its unit in order; lanes with equal digits are ranked by lane.
__global__ void __launch_bounds__(256) sort_scatter_kernel(
    const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, size_t n, int shift,
    const uint32_t* __restrict__ table, size_t n_units
) {
    __shared__ uint32_t base_s[8][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t unit = static_cast<size_t>(blockIdx.x) * 8 + warp;
    if (unit >= n_units) return;
    for (int i = lane; i < 256; i += 32) base_s[warp][i] = table[static_cast<size_t>(i) * n_units + unit];
    __syncwarp();
    const size_t base = unit * kSortUnit;
    const uint32_t lt_mask = (1u << lane) - 1u;
    for (int s = 0; s < kSortUnit / 32; ++s) {
        const size_t idx = base + static_cast<size_t>(s) * 32 + lane;
        const bool valid = idx < n;
        const uint32_t key = valid ? keys_in[idx] : 0u;
        const uint32_t val = valid ? (vals_in ? vals_in[idx] : static_cast<uint32_t>(idx)) : 0u;
        const uint32_t digit = valid ? ((key >> shift) & 255u) : 0xFFFFFFFFu;
        const uint32_t peers = __match_any_sync(0xffffffffu, digit);
        const uint32_t rank = __popc(peers & lt_mask);
        uint32_t pos = 0;
        if (valid) {
            pos = base_s[warp][digit] + rank;
            keys_out[pos] = key;
            vals_out[pos] = val;
        }
        __syncwarp();
        if (valid && rank == 0) base_s[warp][digit] += __popc(peers);
        __syncwarp();
    }
}

// seg_offsets[c] = first sorted position whose key is >= c, for c in [0, k]
__global__ void segment_offsets_kernel(const uint32_t* __restrict__ sorted_keys, size_t n, size_t k, uint32_t* __restrict__ off) {
    const size_t p = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (p >= n) return;
    const uint32_t key = sorted_keys[p];
    const uint32_t lo = (p == 0) ? 0u : sorted_keys[p - 1] + 1u;
    for (uint32_t c = lo; c <= key && c <= k; ++c) off[c] = static_cast<uint32_t>(p);
    if (p == n - 1) {
        for (size_t c = static_cast<size_t>(key) + 1; c <= k; ++c) off[c] = static_cast<uint32_t>(n);
    }
}

__global__ void counts_from_offsets_kernel(const uint32_t* __restrict__ off, size_t k, uint32_t* __restrict__ counts) {
    const size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c < k) counts[c] = off[c + 1] - off[c];
}

// One CTA sums the rows of kUpdateTile consecutive sorted points for a slab of 1024 columns.  The
// first segment of the tile goes to partial slot 2t, the last one (if different) to slot 2t+1, and
// segments that lie strictly inside the tile are final and go straight to `sums`.
template <bool VEC>
__global__ void __launch_bounds__(256) segsum_tile_kernel(
    const float* __restrict__ x, const uint32_t* __restrict__ sorted_keys, const uint32_t* __restrict__ order, size_t n, size_t d, float* __restrict__ sums, float* __restrict__ partials
) {
    __shared__ uint32_t skey[kUpdateTile];
    __shared__ uint32_t sid[kUpdateTile];
    const size_t tile = blockIdx.x;
    const size_t p0 = tile * kUpdateTile;
    const int cnt = static_cast<int>(min(static_cast<size_t>(kUpdateTile), n - p0));
    for (int i = threadIdx.x; i < cnt; i += 256) {
        skey[i] = sorted_keys[p0 + i];
        sid[i] = order[p0 + i];
    }
    __syncthreads();
    const size_t colbase = static_cast<size_t>(blockIdx.y) * 1024;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    size_t col[4];
    bool cv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        col[e] = VEC ? (colbase + static_cast<size_t>(threadIdx.x) * 4 + e) : (colbase + threadIdx.x + 256 * e);
        cv[e] = col[e] < d;
    }
    auto flush = [&](uint32_t key, int kind) {
        float* dst = (kind == 0) ? (partials + (tile * 2) * d) : (kind == 1 ? (partials + (tile * 2 + 1) * d) : (sums + static_cast<size_t>(key) * d));
        if (VEC) {
            if (cv[0]) *reinterpret_cast<float4*>(dst + col[0]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (cv[e]) dst[col[e]] = acc[e];
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    };
    uint32_t cur = skey[0];
    bool first = true;
    constexpr int U = 8;
    for (int i0 = 0; i0 < cnt; i0 += U) {
        float v[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u;
            if (i < cnt) {
                const float* row = x + static_cast<size_t>(sid[i]) * d;
                if (VEC) {
                    if (cv[0]) {
                        const float4 t = __ldg(reinterpret_cast<const float4*>(row + col[0]));
                        v[u][0] = t.x; v[u][1] = t.y; v[u][2] = t.z; v[u][3] = t.w;
                    } else {
                        v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[u][e] = cv[e] ? __ldg(row + col[e]) : 0.f;
                }
            } else {
                v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u;
            if (i < cnt) {
                const uint32_t kk = skey[i];
                if (kk != cur) {
                    flush(cur, first ? 0 : 2);
                    first = false;
                    cur = kk;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] += v[u][e];
            }
        }
    }
    flush(cur, first ? 0 : 1);
}

// Combines the tile partials of every cluster whose points are not strictly inside one tile, in
// tile order; empty clusters get zeros.
template <bool VEC>
__global__ void __launch_bounds__(256) segsum_fix_kernel(const uint32_t* __restrict__ off, size_t n, size_t d, const float* __restrict__ partials, float* __restrict__ sums) {
    const size_t c = blockIdx.x;
    const size_t s = off[c], e = off[c + 1];
    const size_t colbase = static_cast<size_t>(blockIdx.y) * 1024;
    size_t col[4];
    bool cv[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        col[q] = VEC ? (colbase + static_cast<size_t>(threadIdx.x) * 4 + q) : (colbase + threadIdx.x + 256 * q);
        cv[q] = col[q] < d;
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (s < e) {
        const size_t t0 = s / kUpdateTile, t1 = (e - 1) / kUpdateTile;
        const size_t tile_end = min((t0 + 1) * kUpdateTile, n);
        const bool direct = (t0 == t1) && (s > t0 * kUpdateTile) && (e < tile_end);
        if (direct) return;
        for (size_t t = t0; t <= t1; ++t) {
            const size_t slot = (s <= t * kUpdateTile) ? (2 * t) : (2 * t + 1);
            const float* src = partials + slot * d;
            if (VEC) {
                if (cv[0]) {
                    const float4 v = *reinterpret_cast<const float4*>(src + col[0]);
                    acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (cv[q]) acc[q] += src[col[q]];
            }
        }
    }
    float* dst = sums + c * d;
    if (VEC) {
        if (cv[0]) *reinterpret_cast<float4*>(dst + col[0]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (cv[q]) dst[col[q]] = acc[q];
    }
}

// Deterministic reductions of the per-point distance (double) and not-pruned count (u64).
constexpr int kReduceBlocks = 512;
__global__ void __launch_bounds__(256) reduce_stats_kernel(const float* __restrict__ dist, const uint32_t* __restrict__ np, size_t n, double* __restrict__ block_sums) {
    __shared__ double sd[256];
    __shared__ unsigned long long su[256];
    double a = 0.0;
    unsigned long long b = 0;
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<size_t>(kReduceBlocks) * 256) {
        a += static_cast<double>(dist[i]);
        if (np) b += np[i];
    }
    sd[threadIdx.x] = a;
    su[threadIdx.x] = b;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            sd[threadIdx.x] += sd[threadIdx.x + o];
            su[threadIdx.x] += su[threadIdx.x + o];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = sd[0];
        reinterpret_cast<unsigned long long*>(block_sums + kReduceBlocks)[blockIdx.x] = su[0];
    }
}

__global__ void __launch_bounds__(256) reduce_final_kernel(const double* __restrict__ block_sums, int m, double* __restrict__ out_d, unsigned long long* __restrict__ out_u) {
    __shared__ double sd[256];
    __shared__ unsigned long long su[256];
    double a = 0.0;
    unsigned long long b = 0;
    const unsigned long long* bu = reinterpret_cast<const unsigned long long*>(block_sums + kReduceBlocks);
    for (int i = threadIdx.x; i < m; i += 256) {
        a += block_sums[i];
        if (out_u) b += bu[i];
    }
    sd[threadIdx.x] = a;
    su[threadIdx.x] = b;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            sd[threadIdx.x] += sd[threadIdx.x + o];
            su[threadIdx.x] += su[threadIdx.x + o];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (out_d) *out_d = sd[0];
        if (out_u) *out_u = su[0];
    }
}

// Stable LSD radix sort of the indices 0 .. n-1 by key (keys < k): *sorted_keys and *order point into ws.keys_* / ws.vals_*.
void launch_sort_by_key(const uint32_t* keys, size_t n, size_t k, UpdateWorkspace& ws, const uint32_t** sorted_keys_out, const uint32_t** order_out, cudaStream_t stream) {
    const size_t n_units = update_sort_units(n);
    int bits = 1;
    while ((size_t{1} << bits) < k) ++bits;
    const int passes = (bits + 7) / 8;
    const uint32_t* kin = keys;
    const uint32_t* vin = nullptr;
    uint32_t* kout = ws.keys_a;
    uint32_t* vout = ws.vals_a;
    const unsigned unit_blocks = static_cast<unsigned>((n_units + 7) / 8);
    // The scan's block totals live in a dedicated region at the end of digit_table (allocated by the caller).
    uint32_t* scan_totals = ws.digit_table + 256 * n_units;
    for (int pass = 0; pass < passes; ++pass) {
        const int shift = pass * 8;
        sort_hist_kernel<<<unit_blocks, 256, 0, stream>>>(kin, n, shift, ws.digit_table, n_units);
        SKM_LAUNCH_CHECK();
        exclusive_scan_u32(ws.digit_table, 256 * n_units, scan_totals, stream);
        sort_scatter_kernel<<<unit_blocks, 256, 0, stream>>>(kin, vin, kout, vout, n, shift, ws.digit_table, n_units);
        SKM_LAUNCH_CHECK();
        kin = kout;
        vin = vout;
        kout = (kout == ws.keys_a) ? ws.keys_b : ws.keys_a;
        vout = (vout == ws.vals_a) ? ws.vals_b : ws.vals_a;
    }
    *sorted_keys_out = kin;
    *order_out = vin;
}

void launch_update(
    const float* x, const uint32_t* assign, const float* dist, const uint32_t* not_pruned, size_t n, size_t k, size_t d, UpdateWorkspace& ws, float* sums, uint32_t* counts,
    double* wcss, unsigned long long* not_pruned_total, cudaStream_t stream
) {
    if (n == 0) return;
    const uint32_t* sorted_keys = nullptr;
    const uint32_t* order = nullptr;
    launch_sort_by_key(assign, n, k, ws, &sorted_keys, &order, stream);
    segment_offsets_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(sorted_keys, n, k, ws.seg_offsets);
    SKM_LAUNCH_CHECK();
    counts_from_offsets_kernel<<<static_cast<unsigned>((k + 255) / 256), 256, 0, stream>>>(ws.seg_offsets, k, counts);
    SKM_LAUNCH_CHECK();
    const size_t n_tiles = update_tiles(n);
    const unsigned slabs = static_cast<unsigned>((d + 1023) / 1024);
    const bool vec = (d % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (vec) {
        segsum_tile_kernel<true><<<dim3(static_cast<unsigned>(n_tiles), slabs), 256, 0, stream>>>(x, sorted_keys, order, n, d, sums, ws.tile_partials);
        SKM_LAUNCH_CHECK();
        segsum_fix_kernel<true><<<dim3(static_cast<unsigned>(k), slabs), 256, 0, stream>>>(ws.seg_offsets, n, d, ws.tile_partials, sums);
    } else {
        segsum_tile_kernel<false><<<dim3(static_cast<unsigned>(n_tiles), slabs), 256, 0, stream>>>(x, sorted_keys, order, n, d, sums, ws.tile_partials);
        SKM_LAUNCH_CHECK();
        segsum_fix_kernel<false><<<dim3(static_cast<unsigned>(k), slabs), 256, 0, stream>>>(ws.seg_offsets, n, d, ws.tile_partials, sums);
    }
    SKM_LAUNCH_CHECK();
    if (wcss || not_pruned_total) {
        reduce_stats_kernel<<<kReduceBlocks, 256, 0, stream>>>(dist, not_pruned, n, ws.block_sums);
        SKM_LAUNCH_CHECK();
        reduce_final_kernel<<<1, 256, 0, stream>>>(ws.block_sums, kReduceBlocks, wcss, not_pruned ? not_pruned_total : nullptr);
        SKM_LAUNCH_CHECK();
    }
}

// =================================================================================================
// Consolidation
// =================================================================================================
__global__ void scale_by_counts_kernel(float* __restrict__ c, const uint32_t* __restrict__ counts, size_t k, size_t d) {
    const size_t row = blockIdx.x;
    const uint32_t cnt = counts[row];
    if (cnt == 0) return;
    const float mult = static_cast<float>(1.0 / static_cast<double>(cnt));
    float* p = c + row * d;
    for (size_t j = threadIdx.x; j < d; j += blockDim.x) p[j] = __fmul_rn(p[j], mult);
}

void launch_scale_by_counts(float* c, const uint32_t* counts, size_t k, size_t d, cudaStream_t stream) {
    if (k == 0) return;
    scale_by_counts_kernel<<<static_cast<unsigned>(k), 256, 0, stream>>>(c, counts, k, d);
    SKM_LAUNCH_CHECK();
}

// Every thread owns one dimension and replays the row operations in list order.
__global__ void apply_split_ops_kernel(float* __restrict__ c, size_t d, const SplitOpDev* __restrict__ ops, size_t n_ops) {
    const size_t j = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= d) return;
    const float up = 1.0f + (1.0f / 1024.0f), down = 1.0f - (1.0f / 1024.0f);
    for (size_t o = 0; o < n_ops; ++o) {
        const SplitOpDev op = ops[o];
        float* pd = c + static_cast<size_t>(op.dst) * d + j;
        float* ps = c + static_cast<size_t>(op.src) * d + j;
        if (op.kind == 0) {
            const float v = *ps;
            if ((j & 1) == 0) {
                *pd = __fmul_rn(v, up);
                *ps = __fmul_rn(v, down);
            } else {
                *pd = __fmul_rn(v, down);
                *ps = __fmul_rn(v, up);
            }
        } else {
            float val = __fmul_rn(op.wc, *pd);
            val = __fadd_rn(val, *ps);
            *pd = __fdiv_rn(val, __fadd_rn(op.wc, 1.0f));
        }
    }
}

void launch_apply_split_ops(float* c, size_t d, const SplitOpDev* ops, size_t n_ops, cudaStream_t stream) {
    if (n_ops == 0) return;
    apply_split_ops_kernel<<<static_cast<unsigned>((d + 127) / 128), 128, 0, stream>>>(c, d, ops, n_ops);
    SKM_LAUNCH_CHECK();
}

// Spherical k-means post-processing (superkmeans.h:1357-1371): sequential-sum norm per row.
__global__ void normalize_rows_kernel(float* __restrict__ c, size_t k, size_t d) {
    const size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= k) return;
    const int lane = threadIdx.x & 31;
    float* p = c + row * d;
    float s = 0.f;
    for (size_t j = lane; j < d; j += 32) s = fmaf(p[j], p[j], s);
    s = warp_sum(s);
    const float inv = 1.0f / sqrtf(s);
    for (size_t j = lane; j < d; j += 32) p[j] *= inv;
}

void launch_normalize_rows(float* c, size_t k, size_t d, cudaStream_t stream) {
    if (k == 0) return;
    normalize_rows_kernel<<<static_cast<unsigned>((k + 7) / 8), 256, 0, stream>>>(c, k, d);
    SKM_LAUNCH_CHECK();
}

__global__ void pdxify_kernel(const float* __restrict__ c, float* __restrict__ pdx, float* __restrict__ aux, size_t k, size_t d, size_t vertical_d) {
    const size_t row = blockIdx.x;
    const size_t chunk = row / kChunk, v = row % kChunk;
    const size_t cs = min(static_cast<size_t>(kChunk), k - chunk * kChunk);
    const size_t base = chunk * kChunk * d;
    const float* src = c + row * d;
    for (size_t j = threadIdx.x; j < d; j += blockDim.x) {
        const float val = src[j];
        size_t off;
        if (j < vertical_d) {
            off = base + j * cs + v;
            if (aux) aux[row * vertical_d + j] = val;
        } else {
            const size_t h = j - vertical_d;
            off = base + vertical_d * cs + (h / kHBlock) * cs * kHBlock + v * kHBlock + (h % kHBlock);
        }
        pdx[off] = val;
    }
}

void launch_pdxify(const float* c, float* pdx, float* aux, size_t k, size_t d, size_t vertical_d, cudaStream_t stream) {
    if (k == 0) return;
    pdxify_kernel<<<static_cast<unsigned>(k), 256, 0, stream>>>(c, pdx, aux, k, d, vertical_d);
    SKM_LAUNCH_CHECK();
}

__global__ void __launch_bounds__(256) shift_kernel(const float* __restrict__ a, const float* __restrict__ b, size_t k, size_t d, double* __restrict__ block_sums) {
    __shared__ double sd[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    double total = 0.0;
    for (size_t row = static_cast<size_t>(blockIdx.x) * 8 + warp; row < k; row += static_cast<size_t>(gridDim.x) * 8) {
        const float* pa = a + row * d;
        const float* pb = b + row * d;
        float s = 0.f;
        for (size_t j = lane; j < d; j += 32) {
            const float t = pa[j] - pb[j];
            s = fmaf(t, t, s);
        }
        s = warp_sum(s);
        total += static_cast<double>(s);
    }
    if (lane == 0) sd[warp] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += sd[w];
        block_sums[blockIdx.x] = t;
    }
}

void launch_shift(const float* a, const float* b, size_t k, size_t d, double* block_sums, double* out, cudaStream_t stream) {
    const int blocks = static_cast<int>(min(static_cast<size_t>(kReduceBlocks), (k + 7) / 8));
    shift_kernel<<<blocks, 256, 0, stream>>>(a, b, k, d, block_sums);
    SKM_LAUNCH_CHECK();
    reduce_final_kernel<<<1, 256, 0, stream>>>(block_sums, blocks, out, nullptr);
    SKM_LAUNCH_CHECK();
}

// =================================================================================================
// Gather / scatter by index
// =================================================================================================
__global__ void gather_rows_kernel(const float* __restrict__ in, const uint64_t* __restrict__ idx, float* __restrict__ out, size_t n_out, size_t d) {
    const size_t row = blockIdx.x;
    float* dst = out + row * d;
    if (idx[row] == ~uint64_t{0}) {
        // "no row here" (held by another shard): zeros
        for (size_t j = threadIdx.x; j < d; j += blockDim.x) dst[j] = 0.f;
        return;
    }
    const float* src = in + idx[row] * d;
    for (size_t j = threadIdx.x; j < d; j += blockDim.x) dst[j] = src[j];
}

void launch_gather_rows(const float* in, const uint64_t* idx, float* out, size_t n_out, size_t d, cudaStream_t stream) {
    if (n_out == 0) return;
    gather_rows_kernel<<<static_cast<unsigned>(n_out), 256, 0, stream>>>(in, idx, out, n_out, d);
    SKM_LAUNCH_CHECK();
}

__global__ void gather_f32_kernel(const float* __restrict__ in, const uint64_t* __restrict__ idx, float* __restrict__ out, size_t n_out) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n_out) out[i] = in[idx[i]];
}

void launch_gather_f32(const float* in, const uint64_t* idx, float* out, size_t n_out, cudaStream_t stream) {
    if (n_out == 0) return;
    gather_f32_kernel<<<static_cast<unsigned>((n_out + 255) / 256), 256, 0, stream>>>(in, idx, out, n_out);
    SKM_LAUNCH_CHECK();
}

__global__ void scatter_u32_offset_kernel(const uint32_t* __restrict__ in, const uint64_t* __restrict__ idx, uint32_t* __restrict__ out, size_t n, uint32_t offset) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[idx[i]] = in[i] + offset;
}

void launch_scatter_u32_offset(const uint32_t* in, const uint64_t* idx, uint32_t* out, size_t n, uint32_t offset, cudaStream_t stream) {
    if (n == 0) return;
    scatter_u32_offset_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(in, idx, out, n, offset);
    SKM_LAUNCH_CHECK();
}

} // namespace skmb
