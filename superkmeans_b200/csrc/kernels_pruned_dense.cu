// Preparation and dense variant of the pruned assignment (see PruneSplitWorkspace in common.cuh).
//
//   prev_dist_kernel        exact ||x - c_prev||^2 per point: the first ADSampling threshold
//                           (reference: batch_computers.h:372-377)
//   classify_kernel         partial distances to 128 sampled centroids with the tile GEMM; a point whose
//                           first test keeps >= 1/16 of the sample alive is flagged for the dense kernel
//   chain_norms_kernel      cumulative squared norms of every centroid at each checkpoint of the chain
//   assign_pruned_dense_kernel
//                           for flagged points: the same sequence of tests as PDXearch::Prune
//                           (pdx/pdxearch.h:118-217) - after d' dimensions, after every 64 horizontal
//                           dimensions, after the remaining vertical dimensions - evaluated on dense
//                           128 x 128 tiles whose accumulators keep growing along the chain, with the
//                           distance written as ||x||^2 + ||c||^2 - 2 x.c over the dimensions seen so far.
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "device_utils.cuh"
#include "gemm_simt.cuh"

namespace skmb {

constexpr int kSample = 128;
constexpr int kMaxCheckpoints = 64;

uint32_t prune_chain_checkpoints(uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d) {
    return 1u + horizontal_d / kHBlock + (partial_d < vertical_d ? 1u : 0u);
}

size_t prune_split_positions_elems(size_t n) { return n + n / 2048 + 64; }

// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prev_dist_kernel(const float* __restrict__ x, const float* __restrict__ y, const uint32_t* __restrict__ knn, size_t n, size_t d,
                                                        float* __restrict__ best) {
    const size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= n) return;
    const int lane = threadIdx.x & 31;
    const float* __restrict__ xr = x + row * d;
    const float* __restrict__ yr = y + static_cast<size_t>(knn[row]) * d;
    float s = 0.f;
    const bool vec = (d % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    if (vec) {
        for (size_t j = static_cast<size_t>(lane) * 4; j < d; j += 128) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(xr + j));
            const float4 b = __ldg(reinterpret_cast<const float4*>(yr + j));
            float t;
            t = a.x - b.x; s = fmaf(t, t, s);
            t = a.y - b.y; s = fmaf(t, t, s);
            t = a.z - b.z; s = fmaf(t, t, s);
            t = a.w - b.w; s = fmaf(t, t, s);
        }
    } else {
        for (size_t j = lane; j < d; j += 32) {
            const float t = __ldg(xr + j) - __ldg(yr + j);
            s = fmaf(t, t, s);
        }
    }
    s = warp_sum(s);
    if (lane == 0) best[row] = s;
}

// sample[s][:] = y[(s * k) / n_sample][:]
__global__ void gather_sample_kernel(const float* __restrict__ y, size_t k, size_t d, int n_sample, float* __restrict__ sample) {
    const int s = blockIdx.x;
    const size_t c = (static_cast<size_t>(s) * k) / n_sample;
    for (size_t j = threadIdx.x; j < d; j += blockDim.x) sample[static_cast<size_t>(s) * d + j] = y[c * d + j];
}

// One CTA per 128 points: partial distances to the sampled centroids, survivors of the first test
// counted per point.
__global__ void __launch_bounds__(256, 2) classify_kernel(
    const float* __restrict__ x, const float* __restrict__ sample, const float* __restrict__ sample_norms, const float* __restrict__ norms_x, const float* __restrict__ best,
    size_t n, size_t d, uint32_t partial_d, int n_sample, float ratio_first, uint32_t flag_mult, uint32_t* __restrict__ flags, unsigned long long* __restrict__ alive_total
) {
    __shared__ GemmSmem smem;
    __shared__ uint32_t cnt[kTileM];
    const size_t row0 = static_cast<size_t>(blockIdx.x) * kTileM;
    const int m_valid = static_cast<int>(min(static_cast<size_t>(kTileM), n - row0));
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    if (threadIdx.x < kTileM) cnt[threadIdx.x] = 0;
    float acc[8][8];
    gemm_tile_nt(x + row0 * d, d, m_valid, sample, d, n_sample, static_cast<int>(partial_d), smem, acc);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = tile_row_of(ty, i);
        if (r >= m_valid) continue;
        const float thr = best[row0 + r] * ratio_first;
        const float nxv = norms_x[row0 + r];
        uint32_t c_alive = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = tile_col_of(tx, j);
            if (c < n_sample) {
                const float pd = fmaf(-2.0f, acc[i][j], nxv) + __ldg(sample_norms + c);
                c_alive += (pd < thr) ? 1u : 0u;
            }
        }
        if (c_alive) atomicAdd(&cnt[r], c_alive);
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < m_valid) flags[row0 + threadIdx.x] = (cnt[threadIdx.x] * flag_mult >= static_cast<uint32_t>(n_sample)) ? 1u : 0u;
    // total number of sampled pairs that pass the first test (estimates the pass's survival rate)
    if (threadIdx.x < 32) {
        uint32_t s = 0;
        for (int r = threadIdx.x; r < m_valid; r += 32) s += cnt[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (threadIdx.x == 0 && s) atomicAdd(alive_total, static_cast<unsigned long long>(s));
    }
}

__global__ void compact_flags_kernel(const uint32_t* __restrict__ flags, const uint32_t* __restrict__ positions, size_t n, uint32_t* __restrict__ idx, uint32_t* __restrict__ n_out) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (flags[i]) idx[positions[i]] = static_cast<uint32_t>(i);
    if (i == n - 1) *n_out = positions[i] + flags[i];
}

__global__ void copy_u32_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i];
}

// Cumulative squared norm of `row` after each checkpoint of the chain: [0, d'), then each horizontal
// block [vd + 64 b, vd + 64 (b+1)), then [d', vd) when d' < vd.  One warp per row; `out` has n_ck
// entries and is written by lane 0.
__device__ __forceinline__ void chain_norms_row(const float* __restrict__ row, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, int lane, float* out,
                                                size_t out_stride = 1) {
    float cum = 0.f;
    uint32_t ck = 0;
    {
        float s = 0.f;
        for (uint32_t j = lane; j < partial_d; j += 32) s = fmaf(__ldg(row + j), __ldg(row + j), s);
        cum += warp_sum(s);
        if (lane == 0) out[ck * out_stride] = cum;
        ++ck;
    }
    for (uint32_t h = 0; h < horizontal_d; h += kHBlock) {
        const float a = __ldg(row + vertical_d + h + lane), b = __ldg(row + vertical_d + h + 32 + lane);
        cum += warp_sum(fmaf(a, a, b * b));
        if (lane == 0) out[ck * out_stride] = cum;
        ++ck;
    }
    if (partial_d < vertical_d) {
        float s = 0.f;
        for (uint32_t j = partial_d + lane; j < vertical_d; j += 32) s = fmaf(__ldg(row + j), __ldg(row + j), s);
        cum += warp_sum(s);
        if (lane == 0) out[ck * out_stride] = cum;
    }
}

// transposed = false: out[row][checkpoint]; true: out[checkpoint][row]
__global__ void __launch_bounds__(256) chain_norms_kernel(const float* __restrict__ y, size_t k, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d,
                                                          uint32_t n_ck, bool transposed, float* __restrict__ out) {
    const size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= k) return;
    if (transposed) chain_norms_row(y + row * d, partial_d, vertical_d, horizontal_d, threadIdx.x & 31, out + row, k);
    else chain_norms_row(y + row * d, partial_d, vertical_d, horizontal_d, threadIdx.x & 31, out + row * n_ck);
}

// -------------------------------------------------------------------------------------------------
// Dense chain
// -------------------------------------------------------------------------------------------------
struct DenseRowState {
    uint32_t gidx[kTileM];
    float best[kTileM];
    uint32_t bestidx[kTileM];
    uint32_t prev[kTileM];
    uint32_t cnt[kTileM];
    uint32_t npc[kTileM];
    uint32_t prev_first[kTileM];
    unsigned long long chunk_key[kTileM];
};

__global__ void __launch_bounds__(256, 2) assign_pruned_dense_kernel(const PrunedParams p, const uint32_t* __restrict__ hard_idx, size_t n_hard, const float* __restrict__ best_in,
                                                                     const float* __restrict__ chain_norms_y, uint32_t n_ck) {
    __shared__ GemmSmem smem;
    __shared__ DenseRowState st;
    extern __shared__ float nxc[];  // [kTileM][n_ck] cumulative norms of the tile's points
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int lane = tid & 31, warp = tid >> 5;
    const size_t tile0 = static_cast<size_t>(blockIdx.x) * kTileM;
    const int m_valid = static_cast<int>(min(static_cast<size_t>(kTileM), n_hard - tile0));
    const uint32_t n_hblocks = p.horizontal_d / kHBlock;
    const bool has_tail = p.partial_d < p.vertical_d;

    if (tid < kTileM) {
        const bool v = tid < m_valid;
        const uint32_t g = v ? hard_idx[tile0 + tid] : 0u;
        st.gidx[tid] = g;
        st.best[tid] = v ? best_in[g] : -1.0f;
        st.bestidx[tid] = v ? p.knn[g] : 0u;
        st.prev[tid] = v ? p.knn[g] : 0xFFFFFFFFu;
        st.npc[tid] = 0;
    }
    __syncthreads();
    for (int r = warp; r < m_valid; r += 8) chain_norms_row(p.x + static_cast<size_t>(st.gidx[r]) * p.d, p.partial_d, p.vertical_d, p.horizontal_d, lane, nxc + r * n_ck);
    __syncthreads();

    const size_t n_chunks = (p.k + kChunk - 1) / kChunk;
    for (size_t chunk = 0; chunk < n_chunks; ++chunk) {
        const size_t c0 = chunk * kChunk;
        const size_t cs = min(static_cast<size_t>(kChunk), p.k - c0);
        if (tid < kTileM) {
            st.cnt[tid] = 0;
            st.prev_first[tid] = 0;
            st.chunk_key[tid] = ~0ull;
        }
        __syncthreads();
        for (size_t sub0 = 0; sub0 < cs; sub0 += kTileN) {
            const int n_valid = static_cast<int>(min(static_cast<size_t>(kTileN), cs - sub0));
            const float* __restrict__ yb = p.y + (c0 + sub0) * p.d;
            float acc[8][8];
            // ---- checkpoint 0: the first d' dimensions
            gemm_tile_nt_ex<true, true>(p.x, p.d, m_valid, st.gidx, yb, p.d, n_valid, static_cast<int>(p.partial_d), smem, acc);
            unsigned long long alive = 0ull;
            uint32_t dims = p.partial_d;
            {
                const float ratio = __ldg(p.ratios + dims);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = tile_row_of(ty, i);
                    if (r >= m_valid) continue;
                    const float thr = st.best[r] * ratio;
                    const float nxv = nxc[r * n_ck];
                    uint32_t c_alive = 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int c = tile_col_of(tx, j);
                        if (c < n_valid) {
                            const size_t gc = c0 + sub0 + c;
                            const float pd = fmaf(-2.0f, acc[i][j], nxv) + __ldg(chain_norms_y + gc);
                            if (pd < thr) {
                                alive |= 1ull << (i * 8 + j);
                                ++c_alive;
                                if (static_cast<size_t>(st.prev[r]) == gc) st.prev_first[r] = 1;
                            }
                        }
                    }
                    if (c_alive) atomicAdd(&st.cnt[r], c_alive);
                }
            }
            // Nothing of this sub-tile survived the first test: skip its remaining dimensions.
            if (!__syncthreads_or(alive != 0ull)) continue;
            // ---- horizontal blocks, 64 dimensions at a time
            for (uint32_t hb = 0; hb < n_hblocks; ++hb) {
                const size_t off = static_cast<size_t>(p.vertical_d) + static_cast<size_t>(hb) * kHBlock;
                gemm_tile_nt_ex<false, true>(p.x + off, p.d, m_valid, st.gidx, yb + off, p.d, n_valid, kHBlock, smem, acc);
                dims += kHBlock;
                const float ratio = __ldg(p.ratios + dims);
                const uint32_t ck = 1 + hb;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (((alive >> (i * 8)) & 0xFFull) == 0ull) continue;
                    const int r = tile_row_of(ty, i);
                    const float thr = st.best[r] * ratio;
                    const float nxv = nxc[r * n_ck + ck];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (alive & (1ull << (i * 8 + j))) {
                            const size_t gc = c0 + sub0 + tile_col_of(tx, j);
                            const float pd = fmaf(-2.0f, acc[i][j], nxv) + __ldg(chain_norms_y + static_cast<size_t>(ck) * p.k + gc);
                            if (!(pd < thr)) alive &= ~(1ull << (i * 8 + j));
                        }
                    }
                }
                if ((hb & 3u) == 3u && !__syncthreads_or(alive != 0ull)) break;
            }
            // ---- the vertical dimensions not covered by the first checkpoint, then the final pick
            if (has_tail) {
                gemm_tile_nt_ex<false, true>(p.x + p.partial_d, p.d, m_valid, st.gidx, yb + p.partial_d, p.d, n_valid, static_cast<int>(p.vertical_d - p.partial_d), smem, acc);
            }
            const uint32_t ck_last = n_ck - 1;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (((alive >> (i * 8)) & 0xFFull) == 0ull) continue;
                const int r = tile_row_of(ty, i);
                const float b = st.best[r];
                const float nxv = nxc[r * n_ck + ck_last];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (alive & (1ull << (i * 8 + j))) {
                        const size_t gc = c0 + sub0 + tile_col_of(tx, j);
                        const float pd = fmaf(-2.0f, acc[i][j], nxv) + __ldg(chain_norms_y + static_cast<size_t>(ck_last) * p.k + gc);
                        if (pd < b) {  // ratio[d] == 1
                            const unsigned long long key = (static_cast<unsigned long long>(float_to_ordered(pd)) << 32) | static_cast<unsigned long long>(gc);
                            atomicMin(&st.chunk_key[r], key);
                        }
                    }
                }
            }
        }
        __syncthreads();
        if (tid < kTileM) {
            st.npc[tid] += st.cnt[tid];
            const unsigned long long key = st.chunk_key[tid];
            // pdxearch.h:140-143: when the previous centroid is the only survivor of the first test the
            // chunk leaves the candidate untouched
            const bool only_previous = (st.cnt[tid] == 1u) && st.prev_first[tid];
            if (key != ~0ull && !only_previous) {
                st.best[tid] = ordered_to_float(static_cast<uint32_t>(key >> 32));
                st.bestidx[tid] = static_cast<uint32_t>(key & 0xFFFFFFFFull);
            }
        }
        __syncthreads();
    }
    if (tid < m_valid) {
        const uint32_t g = st.gidx[tid];
        p.knn[g] = st.bestidx[tid];
        p.dist[g] = st.best[tid];
        p.not_pruned[g] = st.npc[tid];
    }
}

// -------------------------------------------------------------------------------------------------
void launch_exact_dist(const float* x, const float* y, const uint32_t* knn, size_t n, size_t d, float* out, cudaStream_t stream) {
    if (n == 0) return;
    prev_dist_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(x, y, knn, n, d, out);
    SKM_LAUNCH_CHECK();
}

void launch_pruned_prepare(const PrunedParams& p, PruneSplitWorkspace& ws, cudaStream_t stream) {
    if (p.n == 0) return;
    launch_exact_dist(p.x, p.y, p.knn, p.n, p.d, ws.best, stream);
    const int n_sample = static_cast<int>(std::min<size_t>(p.k, kSample));
    gather_sample_kernel<<<n_sample, 256, 0, stream>>>(p.y, p.k, p.d, n_sample, ws.sample);
    SKM_LAUNCH_CHECK();
    launch_row_sqnorms(ws.sample, n_sample, p.d, p.partial_d, ws.sample_norms, stream);
    const float ratio_first = ws.ratio_first;
    SKM_CUDA(cudaMemsetAsync(ws.alive_total, 0, sizeof(unsigned long long), stream));
    classify_kernel<<<static_cast<unsigned>((p.n + kTileM - 1) / kTileM), 256, 0, stream>>>(p.x, ws.sample, ws.sample_norms, p.norms_x, ws.best, p.n, p.d, p.partial_d, n_sample,
                                                                                             ratio_first, ws.flag_mult, ws.flags, ws.alive_total);
    SKM_LAUNCH_CHECK();
    copy_u32_kernel<<<static_cast<unsigned>((p.n + 255) / 256), 256, 0, stream>>>(ws.flags, ws.positions, p.n);
    SKM_LAUNCH_CHECK();
    exclusive_scan_u32(ws.positions, p.n, ws.positions + p.n, stream);
    compact_flags_kernel<<<static_cast<unsigned>((p.n + 255) / 256), 256, 0, stream>>>(ws.flags, ws.positions, p.n, ws.hard_idx, ws.n_hard_dev);
    SKM_LAUNCH_CHECK();
}

// Rows listed in idx gathered into a compact matrix together with their threshold and previous assignment,
// and the results of a pass over the compact rows scattered back.
__global__ void __launch_bounds__(256) gather_listed_kernel(const float* __restrict__ x, const float* __restrict__ best, const uint32_t* __restrict__ knn,
                                                            const uint32_t* __restrict__ idx, size_t n_listed, size_t d, float* __restrict__ x_out,
                                                            float* __restrict__ best_out, uint32_t* __restrict__ knn_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t i = static_cast<size_t>(blockIdx.x) * 8 + warp;
    if (i >= n_listed) return;
    const size_t row = idx[i];
    const float* src = x + row * d;
    float* dst = x_out + i * d;
    if (d % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_out)) & 15) == 0) {
        for (size_t j = static_cast<size_t>(lane) * 4; j < d; j += 128) *reinterpret_cast<float4*>(dst + j) = __ldg(reinterpret_cast<const float4*>(src + j));
    } else {
        for (size_t j = lane; j < d; j += 32) dst[j] = src[j];
    }
    if (lane == 0) {
        best_out[i] = best[row];
        knn_out[i] = knn[row];
    }
}

__global__ void scatter_listed_kernel(const uint32_t* __restrict__ idx, size_t n_listed, const uint32_t* __restrict__ knn_in, const float* __restrict__ dist_in,
                                      const uint32_t* __restrict__ np_in, uint32_t* __restrict__ knn, float* __restrict__ dist, uint32_t* __restrict__ not_pruned) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_listed) return;
    const size_t row = idx[i];
    knn[row] = knn_in[i];
    dist[row] = dist_in[i];
    not_pruned[row] = np_in[i];
}

void launch_gather_listed(const float* x, const float* best, const uint32_t* knn, const uint32_t* idx, size_t n_listed, size_t d, float* x_out, float* best_out,
                          uint32_t* knn_out, cudaStream_t stream) {
    if (n_listed == 0) return;
    gather_listed_kernel<<<static_cast<unsigned>((n_listed + 7) / 8), 256, 0, stream>>>(x, best, knn, idx, n_listed, d, x_out, best_out, knn_out);
    SKM_LAUNCH_CHECK();
}

void launch_scatter_listed(const uint32_t* idx, size_t n_listed, const uint32_t* knn_in, const float* dist_in, const uint32_t* np_in, uint32_t* knn, float* dist,
                           uint32_t* not_pruned, cudaStream_t stream) {
    if (n_listed == 0) return;
    scatter_listed_kernel<<<static_cast<unsigned>((n_listed + 255) / 256), 256, 0, stream>>>(idx, n_listed, knn_in, dist_in, np_in, knn, dist, not_pruned);
    SKM_LAUNCH_CHECK();
}

// -------------------------------------------------------------------------------------------------
// Helpers of the pass that works on the points in the order of their previous centroid
// -------------------------------------------------------------------------------------------------
// Rows order[b0 .. b0 + cnt) of x, their previous assignment and partial norm, gathered into a compact batch.
__global__ void __launch_bounds__(256) gather_sorted_kernel(const float* __restrict__ x, const uint32_t* __restrict__ order, const uint32_t* __restrict__ knn,
                                                            const float* __restrict__ norms_x, size_t cnt, size_t d, float* __restrict__ xb, uint32_t* __restrict__ knn_b,
                                                            uint32_t* __restrict__ prev_b, float* __restrict__ nx_b) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t i = static_cast<size_t>(blockIdx.x) * 8 + warp;
    if (i >= cnt) return;
    const size_t row = order[i];
    const float* src = x + row * d;
    float* dst = xb + i * d;
    if (d % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xb)) & 15) == 0) {
        for (size_t j = static_cast<size_t>(lane) * 4; j < d; j += 128) *reinterpret_cast<float4*>(dst + j) = __ldg(reinterpret_cast<const float4*>(src + j));
    } else {
        for (size_t j = lane; j < d; j += 32) dst[j] = src[j];
    }
    if (lane == 0) {
        const uint32_t a = knn[row];
        knn_b[i] = a;
        prev_b[i] = a;
        nx_b[i] = norms_x[row];
    }
}

__global__ void scatter_sorted_kernel(const uint32_t* __restrict__ order, size_t cnt, const uint32_t* __restrict__ knn_b, const float* __restrict__ dist_b,
                                      const uint32_t* __restrict__ np_b, uint32_t* __restrict__ knn, float* __restrict__ dist, uint32_t* __restrict__ not_pruned) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= cnt) return;
    const size_t row = order[i];
    knn[row] = knn_b[i];
    dist[row] = dist_b[i];
    not_pruned[row] = np_b[i];
}

// tile_flags[t] = 1 when at least `threshold` of the tile's rows carry a non-zero flag
__global__ void __launch_bounds__(kTileM) tile_flags_kernel(const uint32_t* __restrict__ row_flags, size_t n, uint32_t threshold, uint32_t* __restrict__ tile_flags) {
    const size_t row = static_cast<size_t>(blockIdx.x) * kTileM + threadIdx.x;
    const int c = __syncthreads_count(row < n && row_flags[row] != 0u);
    if (threadIdx.x == 0) tile_flags[blockIdx.x] = static_cast<uint32_t>(c) >= threshold ? 1u : 0u;
}

// What a chain over the listed tiles starts from (and what rows that the chain never reaches keep): the previous
// assignment at its exact distance, no survivors, no runner-ups.
__global__ void __launch_bounds__(kTileM) init_chain_rows_kernel(const uint32_t* __restrict__ tile_map, size_t n, const uint32_t* __restrict__ prev, const float* __restrict__ best,
                                                                 uint32_t* __restrict__ knn, float* __restrict__ dist, uint32_t* __restrict__ not_pruned,
                                                                 uint2* __restrict__ top2) {
    const size_t row = static_cast<size_t>(tile_map[blockIdx.x]) * kTileM + threadIdx.x;
    if (row >= n) return;
    knn[row] = prev[row];
    dist[row] = best[row];
    not_pruned[row] = 0u;
    top2[row] = make_uint2(0xFFFFFFFFu, 0xFFFFFFFFu);
}

void launch_gather_sorted(const float* x, const uint32_t* order, const uint32_t* knn, const float* norms_x, size_t cnt, size_t d, float* xb, uint32_t* knn_b, uint32_t* prev_b,
                          float* nx_b, cudaStream_t stream) {
    if (cnt == 0) return;
    gather_sorted_kernel<<<static_cast<unsigned>((cnt + 7) / 8), 256, 0, stream>>>(x, order, knn, norms_x, cnt, d, xb, knn_b, prev_b, nx_b);
    SKM_LAUNCH_CHECK();
}

void launch_scatter_sorted(const uint32_t* order, size_t cnt, const uint32_t* knn_b, const float* dist_b, const uint32_t* np_b, uint32_t* knn, float* dist,
                           uint32_t* not_pruned, cudaStream_t stream) {
    if (cnt == 0) return;
    scatter_sorted_kernel<<<static_cast<unsigned>((cnt + 255) / 256), 256, 0, stream>>>(order, cnt, knn_b, dist_b, np_b, knn, dist, not_pruned);
    SKM_LAUNCH_CHECK();
}

void launch_tile_flags(const uint32_t* row_flags, size_t n, uint32_t threshold, uint32_t* tile_flags, cudaStream_t stream) {
    if (n == 0) return;
    tile_flags_kernel<<<static_cast<unsigned>((n + kTileM - 1) / kTileM), kTileM, 0, stream>>>(row_flags, n, threshold, tile_flags);
    SKM_LAUNCH_CHECK();
}

void launch_init_chain_rows(const uint32_t* tile_map, size_t n_tiles, size_t n, const uint32_t* prev, const float* best, uint32_t* knn, float* dist, uint32_t* not_pruned,
                            uint2* top2, cudaStream_t stream) {
    if (n_tiles == 0) return;
    init_chain_rows_kernel<<<static_cast<unsigned>(n_tiles), kTileM, 0, stream>>>(tile_map, n, prev, best, knn, dist, not_pruned, top2);
    SKM_LAUNCH_CHECK();
}

// flags / alive_total of launch_pruned_prepare without the exact distances and the compaction (the caller has the former and does not need the latter)
void launch_classify(const PrunedParams& p, PruneSplitWorkspace& ws, cudaStream_t stream) {
    if (p.n == 0) return;
    const int n_sample = static_cast<int>(std::min<size_t>(p.k, kSample));
    gather_sample_kernel<<<n_sample, 256, 0, stream>>>(p.y, p.k, p.d, n_sample, ws.sample);
    SKM_LAUNCH_CHECK();
    launch_row_sqnorms(ws.sample, n_sample, p.d, p.partial_d, ws.sample_norms, stream);
    SKM_CUDA(cudaMemsetAsync(ws.alive_total, 0, sizeof(unsigned long long), stream));
    classify_kernel<<<static_cast<unsigned>((p.n + kTileM - 1) / kTileM), 256, 0, stream>>>(p.x, ws.sample, ws.sample_norms, p.norms_x, ws.best, p.n, p.d, p.partial_d, n_sample,
                                                                                             ws.ratio_first, ws.flag_mult, ws.flags, ws.alive_total);
    SKM_LAUNCH_CHECK();
}

__global__ void iota_u32_kernel(uint32_t* __restrict__ out, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = static_cast<uint32_t>(i);
}

void launch_iota_u32(uint32_t* out, size_t n, cudaStream_t stream) {
    if (n == 0) return;
    iota_u32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(out, n);
    SKM_LAUNCH_CHECK();
}

void launch_compact_flags(const uint32_t* flags, size_t n, PruneSplitWorkspace& ws, cudaStream_t stream) {
    if (n == 0) return;
    copy_u32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(flags, ws.positions, n);
    SKM_LAUNCH_CHECK();
    exclusive_scan_u32(ws.positions, n, ws.positions + n, stream);
    compact_flags_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(flags, ws.positions, n, ws.hard_idx, ws.n_hard_dev);
    SKM_LAUNCH_CHECK();
}

void launch_chain_norms(const float* m, size_t rows, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, bool transposed, float* out,
                        cudaStream_t stream) {
    if (rows == 0) return;
    const uint32_t n_ck = prune_chain_checkpoints(partial_d, vertical_d, horizontal_d);
    chain_norms_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(m, rows, d, partial_d, vertical_d, horizontal_d, n_ck, transposed, out);
    SKM_LAUNCH_CHECK();
}

void launch_assign_pruned_dense(const PrunedParams& p, PruneSplitWorkspace& ws, size_t n_hard, cudaStream_t stream) {
    if (n_hard == 0) return;
    const uint32_t n_ck = prune_chain_checkpoints(p.partial_d, p.vertical_d, p.horizontal_d);
    if (n_ck > kMaxCheckpoints * 4) throw std::invalid_argument("dimensionality too large for the dense pruned kernel");
    launch_chain_norms(p.y, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, true, ws.chain_norms_y, stream);
    const size_t dyn = sizeof(float) * kTileM * n_ck;
    SKM_CUDA(cudaFuncSetAttribute(assign_pruned_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dyn)));
    assign_pruned_dense_kernel<<<static_cast<unsigned>((n_hard + kTileM - 1) / kTileM), 256, dyn, stream>>>(p, ws.hard_idx, n_hard, ws.best, ws.chain_norms_y, n_ck);
    SKM_LAUNCH_CHECK();
}

} // namespace skmb
