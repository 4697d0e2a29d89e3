// Second half of the pruned assignment with candidate lists made on the tensor cores.
//
// The first ADSampling test (after d' dimensions) is evaluated for every (point, centroid) pair by the
// tcgen05 GEMM kernel (first-test epilogue in kernels_tc.cu) against the loosest threshold a point can
// have, the exact distance to its previous centroid times ratio[d'].  Pairs that pass are written to one
// list per group of 32 rows, in centroid order, with the list position at every 1024-centroid boundary.
//
// walk_lists_kernel then does, for a tile of 128 points and chunk after chunk, what the reference's
// search does inside one chunk (pdx/pdxearch.h:118-327, distance_computers/batch_computers.h:297-409):
//   * re-tests every listed pair against the point's CURRENT best (which earlier chunks may have
//     lowered) and counts the survivors per point (the not-pruned counter);
//   * holds the pair with the point's previous centroid back until that count is known and drops it
//     when it is the only survivor;
//   * advances all surviving pairs together, 64 horizontal dimensions at a time (eight lanes per pair,
//     128 contiguous bytes of the PDX block per lane group), re-testing after every block and compacting
//     the list in shared memory, so lanes never idle behind a pair that died early;
//   * adds the vertical dimensions [d', vertical_d), takes the per-point minimum, lowers `best`.
// `best` is constant inside a chunk, so pairs are independent and any processing order gives the same
// result.
#include <cfloat>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "device_utils.cuh"

namespace skmb {

namespace {

constexpr int kWalkThreads = 256;
constexpr int kWalkBatch = 2048;                  // pairs advanced together
constexpr int kWalkListCap = kWalkBatch + kTileM; // + the held-back pairs with the previous centroid

struct WalkShared {
    uint2 list[2][kWalkListCap];   // {local centroid << 7 | row in tile, partial distance}
    float best[kTileM];
    float thr[kTileM];
    float prev_pd[kTileM];
    uint32_t bestidx[kTileM];
    uint32_t prev[kTileM];
    uint32_t cnt[kTileM];
    uint32_t npc[kTileM];
    uint32_t prev_flag[kTileM];
    uint32_t active[kTileM];
    unsigned long long key[kTileM];
    uint32_t count[2];
};

// Appends `ent` for the lanes with keep != 0 (one lane per pair calls with keep set); one shared-memory atomic per warp.
__device__ __forceinline__ void warp_append(uint2* list, uint32_t* counter, bool keep, uint2 ent) {
    const uint32_t m = __ballot_sync(0xffffffffu, keep);
    if (m == 0) return;
    const int lane = threadIdx.x & 31;
    uint32_t base = 0;
    if (lane == __ffs(m) - 1) base = atomicAdd(counter, __popc(m));
    base = __shfl_sync(0xffffffffu, base, __ffs(m) - 1);
    if (keep) list[base + __popc(m & ((1u << lane) - 1u))] = ent;
}

__device__ __forceinline__ float sqdiff8(const float4 a0, const float4 a1, const float4 b0, const float4 b1) {
    float s0, s1, t;
    t = a0.x - b0.x; s0 = t * t;
    t = a0.y - b0.y; s1 = t * t;
    t = a0.z - b0.z; s0 = fmaf(t, t, s0);
    t = a0.w - b0.w; s1 = fmaf(t, t, s1);
    t = a1.x - b1.x; s0 = fmaf(t, t, s0);
    t = a1.y - b1.y; s1 = fmaf(t, t, s1);
    t = a1.z - b1.z; s0 = fmaf(t, t, s0);
    t = a1.w - b1.w; s1 = fmaf(t, t, s1);
    return s0 + s1;
}

__global__ void __launch_bounds__(kWalkThreads, 3) walk_lists_kernel(const WalkParams w) {
    __shared__ WalkShared sh;
    const int tid = threadIdx.x, lane = tid & 31;
    const int g = tid >> 3, gl = tid & 7;            // 32 lane groups of 8
    const uint32_t gmask = 0xFFu << (lane & 24);
    const size_t n_chunks = (w.k + kChunk - 1) / kChunk;
    const size_t n_h = w.horizontal_d / kHBlock;
    const float ratio_first = __ldg(w.ratios + w.partial_d);

    for (size_t tile = blockIdx.x; tile < w.n_tiles; tile += gridDim.x) {
        const size_t row0 = (w.tile0 + tile) * kTileM;
        if (tid < kTileM) {
            const size_t row = row0 + tid;
            const uint32_t overflow = w.list_offs[(tile * 4 + (tid >> 5)) * (n_chunks + 1) + n_chunks] > w.cap_group ? 1u : 0u;
            bool active = row < w.n && !(w.skip && w.skip[row]);
            if (active && overflow) {
                // the group's list did not fit: its points go to the dense kernel
                w.redo[row] = 1u;
                atomicAdd(w.redo_count, 1u);
                active = false;
            }
            sh.active[tid] = active ? 1u : 0u;
            sh.best[tid] = active ? w.best_in[row] : -FLT_MAX;
            sh.bestidx[tid] = active ? w.knn[row] : 0u;
            sh.prev[tid] = active ? w.knn[row] : 0xFFFFFFFFu;
            sh.npc[tid] = 0;
        }
        __syncthreads();

        for (size_t chunk = 0; chunk < n_chunks; ++chunk) {
            const size_t c0 = chunk * kChunk;
            const size_t cs = min(static_cast<size_t>(kChunk), w.k - c0);
            if (tid < kTileM) {
                sh.thr[tid] = sh.best[tid] * ratio_first;
                sh.cnt[tid] = 0;
                sh.prev_flag[tid] = 0;
                sh.key[tid] = ~0ull;
            }
            if (tid == 0) sh.count[0] = 0;
            __syncthreads();

            // The chunk's pairs of the four row groups, taken as one sequence of `total` positions.
            uint32_t gbeg[4], glen[4];
            uint32_t total = 0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t* offs = w.list_offs + (tile * 4 + q) * (n_chunks + 1);
                const bool usable = offs[n_chunks] <= w.cap_group;
                gbeg[q] = offs[chunk];
                glen[q] = usable ? offs[chunk + 1] - offs[chunk] : 0u;
                total += glen[q];
            }
            const uint2* base_list = w.lists + tile * 4 * static_cast<size_t>(w.cap_group);

            uint32_t b0 = 0;
            do {
                const uint32_t b1 = min(b0 + static_cast<uint32_t>(kWalkBatch), total);
                const bool last_batch = b1 == total;
                // ---- load, re-test against the current threshold, count, hold the previous centroid's pair back
                for (uint32_t e0 = b0; e0 < b1; e0 += kWalkThreads) {
                    const uint32_t e = e0 + tid;
                    bool keep = false;
                    uint2 ent = make_uint2(0, 0);
                    if (e < b1) {
                        uint32_t q = 0, off = e - 0u;
                        if (off >= glen[0]) {
                            off -= glen[0];
                            q = 1;
                            if (off >= glen[1]) {
                                off -= glen[1];
                                q = 2;
                                if (off >= glen[2]) {
                                    off -= glen[2];
                                    q = 3;
                                }
                            }
                        }
                        const uint32_t gb = q == 0 ? gbeg[0] : (q == 1 ? gbeg[1] : (q == 2 ? gbeg[2] : gbeg[3]));
                        const uint2 raw = __ldg(base_list + static_cast<size_t>(q) * w.cap_group + gb + off);
                        const uint32_t r = q * 32 + (raw.x & 31u);
                        const uint32_t col = raw.x >> 5;
                        const float pd = __uint_as_float(raw.y);
                        if (pd < sh.thr[r]) {
                            atomicAdd(&sh.cnt[r], 1u);
                            if (col == sh.prev[r]) {
                                sh.prev_pd[r] = pd;
                                sh.prev_flag[r] = 1u;
                            } else {
                                keep = true;
                                ent = make_uint2(((col - static_cast<uint32_t>(c0)) << 7) | r, raw.y);
                            }
                        }
                    }
                    warp_append(sh.list[0], &sh.count[0], keep, ent);
                }
                __syncthreads();
                if (last_batch) {
                    // the survivor counts of the chunk are final now
                    bool keep = false;
                    uint2 ent = make_uint2(0, 0);
                    if (tid < kTileM && sh.prev_flag[tid] && sh.cnt[tid] != 1u) {
                        keep = true;
                        ent = make_uint2(((sh.prev[tid] - static_cast<uint32_t>(c0)) << 7) | tid, __float_as_uint(sh.prev_pd[tid]));
                    }
                    if (tid < kTileM) warp_append(sh.list[0], &sh.count[0], keep, ent);
                    __syncthreads();
                }

                // ---- horizontal blocks, all pairs of the batch in step
                int cur = 0;
                uint32_t m = sh.count[0];
                const float* __restrict__ blk_chunk = w.y_pdx + chunk * kChunk * w.d + static_cast<size_t>(w.vertical_d) * cs;
                if (w.step_hist && tid == 0) atomicAdd(&w.step_hist[30], static_cast<unsigned long long>(b1 - b0));
                for (size_t hb = 0; hb < n_h && m != 0; ++hb) {
                    if (w.step_hist && tid == 0) atomicAdd(&w.step_hist[hb < 29 ? hb : 29], static_cast<unsigned long long>(m));
                    if (tid == 0) sh.count[cur ^ 1] = 0;
                    __syncthreads();
                    const float ratio = __ldg(w.ratios + w.partial_d + (hb + 1) * kHBlock);
                    const float* __restrict__ blk = blk_chunk + hb * cs * kHBlock + gl * 8;
                    const size_t xoff = w.vertical_d + hb * kHBlock + gl * 8;
                    const uint32_t m_pad = (m + 63u) & ~63u;
                    for (uint32_t e = g; e < m_pad; e += 64) {
                        // two pairs per lane group and round, loads of both issued before any arithmetic
                        const uint32_t ea = e, eb = e + 32;
                        const bool va = ea < m, vb = eb < m;
                        const uint2 enta = sh.list[cur][va ? ea : 0];
                        const uint2 entb = sh.list[cur][vb ? eb : 0];
                        const uint32_t ra = enta.x & 127u, rb = entb.x & 127u;
                        const float* ca = blk + static_cast<size_t>(enta.x >> 7) * kHBlock;
                        const float* cb = blk + static_cast<size_t>(entb.x >> 7) * kHBlock;
                        const float* qa = w.x + (row0 + ra) * w.d + xoff;
                        const float* qb = w.x + (row0 + rb) * w.d + xoff;
                        const float4 ca0 = __ldg(reinterpret_cast<const float4*>(ca)), ca1 = __ldg(reinterpret_cast<const float4*>(ca + 4));
                        const float4 cb0 = __ldg(reinterpret_cast<const float4*>(cb)), cb1 = __ldg(reinterpret_cast<const float4*>(cb + 4));
                        const float4 qa0 = __ldg(reinterpret_cast<const float4*>(qa)), qa1 = __ldg(reinterpret_cast<const float4*>(qa + 4));
                        const float4 qb0 = __ldg(reinterpret_cast<const float4*>(qb)), qb1 = __ldg(reinterpret_cast<const float4*>(qb + 4));
                        float sa = sqdiff8(qa0, qa1, ca0, ca1);
                        float sb = sqdiff8(qb0, qb1, cb0, cb1);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 4);
                        sb += __shfl_xor_sync(0xffffffffu, sb, 4);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                        sb += __shfl_xor_sync(0xffffffffu, sb, 2);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                        sb += __shfl_xor_sync(0xffffffffu, sb, 1);
                        const float pda = __uint_as_float(enta.y) + sa;
                        const float pdb = __uint_as_float(entb.y) + sb;
                        const bool ka = va && gl == 0 && pda < sh.best[ra] * ratio;
                        const bool kb = vb && gl == 0 && pdb < sh.best[rb] * ratio;
                        warp_append(sh.list[cur ^ 1], &sh.count[cur ^ 1], ka, make_uint2(enta.x, __float_as_uint(pda)));
                        warp_append(sh.list[cur ^ 1], &sh.count[cur ^ 1], kb, make_uint2(entb.x, __float_as_uint(pdb)));
                    }
                    __syncthreads();
                    cur ^= 1;
                    m = sh.count[cur];
                }

                // ---- vertical dimensions [d', vertical_d) and the minimum of the chunk
                if (w.step_hist && tid == 0) atomicAdd(&w.step_hist[31], static_cast<unsigned long long>(m));
                if (m != 0) {
                    const uint32_t len = w.vertical_d - w.partial_d;
                    for (uint32_t e = g; e < m; e += 32) {
                        const uint2 ent = sh.list[cur][e];
                        const uint32_t r = ent.x & 127u;
                        const size_t c = c0 + (ent.x >> 7);
                        float pd = __uint_as_float(ent.y);
                        if (len != 0) {
                            const float* __restrict__ cp = w.y_aux + c * w.vertical_d + w.partial_d;
                            const float* __restrict__ qp = w.x + (row0 + r) * w.d + w.partial_d;
                            float s = 0.f;
                            for (uint32_t j = gl; j < len; j += 8) {
                                const float t = __ldg(qp + j) - __ldg(cp + j);
                                s = fmaf(t, t, s);
                            }
                            s += __shfl_xor_sync(gmask, s, 4);
                            s += __shfl_xor_sync(gmask, s, 2);
                            s += __shfl_xor_sync(gmask, s, 1);
                            pd += s;
                        }
                        if (gl == 0 && pd < sh.best[r]) {
                            atomicMin(&sh.key[r], (static_cast<unsigned long long>(float_to_ordered(pd)) << 32) | static_cast<unsigned long long>(c));
                        }
                    }
                }
                __syncthreads();
                if (tid == 0) sh.count[0] = 0;
                __syncthreads();
                b0 = b1;
            } while (b0 < total);

            if (tid < kTileM) {
                sh.npc[tid] += sh.cnt[tid];
                const unsigned long long key = sh.key[tid];
                if (key != ~0ull) {
                    sh.best[tid] = ordered_to_float(static_cast<uint32_t>(key >> 32));
                    sh.bestidx[tid] = static_cast<uint32_t>(key & 0xFFFFFFFFull);
                }
            }
            __syncthreads();
        }
        if (tid < kTileM && sh.active[tid]) {
            const size_t row = row0 + tid;
            w.knn[row] = sh.bestidx[tid];
            w.dist[row] = sh.best[tid];
            w.not_pruned[row] = sh.npc[tid];
        }
        __syncthreads();
    }
}

} // namespace

void launch_walk_lists(const WalkParams& w, int device, cudaStream_t stream) {
    if (w.n_tiles == 0) return;
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const unsigned grid = static_cast<unsigned>(std::min<size_t>(w.n_tiles, static_cast<size_t>(sms) * 3));
    static unsigned long long* hist_dev = nullptr;
    const bool want_hist = std::getenv("SKM_WALK_DEBUG") != nullptr;
    WalkParams wp = w;
    wp.step_hist = nullptr;
    if (want_hist) {
        if (!hist_dev) SKM_CUDA(cudaMalloc(&hist_dev, 32 * sizeof(unsigned long long)));
        SKM_CUDA(cudaMemsetAsync(hist_dev, 0, 32 * sizeof(unsigned long long), stream));
        wp.step_hist = hist_dev;
    }
    walk_lists_kernel<<<grid, kWalkThreads, 0, stream>>>(wp);
    SKM_LAUNCH_CHECK();
    if (want_hist) {
        unsigned long long h[32];
        SKM_CUDA(cudaMemcpyAsync(h, hist_dev, sizeof(h), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaStreamSynchronize(stream));
        std::fprintf(stderr, "[walk dbg] listed %llu | alive entering block:", h[30]);
        for (int i = 0; i < 16; ++i) std::fprintf(stderr, " %llu", h[i]);
        std::fprintf(stderr, " | entering tail %llu\n", h[31]);
    }
}

} // namespace skmb
