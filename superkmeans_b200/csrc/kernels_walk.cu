// Second half of the pruned assignment with candidate lists made on the tensor cores.
//
// The first ADSampling test (after d' dimensions) is evaluated for every (point, centroid) pair by the
// tcgen05 GEMM kernel (first-test epilogue in kernels_tc.cu) against the loosest threshold a point can
// have, the exact distance to its previous centroid times ratio[d'].  Pairs that pass are written to eight
// lists per tile of 128 points (32 rows x the lower or upper 128 columns of every 256-centroid tile), in
// centroid-tile order, with the list position at every 1024-centroid boundary.
//
// walk_lists_kernel then does, for a tile of 128 points and chunk after chunk, what the reference's
// search does inside one chunk (pdx/pdxearch.h:118-327, distance_computers/batch_computers.h:297-409):
//   * re-tests every listed pair against the point's CURRENT best (which earlier chunks may have
//     lowered) and counts the survivors per point (the not-pruned counter);
//   * holds the pair with the point's previous centroid back until that count is known and drops it
//     when it is the only survivor;
//   * keeps the surviving pairs of a batch in shared memory sorted by point and gives every group of eight
//     lanes a contiguous run of them; a group advances its run 64 horizontal dimensions at a time (128
//     contiguous bytes of the PDX block per load, the point's slice held in registers while the point does
//     not change), re-tests after every block and compacts the run in place, so no lane idles behind a pair
//     that died early and no block-wide barrier is needed between blocks; the runs are evened out twice
//     on the way (after the second and the sixth block);
//   * adds the vertical dimensions [d', vertical_d), recomputes in fp32 any final distance that comes within
//     rounding of the tensor-core part of `best`, takes the per-point minimum, lowers `best`.
// `best` is constant inside a chunk, so pairs are independent and any processing order gives the same
// result.
#include <cfloat>

#include "common.cuh"
#include "device_utils.cuh"

namespace skmb {

namespace {

constexpr int kWalkThreads = 256;
constexpr int kWalkGroups = kWalkThreads / 8;     // lane groups of eight, one pair at a time each
constexpr int kWalkPerThread = 8;                 // listed pairs a thread loads per batch
constexpr int kWalkBatch = kWalkThreads * kWalkPerThread;
constexpr int kWalkListCap = kWalkBatch + kTileM; // + the held-back pairs with the previous centroid

struct WalkShared {
    uint2 list[2][kWalkListCap];   // {local centroid << 7 | row in tile, partial distance}, sorted by row
    float best[kTileM];
    float thr[kTileM];
    float prev_pd[kTileM];
    float margin[kTileM];          // how close to `best` a final distance must be to be recomputed exactly
    float nx[kTileM];              // squared norm of the point over the first d' dimensions
    uint32_t bestidx[kTileM];
    uint32_t prev[kTileM];
    uint32_t cnt[kTileM];          // survivors of the first test in this chunk
    uint32_t npc[kTileM];
    uint32_t prev_flag[kTileM];
    uint32_t active[kTileM];
    uint32_t hist[kTileM];         // survivors per row in this batch, then their first position
    uint32_t cursor[kTileM];
    uint32_t warp_tot[4];
    uint32_t gcount[kWalkGroups];
    uint32_t gbeg[8], glen[8];     // this chunk's slice of each of the tile's eight lists
    unsigned long long key[kTileM];
    uint32_t m;
};

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

__device__ __forceinline__ float group_sum(float s, uint32_t gmask) {
    s += __shfl_xor_sync(gmask, s, 4);
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 1);
    return s;
}

// One 64-dimension block for the run [beg, beg + cnt) of `list`, compacted in place; returns the new length.
// All eight lanes of the group execute this together, two pairs per trip so that four 128-byte gathers are in
// flight per lane group.  The point's slice of the block is loaded only when the point changes (the list is
// sorted by point).
__device__ __forceinline__ uint32_t walk_block(uint2* list, uint32_t beg, uint32_t cnt, const float* __restrict__ blk, const float* __restrict__ xblk, size_t d,
                                               const float* best, float ratio, int gl, uint32_t gmask) {
    constexpr int U = 2;
    uint32_t j = 0, xrow = 0xFFFFFFFFu;
    float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
    for (uint32_t i = 0; i < cnt; i += U) {
        uint2 e[U];
        float4 c0[U], c1[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            e[u] = list[beg + min(i + u, cnt - 1)];
            const float* c = blk + static_cast<size_t>(e[u].x >> 7) * kHBlock;
            c0[u] = __ldg(reinterpret_cast<const float4*>(c));
            c1[u] = __ldg(reinterpret_cast<const float4*>(c + 4));
        }
        float s[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = e[u].x & 127u;
            if (r != xrow) {
                const float* q = xblk + static_cast<size_t>(r) * d;
                x0 = __ldg(reinterpret_cast<const float4*>(q));
                x1 = __ldg(reinterpret_cast<const float4*>(q + 4));
                xrow = r;
            }
            s[u] = sqdiff8(x0, x1, c0[u], c1[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) s[u] = group_sum(s[u], gmask);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float pd = __uint_as_float(e[u].y) + s[u];
            const bool keep = (i + u < cnt) && pd < best[e[u].x & 127u] * ratio;
            if (keep && gl == 0) list[beg + j] = make_uint2(e[u].x, __float_as_uint(pd));
            j += keep ? 1u : 0u;
        }
    }
    __syncwarp(gmask);
    return j;
}

// Four CTAs per SM: the kernel waits on gathers most of the time, and more resident warps hide more of that (three
// CTAs were 12 % slower, five no faster; gathers that bypass L1 were 25 % slower).
constexpr int kWalkCtasPerSm = 4;

__global__ void __launch_bounds__(kWalkThreads, kWalkCtasPerSm) walk_lists_kernel(const WalkParams w) {
    __shared__ WalkShared sh;
    if (w.upstream_error && *reinterpret_cast<const volatile int*>(w.upstream_error) != 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = tid >> 3, gl = tid & 7;
    const uint32_t gmask = 0xFFu << (lane & 24);
    const size_t n_chunks = (w.k + kChunk - 1) / kChunk;
    const size_t n_h = w.horizontal_d / kHBlock;
    const float ratio_first = __ldg(w.ratios + w.partial_d);
    unsigned long long steps_done = 0;

    for (size_t tile = blockIdx.x; tile < w.n_tiles; tile += gridDim.x) {
        const size_t row0 = (w.tile_map ? static_cast<size_t>(w.tile_map[tile]) : w.tile0 + tile) * kTileM;
        if (tid < kTileM) {
            const size_t row = row0 + tid;
            const uint32_t overflow = (w.list_offs[(tile * 8 + (tid >> 5)) * (n_chunks + 1) + n_chunks] > w.cap_group ||
                                       w.list_offs[(tile * 8 + 4 + (tid >> 5)) * (n_chunks + 1) + n_chunks] > w.cap_group)
                                          ? 1u
                                          : 0u;
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
            sh.nx[tid] = active ? w.norms_x[row] : 0.f;
            sh.npc[tid] = 0;
        }
        __syncthreads();

        for (size_t chunk = 0; chunk < n_chunks; ++chunk) {
            const size_t c0 = chunk * kChunk;
            const size_t cs = min(static_cast<size_t>(kChunk), w.k - c0);
            if (tid < kTileM) {
                sh.thr[tid] = sh.best[tid] * ratio_first;
                sh.margin[tid] = 1e-5f * sh.nx[tid];   // the tensor-core part of a distance is within ~3e-6 of the norms over d'
                sh.cnt[tid] = 0;
                sh.prev_flag[tid] = 0;
                sh.key[tid] = ~0ull;
                sh.hist[tid] = 0;
            }

            // The chunk's pairs of the tile's eight lists, taken as one sequence of `total` positions.
            if (tid < 8) {
                const uint32_t* offs = w.list_offs + (tile * 8 + tid) * (n_chunks + 1);
                const uint32_t* offs_other = w.list_offs + (tile * 8 + (tid ^ 4)) * (n_chunks + 1);
                const bool usable = offs[n_chunks] <= w.cap_group && offs_other[n_chunks] <= w.cap_group;
                sh.gbeg[tid] = offs[chunk];
                sh.glen[tid] = usable ? offs[chunk + 1] - offs[chunk] : 0u;
            }
            __syncthreads();
            uint32_t total = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) total += sh.glen[q];
            const uint2* base_list = w.lists + tile * 8 * static_cast<size_t>(w.cap_group);
            const float* __restrict__ blk_chunk = w.y_pdx + chunk * kChunk * w.d + static_cast<size_t>(w.vertical_d) * cs;

            uint32_t b0 = 0;
            do {
                const uint32_t b1 = min(b0 + static_cast<uint32_t>(kWalkBatch), total);
                const bool last_batch = b1 == total;
                // (sh.hist is zero here: cleared at the start of the chunk and at the end of every batch)
                // ---- load, re-test against the current threshold, count; the previous centroid's pair is held back
                uint2 mine[kWalkPerThread];
                uint32_t keep = 0;
#pragma unroll
                for (int u = 0; u < kWalkPerThread; ++u) {
                    const uint32_t e = b0 + u * kWalkThreads + tid;
                    mine[u] = make_uint2(0, 0);
                    if (e < b1) {
                        uint32_t q = 0, off = e;
                        while (q < 7 && off >= sh.glen[q]) {
                            off -= sh.glen[q];
                            ++q;
                        }
                        const uint2 raw = __ldg(base_list + static_cast<size_t>(q) * w.cap_group + sh.gbeg[q] + off);
                        const uint32_t r = (q & 3u) * 32 + (raw.x & 31u);
                        const uint32_t col = raw.x >> 5;
                        const float pd = __uint_as_float(raw.y);
                        if (pd < sh.thr[r]) {
                            atomicAdd(&sh.cnt[r], 1u);
                            if (col == sh.prev[r]) {
                                sh.prev_pd[r] = pd;
                                sh.prev_flag[r] = 1u;
                            } else {
                                keep |= 1u << u;
                                mine[u] = make_uint2(((col - static_cast<uint32_t>(c0)) << 7) | r, raw.y);
                                atomicAdd(&sh.hist[r], 1u);
                            }
                        }
                    }
                }
                __syncthreads();
                // the held-back pairs join the last batch, once the survivor counts of the chunk are final
                bool add_prev = false;
                if (last_batch && tid < kTileM && sh.prev_flag[tid] && sh.cnt[tid] != 1u) {
                    add_prev = true;
                    sh.hist[tid] += 1u;   // only this thread touches its row's counter here
                }
                // ---- exclusive scan of the per-row counts: pairs are stored sorted by row
                if (tid < kTileM) {
                    const uint32_t v = sh.hist[tid];
                    uint32_t incl = v;
#pragma unroll
                    for (int off = 1; off < 32; off <<= 1) {
                        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, off);
                        if (lane >= off) incl += t;
                    }
                    if (lane == 31) sh.warp_tot[warp] = incl;
                    sh.cursor[tid] = incl - v;   // exclusive inside the warp for now
                }
                __syncthreads();
                if (tid < kTileM) {
                    uint32_t base = 0;
                    for (int q = 0; q < warp; ++q) base += sh.warp_tot[q];
                    const uint32_t start = base + sh.cursor[tid];
                    sh.hist[tid] = start;
                    // the held-back pair takes the first slot of its row (nobody reads the list yet)
                    if (add_prev) sh.list[0][start] = make_uint2(((sh.prev[tid] - static_cast<uint32_t>(c0)) << 7) | tid, __float_as_uint(sh.prev_pd[tid]));
                    sh.cursor[tid] = add_prev ? 1u : 0u;
                }
                __syncthreads();
                if (tid == 0) sh.m = sh.warp_tot[0] + sh.warp_tot[1] + sh.warp_tot[2] + sh.warp_tot[3];
#pragma unroll
                for (int u = 0; u < kWalkPerThread; ++u) {
                    if ((keep >> u) & 1u) {
                        const uint32_t r = mine[u].x & 127u;
                        sh.list[0][sh.hist[r] + atomicAdd(&sh.cursor[r], 1u)] = mine[u];
                    }
                }
                __syncthreads();

                // ---- horizontal blocks: every lane group owns a contiguous run of the sorted list
                int cur = 0;
                uint32_t m = sh.m;
                uint32_t run = (m + kWalkGroups - 1) / kWalkGroups;
                uint32_t beg = min(static_cast<uint32_t>(g) * run, m);
                uint32_t len = min(run, m - beg);
                for (size_t hb = 0; hb < n_h; ++hb) {
                    steps_done += (gl == 0) ? len : 0u;
                    len = walk_block(sh.list[cur], beg, len, blk_chunk + hb * cs * kHBlock + gl * 8, w.x + row0 * w.d + w.vertical_d + hb * kHBlock + gl * 8, w.d, sh.best,
                                     __ldg(w.ratios + w.partial_d + (hb + 1) * kHBlock), gl, gmask);
                    if (((w.rebalance_mask >> hb) & 1u) && hb + 1 < n_h) {
                        // even the runs out (the only block-wide barriers between blocks): runs that hold pairs of
                        // a point with a loose threshold keep everything, others die out
                        if (gl == 0) sh.gcount[g] = len;
                        __syncthreads();
                        uint32_t off = 0, tot = 0;
                        for (int q = 0; q < kWalkGroups; ++q) {
                            const uint32_t c = sh.gcount[q];
                            off += (q < g) ? c : 0u;
                            tot += c;
                        }
                        for (uint32_t i = gl; i < len; i += 8) sh.list[cur ^ 1][off + i] = sh.list[cur][beg + i];
                        __syncthreads();
                        cur ^= 1;
                        m = tot;
                        run = (m + kWalkGroups - 1) / kWalkGroups;
                        beg = min(static_cast<uint32_t>(g) * run, m);
                        len = min(run, m - beg);
                    }
                }

                // ---- vertical dimensions [d', vertical_d) and the minimum of the chunk
                {
                    const uint32_t vlen = w.vertical_d - w.partial_d;
                    for (uint32_t i = 0; i < len; ++i) {
                        const uint2 ent = sh.list[cur][beg + i];
                        const uint32_t r = ent.x & 127u;
                        const size_t c = c0 + (ent.x >> 7);
                        float pd = __uint_as_float(ent.y);
                        if (vlen != 0) {
                            const float* __restrict__ cp = w.y_aux + c * w.vertical_d + w.partial_d;
                            const float* __restrict__ qp = w.x + (row0 + r) * w.d + w.partial_d;
                            // scalar head up to a 16-byte boundary (both rows start at a multiple of four floats, so
                            // they share it), float4 body, scalar rest
                            const uint32_t head = min(vlen, (4u - (w.partial_d & 3u)) & 3u);
                            const uint32_t n4 = (vlen - head) >> 2;
                            const uint32_t rest0 = head + (n4 << 2);
                            float s = 0.f;
                            if (static_cast<uint32_t>(gl) < head) {
                                const float t = __ldg(qp + gl) - __ldg(cp + gl);
                                s = t * t;
                            }
                            if (rest0 + gl < vlen) {
                                const float t = __ldg(qp + rest0 + gl) - __ldg(cp + rest0 + gl);
                                s = fmaf(t, t, s);
                            }
                            const float4* q4 = reinterpret_cast<const float4*>(qp + head);
                            const float4* c4 = reinterpret_cast<const float4*>(cp + head);
                            for (uint32_t jj = gl; jj < n4; jj += 8) {
                                const float4 a = __ldg(q4 + jj), b = __ldg(c4 + jj);
                                float t;
                                t = a.x - b.x; s = fmaf(t, t, s);
                                t = a.y - b.y; s = fmaf(t, t, s);
                                t = a.z - b.z; s = fmaf(t, t, s);
                                t = a.w - b.w; s = fmaf(t, t, s);
                            }
                            pd += group_sum(s, gmask);
                        }
                        // The first d' dimensions of pd come from the tensor cores (three TF32 products, truncating
                        // accumulator: a few 1e-6 of the norms off).  A pair that would win, or lose, by less than that
                        // is settled with the distance recomputed from direct differences in fp32.
                        // (The pair with the previous centroid needs none of this: its exact distance is `best` itself,
                        // which it cannot undercut.)
                        if (pd < sh.best[r] + sh.margin[r] && static_cast<uint32_t>(c) != sh.prev[r]) {
                            const float4* q4 = reinterpret_cast<const float4*>(w.x + (row0 + r) * w.d);
                            const float4* c4 = reinterpret_cast<const float4*>(w.y + c * w.d);
                            float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
                            for (uint32_t jj = gl; jj < w.d / 4; jj += 8) {
                                const float4 a = __ldg(q4 + jj), b = __ldg(c4 + jj);
                                float t;
                                t = a.x - b.x; s0 = fmaf(t, t, s0);
                                t = a.y - b.y; s1 = fmaf(t, t, s1);
                                t = a.z - b.z; s0 = fmaf(t, t, s0);
                                t = a.w - b.w; s1 = fmaf(t, t, s1);
                            }
                            const float exact = group_sum(s0 + s1, gmask);
                            if (gl == 0 && exact < sh.best[r]) {
                                atomicMin(&sh.key[r], (static_cast<unsigned long long>(float_to_ordered(exact)) << 32) | static_cast<unsigned long long>(c));
                            }
                        }
                    }
                }
                if (tid < kTileM) sh.hist[tid] = 0;
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
    if (gl == 0 && steps_done) atomicAdd(w.pair_steps, steps_done);
}

} // namespace

void launch_walk_lists(const WalkParams& w, int device, cudaStream_t stream) {
    if (w.n_tiles == 0) return;
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const unsigned grid = static_cast<unsigned>(std::min<size_t>(w.n_tiles, static_cast<size_t>(sms) * kWalkCtasPerSm));
    walk_lists_kernel<<<grid, kWalkThreads, 0, stream>>>(w);
    SKM_LAUNCH_CHECK();
}

} // namespace skmb
