// Pruned assignment as an ADSampling chain over the centroids that can matter to a tile of points.
//
// The dense chain (chain_tc_kernel in kernels_tc.cu) grows a full X * C^T product for every point it is given, because
// a point with a loose threshold keeps a sizeable share of all centroids alive.  Which centroids those are is not
// random: they are the centroids near the point's previous centroid, and points that share a previous centroid keep
// (almost) the same ones.  So the points are processed in the order of their previous centroid, and for every tile
// of 128 such points:
//   1. a first-test pass over the first d' dimensions (gemm_tc_kernel<MODE_UNION>) records, per 1024-centroid chunk,
//      the set of centroids that pass the test for at least one row of the tile;
//   2. build_cols_kernel turns the bit sets into ascending index lists;
//   3. sparse_chain_kernel (here) runs the chain of the dense kernel - same checkpoints, same thresholds, `best` fixed
//      inside a chunk and lowered at its end (pdx/pdxearch.h:118-217, :290-324) - but only over the listed centroids,
//      in units of up to 256 of them.  A centroid that is not listed fails the first test for every row of the tile,
//      so leaving it out changes neither the survivor counts nor the winners.
//
// Kernel roles (512 threads, one persistent CTA per SM), stage layout and accumulators are those of the dense chain:
//   warp 0      TMA producer of the X tile (128 points x 16 dimensions per stage);
//   warp 1      MMA issuer: tcgen05.mma kind::tf32, M = 128, N = the unit's column count rounded up to 16;
//   warps 2-3   split the X tile into tf32 hi / lo parts in place;
//   warps 4-7   gather the unit's centroid rows: asynchronous 16-byte copies (cp.async) of the hi and lo parts from the
//               pre-split centroid matrix (global memory, L2 resident) into the stage, in the 64-byte swizzled layout
//               the MMA descriptors expect (16-byte unit u of row r at unit u ^ ((r >> 1) & 3)); up to three stages
//               of copies are in flight, and a stage is announced once its copies have landed;
//   warps 8-15  the rows' threads: two per point (columns 0-127 and 128-255 of a unit); tests after every segment,
//               merge at chunk ends, as in the dense chain.
// Every wait is bounded; on expiry the kernel records a code, every role leaves its loops, tensor memory is released
// and the kernel returns.
#include <cfloat>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels_tc.cuh"
#include "tc_ptx.cuh"

namespace skmb {
namespace tc {

namespace {

struct SparseParams {
    size_t n, k;
    uint32_t d, partial_d, vertical_d, horizontal_d;
    uint32_t n_seg;                 // 1 + horizontal_d / 64 + (partial_d < vertical_d)
    uint32_t n_chunks;
    const float* chain_norms_x;     // n x n_seg cumulative squared norms of the points
    const float* chain_norms_y;     // n_seg x k (checkpoint-major), of the centroids
    const float* ratios;            // d + 1
    const float* best_in;           // exact distance to the previous centroid
    uint32_t* knn;                  // in: previous assignment, out: new
    float* dist;
    uint32_t* not_pruned;
    uint2* top2;                    // out: the two smallest final distances seen by the chain, per point
    uint32_t* dirty;                // optimistic pass only, out: 1 = the point's best candidate can move
    uint32_t* cand;                 // optimistic pass only, out: per point two lists (one per thread of the row) of cand_cap centroid indices
    uint32_t* cand_meta;            //   list lengths in bits 0..7 and 8..15, bit 16 = a list overflowed
    uint32_t cand_cap;
    const float* y_hi;              // k x d, tf32 hi parts of the centroids
    const float* y_lo;              // k x d, tf32 lo parts
    const uint32_t* tile_map;       // n_tiles row-tile indices
    size_t n_tiles;
    const uint16_t* cols;           // [n_tiles][cols_stride]
    const uint32_t* col_counts;     // [n_tiles][n_chunks]
    size_t cols_stride;
    int* error;
    long long wait_limit;
};

// Where the roles of sparse_chain_kernel spend their cycles, summed over the CTAs of all launches since the last read
// (one representative thread per role): see role_cycles().
__device__ unsigned long long g_role_cycles[16];

__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w, int code, long long& acc) {
    const long long t0 = clock64();
    const bool ok = mbar_wait(bar, parity, w, code);
    acc += clock64() - t0;
    return ok;
}
// for the roles that run ahead of the tensor pipe (TMA producer, X splitter, centroid gather)
__device__ __forceinline__ bool timed_wait_relaxed(uint64_t* bar, uint32_t parity, const WaitCtx& w, int code, long long& acc) {
    const long long t0 = clock64();
    const bool ok = mbar_wait_relaxed(bar, parity, w, code);
    acc += clock64() - t0;
    return ok;
}

struct SparseMaps {
    CUtensorMap x[3];     // points, visible extent d' / vertical_d / d
};

struct Seg {
    uint32_t x_begin;     // first column fetched (multiple of 4)
    uint32_t n_kb;        // 16-column blocks
    uint32_t map;         // 0 = front (extent d'), 1 = vertical (extent vertical_d), 2 = full
    uint32_t mask_below;  // columns below this value are zeroed in the first block (tail segment only)
    uint32_t dims_after;
};

__device__ __forceinline__ Seg sparse_segment(const SparseParams& p, uint32_t seg) {
    Seg s;
    const uint32_t n_h = p.horizontal_d / 64;
    if (seg == 0) {
        s.x_begin = 0;
        s.n_kb = (p.partial_d + BK - 1) / BK;
        s.map = 0;
        s.mask_below = 0;
        s.dims_after = p.partial_d;
    } else if (seg <= n_h) {
        s.x_begin = p.vertical_d + (seg - 1) * 64;
        s.n_kb = 64 / BK;
        s.map = 2;
        s.mask_below = 0;
        s.dims_after = p.partial_d + seg * 64;
    } else {
        s.x_begin = p.partial_d & ~3u;
        s.n_kb = (p.vertical_d - s.x_begin + BK - 1) / BK;
        s.map = 1;
        s.mask_below = p.partial_d;
        s.dims_after = p.d;
    }
    return s;
}

// What the two threads of a row (one per half of a unit's columns) tell each other at the end of a chunk.
struct RowPartial {
    uint32_t cnt;          // survivors of the first test in this chunk
    uint32_t prev_first;   // the previous centroid is among them
    float cb;              // best final distance of the chunk, FLT_MAX if none
    uint32_t cbi;
    float t1, t2;          // the two smallest final distances of the row so far (candidates for the refinement)
    uint32_t i1, i2;
};

struct SparseCtrl {
    uint64_t full[STAGES];
    uint64_t conv[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_ready[2];    // MMA -> rows: accumulator a holds the chain up to the current segment
    uint64_t acc_loaded[2];   // rows -> MMA: every row has read it
    uint64_t xchg_bar;        // the 256 row threads have published their RowPartial
    uint32_t tmem_base;
    uint32_t pad;
    alignas(16) float ny[8][BN / 2];      // per row warp: centroid norms of its share of the unit's columns at the current checkpoint
    float seg_ratio[64];                  // ratios[dimensions seen after segment s]
    alignas(16) uint16_t colid[8][2][BN / 2]; // per row warp and accumulator: local centroid index of each column of its share
    uint32_t rowoff[1][2][BN];            // per accumulator: element offset (centroid * d) of each unit column (entry r belongs to one gather thread)
    alignas(16) RowPartial xchg[2][2][BM];   // [use parity][column half][row]
};
constexpr uint32_t S_CTRL_BYTES = 30720;
static_assert(sizeof(SparseCtrl) <= S_CTRL_BYTES, "control block too large");
constexpr uint32_t S_SMEM_BYTES = STAGES * STAGE_BYTES + S_CTRL_BYTES + 1024;
static_assert(S_SMEM_BYTES <= 232448, "over the shared memory of one CTA");
constexpr uint32_t SPARSE_MAX_SEGMENTS = 64;
constexpr int SPARSE_THREADS = 512;
// warps: 0 TMA producer, 1 MMA issuer, 2-3 X splitter, 4-7 centroid gather, 8-15 rows
constexpr int kGatherThreads = 128;
constexpr int kRowWarp0 = 8;

// Order of work shared by all roles: listed tile, chunk of 1024 centroids (skipped when it lists nothing), pair of
// units, segment, unit of the pair.  A chunk's listed centroids are cut into units of equal width (a multiple of 16, at
// most 256).  `a` (0 / 1) is the unit's accumulator, `nu` its number of listed centroids and `nmma` that number
// rounded up to the tensor cores' multiple of 16.
#define SPARSE_FOR_EACH_UNIT_SEGMENT(...)                                                                 \
    for (size_t lt = blockIdx.x; lt < p.n_tiles && ok; lt += gridDim.x) {                                 \
        [[maybe_unused]] const size_t rt = static_cast<size_t>(__ldg(p.tile_map + lt));                               \
        for (uint32_t chunk = 0; chunk < p.n_chunks && ok; ++chunk) {                                     \
            const uint32_t n_listed = __ldg(p.col_counts + lt * p.n_chunks + chunk);                      \
            if (n_listed == 0) continue;                                                                  \
            const size_t c0 = static_cast<size_t>(chunk) * kChunk;                                        \
            const uint16_t* chunk_cols = p.cols + lt * p.cols_stride + c0;                                \
            /* at least two units whenever there is enough to split, so that one unit's tests overlap the other's products */ \
            const uint32_t n_units = n_listed <= 16u ? 1u : max(2u, (n_listed + BN - 1) / BN);            \
            const uint32_t unit_w = (((n_listed + n_units - 1) / n_units) + 15u) & ~15u;                  \
            for (uint32_t pair = 0; pair * 2 < n_units && ok; ++pair) {                                   \
                for (uint32_t seg = 0; seg < p.n_seg && ok; ++seg) {                                      \
                    const Seg si = sparse_segment(p, seg);                                                \
                    for (uint32_t a = 0; a < 2 && ok; ++a) {                                              \
                        const uint32_t unit = pair * 2 + a;                                               \
                        if (unit >= n_units || unit * unit_w >= n_listed) break;                          \
                        [[maybe_unused]] const uint32_t nu = min(unit_w, n_listed - unit * unit_w);      \
                        [[maybe_unused]] const uint32_t nmma = (nu + 15u) & ~15u;                         \
                        [[maybe_unused]] const uint16_t* unit_cols = chunk_cols + unit * unit_w;          \
                        __VA_ARGS__                                                                       \
                    }                                                                                     \
                }                                                                                         \
            }                                                                                             \
        }                                                                                                 \
    }

// MERGED = false: the exact chain, chunk by chunk.  MERGED = true: the optimistic pass (see merged_rows below): the
// lists are one per tile (n_chunks = 1, global centroid indices), and the rows' threads only count and look for a winner.
template <bool MERGED>
__global__ void __launch_bounds__(SPARSE_THREADS, 1) sparse_chain_kernel(const __grid_constant__ SparseMaps maps, const SparseParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    SparseCtrl* ctrl = reinterpret_cast<SparseCtrl*>(smem + STAGES * STAGE_BYTES);
    const WaitCtx wctx{p.error, p.wait_limit};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctrl->full[s], 1);
            mbar_init(&ctrl->conv[s], 64 + kGatherThreads);   // 64 X-splitter threads + the gather threads
            mbar_init(&ctrl->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&ctrl->acc_ready[a], 1);
            mbar_init(&ctrl->acc_loaded[a], 256);
        }
        mbar_init(&ctrl->xchg_bar, 256);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + SPARSE_MAX_SEGMENTS && threadIdx.x - 64 < p.n_seg) {
        ctrl->seg_ratio[threadIdx.x - 64] = __ldg(p.ratios + sparse_segment(p, threadIdx.x - 64).dims_after);
    }
    if (warp == 1) tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (points only)
        if (lane == 0) {
            uint32_t kbt = 0;
            bool ok = true;
            long long w_empty = 0;
            SPARSE_FOR_EACH_UNIT_SEGMENT({
                const CUtensorMap* mx = &maps.x[si.map];
                for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                    const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                    if (!timed_wait_relaxed(&ctrl->empty[s], ph ^ 1u, wctx, 21, w_empty)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&ctrl->full[s], A_TILE_BYTES);
                    tma_load_2d(smem_base + s * STAGE_BYTES + OFF_A_HI, mx, &ctrl->full[s], static_cast<int>(si.x_begin + kb * BK), static_cast<int>(rt * BM));
                }
            })
            atomicAdd(&g_role_cycles[11], static_cast<unsigned long long>(w_empty));
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t kbt = 0;
            uint32_t uses[2] = {0, 0};
            bool unread[2] = {false, false};   // accumulator a was handed to the rows and they have not confirmed reading it
            bool ok = true;
            long long w_loaded = 0, w_conv = 0, n_steps = 0;
            const long long t_begin = clock64();
            SPARSE_FOR_EACH_UNIT_SEGMENT({
                ++n_steps;
                // the rows must have read this accumulator's previous checkpoint before it grows (or restarts)
                if (unread[a]) {
                    if (!timed_wait(&ctrl->acc_loaded[a], (uses[a] - 1) & 1u, wctx, 22, w_loaded)) {
                        ok = false;
                        break;
                    }
                    unread[a] = false;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + a * BN;
                const uint32_t idesc = make_idesc(nmma);
                for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                    const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                    if (!timed_wait(&ctrl->conv[s], ph, wctx, 23, w_conv)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_base + s * STAGE_BYTES;
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / 8; ++kk) {
                        const uint64_t a_hi = make_desc(st + OFF_A_HI + kk * 32);
                        const uint64_t a_lo = make_desc(st + OFF_A_LO + kk * 32);
                        const uint64_t b_hi = make_desc(st + OFF_B_HI + kk * 32);
                        const uint64_t b_lo = make_desc(st + OFF_B_LO + kk * 32);
                        umma_tf32(acc, a_hi, b_hi, (seg | kb | kk) != 0 ? 1u : 0u, idesc);
                        umma_tf32(acc, a_hi, b_lo, 1u, idesc);
                        umma_tf32(acc, a_lo, b_hi, 1u, idesc);
                    }
                    umma_commit(&ctrl->empty[s]);
                }
                // The optimistic pass looks at the accumulator after the first segment (first test, counts) and after the
                // last one (could another centroid win) only: a test in between can only clear a row that the last one
                // would flag, never the other way round, so the segments in between accumulate without a hand-over.
                if (!MERGED || seg == 0 || seg + 1 == p.n_seg) {
                    if (ok) umma_commit(&ctrl->acc_ready[a]);
                    ++uses[a];
                    unread[a] = true;
                }
            })
            atomicAdd(&g_role_cycles[0], static_cast<unsigned long long>(w_loaded));
            atomicAdd(&g_role_cycles[1], static_cast<unsigned long long>(w_conv));
            atomicAdd(&g_role_cycles[2], static_cast<unsigned long long>(clock64() - t_begin));
            atomicAdd(&g_role_cycles[12], static_cast<unsigned long long>(n_steps));
            atomicAdd(&g_role_cycles[13], 1ull);
        }
    } else if (warp < 4) {
        // ---------------------------------------------------------------- X splitter (warps 2, 3)
        const int cid = threadIdx.x - 64;   // 0 .. 63
        uint32_t kbt = 0;
        bool ok = true;
        long long w_full = 0;
        SPARSE_FOR_EACH_UNIT_SEGMENT({
            for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                if (!timed_wait_relaxed(&ctrl->full[s], ph, wctx, 24, w_full)) {
                    ok = false;
                    break;
                }
                uint8_t* st = smem + s * STAGE_BYTES;
                float4* a_hi = reinterpret_cast<float4*>(st + OFF_A_HI);
                float4* a_lo = reinterpret_cast<float4*>(st + OFF_A_LO);
                const bool mask = (kb == 0) && (si.mask_below > si.x_begin);
#pragma unroll
                for (int i = 0; i < static_cast<int>(A_TILE_BYTES / 16 / 64); ++i) {
                    const int q = cid + 64 * i;
                    float4 v = a_hi[q];
                    if (mask) {
                        // 64-byte swizzle: 16-byte unit u of row r sits at unit u ^ ((r >> 1) & 3)
                        const int r = q >> 2;
                        const uint32_t col = si.x_begin + 4u * static_cast<uint32_t>((q & 3) ^ ((r >> 1) & 3));
                        if (col + 0 < si.mask_below) v.x = 0.f;
                        if (col + 1 < si.mask_below) v.y = 0.f;
                        if (col + 2 < si.mask_below) v.z = 0.f;
                        if (col + 3 < si.mask_below) v.w = 0.f;
                    }
                    float4 hi, lo;
                    split4(v, hi, lo);
                    a_hi[q] = hi;
                    a_lo[q] = lo;
                }
                fence_proxy_async();
                mbar_arrive(&ctrl->conv[s]);
            }
        })
        if (cid == 0) atomicAdd(&g_role_cycles[10], static_cast<unsigned long long>(w_full));
    } else if (warp < kRowWarp0) {
        // ---------------------------------------------------------------- centroid gather (warps 4 .. 7)
        // Asynchronous 16-byte copies (cp.async) from the pre-split centroid matrix straight into the stage, in the
        // swizzled layout; no registers are tied up, so the copies of up to three stages are in flight per thread.  A
        // thread copies unit c16 of the hi and of the lo part of rows r0, r0 + 32, ..., r0 + 224 (four warps: the copies
        // issue rate, ~50 cycles per warp instruction of 32 scattered 16-byte pieces, was the kernel's limit with two).
        // A stage is announced
        // to the MMA warp two stages after its copies were issued, once cp.async.wait_group says they have landed.
        const uint32_t gid = threadIdx.x - 128u;   // 0 .. kGatherThreads - 1
        const uint32_t c16 = gid & 3u;
        const uint32_t r0 = gid >> 2;              // 0 .. kGatherThreads / 4 - 1
        uint32_t* rowoff = ctrl->rowoff[0][0];
        uint32_t kbt = 0;
        bool ok = true;
        long long w_empty = 0, w_group = 0;
        const long long t_begin = clock64();
        SPARSE_FOR_EACH_UNIT_SEGMENT({
            if (seg == 0) {
                // element offsets of this thread's centroid rows; rows past the unit's last centroid repeat it (finite
                // values; their columns are never tested).  Entry r is written and read by this thread only.
#pragma unroll
                for (int i = 0; i < static_cast<int>(BN * 4 / kGatherThreads); ++i) {
                    const uint32_t r = r0 + static_cast<uint32_t>(kGatherThreads / 4) * i;
                    if (r < nmma) rowoff[a * BN + r] = (static_cast<uint32_t>(c0) + __ldg(unit_cols + min(r, nu - 1u))) * p.d;
                }
            }
            for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                // the MMAs that read this stage four k-blocks ago must be done before it is overwritten
                if (!timed_wait_relaxed(&ctrl->empty[s], ph ^ 1u, wctx, 27, w_empty)) {
                    ok = false;
                    break;
                }
                const uint32_t xc = si.x_begin + kb * BK + c16 * 4u;
                const uint32_t st = smem_base + s * STAGE_BYTES;
#pragma unroll
                for (int i = 0; i < static_cast<int>(BN * 4 / kGatherThreads); ++i) {
                    const uint32_t r = r0 + static_cast<uint32_t>(kGatherThreads / 4) * i;
                    if (r < nmma) {
                        const uint32_t off = rowoff[a * BN + r] + xc;
                        const uint32_t slot = (r * 4u + (c16 ^ ((r >> 1) & 3u))) * 16u;
                        cp_async_16(st + OFF_B_HI + slot, p.y_hi + off);
                        cp_async_16(st + OFF_B_LO + slot, p.y_lo + off);
                    }
                }
                cp_async_commit();
                if (kbt >= 2) {
                    const long long t0 = clock64();
                    cp_async_wait_group<2>();   // everything but the two newest groups: the stage of two k-blocks ago
                    w_group += clock64() - t0;
                    fence_proxy_async();
                    mbar_arrive(&ctrl->conv[(kbt - 2) % STAGES]);
                }
            }
        })
        // the last two stages
        cp_async_wait_group<0>();
        if (ok) {
            fence_proxy_async();
            if (kbt >= 2) mbar_arrive(&ctrl->conv[(kbt - 2) % STAGES]);
            if (kbt >= 1) mbar_arrive(&ctrl->conv[(kbt - 1) % STAGES]);
        }
        if (gid == 0) {
            atomicAdd(&g_role_cycles[7], static_cast<unsigned long long>(w_empty));
            atomicAdd(&g_role_cycles[8], static_cast<unsigned long long>(w_group));
            atomicAdd(&g_role_cycles[9], static_cast<unsigned long long>(clock64() - t_begin));
        }
    } else if (MERGED) {
        // (warps 8 .. 15)
        // ---------------------------------------------------------------- rows, optimistic pass
        // The chain is run once over ALL the centroids a tile can still reach, in units that ignore the 1024-centroid
        // chunks, with every threshold taken from the distance to the previous centroid.  That is exactly what the
        // chunk-by-chunk search does for a point whose `best` never changes on the way - the common case once the
        // clustering settles.  A point for which some other centroid survives every test and ends below that distance
        // would have had its `best` lowered at that centroid's chunk, and its later chunks tested more strictly: it is
        // flagged (`dirty`) and redone by the exact kernel; for all others the survivor count and the (unchanged)
        // assignment are final.  Only two checkpoints are looked at: the first (survivor count, survivor mask) and the
        // last (does a first-test survivor other than the previous centroid end below the bar).  The tests in between could
        // only take candidates away, i.e. clear a flag, and they rarely do (a candidate that ends below `best` yet fails
        // a test on the way is an ADSampling false prune); leaving them out flags a few more rows and saves the rows'
        // threads twelve of fourteen passes over the accumulator at d = 1024.
        const uint32_t half = static_cast<uint32_t>(warp - kRowWarp0) >> 2;
        const uint32_t quarter = static_cast<uint32_t>(warp) & 3u;
        const uint32_t lane_base = 32u * quarter;
        const uint32_t row_in_tile = lane_base + lane;
        uint32_t uses[2] = {0, 0};
        uint32_t xchg_uses = 0;
        bool ok = true;
        long long w_ready = 0, w_xchg = 0, t_norms = 0;
        const long long t_begin = clock64();
        size_t cur_lt = ~size_t{0};
        size_t row = 0;
        bool row_valid = false;
        float best = -1.f;
        uint32_t prev = 0xFFFFFFFFu, cnt = 0, dirty = 0;
        constexpr int HS = BN / 64;
        uint32_t alive0[HS], alive1[HS];
#pragma unroll
        for (int q = 0; q < HS; ++q) alive0[q] = alive1[q] = 0;
        float* ny = ctrl->ny[warp - kRowWarp0];
        uint32_t ncand = 0;   // competitors this thread found for its row in the current tile
        auto close_row = [&]() -> bool {
            RowPartial mine{};
            mine.cnt = cnt;
            mine.prev_first = dirty;
            mine.cbi = ncand;
            const uint32_t slot = xchg_uses & 1u;
            ctrl->xchg[slot][half][row_in_tile] = mine;
            __threadfence_block();
            mbar_arrive(&ctrl->xchg_bar);
            if (!__all_sync(0xffffffffu, timed_wait(&ctrl->xchg_bar, xchg_uses & 1u, wctx, 26, w_xchg))) return false;
            ++xchg_uses;
            if (row_valid && half == 0) {
                const RowPartial other = ctrl->xchg[slot][1][row_in_tile];
                p.not_pruned[row] = cnt + other.cnt;
                p.dirty[row] = (dirty | other.prev_first) ? 1u : 0u;
                if (p.cand_meta) {
                    const uint32_t over = (ncand > p.cand_cap || other.cbi > p.cand_cap) ? 1u : 0u;
                    p.cand_meta[row] = min(ncand, p.cand_cap) | (min(other.cbi, p.cand_cap) << 8) | (over << 16);
                }
            }
            return true;
        };
        SPARSE_FOR_EACH_UNIT_SEGMENT({
            if (lt != cur_lt) {
                if (cur_lt != ~size_t{0} && !close_row()) {
                    ok = false;
                    break;
                }
                cur_lt = lt;
                row = rt * BM + row_in_tile;
                row_valid = row < p.n;
                best = row_valid ? p.best_in[row] : -1.f;
                prev = row_valid ? p.knn[row] : 0xFFFFFFFFu;
                cnt = 0;
                dirty = 0;
                ncand = 0;
            }
            const bool first = seg == 0, last = (seg + 1 == p.n_seg);
            if (!first && !last) continue;   // no hand-over in between (see the MMA warp)
            const uint32_t hw = ((nu + 63u) >> 6) << 5;
            const uint32_t hb = half * hw;
            const uint32_t my_cols = nu > hb ? min(hw, nu - hb) : 0u;
            const uint32_t n_sl = (my_cols + 31u) >> 5;
            uint16_t* colid = ctrl->colid[warp - kRowWarp0][a];
            uint32_t cidx[HS];
            if (first) {
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) {
                    const uint32_t j = q * 32 + lane;
                    cidx[q] = j < my_cols ? static_cast<uint32_t>(__ldg(unit_cols + hb + j)) : 0u;
                    colid[j] = static_cast<uint16_t>(cidx[q]);
                }
                __syncwarp();
            } else {
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) cidx[q] = colid[q * 32 + lane];
            }
            const float thr = best * ctrl->seg_ratio[seg];
            const float nxv = row_valid ? __ldg(p.chain_norms_x + row * p.n_seg + seg) : 0.f;
            const long long t_norms0 = clock64();
            {
                const float* __restrict__ src = p.chain_norms_y + static_cast<size_t>(seg) * p.k;
                float cur[HS];
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) cur[q] = (q * 32 + lane < my_cols) ? __ldg(src + cidx[q]) : 0.f;
                __syncwarp();
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) ny[q * 32 + lane] = cur[q];
                __syncwarp();
            }
            t_norms += clock64() - t_norms0;
            if (!__all_sync(0xffffffffu, timed_wait(&ctrl->acc_ready[a], uses[a] & 1u, wctx, 25, w_ready))) {
                ok = false;
                break;
            }
            ++uses[a];
            tc_fence_after();
            const uint32_t taddr = tmem_base + (lane_base << 16) + a * BN + hb;
            uint32_t alive[HS];
#pragma unroll
            for (int q = 0; q < HS; ++q) alive[q] = a ? alive1[q] : alive0[q];
            // At the last checkpoint the question is not the test itself but "could this centroid beat the previous one":
            // distances from the tensor-memory accumulator sit too high by an amount that grows with the number of
            // accumulation steps (up to ~2e-5 of the norms at d = 1024, ~6e-5 at d = 1536), and the exact pass settles
            // such near-misses with fp32 distances of its runner-ups, so the bar is raised by that much.
            const float near_bar = last ? fmaf(best, 1e-4f, best) + (3e-8f * static_cast<float>(p.d)) * nxv : thr;
            auto test_slice = [&](const uint32_t sl, const uint32_t (&r)[32], uint32_t& alive_ch) {
                const uint32_t cb0 = sl * 32;
                uint32_t w = 0;
#pragma unroll
                for (uint32_t j = 0; j < 32; j += 4) {
                    const float4 nyv = *reinterpret_cast<const float4*>(ny + cb0 + j);
                    const float p0 = fmaf(-2.0f, __uint_as_float(r[j + 0]), nxv) + nyv.x;
                    const float p1 = fmaf(-2.0f, __uint_as_float(r[j + 1]), nxv) + nyv.y;
                    const float p2 = fmaf(-2.0f, __uint_as_float(r[j + 2]), nxv) + nyv.z;
                    const float p3 = fmaf(-2.0f, __uint_as_float(r[j + 3]), nxv) + nyv.w;
                    w |= (p0 < near_bar ? (1u << j) : 0u) | (p1 < near_bar ? (2u << j) : 0u) | (p2 < near_bar ? (4u << j) : 0u) | (p3 < near_bar ? (8u << j) : 0u);
                }
                if (first) {
                    const uint32_t lo = sl * 32;
                    const uint32_t valid = (my_cols >= lo + 32) ? 0xFFFFFFFFu : (my_cols > lo ? ((1u << (my_cols - lo)) - 1u) : 0u);
                    alive_ch = w & valid;
                    cnt += __popc(alive_ch);
                } else {
                    alive_ch &= w;
                }
                if (last) {
                    // survivors of every test that end below (or within rounding of) the distance to the previous centroid:
                    // any of them other than the previous centroid itself means `best` could have moved
                    uint32_t m = alive_ch;
                    while (m) {
                        const uint32_t j = __ffs(m) - 1;
                        m &= m - 1;
                        const uint32_t col = colid[cb0 + j];
                        if (col != prev) {
                            dirty = 1u;
                            if (p.cand && ncand < p.cand_cap) p.cand[(row * 2 + half) * p.cand_cap + ncand] = col;
                            ++ncand;
                        }
                    }
                }
            };
            uint32_t ra[32], rb[32];
            if (n_sl <= 2) {
                if (n_sl > 0) tmem_ld32_issue(taddr, ra);
                if (n_sl > 1) tmem_ld32_issue(taddr + 32, rb);
                if (n_sl > 0) tmem_ld_wait(ra);
                if (n_sl > 1) tmem_ld_wait(rb);
                tc_fence_before();
                mbar_arrive(&ctrl->acc_loaded[a]);
                if (n_sl > 0) test_slice(0, ra, alive[0]);
                if (n_sl > 1) test_slice(1, rb, alive[1]);
            } else {
                tmem_ld32_issue(taddr, ra);
                tmem_ld_wait(ra);
                bool handed_back = false;
#pragma unroll 1
                for (uint32_t ch = 0; ch < HS; ch += 2) {
                    const bool has0 = ch < n_sl, has1 = ch + 1 < n_sl, has2 = ch + 2 < n_sl;
                    if (has1) tmem_ld32_issue(taddr + (ch + 1) * 32, rb);
                    if (has0) test_slice(ch, ra, alive[0]);
                    if (has1) tmem_ld_wait(rb);
                    if (has2) {
                        tmem_ld32_issue(taddr + (ch + 2) * 32, ra);
                    } else if (!handed_back) {
                        tc_fence_before();
                        mbar_arrive(&ctrl->acc_loaded[a]);
                        handed_back = true;
                    }
                    if (has1) test_slice(ch + 1, rb, alive[1]);
                    if (has2) tmem_ld_wait(ra);
                    const uint32_t m0 = alive[0], m1 = alive[1];
#pragma unroll
                    for (int q = 0; q < HS - 2; ++q) alive[q] = alive[q + 2];
                    alive[HS - 2] = m0;
                    alive[HS - 1] = m1;
                }
            }
#pragma unroll
            for (int q = 0; q < HS; ++q) {
                if (a) alive1[q] = alive[q];
                else alive0[q] = alive[q];
            }
        })
        if (ok && cur_lt != ~size_t{0}) close_row();
        if (warp == kRowWarp0 && lane == 0) {
            atomicAdd(&g_role_cycles[3], static_cast<unsigned long long>(w_ready));
            atomicAdd(&g_role_cycles[4], static_cast<unsigned long long>(t_norms));
            atomicAdd(&g_role_cycles[5], static_cast<unsigned long long>(clock64() - t_begin));
            atomicAdd(&g_role_cycles[6], static_cast<unsigned long long>(w_xchg));
        }
    } else {
        // (warps 8 .. 15)
        // ---------------------------------------------------------------- rows: tests at every checkpoint
        const uint32_t half = static_cast<uint32_t>(warp - kRowWarp0) >> 2;   // which 128 of a unit's 256 columns
        const uint32_t quarter = static_cast<uint32_t>(warp) & 3u;
        const uint32_t lane_base = 32u * quarter;
        const uint32_t row_in_tile = lane_base + lane;
        uint32_t uses[2] = {0, 0};
        uint32_t xchg_uses = 0;
        bool ok = true;
        long long w_ready = 0, w_xchg = 0, t_norms = 0;
        const long long t_begin = clock64();
        size_t cur_lt = ~size_t{0};
        uint32_t cur_chunk = 0xFFFFFFFFu;
        size_t row = 0;
        bool row_valid = false;
        float best = -1.f, cb = FLT_MAX, t1 = FLT_MAX, t2 = FLT_MAX;
        uint32_t bestidx = 0, prev = 0xFFFFFFFFu, npc = 0, cnt = 0, cbi = 0, i1 = 0xFFFFFFFFu, i2 = 0xFFFFFFFFu;
        uint32_t o1 = 0xFFFFFFFFu, o2 = 0xFFFFFFFFu;   // merged runner-ups of the row, set at every chunk end
        bool prev_first = false;
        constexpr int HS = BN / 64;   // 32-column slices per half
        // per accumulator: survivor masks of the unit in flight and where among this half's columns the row's previous
        // centroid sits (or none)
        uint32_t alive0[HS], alive1[HS];
        uint32_t prevpos0 = 0xFFFFFFFFu, prevpos1 = 0xFFFFFFFFu;
#pragma unroll
        for (int q = 0; q < HS; ++q) alive0[q] = alive1[q] = 0;
        float* ny = ctrl->ny[warp - kRowWarp0];
        // End of a chunk: the two threads of the row exchange what they found in their halves of the columns and
        // both apply the same update.  Returns false when the wait ran out.
        auto close_chunk = [&]() -> bool {
            RowPartial mine;
            mine.cnt = cnt;
            mine.prev_first = prev_first ? 1u : 0u;
            mine.cb = cb;
            mine.cbi = cbi;
            mine.t1 = t1;
            mine.t2 = t2;
            mine.i1 = i1;
            mine.i2 = i2;
            const uint32_t slot = xchg_uses & 1u;
            ctrl->xchg[slot][half][row_in_tile] = mine;
            __threadfence_block();
            mbar_arrive(&ctrl->xchg_bar);
            if (!__all_sync(0xffffffffu, timed_wait(&ctrl->xchg_bar, xchg_uses & 1u, wctx, 26, w_xchg))) return false;
            ++xchg_uses;
            const RowPartial other = ctrl->xchg[slot][half ^ 1u][row_in_tile];
            const uint32_t cnt_all = cnt + other.cnt;
            const bool prev_all = prev_first || other.prev_first != 0u;
            float mb = cb;
            uint32_t mbi = cbi;
            if (other.cb < mb || (other.cb == mb && other.cbi < mbi)) {
                mb = other.cb;
                mbi = other.cbi;
            }
            npc += cnt_all;
            // pdxearch.h:140-143: the previous centroid as the only survivor leaves the candidate untouched
            if (mb < FLT_MAX && !(cnt_all == 1u && prev_all)) {
                best = mb;
                bestidx = mbi;
            }
            // the two smallest of both halves, for the end of the row
            if (other.t1 < t1) {
                o2 = (t1 < other.t2) ? i1 : other.i2;
                o1 = other.i1;
            } else {
                o1 = i1;
                o2 = (other.t1 < t2) ? other.i1 : i2;
            }
            cnt = 0;
            prev_first = false;
            cb = FLT_MAX;
            cbi = 0;
            return true;
        };
        auto close_row = [&]() {
            if (row_valid && half == 0) {
                p.knn[row] = bestidx;
                p.dist[row] = best;
                p.not_pruned[row] = npc;
                p.top2[row] = make_uint2(o1, o2);
            }
        };
        SPARSE_FOR_EACH_UNIT_SEGMENT({
            if (lt != cur_lt) {
                if (cur_lt != ~size_t{0}) {
                    if (!close_chunk()) {
                        ok = false;
                        break;
                    }
                    close_row();
                }
                cur_lt = lt;
                cur_chunk = chunk;
                row = rt * BM + row_in_tile;
                row_valid = row < p.n;
                best = row_valid ? p.best_in[row] : -1.f;
                prev = row_valid ? p.knn[row] : 0xFFFFFFFFu;
                bestidx = row_valid ? prev : 0u;
                npc = 0;
                cnt = 0;
                prev_first = false;
                cb = FLT_MAX;
                cbi = 0;
                t1 = t2 = FLT_MAX;
                i1 = i2 = 0xFFFFFFFFu;
                o1 = o2 = 0xFFFFFFFFu;
            } else if (chunk != cur_chunk) {
                if (!close_chunk()) {
                    ok = false;
                    break;
                }
                cur_chunk = chunk;
            }
            const bool first = seg == 0, last = (seg + 1 == p.n_seg);
            // The unit's columns are shared between the two threads of a row: the first hw columns (a multiple of 32) and
            // the rest.  my_cols: how many belong to this thread, n_sl: the 32-column slices they fill.
            const uint32_t hw = ((nu + 63u) >> 6) << 5;
            const uint32_t hb = half * hw;   // first column of this thread's share
            const uint32_t my_cols = nu > hb ? min(hw, nu - hb) : 0u;
            const uint32_t n_sl = (my_cols + 31u) >> 5;
            uint16_t* colid = ctrl->colid[warp - kRowWarp0][a];
            uint32_t cidx[HS];
            uint32_t prevpos;
            if (first) {
                // Local centroid indices of this warp's share of the unit's columns, into the warp's own table: read back per
                // lane for the norm gathers of every segment, and per column when a survivor needs its centroid.
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) {
                    const uint32_t j = q * 32 + lane;
                    cidx[q] = j < my_cols ? static_cast<uint32_t>(__ldg(unit_cols + hb + j)) : 0u;
                    colid[j] = static_cast<uint16_t>(cidx[q]);
                }
                __syncwarp();
                // where the row's previous centroid sits among this half's columns (ascending indices: binary search)
                prevpos = 0xFFFFFFFFu;
                if (prev >= c0 && prev < c0 + kChunk && my_cols != 0) {
                    const uint32_t want = prev - static_cast<uint32_t>(c0);
                    uint32_t lo = 0, hi = my_cols;
                    while (lo < hi) {
                        const uint32_t mid = (lo + hi) >> 1;
                        if (colid[mid] < want) lo = mid + 1;
                        else hi = mid;
                    }
                    if (lo < my_cols && colid[lo] == want) prevpos = lo;
                }
                if (a) prevpos1 = prevpos;
                else prevpos0 = prevpos;
            } else {
                // this lane's columns (q * 32 + lane of this half), from the copy the first segment left
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) cidx[q] = colid[q * 32 + lane];
                prevpos = a ? prevpos1 : prevpos0;
            }
            const float thr = best * ctrl->seg_ratio[seg];
            const float nxv = row_valid ? __ldg(p.chain_norms_x + row * p.n_seg + seg) : 0.f;
            // centroid norms of this warp's share of the unit's columns at this checkpoint
            const long long t_norms0 = clock64();
            {
                const float* __restrict__ src = p.chain_norms_y + static_cast<size_t>(seg) * p.k + c0;
                float cur[HS];
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) cur[q] = (q * 32 + lane < my_cols) ? __ldg(src + cidx[q]) : 0.f;
                __syncwarp();
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) ny[q * 32 + lane] = cur[q];
                __syncwarp();
            }
            t_norms += clock64() - t_norms0;
            if (!__all_sync(0xffffffffu, timed_wait(&ctrl->acc_ready[a], uses[a] & 1u, wctx, 25, w_ready))) {
                ok = false;
                break;
            }
            ++uses[a];
            tc_fence_after();
            const uint32_t taddr = tmem_base + (lane_base << 16) + a * BN + hb;
            uint32_t alive[HS];
#pragma unroll
            for (int q = 0; q < HS; ++q) alive[q] = a ? alive1[q] : alive0[q];
            // One 32-column slice (slice `sl` of this half) is tested while the next one is on its way from tensor memory.
            auto test_slice = [&](const uint32_t sl, uint32_t (&r)[32], uint32_t& alive_ch) {
                const uint32_t cb0 = sl * 32;   // first column of the slice inside this thread's share of the unit
                // bit j of w = (partial distance of column cb0 + j < threshold), branch-free
                uint32_t w = 0;
#pragma unroll
                for (uint32_t j = 0; j < 32; j += 4) {
                    const float4 nyv = *reinterpret_cast<const float4*>(ny + cb0 + j);
                    const float p0 = fmaf(-2.0f, __uint_as_float(r[j + 0]), nxv) + nyv.x;
                    const float p1 = fmaf(-2.0f, __uint_as_float(r[j + 1]), nxv) + nyv.y;
                    const float p2 = fmaf(-2.0f, __uint_as_float(r[j + 2]), nxv) + nyv.z;
                    const float p3 = fmaf(-2.0f, __uint_as_float(r[j + 3]), nxv) + nyv.w;
                    w |= (p0 < thr ? (1u << j) : 0u) | (p1 < thr ? (2u << j) : 0u) | (p2 < thr ? (4u << j) : 0u) | (p3 < thr ? (8u << j) : 0u);
                    r[j + 0] = __float_as_uint(p0);
                    r[j + 1] = __float_as_uint(p1);
                    r[j + 2] = __float_as_uint(p2);
                    r[j + 3] = __float_as_uint(p3);
                }
                if (first) {
                    const uint32_t lo = sl * 32;
                    const uint32_t valid = (my_cols >= lo + 32) ? 0xFFFFFFFFu : (my_cols > lo ? ((1u << (my_cols - lo)) - 1u) : 0u);
                    const uint32_t al = w & valid;
                    alive_ch = al;
                    cnt += __popc(al);
                    if (prevpos >= lo && prevpos < lo + 32) {
                        if ((al >> (prevpos & 31u)) & 1u) prev_first = true;
                    }
                }
                if (!first && !last) alive_ch &= w;
                if (last) {
                    // Last checkpoint: the pairs still alive compete.  thr == best here (ratio[d] == 1).  With a
                    // single segment (first and last at once) alive_ch has just been set above.
                    uint32_t m = alive_ch;
                    if (m) {
                        float pdv[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) pdv[j] = __uint_as_float(r[j]);
                        while (m) {
                            const uint32_t j = __ffs(m) - 1;
                            m &= m - 1;
                            const float pd = pdv[j];
                            const uint32_t gc = static_cast<uint32_t>(c0) + colid[cb0 + j];
                            if (pd < t2) {
                                // runner-ups by the chain's own (slightly truncated) distances; the fp32
                                // refinement afterwards decides among them and the chain's winner
                                if (pd < t1) {
                                    t2 = t1;
                                    i2 = i1;
                                    t1 = pd;
                                    i1 = gc;
                                } else {
                                    t2 = pd;
                                    i2 = gc;
                                }
                            }
                            if (pd < thr && pd < cb) {
                                cb = pd;
                                cbi = gc;
                            }
                        }
                    }
                }
            };
            uint32_t ra[32], rb[32];
            if (n_sl <= 2) {
                // At most two slices: both fit in registers, so the accumulator goes back to the MMA warp before any test.
                if (n_sl > 0) tmem_ld32_issue(taddr, ra);
                if (n_sl > 1) tmem_ld32_issue(taddr + 32, rb);
                if (n_sl > 0) tmem_ld_wait(ra);
                if (n_sl > 1) tmem_ld_wait(rb);
                tc_fence_before();
                mbar_arrive(&ctrl->acc_loaded[a]);
                if (n_sl > 0) test_slice(0, ra, alive[0]);
                if (n_sl > 1) test_slice(1, rb, alive[1]);
            } else {
                tmem_ld32_issue(taddr, ra);
                tmem_ld_wait(ra);
                // Two slices per trip, always HS / 2 trips so that the survivor masks, which rotate through alive[0] and
                // alive[1] to stay in registers, are back in place afterwards; slices beyond the unit's columns are skipped.
                // The accumulator is handed back as soon as this thread's last slice is in registers.
                bool handed_back = false;
#pragma unroll 1
                for (uint32_t ch = 0; ch < HS; ch += 2) {
                    const bool has0 = ch < n_sl, has1 = ch + 1 < n_sl, has2 = ch + 2 < n_sl;
                    if (has1) tmem_ld32_issue(taddr + (ch + 1) * 32, rb);
                    if (has0) test_slice(ch, ra, alive[0]);
                    if (has1) tmem_ld_wait(rb);
                    if (has2) {
                        tmem_ld32_issue(taddr + (ch + 2) * 32, ra);
                    } else if (!handed_back) {
                        // everything of this checkpoint is in registers: the accumulator may grow again
                        tc_fence_before();
                        mbar_arrive(&ctrl->acc_loaded[a]);
                        handed_back = true;
                    }
                    if (has1) test_slice(ch + 1, rb, alive[1]);
                    if (has2) tmem_ld_wait(ra);
                    const uint32_t m0 = alive[0], m1 = alive[1];
#pragma unroll
                    for (int q = 0; q < HS - 2; ++q) alive[q] = alive[q + 2];
                    alive[HS - 2] = m0;
                    alive[HS - 1] = m1;
                }
            }
#pragma unroll
            for (int q = 0; q < HS; ++q) {
                if (a) alive1[q] = alive[q];
                else alive0[q] = alive[q];
            }
        })
        if (ok && cur_lt != ~size_t{0}) {
            if (close_chunk()) close_row();
        }
        if (warp == kRowWarp0 && lane == 0) {
            atomicAdd(&g_role_cycles[3], static_cast<unsigned long long>(w_ready));
            atomicAdd(&g_role_cycles[4], static_cast<unsigned long long>(t_norms));
            atomicAdd(&g_role_cycles[5], static_cast<unsigned long long>(clock64() - t_begin));
            atomicAdd(&g_role_cycles[6], static_cast<unsigned long long>(w_xchg));
        }
    }
#undef SPARSE_FOR_EACH_UNIT_SEGMENT

    cp_async_wait_group<0>();   // no copy may still be on its way into shared memory when the CTA ends
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// One warp per (tile, chunk): the set bits of the chunk's 1024 union bits as ascending local indices.
__global__ void __launch_bounds__(256) build_cols_kernel(const uint32_t* __restrict__ union_bits, uint32_t union_words, size_t n_tiles, uint32_t n_chunks, size_t k,
                                                         uint16_t* __restrict__ cols, uint32_t* __restrict__ col_counts, size_t cols_stride,
                                                         unsigned long long* __restrict__ total_cols) {
    const size_t wid = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wid >= n_tiles * n_chunks) return;
    const size_t t = wid / n_chunks;
    const uint32_t chunk = static_cast<uint32_t>(wid % n_chunks);
    const uint32_t word = chunk * 32u + lane;   // 32 words of 32 bits per chunk
    uint32_t bits = word < union_words ? union_bits[t * union_words + word] : 0u;
    // bits past the last centroid cannot be set (the union pass masks them); keep that explicit
    const size_t first = static_cast<size_t>(word) * 32;
    if (first + 32 > k) bits &= first >= k ? 0u : ((1u << (k - first)) - 1u);
    const uint32_t c = __popc(bits);
    uint32_t incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
    }
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    uint16_t* out = cols + t * cols_stride + static_cast<size_t>(chunk) * kChunk + (incl - c);
    uint32_t m = bits;
    while (m) {
        const uint32_t b = __ffs(m) - 1;
        m &= m - 1;
        *out++ = static_cast<uint16_t>(lane * 32 + b);
    }
    if (lane == 0) {
        col_counts[t * n_chunks + chunk] = total;
        if (total_cols && total) {
            // columns as the tensor cores see them: the chunk's units (cut as in sparse_chain_kernel), each rounded up to 16
            const uint32_t n_units = total <= 16u ? 1u : max(2u, (total + BN - 1) / BN);
            const uint32_t unit_w = (((total + n_units - 1) / n_units) + 15u) & ~15u;
            unsigned long long cols16 = 0;
            for (uint32_t u = 0; u * unit_w < total; ++u) cols16 += (min(unit_w, total - u * unit_w) + 15u) & ~15u;
            atomicAdd(total_cols, cols16);
        }
    }
}

} // namespace

// Reads and clears the role cycle counters of the current device: [0] MMA thread waiting for the rows to hand an
// accumulator back, [1] waiting for a stage, [2] its whole loop; [3] a row warp waiting for an accumulator, [4] fetching
// centroid norms, [5] its whole loop, [6] waiting for its partner at chunk ends; [7] a gather thread waiting for a free
// stage, [8] for its copies, [9] its whole loop; [10] an X splitter waiting for its tile; [11] the producer waiting for a
// free stage; [12] (unit, segment) steps; [13] CTAs.
void role_cycles(unsigned long long out[16]) {
    SKM_CUDA(cudaMemcpyFromSymbol(out, g_role_cycles, sizeof(unsigned long long) * 16));
    unsigned long long zero[16] = {};
    SKM_CUDA(cudaMemcpyToSymbol(g_role_cycles, zero, sizeof(zero)));
}

void launch_build_cols(const uint32_t* union_bits, uint32_t union_words, size_t n_tiles, size_t k, uint16_t* cols, uint32_t* col_counts, size_t cols_stride,
                       unsigned long long* total_cols, cudaStream_t stream) {
    if (n_tiles == 0 || k == 0) return;
    const uint32_t n_chunks = static_cast<uint32_t>((k + kChunk - 1) / kChunk);
    const size_t warps = n_tiles * n_chunks;
    build_cols_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(union_bits, union_words, n_tiles, n_chunks, k, cols, col_counts, cols_stride, total_cols);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_sparse_chain(const float* x, size_t n, size_t k, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, const float* chain_norms_x,
                         const float* chain_norms_y, const float* ratios, const float* best_in, uint32_t* knn, float* dist, uint32_t* not_pruned, uint2* top2_scratch,
                         const float* y_split, const uint32_t* tile_map, size_t n_tiles, const uint16_t* cols, const uint32_t* col_counts, size_t cols_stride,
                         cudaStream_t stream, uint32_t* dirty, uint32_t* cand, uint32_t* cand_meta, uint32_t cand_cap) {
    if (n_tiles == 0 || n == 0 || k == 0) return;
    if (k * d >= (size_t{1} << 32)) throw std::invalid_argument("centroid matrix too large for the gathered chain (k * d must stay below 2^32)");
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    SparseMaps maps;
    const size_t extents[3] = {partial_d, vertical_d, d};
    for (int i = 0; i < 3; ++i) maps.x[i] = make_row_major_tmap(x, extents[i], n, d, BM);
    SparseParams p{};
    p.n = n;
    p.k = k;
    p.d = static_cast<uint32_t>(d);
    p.partial_d = partial_d;
    p.vertical_d = vertical_d;
    p.horizontal_d = horizontal_d;
    p.n_seg = 1u + horizontal_d / 64u + (partial_d < vertical_d ? 1u : 0u);
    if (p.n_seg > SPARSE_MAX_SEGMENTS) throw std::invalid_argument("dimensionality too large for the tensor-core chain");
    p.n_chunks = static_cast<uint32_t>((k + kChunk - 1) / kChunk);
    p.chain_norms_x = chain_norms_x;
    p.chain_norms_y = chain_norms_y;
    p.ratios = ratios;
    p.best_in = best_in;
    p.knn = knn;
    p.dist = dist;
    p.not_pruned = not_pruned;
    p.top2 = top2_scratch;
    p.y_hi = y_split;
    p.y_lo = y_split + k * d;
    p.tile_map = tile_map;
    p.n_tiles = n_tiles;
    p.cols = cols;
    p.col_counts = col_counts;
    p.cols_stride = cols_stride;
    p.error = error_word();
    p.wait_limit = wait_limit();
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int grid = static_cast<int>(std::min<size_t>(n_tiles, static_cast<size_t>(sms)));
    if (dirty) {
        // optimistic pass: one list per tile, global indices
        if (k > 65536) throw std::invalid_argument("the optimistic chain pass indexes centroids with 16 bits (k <= 65536)");
        p.n_chunks = 1;
        p.dirty = dirty;
        p.cand = cand;
        p.cand_meta = cand_meta;
        p.cand_cap = cand_cap;
        SKM_CUDA(cudaFuncSetAttribute(sparse_chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S_SMEM_BYTES)));
        sparse_chain_kernel<true><<<grid, SPARSE_THREADS, S_SMEM_BYTES, stream>>>(maps, p);
    } else {
        SKM_CUDA(cudaFuncSetAttribute(sparse_chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S_SMEM_BYTES)));
        sparse_chain_kernel<false><<<grid, SPARSE_THREADS, S_SMEM_BYTES, stream>>>(maps, p);
    }
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

// One warp per tile: all set bits of the tile's union words as ascending global centroid indices, and their number.
__global__ void __launch_bounds__(256) build_flat_cols_kernel(const uint32_t* __restrict__ union_bits, uint32_t union_words, size_t n_tiles, size_t k,
                                                              uint16_t* __restrict__ cols, uint32_t* __restrict__ totals, size_t cols_stride,
                                                              unsigned long long* __restrict__ total_cols) {
    const size_t t = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= n_tiles) return;
    uint32_t base = 0;
    uint16_t* out_tile = cols + t * cols_stride;
    for (uint32_t w0 = 0; w0 < union_words; w0 += 32) {
        const uint32_t word = w0 + lane;
        uint32_t bits = word < union_words ? union_bits[t * union_words + word] : 0u;
        const size_t first = static_cast<size_t>(word) * 32;
        if (first + 32 > k) bits &= first >= k ? 0u : ((1u << (k - first)) - 1u);
        const uint32_t c = __popc(bits);
        uint32_t incl = c;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        uint16_t* out = out_tile + base + (incl - c);
        uint32_t m = bits;
        while (m) {
            const uint32_t b = __ffs(m) - 1;
            m &= m - 1;
            *out++ = static_cast<uint16_t>(first + b);
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
        totals[t] = base;
        if (total_cols && base) {
            const uint32_t n_units = base <= 16u ? 1u : max(2u, (base + BN - 1) / BN);
            const uint32_t unit_w = (((base + n_units - 1) / n_units) + 15u) & ~15u;
            unsigned long long cols16 = 0;
            for (uint32_t u = 0; u * unit_w < base; ++u) cols16 += (min(unit_w, base - u * unit_w) + 15u) & ~15u;
            atomicAdd(total_cols, cols16);
        }
    }
}

void launch_build_flat_cols(const uint32_t* union_bits, uint32_t union_words, size_t n_tiles, size_t k, uint16_t* cols, uint32_t* totals, size_t cols_stride,
                            unsigned long long* total_cols, cudaStream_t stream) {
    if (n_tiles == 0 || k == 0) return;
    build_flat_cols_kernel<<<static_cast<unsigned>((n_tiles + 7) / 8), 256, 0, stream>>>(union_bits, union_words, n_tiles, k, cols, totals, cols_stride, total_cols);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

} // namespace tc
} // namespace skmb
