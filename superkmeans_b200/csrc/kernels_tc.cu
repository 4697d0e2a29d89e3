// Tensor-core (tcgen05) kernels for sm_100a: X * Y^T with fp32 operands and fp32-level accuracy.
//
// Every fp32 operand value v is split into hi = tf32(v) and lo = tf32(v - hi); the product is accumulated as
// hi*hi + hi*lo + lo*hi (three kind::tf32 MMAs per k-step, fp32 accumulation in tensor memory), which restores
// fp32-level accuracy of the products.  The points (X) are split in shared memory by splitter warps; the
// centroids (Y), which every CTA re-reads, can arrive already split from global memory (split_tf32_kernel).
//
// gemm_tc_kernel: one persistent CTA per SM, 448 threads:
//   warp 0       TMA producer: cp.async.bulk.tensor loads of a 128 x 16 tile of X and a 256 x 16 tile of Y
//                (hi and lo when pre-split; 64-byte swizzle) into a 4-stage ring;
//   warp 1       MMA issuer: tcgen05.mma (M = 128, N = 256, K = 8) into one of two 256-column accumulators in
//                tensor memory, tcgen05.commit to release stages / publish tiles;
//   warps 2-5    splitters: rewrite each landed X (and raw Y) tile in place as its hi part and write the lo part
//                beside it (element-wise, so the swizzle pattern never has to be decoded);
//   warps 6-9    epilogue: tcgen05.ld, one thread per row.  Three epilogues: the two smallest
//                ||x||^2 + ||y||^2 - 2 x.y per row (exact assignment), a plain store, and the first ADSampling
//                test with survivor lists;
//   warps 10-13  second half of the epilogue warps in the first-test mode (idle otherwise).
// chain_tc_kernel (320 threads, same roles) grows its accumulators segment by segment and tests after each.
// Rows / columns / k beyond the matrix edges are zero-filled by TMA, so any n, k and K work as long as the row
// pitch is a multiple of 16 bytes.
//
// Every wait on an mbarrier is bounded: on expiry the kernel records an error code, all roles leave their loops,
// tensor memory is released and the kernel returns.
#include <cuda.h>

#include <cfloat>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <stdexcept>

#include "common.cuh"
#include "kernels_tc.cuh"
#include "tc_ptx.cuh"

namespace skmb {
namespace tc {

struct Params {
    size_t n;         // rows of X
    size_t k;         // rows of Y
    uint32_t kdim;    // reduction length
    // arg-min epilogue
    const float* norms_x;
    const float* norms_y;
    uint32_t* out_knn;
    float* out_dist;
    uint2* out_top2;  // per row: the two best candidate indices found by the tensor-core pass
    // store epilogue
    float* out;
    size_t ldo;
    int* error;
    long long wait_limit;   // SM cycles after which a wait gives up
    // first-test epilogue (MODE_PRUNE): rows [tile0 * 128, (tile0 + n_tiles) * 128) are processed; norms_x / norms_y
    // hold the norms over the first kdim dimensions
    size_t tile0;
    size_t n_tiles;        // 0 = all row tiles (other modes)
    const float* best_in;  // n: exact distance to the previous centroid
    const uint32_t* skip;  // n or null: 1 = row handled elsewhere
    float ratio_first;     // ratios[kdim]
    // eight lists per row tile: list (h * 4 + q) holds the pairs of rows 32q..32q+31 with the centroids of columns
    // 128h..128h+127 of every 256-column tile; entries {centroid << 5 | row in the 32-row group, partial distance}
    uint2* lists;
    uint32_t* list_offs;   // per list: (n_chunks + 1) entry counts at the start of every 1024-centroid chunk
    uint32_t cap_group;    // capacity of one list
    // first-test and union modes: when set, entry t of the launch's tile range works on row tile tile_map[t]
    // (rows tile_map[t] * 128 ...) instead of row tile tile0 + t; lists and union words stay indexed by t
    const uint32_t* tile_map;
    // union epilogue (MODE_UNION): bit c of union_bits[t * union_words + c / 32] is set when at least one row of the
    // tile passes the (slightly widened) first test against centroid c
    uint32_t* union_bits;
    uint32_t union_words;
    // counting epilogue (MODE_COUNT): count_out[row] += number of centroids whose partial distance over the first kdim
    // dimensions is below thr_rows[row * thr_chunks + chunk of 1024 the centroid lies in]
    const float* thr_rows;
    uint32_t thr_chunks;
    uint32_t* count_out;
    // Y arrives already split: tmap_y covers the hi parts, tmap_ylo the lo parts, and the splitter warps
    // only treat X
    bool y_presplit;
    // test hook: when non-zero the producer stops after this many k-blocks, so that the roles behind it wait for
    // data that never arrives, run into the wait limit and the kernel returns with an error code
    uint32_t debug_producer_stop;
};

enum { MODE_ARGMIN = 0, MODE_STORE = 1, MODE_PRUNE = 2, MODE_UNION = 3, MODE_COUNT = 4 };
constexpr float kUnionSlack = 1.0f / 512.0f;   // see the union epilogue

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                                                                 const __grid_constant__ CUtensorMap tmap_ylo, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * STAGE_BYTES);
    const WaitCtx wctx{p.error, p.wait_limit};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctrl->full[s], 1);
            mbar_init(&ctrl->conv[s], 128);
            mbar_init(&ctrl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctrl->tmem_full[b], 1);
            mbar_init(&ctrl->tmem_empty[b], (MODE == MODE_PRUNE || MODE == MODE_UNION || MODE == MODE_COUNT) ? 256 : 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    constexpr bool kTiled = (MODE == MODE_PRUNE || MODE == MODE_UNION || MODE == MODE_COUNT);   // works on a given range / list of row tiles
    const size_t rt_begin = kTiled ? p.tile0 : 0;
    const size_t n_row_tiles = kTiled ? p.tile0 + p.n_tiles : (p.n + BM - 1) / BM;
    // row tile that entry rt of the loops below stands for
    auto tile_of = [&](size_t rt) -> size_t { return (kTiled && p.tile_map) ? static_cast<size_t>(__ldg(p.tile_map + (rt - rt_begin))) : rt; };
    const uint32_t n_col_tiles = static_cast<uint32_t>((p.k + BN - 1) / BN);
    const uint32_t nkb = (p.kdim + BK - 1) / BK;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t kbt = 0;
            bool ok = true;
            for (size_t rt = rt_begin + blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
                const size_t x_row = tile_of(rt) * BM;
                for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt) {
                    for (uint32_t kb = 0; kb < nkb; ++kb, ++kbt) {
                        const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                        if (p.debug_producer_stop != 0 && kbt >= p.debug_producer_stop) {
                            ok = false;
                            break;
                        }
                        if (!mbar_wait(&ctrl->empty[s], ph ^ 1u, wctx, 1)) {
                            ok = false;
                            break;
                        }
                        // (the union pass multiplies hi parts only and never loads the lo parts of Y)
                        const bool load_ylo = p.y_presplit && MODE != MODE_UNION;
                        mbar_arrive_expect_tx(&ctrl->full[s], A_TILE_BYTES + (load_ylo ? 2 * B_TILE_BYTES : B_TILE_BYTES));
                        const uint32_t st = smem_base + s * STAGE_BYTES;
                        tma_load_2d(st + OFF_A_HI, &tmap_x, &ctrl->full[s], static_cast<int>(kb * BK), static_cast<int>(x_row));
                        tma_load_2d(st + OFF_B_HI, &tmap_y, &ctrl->full[s], static_cast<int>(kb * BK), static_cast<int>(nt * BN));
                        if (load_ylo) tma_load_2d(st + OFF_B_LO, &tmap_ylo, &ctrl->full[s], static_cast<int>(kb * BK), static_cast<int>(nt * BN));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t kbt = 0, t = 0;
            bool ok = true;
            for (size_t rt = rt_begin + blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
                for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt, ++t) {
                    const uint32_t b = t & 1u, tph = (t >> 1) & 1u;
                    if (!mbar_wait(&ctrl->tmem_empty[b], tph ^ 1u, wctx, 2)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t acc = tmem_base + b * BN;
                    for (uint32_t kb = 0; kb < nkb; ++kb, ++kbt) {
                        const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                        if (!mbar_wait(&ctrl->conv[s], ph, wctx, 3)) {
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
                            umma_tf32(acc, a_hi, b_hi, (kb | kk) != 0 ? 1u : 0u);
                            if (MODE != MODE_UNION) {
                                umma_tf32(acc, a_hi, b_lo, 1u);
                                umma_tf32(acc, a_lo, b_hi, 1u);
                            }
                        }
                        umma_commit(&ctrl->empty[s]);
                    }
                    if (ok) umma_commit(&ctrl->tmem_full[b]);
                }
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- hi / lo splitters
        const int cid = threadIdx.x - 64;
        uint32_t kbt = 0;
        bool ok = true;
        for (size_t rt = rt_begin + blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
            for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt) {
                for (uint32_t kb = 0; kb < nkb; ++kb, ++kbt) {
                    const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                    if (!mbar_wait(&ctrl->full[s], ph, wctx, 4)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = smem + s * STAGE_BYTES;
                    float4* a_hi = reinterpret_cast<float4*>(st + OFF_A_HI);
                    float4* a_lo = reinterpret_cast<float4*>(st + OFF_A_LO);
                    float4* b_hi = reinterpret_cast<float4*>(st + OFF_B_HI);
                    float4* b_lo = reinterpret_cast<float4*>(st + OFF_B_LO);
#pragma unroll
                    for (int i = 0; i < static_cast<int>(A_TILE_BYTES / 16 / 128); ++i) {
                        float4 hi, lo;
                        split4(a_hi[cid + 128 * i], hi, lo);
                        a_hi[cid + 128 * i] = hi;
                        a_lo[cid + 128 * i] = lo;
                    }
                    if (!p.y_presplit) {
#pragma unroll
                        for (int i = 0; i < static_cast<int>(B_TILE_BYTES / 16 / 128); ++i) {
                            float4 hi, lo;
                            split4(b_hi[cid + 128 * i], hi, lo);
                            b_hi[cid + 128 * i] = hi;
                            b_lo[cid + 128 * i] = lo;
                        }
                    }
                    fence_proxy_async();
                    mbar_arrive(&ctrl->conv[s]);
                }
            }
        }
    } else if (warp < 10 || kTiled) {
        // ---------------------------------------------------------------- epilogue
        // First-test mode: eight warps, two per quarter of the tile's rows; warps 6-9 take columns 0-127 of
        // every 256-column tile, warps 10-13 columns 128-255, each with a candidate list of its own.
        const uint32_t half = kTiled ? static_cast<uint32_t>(warp - 6) >> 2 : 0u;
        const uint32_t lane_base = 32u * (warp & 3);    // tensor-memory lanes this warp may read
        const uint32_t row_in_tile = lane_base + lane;
        uint32_t t = 0;
        bool ok = true;
        for (size_t rt = rt_begin + blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
            const size_t row = tile_of(rt) * BM + row_in_tile;
            const bool row_valid = row < p.n;
            // Best and runner-up of the tensor-core distances.  They are only candidates: the accumulator
            // in tensor memory truncates, which biases long sums by up to ~1e-5 relative, so the winner and
            // its distance are settled afterwards in fp32 by refine_top2_kernel.
            float nx = 0.f, d1 = FLT_MAX, d2 = FLT_MAX;
            uint32_t i1 = 0, i2 = 0xFFFFFFFFu;
            if ((MODE == MODE_ARGMIN || kTiled) && row_valid) nx = p.norms_x[row];
            // first-test epilogue: this warp's 32 rows share one candidate list; `filled` is warp-uniform
            float thr = -FLT_MAX;
            uint32_t filled = 0;
            uint2* my_list = nullptr;
            uint32_t* my_offs = nullptr;
            if (MODE == MODE_PRUNE) {
                const size_t group = (rt - rt_begin) * 8 + half * 4 + (warp & 3);
                my_list = p.lists + group * p.cap_group;
                my_offs = p.list_offs + group * ((p.k + 1023) / 1024 + 1);
                if (row_valid && !(p.skip && p.skip[row])) thr = p.best_in[row] * p.ratio_first;
            }
            uint32_t* my_union = nullptr;
            if (MODE == MODE_UNION) {
                my_union = p.union_bits + (rt - rt_begin) * static_cast<size_t>(p.union_words);
                // The union must contain every pair that the chain kernel's own first test will pass.  This pass multiplies
                // the tf32 hi parts only (one product instead of three): x.c is then off by at most 2^-10 |x| |c|, the
                // partial distance by at most 2^-10 (|x|^2 + |c|^2).  The test is widened by twice that (kUnionSlack; the
                // |c|^2 share is folded into the centroid norms below), plus a little for norms summed in another order.
                if (row_valid && !(p.skip && p.skip[row])) {
                    const float t0 = p.best_in[row] * p.ratio_first;
                    thr = fmaf(t0, 1e-4f, t0) + (kUnionSlack + 1e-6f) * nx;
                }
            }
            uint32_t counted = 0;   // MODE_COUNT
            for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt, ++t) {
                const uint32_t b = t & 1u, tph = (t >> 1) & 1u;
                const size_t col0 = static_cast<size_t>(nt) * BN;
                float* ny = ctrl->ny[warp & 3][b];
                if (MODE == MODE_PRUNE && (nt & 3u) == 0 && lane == 0) my_offs[nt >> 2] = filled;
                if (MODE == MODE_COUNT && (nt & 3u) == 0) thr = row_valid ? __ldg(p.thr_rows + row * p.thr_chunks + (nt >> 2)) : -FLT_MAX;
                if (MODE == MODE_ARGMIN) {
                    // each warp keeps its own copy, so no cross-warp barrier is needed
                    for (int j = lane; j < BN; j += 32) ny[j] = (col0 + j < p.k) ? __ldg(p.norms_y + col0 + j) : 0.f;
                    __syncwarp();
                }
                if (kTiled) {
                    // the two warps of a row quarter fill (and read) disjoint halves of the shared copy
                    const float ny_scale = MODE == MODE_UNION ? 1.0f - kUnionSlack : 1.0f;
                    for (int j = half * (BN / 2) + lane; j < static_cast<int>((half + 1) * (BN / 2)); j += 32) ny[j] = (col0 + j < p.k) ? ny_scale * __ldg(p.norms_y + col0 + j) : 0.f;
                    __syncwarp();
                }
                // warp-uniform outcome: the tensor-memory loads below must be executed by the whole warp
                if (!__all_sync(0xffffffffu, mbar_wait(&ctrl->tmem_full[b], tph, wctx, 5))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (lane_base << 16) + b * BN;
                const int ch_begin = kTiled ? static_cast<int>(half) * (BN / 64) : 0;
                const int ch_end = kTiled ? ch_begin + BN / 64 : BN / 32;
#pragma unroll 1
                for (int ch = ch_begin; ch < ch_end; ++ch) {
                    uint32_t r[32];
                    tmem_ld32(taddr + ch * 32, r);
                    if (MODE == MODE_ARGMIN) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const size_t c = col0 + ch * 32 + j;
                            if (c < p.k) {
                                const float dist = fmaf(-2.0f, __uint_as_float(r[j]), nx) + ny[ch * 32 + j];
                                if (dist < d2) {
                                    if (dist < d1) {
                                        d2 = d1;
                                        i2 = i1;
                                        d1 = dist;
                                        i1 = static_cast<uint32_t>(c);
                                    } else {
                                        d2 = dist;
                                        i2 = static_cast<uint32_t>(c);
                                    }
                                }
                            }
                        }
                    } else if (MODE == MODE_UNION) {
                        // first test for 32 centroids; only which centroids pass for ANY row of the tile is kept
                        uint32_t mask = 0;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 nyv = *reinterpret_cast<const float4*>(ny + ch * 32 + j);
                            const float p0 = fmaf(-2.0f, __uint_as_float(r[j + 0]), nx) + nyv.x;
                            const float p1 = fmaf(-2.0f, __uint_as_float(r[j + 1]), nx) + nyv.y;
                            const float p2 = fmaf(-2.0f, __uint_as_float(r[j + 2]), nx) + nyv.z;
                            const float p3 = fmaf(-2.0f, __uint_as_float(r[j + 3]), nx) + nyv.w;
                            mask |= (p0 < thr ? (1u << j) : 0u) | (p1 < thr ? (2u << j) : 0u) | (p2 < thr ? (4u << j) : 0u) | (p3 < thr ? (8u << j) : 0u);
                        }
                        const size_t first = col0 + static_cast<size_t>(ch) * 32;
                        const uint32_t n_valid = first >= p.k ? 0u : static_cast<uint32_t>(min(static_cast<size_t>(32), p.k - first));
                        mask &= n_valid >= 32u ? 0xFFFFFFFFu : ((1u << n_valid) - 1u);
                        const uint32_t any = __reduce_or_sync(0xffffffffu, mask);
                        if (any != 0 && lane == 0) atomicOr(my_union + (first >> 5), any);
                    } else if (MODE == MODE_COUNT) {
                        uint32_t mask = 0;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 nyv = *reinterpret_cast<const float4*>(ny + ch * 32 + j);
                            const float p0 = fmaf(-2.0f, __uint_as_float(r[j + 0]), nx) + nyv.x;
                            const float p1 = fmaf(-2.0f, __uint_as_float(r[j + 1]), nx) + nyv.y;
                            const float p2 = fmaf(-2.0f, __uint_as_float(r[j + 2]), nx) + nyv.z;
                            const float p3 = fmaf(-2.0f, __uint_as_float(r[j + 3]), nx) + nyv.w;
                            mask |= (p0 < thr ? (1u << j) : 0u) | (p1 < thr ? (2u << j) : 0u) | (p2 < thr ? (4u << j) : 0u) | (p3 < thr ? (8u << j) : 0u);
                        }
                        const size_t first = col0 + static_cast<size_t>(ch) * 32;
                        const uint32_t n_valid = first >= p.k ? 0u : static_cast<uint32_t>(min(static_cast<size_t>(32), p.k - first));
                        mask &= n_valid >= 32u ? 0xFFFFFFFFu : ((1u << n_valid) - 1u);
                        counted += __popc(mask);
                    } else if (MODE == MODE_PRUNE) {
                        // test of the first checkpoint for 32 centroids, then a warp scan places every row's
                        // survivors behind those of the lower lanes
                        uint32_t mask = 0;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 nyv = *reinterpret_cast<const float4*>(ny + ch * 32 + j);
                            const float p0 = fmaf(-2.0f, __uint_as_float(r[j + 0]), nx) + nyv.x;
                            const float p1 = fmaf(-2.0f, __uint_as_float(r[j + 1]), nx) + nyv.y;
                            const float p2 = fmaf(-2.0f, __uint_as_float(r[j + 2]), nx) + nyv.z;
                            const float p3 = fmaf(-2.0f, __uint_as_float(r[j + 3]), nx) + nyv.w;
                            r[j + 0] = __float_as_uint(p0);
                            r[j + 1] = __float_as_uint(p1);
                            r[j + 2] = __float_as_uint(p2);
                            r[j + 3] = __float_as_uint(p3);
                            mask |= (p0 < thr ? (1u << j) : 0u) | (p1 < thr ? (2u << j) : 0u) | (p2 < thr ? (4u << j) : 0u) | (p3 < thr ? (8u << j) : 0u);
                        }
                        {
                            // columns past the last centroid (zero-filled by TMA) never count
                            const size_t first = col0 + static_cast<size_t>(ch) * 32;
                            const uint32_t n_valid = first >= p.k ? 0u : static_cast<uint32_t>(min(static_cast<size_t>(32), p.k - first));
                            mask &= n_valid >= 32u ? 0xFFFFFFFFu : ((1u << n_valid) - 1u);
                        }
                        const uint32_t cnt = __popc(mask);
                        uint32_t incl = cnt;
#pragma unroll
                        for (int off = 1; off < 32; off <<= 1) {
                            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
                            if (lane >= off) incl += v;
                        }
                        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
                        if (total != 0) {
                            const uint32_t colbits = static_cast<uint32_t>(col0 + ch * 32) << 5;
                            if (total <= STAGE_ENTRIES) {
                                // survivors are packed in shared memory first (predicated stores, no divergence) and
                                // leave for global memory as contiguous runs
                                uint2* stg = reinterpret_cast<uint2*>(smem + STAGES * STAGE_BYTES + SMEM_CTRL_BYTES) + (warp - 6) * STAGE_ENTRIES;
                                // slot of column j = this lane's first slot + number of its survivors below j: no chain
                                // of dependent additions through the 32 columns
                                const uint32_t base = incl - cnt;
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    if ((mask >> j) & 1u) stg[base + __popc(mask & ((1u << j) - 1u))] = make_uint2((colbits + (static_cast<uint32_t>(j) << 5)) | lane, r[j]);
                                }
                                __syncwarp();
                                for (uint32_t i = lane; i < total; i += 32)
                                    if (filled + i < p.cap_group) my_list[filled + i] = stg[i];
                                __syncwarp();
                            } else {
                                // dense case (more than a quarter of the 32 x 32 block passes): eight columns at a time,
                                // which always fit in the staging area
                                uint2* stg = reinterpret_cast<uint2*>(smem + STAGES * STAGE_BYTES + SMEM_CTRL_BYTES) + (warp - 6) * STAGE_ENTRIES;
                                uint32_t done = 0;
#pragma unroll
                                for (int sb = 0; sb < 4; ++sb) {
                                    const uint32_t sub = (mask >> (8 * sb)) & 0xFFu;
                                    const uint32_t c8 = __popc(sub);
                                    uint32_t in8 = c8;
#pragma unroll
                                    for (int off = 1; off < 32; off <<= 1) {
                                        const uint32_t v = __shfl_up_sync(0xffffffffu, in8, off);
                                        if (lane >= off) in8 += v;
                                    }
                                    const uint32_t tot8 = __shfl_sync(0xffffffffu, in8, 31);
                                    uint32_t pos = in8 - c8;
#pragma unroll
                                    for (int j = 8 * sb; j < 8 * sb + 8; ++j) {
                                        const uint32_t bit = (mask >> j) & 1u;
                                        if (bit) stg[pos] = make_uint2((colbits + (static_cast<uint32_t>(j) << 5)) | lane, r[j]);
                                        pos += bit;
                                    }
                                    __syncwarp();
                                    for (uint32_t i = lane; i < tot8; i += 32)
                                        if (filled + done + i < p.cap_group) my_list[filled + done + i] = stg[i];
                                    __syncwarp();
                                    done += tot8;
                                }
                            }
                            filled += total;
                        }
                    } else if (row_valid) {
                        float* orow = p.out + row * p.ldo + col0 + ch * 32;
                        const size_t left = (col0 + ch * 32 < p.k) ? (p.k - (col0 + ch * 32)) : 0;
                        if (left >= 32 && (p.ldo % 4 == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(orow + j) =
                                    make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (static_cast<size_t>(j) < left) orow[j] = __uint_as_float(r[j]);
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(&ctrl->tmem_empty[b]);
            }
            if (MODE == MODE_ARGMIN && ok && row_valid) p.out_top2[row] = make_uint2(i1, i2);
            if (MODE == MODE_PRUNE && ok && lane == 0) my_offs[(n_col_tiles + 3) / 4] = filled;
            if (MODE == MODE_COUNT && ok && row_valid && counted != 0) atomicAdd(p.count_out + row, counted);   // the row's other half adds its own
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// =================================================================================================
// Dense ADSampling chain on the tensor cores (pruned assignment without candidate lists).
//
// For a tile of 128 points and a chunk of 1024 centroids the reference evaluates, for every pair,
// a sequence of tests "partial distance < best * ratio[dimensions seen]": after the first d'
// dimensions, after every further 64 horizontal dimensions, and after the remaining vertical
// dimensions (pdx/pdxearch.h:118-217); `best` is fixed inside the chunk and lowered at its end
// (:290-324).  Here the partial distances come from accumulators that keep growing along that same
// order of dimensions: the MMA warp walks the reduction dimension segment by segment and publishes
// the accumulator after each one; the epilogue thread of a row reads it (without clearing it), 32
// columns at a time, turns it into ||x||^2 + ||c||^2 - 2 x.c over the dimensions seen so far with
// precomputed cumulative norms, and updates a bit mask of surviving centroids.  Every quantity a row
// needs (survivor masks, survivor count, chunk minimum) is private to its thread.
// =================================================================================================
struct ChainParams {
    size_t n, k;
    uint32_t d, partial_d, vertical_d, horizontal_d;
    uint32_t n_seg;                 // 1 + horizontal_d / 64 + (partial_d < vertical_d)
    const float* chain_norms_x;     // n x n_seg cumulative squared norms of the points
    const float* chain_norms_y;     // n_seg x k (checkpoint-major), of the centroids
    const float* ratios;            // d + 1
    const float* best_in;           // exact distance to the previous centroid
    uint32_t* knn;                  // in: previous assignment, out: new
    float* dist;
    uint32_t* not_pruned;
    uint2* top2;                    // out: the two smallest final distances seen by the chain, per point
    int* error;
    long long wait_limit;
};

struct SegInfo {
    uint32_t x_begin;   // first column fetched (multiple of 4)
    uint32_t n_kb;      // 16-column blocks
    uint32_t map;       // 0 = front (extent d'), 1 = vertical (extent vertical_d), 2 = full
    uint32_t mask_below;  // columns below this value are zeroed in the first block (tail segment only)
    uint32_t dims_after;
};

__device__ __forceinline__ SegInfo chain_segment(const ChainParams& p, uint32_t seg) {
    SegInfo s;
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

struct ChainMaps {
    CUtensorMap x[3];     // points, visible extent d' / vertical_d / d
    CUtensorMap yhi[3];   // tf32 hi parts of the centroids, same extents
    CUtensorMap ylo[3];   // tf32 lo parts
};

// Chain kernel geometry: units of 128 points x 256 centroids, the stage layout of the GEMM kernel (X raw ->
// hi/lo by the splitter warps, Y hi and lo straight from global memory), two accumulators of 256 columns.
// The two accumulators belong to two neighbouring centroid units that advance through the segments in
// turn, so the tensor pipe works on one unit while the rows' threads test the other.
// What the two threads of a row (one per half of the columns) tell each other at the end of a chunk.
struct ChainPartial {
    uint32_t cnt;          // survivors of the first test in this chunk
    uint32_t prev_first;   // the previous centroid is among them
    float cb;              // best final distance of the chunk, FLT_MAX if none
    uint32_t cbi;
    float t1, t2;          // the two smallest final distances of the row so far (candidates for the refinement)
    uint32_t i1, i2;
};

struct ChainCtrl {
    uint64_t full[STAGES];
    uint64_t conv[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_ready[2];    // MMA -> epilogue: accumulator a holds the chain up to the current segment
    uint64_t acc_loaded[2];   // epilogue -> MMA: every row has read it
    uint64_t xchg_bar;        // the 256 row threads have published their ChainPartial
    uint32_t tmem_base;
    uint32_t pad;
    alignas(16) float ny[4][BN];   // per quarter of the rows: centroid norms of the unit at the current checkpoint
    float seg_ratio[64];           // ratios[dimensions seen after segment s]
    alignas(16) ChainPartial xchg[2][2][BM];   // [use parity][column half][row]
};
constexpr uint32_t C_CTRL_BYTES = 24576;
static_assert(sizeof(ChainCtrl) <= C_CTRL_BYTES, "control block too large");
constexpr uint32_t C_SMEM_BYTES = STAGES * STAGE_BYTES + C_CTRL_BYTES + 1024;
constexpr uint32_t CHAIN_MAX_SEGMENTS = 64;
// producer, MMA issuer, four splitter warps, eight row warps: warps 6-9 test columns 0-127 of every 256-centroid
// unit, warps 10-13 columns 128-255; the two threads of a row merge their findings at the end of every chunk
constexpr int CHAIN_THREADS = 448;

// Order of work shared by all roles: row tile, chunk of 1024 centroids, pair of 256-centroid units, segment,
// unit of the pair.  `a` (0 / 1) is the unit's accumulator.
#define CHAIN_FOR_EACH_UNIT_SEGMENT(...)                                                                  \
    for (size_t rt = blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {                               \
        for (uint32_t chunk = 0; chunk < n_chunks && ok; ++chunk) {                                       \
            const size_t c0 = static_cast<size_t>(chunk) * kChunk;                                        \
            const uint32_t cs = static_cast<uint32_t>(min(static_cast<size_t>(kChunk), p.k - c0));        \
            const uint32_t n_units = (cs + BN - 1) / BN;                                                  \
            for (uint32_t pair = 0; pair * 2 < n_units && ok; ++pair) {                                   \
                for (uint32_t seg = 0; seg < p.n_seg && ok; ++seg) {                                      \
                    const SegInfo si = chain_segment(p, seg);                                             \
                    for (uint32_t a = 0; a < 2 && ok; ++a) {                                              \
                        const uint32_t unit = pair * 2 + a;                                               \
                        if (unit >= n_units) break;                                                       \
                        __VA_ARGS__                                                                       \
                    }                                                                                     \
                }                                                                                         \
            }                                                                                             \
        }                                                                                                 \
    }

__global__ void __launch_bounds__(CHAIN_THREADS, 1) chain_tc_kernel(const __grid_constant__ ChainMaps maps, const ChainParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    ChainCtrl* ctrl = reinterpret_cast<ChainCtrl*>(smem + STAGES * STAGE_BYTES);
    const WaitCtx wctx{p.error, p.wait_limit};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctrl->full[s], 1);
            mbar_init(&ctrl->conv[s], 128);
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
    if (threadIdx.x >= 64 && threadIdx.x < 64 + CHAIN_MAX_SEGMENTS && threadIdx.x - 64 < p.n_seg) {
        ctrl->seg_ratio[threadIdx.x - 64] = __ldg(p.ratios + chain_segment(p, threadIdx.x - 64).dims_after);
    }
    if (warp == 1) tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    const size_t n_row_tiles = (p.n + BM - 1) / BM;
    const uint32_t n_chunks = static_cast<uint32_t>((p.k + kChunk - 1) / kChunk);

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t kbt = 0;
            bool ok = true;
            CHAIN_FOR_EACH_UNIT_SEGMENT({
                const CUtensorMap* mx = &maps.x[si.map];
                const CUtensorMap* mh = &maps.yhi[si.map];
                const CUtensorMap* ml = &maps.ylo[si.map];
                const int yrow = static_cast<int>(c0 + static_cast<size_t>(unit) * BN);
                for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                    const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                    if (!mbar_wait(&ctrl->empty[s], ph ^ 1u, wctx, 11)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&ctrl->full[s], A_TILE_BYTES + 2 * B_TILE_BYTES);
                    const uint32_t st = smem_base + s * STAGE_BYTES;
                    const int xc = static_cast<int>(si.x_begin + kb * BK);
                    tma_load_2d(st + OFF_A_HI, mx, &ctrl->full[s], xc, static_cast<int>(rt * BM));
                    tma_load_2d(st + OFF_B_HI, mh, &ctrl->full[s], xc, yrow);
                    tma_load_2d(st + OFF_B_LO, ml, &ctrl->full[s], xc, yrow);
                }
            })
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t kbt = 0;
            uint32_t uses[2] = {0, 0};
            bool ok = true;
            CHAIN_FOR_EACH_UNIT_SEGMENT({
                // the rows must have read this accumulator's previous checkpoint before it grows (or restarts)
                if (uses[a] > 0 && !mbar_wait(&ctrl->acc_loaded[a], (uses[a] - 1) & 1u, wctx, 12)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + a * BN;
                for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                    const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                    if (!mbar_wait(&ctrl->conv[s], ph, wctx, 13)) {
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
                        umma_tf32(acc, a_hi, b_hi, (seg | kb | kk) != 0 ? 1u : 0u);
                        umma_tf32(acc, a_hi, b_lo, 1u);
                        umma_tf32(acc, a_lo, b_hi, 1u);
                    }
                    umma_commit(&ctrl->empty[s]);
                }
                if (ok) umma_commit(&ctrl->acc_ready[a]);
                ++uses[a];
            })
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- hi / lo splitter of the X tile
        const int cid = threadIdx.x - 64;
        uint32_t kbt = 0;
        bool ok = true;
        CHAIN_FOR_EACH_UNIT_SEGMENT({
            for (uint32_t kb = 0; kb < si.n_kb; ++kb, ++kbt) {
                const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                if (!mbar_wait(&ctrl->full[s], ph, wctx, 14)) {
                    ok = false;
                    break;
                }
                uint8_t* st = smem + s * STAGE_BYTES;
                float4* a_hi = reinterpret_cast<float4*>(st + OFF_A_HI);
                float4* a_lo = reinterpret_cast<float4*>(st + OFF_A_LO);
                const bool mask = (kb == 0) && (si.mask_below > si.x_begin);
#pragma unroll
                for (int i = 0; i < static_cast<int>(A_TILE_BYTES / 16 / 128); ++i) {
                    const int q = cid + 128 * i;
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
    } else {
        // (warps 6 .. 13)
        // ---------------------------------------------------------------- rows: tests at every checkpoint
        const uint32_t half = static_cast<uint32_t>(warp - 6) >> 2;   // which 128 of a unit's 256 columns
        const uint32_t lane_base = 32u * (warp & 3);
        const uint32_t row_in_tile = lane_base + lane;
        uint32_t uses[2] = {0, 0};
        uint32_t xchg_uses = 0;
        bool ok = true;
        size_t cur_rt = ~size_t{0};
        uint32_t cur_chunk = 0xFFFFFFFFu;
        size_t row = 0;
        bool row_valid = false;
        float best = -1.f, cb = FLT_MAX, t1 = FLT_MAX, t2 = FLT_MAX;
        uint32_t bestidx = 0, prev = 0xFFFFFFFFu, npc = 0, cnt = 0, cbi = 0, i1 = 0xFFFFFFFFu, i2 = 0xFFFFFFFFu;
        uint32_t o1 = 0xFFFFFFFFu, o2 = 0xFFFFFFFFu;   // merged runner-ups of the row, set at every chunk end
        bool prev_first = false;
        constexpr int HS = BN / 64;   // 32-column slices per half
        // survivor masks of the two units in flight (kept apart so that both stay in registers)
        uint32_t alive0[HS], alive1[HS];
#pragma unroll
        for (int q = 0; q < HS; ++q) alive0[q] = alive1[q] = 0;
        float* ny = ctrl->ny[warp & 3];
        // End of a chunk: the two threads of the row exchange what they found in their halves of the columns and
        // both apply the same update.  Returns false when the wait ran out.
        auto close_chunk = [&]() -> bool {
            ChainPartial mine;
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
            if (!__all_sync(0xffffffffu, mbar_wait(&ctrl->xchg_bar, xchg_uses & 1u, wctx, 16))) return false;
            ++xchg_uses;
            const ChainPartial other = ctrl->xchg[slot][half ^ 1u][row_in_tile];
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
            // the two smallest of both halves, for the end of the row (the halves' own pairs cover disjoint columns
            // and stay as they are)
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
        CHAIN_FOR_EACH_UNIT_SEGMENT({
            if (rt != cur_rt) {
                if (cur_rt != ~size_t{0}) {
                    if (!close_chunk()) {
                        ok = false;
                        break;
                    }
                    close_row();
                }
                cur_rt = rt;
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
            } else if (chunk != cur_chunk) {
                if (!close_chunk()) {
                    ok = false;
                    break;
                }
                cur_chunk = chunk;
            }
            const size_t col0 = c0 + static_cast<size_t>(unit) * BN;
            const uint32_t cols_valid = static_cast<uint32_t>(min(static_cast<size_t>(BN), p.k - col0));
            const float thr = best * ctrl->seg_ratio[seg];
            const float nxv = row_valid ? __ldg(p.chain_norms_x + row * p.n_seg + seg) : 0.f;
            const bool first = seg == 0, last = (seg + 1 == p.n_seg);
            // centroid norms of the unit at this checkpoint: the two warps of a row quarter fill (and read) disjoint
            // halves of the quarter's copy
            {
                const float* __restrict__ src = p.chain_norms_y + static_cast<size_t>(seg) * p.k + col0 + half * (BN / 2);
                float cur[HS];
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) cur[q] = (half * (BN / 2) + q * 32 + lane < cols_valid) ? __ldg(src + q * 32 + lane) : 0.f;
                __syncwarp();
#pragma unroll
                for (uint32_t q = 0; q < HS; ++q) ny[half * (BN / 2) + q * 32 + lane] = cur[q];
                __syncwarp();
            }
            if (!__all_sync(0xffffffffu, mbar_wait(&ctrl->acc_ready[a], uses[a] & 1u, wctx, 15))) {
                ok = false;
                break;
            }
            ++uses[a];
            tc_fence_after();
            const uint32_t taddr = tmem_base + (lane_base << 16) + a * BN + half * (BN / 2);
            uint32_t alive[HS];
#pragma unroll
            for (int q = 0; q < HS; ++q) alive[q] = a ? alive1[q] : alive0[q];
            // One 32-column slice is tested while the next one is on its way from tensor memory.
            auto test_slice = [&](const uint32_t ch, uint32_t (&r)[32], uint32_t& alive_ch) {
                // bit j of w = (partial distance of column ch * 32 + j < threshold), branch-free
                uint32_t w = 0;
#pragma unroll
                for (uint32_t j = 0; j < 32; j += 4) {
                    const float4 nyv = *reinterpret_cast<const float4*>(ny + ch * 32 + j);
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
                    const uint32_t lo = ch * 32;
                    const uint32_t valid = (cols_valid >= lo + 32) ? 0xFFFFFFFFu : (cols_valid > lo ? ((1u << (cols_valid - lo)) - 1u) : 0u);
                    const uint32_t al = w & valid;
                    alive_ch = al;
                    cnt += __popc(al);
                    if (static_cast<size_t>(prev) >= col0 + lo && static_cast<size_t>(prev) < col0 + lo + 32) {
                        if ((al >> (static_cast<uint32_t>(prev - col0) & 31u)) & 1u) prev_first = true;
                    }
                }
                if (!first && !last) alive_ch &= w;
                if (last) {
                    // Last checkpoint: the pairs still alive compete.  thr == best here (ratio[d] == 1).  With a
                    // single segment (first and last at once) alive[] has just been set above.
                    uint32_t m = alive_ch;
                    if (m) {
                        float pdv[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) pdv[j] = __uint_as_float(r[j]);
                        while (m) {
                            const uint32_t j = __ffs(m) - 1;
                            m &= m - 1;
                            const float pd = pdv[j];
                            const uint32_t gc = static_cast<uint32_t>(col0 + ch * 32 + j);
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
            tmem_ld32_issue(taddr, ra);
            tmem_ld_wait(ra);
            // Rolled on purpose (two slices per trip): unrolled, the tests of a whole unit do not fit the instruction
            // cache.  The survivor masks rotate through alive[0] and alive[1] so that they stay in registers.
            const uint32_t slice0 = half * HS;   // first of this thread's slices inside the unit
#pragma unroll 1
            for (uint32_t ch = 0; ch < HS; ch += 2) {
                tmem_ld32_issue(taddr + (ch + 1) * 32, rb);
                test_slice(slice0 + ch, ra, alive[0]);
                tmem_ld_wait(rb);
                if (ch + 2 < HS) {
                    tmem_ld32_issue(taddr + (ch + 2) * 32, ra);
                } else {
                    // everything of this checkpoint is in registers: the accumulator may grow again
                    tc_fence_before();
                    mbar_arrive(&ctrl->acc_loaded[a]);
                }
                test_slice(slice0 + ch + 1, rb, alive[1]);
                if (ch + 2 < HS) tmem_ld_wait(ra);
                const uint32_t m0 = alive[0], m1 = alive[1];
#pragma unroll
                for (int q = 0; q < HS - 2; ++q) alive[q] = alive[q + 2];
                alive[HS - 2] = m0;
                alive[HS - 1] = m1;
            }
#pragma unroll
            for (int q = 0; q < HS; ++q) {
                if (a) alive1[q] = alive[q];
                else alive0[q] = alive[q];
            }
        })
        if (ok && cur_rt != ~size_t{0}) {
            if (close_chunk()) close_row();
        }
    }
#undef CHAIN_FOR_EACH_UNIT_SEGMENT

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// After the chain: the exact squared distance (direct differences, fp32) of a point to the chain's
// winner and to the two runner-ups; the smallest wins, the winner keeps its place on ties.
__global__ void __launch_bounds__(256) refine_chain_kernel(const float* __restrict__ x, const float* __restrict__ y, size_t n, size_t k, size_t d,
                                                           const uint2* __restrict__ top2, uint32_t* __restrict__ knn, float* __restrict__ dist,
                                                           const int* __restrict__ error, const uint32_t* __restrict__ tile_map) {
    // with a tile map the grid covers the rows of the listed 128-row tiles, else rows 0 .. n-1
    size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (tile_map) row = static_cast<size_t>(tile_map[row / BM]) * BM + (row % BM);
    if (row >= n) return;
    // a chain kernel that gave up on a wait leaves its outputs unwritten: nothing to refine, and no index to trust
    if (*reinterpret_cast<const volatile int*>(error) != 0) return;
    const int lane = threadIdx.x & 31;
    const uint32_t w = knn[row];
    const uint2 t = top2[row];
    if (w >= k) return;
    uint32_t cand[3] = {w, t.x < k ? t.x : 0xFFFFFFFFu, t.y < k ? t.y : 0xFFFFFFFFu};
    if (cand[1] == 0xFFFFFFFFu || cand[1] == w) cand[1] = w;
    if (cand[2] == 0xFFFFFFFFu || cand[2] == w) cand[2] = w;
    const float* xr = x + row * d;
    const float* y0 = y + static_cast<size_t>(cand[0]) * d;
    const float* y1 = y + static_cast<size_t>(cand[1]) * d;
    const float* y2 = y + static_cast<size_t>(cand[2]) * d;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    for (size_t j = static_cast<size_t>(lane) * 4; j < d; j += 128) {
        const float4 xv = __ldg(reinterpret_cast<const float4*>(xr + j));
        const float4 a = __ldg(reinterpret_cast<const float4*>(y0 + j));
        const float4 b = __ldg(reinterpret_cast<const float4*>(y1 + j));
        const float4 c = __ldg(reinterpret_cast<const float4*>(y2 + j));
        float u;
        u = xv.x - a.x; s0 = fmaf(u, u, s0); u = xv.y - a.y; s0 = fmaf(u, u, s0); u = xv.z - a.z; s0 = fmaf(u, u, s0); u = xv.w - a.w; s0 = fmaf(u, u, s0);
        u = xv.x - b.x; s1 = fmaf(u, u, s1); u = xv.y - b.y; s1 = fmaf(u, u, s1); u = xv.z - b.z; s1 = fmaf(u, u, s1); u = xv.w - b.w; s1 = fmaf(u, u, s1);
        u = xv.x - c.x; s2 = fmaf(u, u, s2); u = xv.y - c.y; s2 = fmaf(u, u, s2); u = xv.z - c.z; s2 = fmaf(u, u, s2); u = xv.w - c.w; s2 = fmaf(u, u, s2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) {
        uint32_t bi = cand[0];
        float bd = s0;
        if (s1 < bd || (s1 == bd && cand[1] < bi && cand[1] != w && bi != w)) {
            bd = s1;
            bi = cand[1];
        }
        if (s2 < bd || (s2 == bd && cand[2] < bi && bi != w)) {
            bd = s2;
            bi = cand[2];
        }
        knn[row] = bi;
        dist[row] = bd;
    }
}

// Settles the assignment in fp32: one warp per row recomputes ||x||^2 + ||y||^2 - 2 x.y for the two
// candidates with fp32 fused multiply-adds, keeps the smaller (the lower index on a tie) and stores
// the distance clamped at zero, as the reference does (batch_computers.h:160-166).
__global__ void __launch_bounds__(256) refine_top2_kernel(
    const float* __restrict__ x, const float* __restrict__ y, size_t n, size_t k, size_t d, const float* __restrict__ norms_x, const float* __restrict__ norms_y,
    const uint2* __restrict__ top2, uint32_t* __restrict__ out_knn, float* __restrict__ out_dist, const int* __restrict__ error
) {
    const size_t row = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= n) return;
    // a tensor-core pass that gave up on a wait leaves the candidate pairs unwritten
    if (*reinterpret_cast<const volatile int*>(error) != 0) return;
    const int lane = threadIdx.x & 31;
    const uint2 cand = top2[row];
    if (cand.x >= k) return;
    const bool two = cand.y < k;
    const float* xr = x + row * d;
    const float* y1 = y + static_cast<size_t>(cand.x) * d;
    const float* y2 = y + static_cast<size_t>(two ? cand.y : cand.x) * d;
    float a1 = 0.f, a2 = 0.f;
    for (size_t j = static_cast<size_t>(lane) * 4; j < d; j += 128) {  // d % 4 == 0 on this path
        const float4 xv = __ldg(reinterpret_cast<const float4*>(xr + j));
        const float4 u = __ldg(reinterpret_cast<const float4*>(y1 + j));
        const float4 v = __ldg(reinterpret_cast<const float4*>(y2 + j));
        a1 = fmaf(xv.x, u.x, a1); a1 = fmaf(xv.y, u.y, a1); a1 = fmaf(xv.z, u.z, a1); a1 = fmaf(xv.w, u.w, a1);
        a2 = fmaf(xv.x, v.x, a2); a2 = fmaf(xv.y, v.y, a2); a2 = fmaf(xv.z, v.z, a2); a2 = fmaf(xv.w, v.w, a2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a1 += __shfl_xor_sync(0xffffffffu, a1, o);
        a2 += __shfl_xor_sync(0xffffffffu, a2, o);
    }
    if (lane == 0) {
        const float nx = norms_x[row];
        float e1 = fmaf(-2.0f, a1, nx) + norms_y[cand.x];
        uint32_t w = cand.x;
        if (two) {
            float e2 = fmaf(-2.0f, a2, nx) + norms_y[cand.y];
            if (fabsf(e1 - e2) <= 1e-4f * fmaxf(fabsf(e1), fabsf(e2))) {
                // Near-tie (typically the twin centroids left by a cluster split): settle it with the dot
                // products accumulated strictly in index order, the order of the fp32 SIMT kernel.
                float s1 = 0.f, s2 = 0.f;
                for (size_t j = 0; j < d; ++j) {
                    const float xv = xr[j];
                    s1 = fmaf(xv, y1[j], s1);
                    s2 = fmaf(xv, y2[j], s2);
                }
                e1 = fmaf(-2.0f, s1, nx) + norms_y[cand.x];
                e2 = fmaf(-2.0f, s2, nx) + norms_y[cand.y];
            }
            if (e2 < e1 || (e2 == e1 && cand.y < cand.x)) {
                e1 = e2;
                w = cand.y;
            }
        }
        out_knn[row] = w;
        out_dist[row] = fmaxf(0.0f, e1);
    }
}

// hi = tf32(v), lo = tf32(v - hi) for every element (the split the splitter warps would do in shared memory)
__global__ void __launch_bounds__(256) split_tf32_kernel(const float4* __restrict__ in, float4* __restrict__ hi, float4* __restrict__ lo, size_t n4) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 h, l;
    split4(__ldg(in + i), h, l);
    hi[i] = h;
    lo[i] = l;
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    if (!fn) throw CudaError("cuTensorMapEncodeTiled is not available from this driver");
    return fn;
}

// Row-major fp32 matrix [rows][ld] of which the first `extent` columns are visible; boxes of 16
// columns x box_rows rows, 64-byte swizzle, zero fill outside.
CUtensorMap make_tmap(const float* base, size_t extent, size_t rows, size_t ld, uint32_t box_rows) {
    CUtensorMap m;
    const cuuint64_t dims[2] = {extent, rows};
    const cuuint64_t strides[1] = {ld * sizeof(float)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
    return m;
}

// Splits y (rows x ld, 16-byte aligned, ld % 4 == 0) into y_split[0 .. rows*ld) = hi and y_split[rows*ld ..) = lo.
void presplit(const float* y, size_t rows, size_t ld, float* y_split, cudaStream_t stream) {
    const size_t n4 = rows * ld / 4;
    if (n4 == 0) return;
    split_tf32_kernel<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const float4*>(y), reinterpret_cast<float4*>(y_split),
                                                                                   reinterpret_cast<float4*>(y_split + rows * ld), n4);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

int* error_flag(int device) {
    static std::mutex mu;
    static int* flags[64] = {nullptr};
    std::lock_guard<std::mutex> lock(mu);
    if (!flags[device]) {
        note_device_alloc();
        SKM_CUDA(cudaMalloc(&flags[device], sizeof(int)));
        SKM_CUDA(cudaMemset(flags[device], 0, sizeof(int)));
    }
    return flags[device];
}

int sm_count(int device) {
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    return sms;
}

template <int MODE>
void launch(const CUtensorMap& tx, const CUtensorMap& ty, const CUtensorMap& tylo, const Params& p, cudaStream_t stream) {
    SKM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES)));
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const size_t row_tiles = (p.n + BM - 1) / BM;
    const int grid = static_cast<int>(std::min<size_t>(row_tiles, static_cast<size_t>(sm_count(device))));
    gemm_tc_kernel<MODE><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tx, ty, tylo, p);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

bool g_enabled = true;
uint32_t g_debug_producer_stop = 0;
long long g_wait_limit = WAIT_LIMIT_CYCLES;

} // namespace

long long wait_limit() { return g_wait_limit; }

void set_debug_wait_injection(long long wait_limit_cycles, uint32_t producer_stops_after_kblocks) {
    g_wait_limit = wait_limit_cycles > 0 ? wait_limit_cycles : WAIT_LIMIT_CYCLES;
    g_debug_producer_stop = producer_stops_after_kblocks;
}

void launch_presplit(const float* y, size_t rows, size_t ld, float* y_split, cudaStream_t stream) { presplit(y, rows, ld, y_split, stream); }

CUtensorMap make_row_major_tmap(const float* base, size_t extent, size_t rows, size_t ld, uint32_t box_rows) { return make_tmap(base, extent, rows, ld, box_rows); }

int* error_word() {
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    return error_flag(device);
}

void set_enabled(bool on) { g_enabled = on; }
bool enabled() { return g_enabled; }

bool eligible(const float* x, size_t ldx, const float* y, size_t ldy) {
    if (!g_enabled) return false;
    if (ldx % 4 != 0 || ldy % 4 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return false;
    return true;
}

void launch_assign_full(const float* x, const float* y, size_t n, size_t k, size_t d, const float* norms_x, const float* norms_y, uint32_t* out_knn, float* out_dist,
                        uint2* top2_scratch, cudaStream_t stream, float* y_split) {
    if (n == 0 || k == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    if (y_split) presplit(y, k, d, y_split, stream);
    const CUtensorMap tx = make_tmap(x, d, n, d, BM);
    const CUtensorMap ty = make_tmap(y_split ? y_split : y, d, k, d, BN);
    const CUtensorMap tylo = y_split ? make_tmap(y_split + k * d, d, k, d, BN) : ty;
    Params p{};
    p.y_presplit = y_split != nullptr;
    p.n = n;
    p.k = k;
    p.kdim = static_cast<uint32_t>(d);
    p.norms_x = norms_x;
    p.norms_y = norms_y;
    p.out_knn = out_knn;
    p.out_dist = out_dist;
    p.out_top2 = top2_scratch;
    p.error = error_flag(device);
    p.wait_limit = g_wait_limit;
    p.debug_producer_stop = g_debug_producer_stop;
    launch<MODE_ARGMIN>(tx, ty, tylo, p, stream);
    refine_top2_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(x, y, n, k, d, norms_x, norms_y, top2_scratch, out_knn, out_dist, p.error);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_assign_full_flagged(const float* x, const float* y, size_t n, size_t k, size_t d, const float* norms_x, const float* norms_y, uint32_t* out_knn, float* out_dist,
                                uint2* top2_scratch, int* error_word, cudaStream_t stream) {
    if (n == 0 || k == 0) return;
    const CUtensorMap tx = make_tmap(x, d, n, d, BM);
    const CUtensorMap ty = make_tmap(y, d, k, d, BN);
    Params p{};
    p.n = n;
    p.k = k;
    p.kdim = static_cast<uint32_t>(d);
    p.norms_x = norms_x;
    p.norms_y = norms_y;
    p.out_knn = out_knn;
    p.out_dist = out_dist;
    p.out_top2 = top2_scratch;
    p.error = error_word;
    p.wait_limit = g_wait_limit;
    launch<MODE_ARGMIN>(tx, ty, ty, p, stream);
    refine_top2_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(x, y, n, k, d, norms_x, norms_y, top2_scratch, out_knn, out_dist, p.error);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_first_test(const float* x, const float* y, size_t n, size_t k, size_t d, uint32_t partial_d, const float* norms_x, const float* norms_y, const float* best_in,
                       const uint32_t* skip, float ratio_first, size_t tile0, size_t n_tiles, uint2* lists, uint32_t* list_offs, uint32_t cap_group, cudaStream_t stream,
                       const float* y_split, const uint32_t* tile_map) {
    if (n_tiles == 0 || k == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const CUtensorMap tx = make_tmap(x, partial_d, n, d, BM);
    const CUtensorMap ty = make_tmap(y_split ? y_split : y, partial_d, k, d, BN);
    const CUtensorMap tylo = y_split ? make_tmap(y_split + k * d, partial_d, k, d, BN) : ty;
    Params p{};
    p.y_presplit = y_split != nullptr;
    p.n = n;
    p.k = k;
    p.kdim = partial_d;
    p.norms_x = norms_x;
    p.norms_y = norms_y;
    p.error = error_flag(device);
    p.wait_limit = g_wait_limit;
    p.tile0 = tile0;
    p.n_tiles = n_tiles;
    p.best_in = best_in;
    p.skip = skip;
    p.ratio_first = ratio_first;
    p.lists = lists;
    p.list_offs = list_offs;
    p.cap_group = cap_group;
    p.tile_map = tile_map;
    SKM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<MODE_PRUNE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES)));
    const int grid = static_cast<int>(std::min<size_t>(n_tiles, static_cast<size_t>(sm_count(device))));
    gemm_tc_kernel<MODE_PRUNE><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tx, ty, tylo, p);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_count_first_test(const float* x, size_t n, size_t k, size_t d, uint32_t partial_d, const float* norms_x, const float* norms_y, const float* thr_rows,
                             uint32_t thr_chunks, uint32_t* count_out, const float* y_split, cudaStream_t stream) {
    if (n == 0 || k == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const CUtensorMap tx = make_tmap(x, partial_d, n, d, BM);
    const CUtensorMap ty = make_tmap(y_split, partial_d, k, d, BN);
    const CUtensorMap tylo = make_tmap(y_split + k * d, partial_d, k, d, BN);
    Params p{};
    p.y_presplit = true;
    p.n = n;
    p.k = k;
    p.kdim = partial_d;
    p.norms_x = norms_x;
    p.norms_y = norms_y;
    p.error = error_flag(device);
    p.wait_limit = g_wait_limit;
    p.tile0 = 0;
    p.n_tiles = (n + BM - 1) / BM;
    p.thr_rows = thr_rows;
    p.thr_chunks = thr_chunks;
    p.count_out = count_out;
    SKM_CUDA(cudaMemsetAsync(count_out, 0, sizeof(uint32_t) * n, stream));
    SKM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<MODE_COUNT>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES)));
    const int grid = static_cast<int>(std::min<size_t>(p.n_tiles, static_cast<size_t>(sm_count(device))));
    gemm_tc_kernel<MODE_COUNT><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tx, ty, tylo, p);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_union(const float* x, size_t n, size_t k, size_t d, uint32_t partial_d, const float* norms_x, const float* norms_y, const float* best_in, float ratio_first,
                  const uint32_t* tile_map, size_t n_tiles, uint32_t* union_bits, uint32_t union_words, const float* y_split, cudaStream_t stream) {
    if (n_tiles == 0 || k == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const CUtensorMap tx = make_tmap(x, partial_d, n, d, BM);
    const CUtensorMap ty = make_tmap(y_split, partial_d, k, d, BN);
    const CUtensorMap tylo = make_tmap(y_split + k * d, partial_d, k, d, BN);
    Params p{};
    p.y_presplit = true;
    p.n = n;
    p.k = k;
    p.kdim = partial_d;
    p.norms_x = norms_x;
    p.norms_y = norms_y;
    p.error = error_flag(device);
    p.wait_limit = g_wait_limit;
    p.tile0 = 0;
    p.n_tiles = n_tiles;
    p.best_in = best_in;
    p.ratio_first = ratio_first;
    p.tile_map = tile_map;
    p.union_bits = union_bits;
    p.union_words = union_words;
    SKM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<MODE_UNION>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES)));
    const int grid = static_cast<int>(std::min<size_t>(n_tiles, static_cast<size_t>(sm_count(device))));
    gemm_tc_kernel<MODE_UNION><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tx, ty, tylo, p);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_gemm_nt(const float* a, size_t lda, const float* b, size_t ldb, float* out, size_t ldo, size_t n, size_t n_out, size_t k_dim, cudaStream_t stream) {
    if (n == 0 || n_out == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const CUtensorMap tx = make_tmap(a, k_dim, n, lda, BM);
    const CUtensorMap ty = make_tmap(b, k_dim, n_out, ldb, BN);
    Params p{};
    p.n = n;
    p.k = n_out;
    p.kdim = static_cast<uint32_t>(k_dim);
    p.out = out;
    p.ldo = ldo;
    p.error = error_flag(device);
    p.wait_limit = g_wait_limit;
    launch<MODE_STORE>(tx, ty, ty, p, stream);
}

void launch_chain(const float* x, const float* y, size_t n, size_t k, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, const float* chain_norms_x,
                  const float* chain_norms_y, const float* ratios, const float* best_in, uint32_t* knn, float* dist, uint32_t* not_pruned, uint2* top2_scratch,
                  float* y_split, cudaStream_t stream) {
    if (n == 0 || k == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    presplit(y, k, d, y_split, stream);
    ChainMaps maps;
    const size_t extents[3] = {partial_d, vertical_d, d};
    for (int i = 0; i < 3; ++i) {
        maps.x[i] = make_tmap(x, extents[i], n, d, BM);
        maps.yhi[i] = make_tmap(y_split, extents[i], k, d, BN);
        maps.ylo[i] = make_tmap(y_split + k * d, extents[i], k, d, BN);
    }
    ChainParams p{};
    p.n = n;
    p.k = k;
    p.d = static_cast<uint32_t>(d);
    p.partial_d = partial_d;
    p.vertical_d = vertical_d;
    p.horizontal_d = horizontal_d;
    p.n_seg = 1u + horizontal_d / 64u + (partial_d < vertical_d ? 1u : 0u);
    if (p.n_seg > CHAIN_MAX_SEGMENTS) throw std::invalid_argument("dimensionality too large for the tensor-core chain");
    p.chain_norms_x = chain_norms_x;
    p.chain_norms_y = chain_norms_y;
    p.ratios = ratios;
    p.best_in = best_in;
    p.knn = knn;
    p.dist = dist;
    p.not_pruned = not_pruned;
    p.top2 = top2_scratch;
    p.error = error_flag(device);
    p.wait_limit = g_wait_limit;
    SKM_CUDA(cudaFuncSetAttribute(chain_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(C_SMEM_BYTES)));
    const size_t row_tiles = (n + BM - 1) / BM;
    const int grid = static_cast<int>(std::min<size_t>(row_tiles, static_cast<size_t>(sm_count(device))));
    chain_tc_kernel<<<grid, CHAIN_THREADS, C_SMEM_BYTES, stream>>>(maps, p);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
    refine_chain_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(x, y, n, k, d, top2_scratch, knn, dist, p.error, nullptr);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

void launch_refine_chain_tiles(const float* x, const float* y, size_t n, size_t k, size_t d, const uint2* top2, uint32_t* knn, float* dist, const uint32_t* tile_map,
                               size_t n_tiles, cudaStream_t stream) {
    if (n_tiles == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    refine_chain_kernel<<<static_cast<unsigned>(n_tiles * (BM / 8)), 256, 0, stream>>>(x, y, n, k, d, top2, knn, dist, error_flag(device), tile_map);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

// Reads (and clears) the error code left by the last kernels on this device.  Synchronises `stream`.
int fetch_error(cudaStream_t stream) {
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    int* flag = error_flag(device);
    int host = 0;
    SKM_CUDA(cudaMemcpyAsync(&host, flag, sizeof(int), cudaMemcpyDeviceToHost, stream));
    SKM_CUDA(cudaStreamSynchronize(stream));
    if (host != 0) SKM_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), stream));
    return host;
}

} // namespace tc
} // namespace skmb
