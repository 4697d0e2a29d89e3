// Rotation on the tensor cores: out = A * B^T for row-major fp32 A [n][K] and B [n_out][K] (ADSamplingPruner::Rotate with
// B = M, Unrotate with B = M^T; adsampling.h:191-215, :273-298), with fp32-level accuracy.
//
// Both operands are split into tf32 hi + lo parts in shared memory and multiplied as hi*hi + hi*lo + lo*hi (see
// kernels_tc.cu).  What limits the accuracy of that scheme is the accumulator in tensor memory, which truncates on every
// addition: a chain of K products ends up about K * 1e-8 (relative to |a| |b|) low.  Rotated rows feed every distance
// computed afterwards, so the chain is cut: the reduction dimension is divided among kAcc accumulators, each summing a
// quarter of K, and the epilogue adds the four partial sums in fp32 registers.  With K = 1024 that leaves ~2e-6, the
// level of a sequential fp32 accumulation.
//
// One persistent CTA per SM, 320 threads, tiles of 128 rows x 128 output columns:
//   warp 0      TMA producer (A tile 128 x 16 and B tile 128 x 16 per stage, 64-byte swizzle);
//   warp 1      MMA issuer (M = 128, N = 128, K = 8; accumulator kb / blocks-per-accumulator);
//   warps 2-5   split both tiles of a stage into hi / lo parts in place;
//   warps 6-9   epilogue, one thread per row: sums the accumulators 32 columns at a time, stores the row segment and
//               (optionally) accumulates the squared norm of the output row.
// Every wait is bounded (see kernels_tc.cu).
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "kernels_tc.cuh"
#include "tc_ptx.cuh"

namespace skmb {
namespace tc {

namespace {

constexpr int RN = 128;                  // output columns per tile
constexpr int kAcc = 4;                  // accumulators, RN columns each (all 512 columns of tensor memory)
constexpr int ROT_THREADS = 320;
constexpr uint32_t ROT_B_BYTES = RN * BK * 4;   // 8192 per part
constexpr uint32_t ROT_CTRL_BYTES = 1024;
constexpr uint32_t ROT_SMEM_BYTES = STAGES * STAGE_BYTES + ROT_CTRL_BYTES + 1024;

struct RotParams {
    size_t n, n_out;
    uint32_t kdim;
    float* out;
    size_t ldo;
    float* out_sqnorms;   // optional: squared norm of every output row
    int* error;
    long long wait_limit;
};

struct RotCtrl {
    uint64_t full[STAGES];
    uint64_t conv[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full;
    uint64_t acc_empty;
    uint32_t tmem_base;
};
static_assert(sizeof(RotCtrl) <= ROT_CTRL_BYTES, "control block too large");

__global__ void __launch_bounds__(ROT_THREADS, 1) rotate_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const RotParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    RotCtrl* ctrl = reinterpret_cast<RotCtrl*>(smem + STAGES * STAGE_BYTES);
    const WaitCtx wctx{p.error, p.wait_limit};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctrl->full[s], 1);
            mbar_init(&ctrl->conv[s], 128);
            mbar_init(&ctrl->empty[s], 1);
        }
        mbar_init(&ctrl->acc_full, 1);
        mbar_init(&ctrl->acc_empty, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    const size_t n_row_tiles = (p.n + BM - 1) / BM;
    const uint32_t n_col_tiles = static_cast<uint32_t>((p.n_out + RN - 1) / RN);
    const uint32_t nkb = (p.kdim + BK - 1) / BK;
    const uint32_t kb_per_acc = (nkb + kAcc - 1) / kAcc;
    constexpr uint32_t idesc = make_idesc(RN);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t kbt = 0;
            bool ok = true;
            for (size_t rt = blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
                for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt) {
                    for (uint32_t kb = 0; kb < nkb; ++kb, ++kbt) {
                        const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                        if (!mbar_wait(&ctrl->empty[s], ph ^ 1u, wctx, 31)) {
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(&ctrl->full[s], A_TILE_BYTES + ROT_B_BYTES);
                        const uint32_t st = smem_base + s * STAGE_BYTES;
                        tma_load_2d(st + OFF_A_HI, &tmap_a, &ctrl->full[s], static_cast<int>(kb * BK), static_cast<int>(rt * BM));
                        tma_load_2d(st + OFF_B_HI, &tmap_b, &ctrl->full[s], static_cast<int>(kb * BK), static_cast<int>(nt * RN));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t kbt = 0, t = 0;
            bool ok = true;
            for (size_t rt = blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
                for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt, ++t) {
                    // the epilogue must have read the previous tile's accumulators
                    if (t > 0 && !mbar_wait(&ctrl->acc_empty, (t - 1) & 1u, wctx, 32)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    for (uint32_t kb = 0; kb < nkb; ++kb, ++kbt) {
                        const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                        if (!mbar_wait(&ctrl->conv[s], ph, wctx, 33)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t st = smem_base + s * STAGE_BYTES;
                        const uint32_t acc = tmem_base + (kb / kb_per_acc) * RN;
                        const bool fresh = (kb % kb_per_acc) == 0;
#pragma unroll
                        for (uint32_t kk = 0; kk < BK / 8; ++kk) {
                            const uint64_t a_hi = make_desc(st + OFF_A_HI + kk * 32);
                            const uint64_t a_lo = make_desc(st + OFF_A_LO + kk * 32);
                            const uint64_t b_hi = make_desc(st + OFF_B_HI + kk * 32);
                            const uint64_t b_lo = make_desc(st + OFF_B_LO + kk * 32);
                            umma_tf32(acc, a_hi, b_hi, (fresh && kk == 0) ? 0u : 1u, idesc);
                            umma_tf32(acc, a_hi, b_lo, 1u, idesc);
                            umma_tf32(acc, a_lo, b_hi, 1u, idesc);
                        }
                        umma_commit(&ctrl->empty[s]);
                    }
                    if (ok) umma_commit(&ctrl->acc_full);
                }
            }
        }
    } else if (warp < 6) {
        const int cid = threadIdx.x - 64;
        uint32_t kbt = 0;
        bool ok = true;
        for (size_t rt = blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
            for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt) {
                for (uint32_t kb = 0; kb < nkb; ++kb, ++kbt) {
                    const uint32_t s = kbt % STAGES, ph = (kbt / STAGES) & 1u;
                    if (!mbar_wait(&ctrl->full[s], ph, wctx, 34)) {
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
#pragma unroll
                    for (int i = 0; i < static_cast<int>(ROT_B_BYTES / 16 / 128); ++i) {
                        float4 hi, lo;
                        split4(b_hi[cid + 128 * i], hi, lo);
                        b_hi[cid + 128 * i] = hi;
                        b_lo[cid + 128 * i] = lo;
                    }
                    fence_proxy_async();
                    mbar_arrive(&ctrl->conv[s]);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 6 .. 9)
        const uint32_t lane_base = 32u * (warp & 3);
        const uint32_t row_in_tile = lane_base + lane;
        // accumulators that received at least one k-block
        const uint32_t n_used = (nkb + kb_per_acc - 1) / kb_per_acc;
        uint32_t t = 0;
        bool ok = true;
        for (size_t rt = blockIdx.x; rt < n_row_tiles && ok; rt += gridDim.x) {
            const size_t row = rt * BM + row_in_tile;
            const bool row_valid = row < p.n;
            float sq = 0.f;
            for (uint32_t nt = 0; nt < n_col_tiles && ok; ++nt, ++t) {
                if (!__all_sync(0xffffffffu, mbar_wait(&ctrl->acc_full, t & 1u, wctx, 35))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (lane_base << 16);
                const size_t col0 = static_cast<size_t>(nt) * RN;
#pragma unroll 1
                for (int ch = 0; ch < RN / 32; ++ch) {
                    uint32_t r[32], q[32];
                    tmem_ld32(taddr + ch * 32, r);
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    for (uint32_t a = 1; a < n_used; ++a) {
                        tmem_ld32(taddr + a * RN + ch * 32, q);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(q[j]);
                    }
                    if (ch == RN / 32 - 1) {
                        // everything of this tile is in registers: the accumulators may be overwritten
                        tc_fence_before();
                        mbar_arrive(&ctrl->acc_empty);
                    }
                    if (row_valid) {
                        float* orow = p.out + row * p.ldo + col0 + ch * 32;
                        const size_t left = (col0 + ch * 32 < p.n_out) ? (p.n_out - (col0 + ch * 32)) : 0;
                        if (left >= 32 && (p.ldo % 4 == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(orow + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
#pragma unroll
                            for (int j = 0; j < 32; ++j) sq = fmaf(v[j], v[j], sq);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (static_cast<size_t>(j) < left) {
                                    orow[j] = v[j];
                                    sq = fmaf(v[j], v[j], sq);
                                }
                            }
                        }
                    }
                }
            }
            if (ok && row_valid && p.out_sqnorms) p.out_sqnorms[row] = sq;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

} // namespace

void launch_rotate(const float* a, size_t lda, const float* b, size_t ldb, float* out, size_t ldo, size_t n, size_t n_out, size_t k_dim, float* out_sqnorms,
                   cudaStream_t stream) {
    if (n == 0 || n_out == 0) return;
    int device = 0;
    SKM_CUDA(cudaGetDevice(&device));
    const CUtensorMap ta = make_row_major_tmap(a, k_dim, n, lda, BM);
    const CUtensorMap tb = make_row_major_tmap(b, k_dim, n_out, ldb, RN);
    RotParams p{};
    p.n = n;
    p.n_out = n_out;
    p.kdim = static_cast<uint32_t>(k_dim);
    p.out = out;
    p.ldo = ldo;
    p.out_sqnorms = out_sqnorms;
    p.error = error_word();
    p.wait_limit = wait_limit();
    SKM_CUDA(cudaFuncSetAttribute(rotate_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ROT_SMEM_BYTES)));
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const size_t row_tiles = (n + BM - 1) / BM;
    const int grid = static_cast<int>(std::min<size_t>(row_tiles, static_cast<size_t>(sms)));
    rotate_tc_kernel<<<grid, ROT_THREADS, ROT_SMEM_BYTES, stream>>>(ta, tb, p);
    note_kernel_launch();
    SKM_CUDA(cudaGetLastError());
}

} // namespace tc
} // namespace skmb
