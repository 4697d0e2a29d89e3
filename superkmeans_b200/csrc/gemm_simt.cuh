// fp32 SIMT tile GEMM core shared by the rotation, exact-assignment and pruned-assignment kernels.
//
// A CTA of 256 threads computes a 128 x 128 tile of A * B^T where A (points) and B (centroids or
// the rotation matrix) are both row-major with the reduction dimension contiguous.  The reduction
// length K is arbitrary (d' changes every iteration and is not a multiple of anything); rows past
// m_valid / n_valid and columns past K read as zero.  Operands are staged through shared memory in
// k-major order, double buffered, with the next k-step prefetched into registers during the math.
//
// Thread (ty, tx) = (tid / 16, tid % 16) owns rows {4ty..4ty+3, 64+4ty..64+4ty+3} and columns
// {4tx..4tx+3, 64+4tx..64+4tx+3} of the tile, which keeps every shared-memory float4 read
// conflict-free.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace skmb {

constexpr int kGemmBK = 16;
constexpr int kGemmPad = 4;
constexpr int kGemmLd = 128 + kGemmPad;

struct GemmSmem {
    float a[2][kGemmBK][kGemmLd];
    float b[2][kGemmBK][kGemmLd];
};

__device__ __forceinline__ int tile_row_of(int ty, int i) { return (i < 4) ? (ty * 4 + i) : (64 + ty * 4 + (i - 4)); }
__device__ __forceinline__ int tile_col_of(int tx, int j) { return (j < 4) ? (tx * 4 + j) : (64 + tx * 4 + (j - 4)); }

// `grow` is the row of the matrix that tile row `row` maps to (identity unless rows are indirect).
__device__ __forceinline__ float4 gemm_load4(const float* __restrict__ base, size_t ld, int row, size_t grow, int rows_valid, int k0, int K, bool vec_ok) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < rows_valid && k0 < K) {
        const float* p = base + grow * ld + k0;
        if (vec_ok && k0 + 3 < K) {
            v = __ldg(reinterpret_cast<const float4*>(p));
        } else {
            v.x = __ldg(p);
            if (k0 + 1 < K) v.y = __ldg(p + 1);
            if (k0 + 2 < K) v.z = __ldg(p + 2);
            if (k0 + 3 < K) v.w = __ldg(p + 3);
        }
    }
    return v;
}

__device__ __forceinline__ void gemm_store4(float (*dst)[kGemmLd], int kq, int row, float4 v) {
    dst[kq + 0][row] = v.x;
    dst[kq + 1][row] = v.y;
    dst[kq + 2][row] = v.z;
    dst[kq + 3][row] = v.w;
}

// acc[i][j] (+)= sum_{k < K} A[row(tile_row_of(ty,i))][k] * B[tile_col_of(tx,j)][k]
// A, B point at the first row of the tile (A at row 0 of the matrix when INDIRECT, in which case
// row_idx[r] in shared memory names the matrix row of tile row r).  ZERO_ACC clears the accumulators
// first; otherwise the products are added to what they hold, which lets a caller walk the reduction
// dimension in several segments.  Must be called by all 256 threads of the CTA.
template <bool ZERO_ACC, bool INDIRECT>
__device__ __forceinline__ void gemm_tile_nt_ex(
    const float* __restrict__ A, size_t lda, int m_valid, const uint32_t* row_idx, const float* __restrict__ B, size_t ldb, int n_valid, int K, GemmSmem& s,
    float (&acc)[8][8]
) {
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int lr = tid >> 2;         // 0..63
    const int kq = (tid & 3) * 4;    // 0,4,8,12
    const bool vec_a = (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    const bool vec_b = (ldb % 4 == 0) && ((reinterpret_cast<uintptr_t>(B) & 15) == 0);
    if (ZERO_ACC) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    }
    const size_t ga0 = INDIRECT ? ((lr < m_valid) ? row_idx[lr] : 0) : static_cast<size_t>(lr);
    const size_t ga1 = INDIRECT ? ((lr + 64 < m_valid) ? row_idx[lr + 64] : 0) : static_cast<size_t>(lr + 64);

    const int nk = (K + kGemmBK - 1) / kGemmBK;
    float4 ra0 = gemm_load4(A, lda, lr, ga0, m_valid, kq, K, vec_a);
    float4 ra1 = gemm_load4(A, lda, lr + 64, ga1, m_valid, kq, K, vec_a);
    float4 rb0 = gemm_load4(B, ldb, lr, lr, n_valid, kq, K, vec_b);
    float4 rb1 = gemm_load4(B, ldb, lr + 64, lr + 64, n_valid, kq, K, vec_b);
    gemm_store4(s.a[0], kq, lr, ra0);
    gemm_store4(s.a[0], kq, lr + 64, ra1);
    gemm_store4(s.b[0], kq, lr, rb0);
    gemm_store4(s.b[0], kq, lr + 64, rb1);
    __syncthreads();

    for (int ks = 0; ks < nk; ++ks) {
        const int cur = ks & 1;
        const bool more = (ks + 1 < nk);
        if (more) {
            const int k0 = (ks + 1) * kGemmBK + kq;
            ra0 = gemm_load4(A, lda, lr, ga0, m_valid, k0, K, vec_a);
            ra1 = gemm_load4(A, lda, lr + 64, ga1, m_valid, k0, K, vec_a);
            rb0 = gemm_load4(B, ldb, lr, lr, n_valid, k0, K, vec_b);
            rb1 = gemm_load4(B, ldb, lr + 64, lr + 64, n_valid, k0, K, vec_b);
        }
#pragma unroll
        for (int k = 0; k < kGemmBK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&s.a[cur][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&s.a[cur][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&s.b[cur][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&s.b[cur][k][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (more) {
            gemm_store4(s.a[cur ^ 1], kq, lr, ra0);
            gemm_store4(s.a[cur ^ 1], kq, lr + 64, ra1);
            gemm_store4(s.b[cur ^ 1], kq, lr, rb0);
            gemm_store4(s.b[cur ^ 1], kq, lr + 64, rb1);
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void gemm_tile_nt(
    const float* __restrict__ A, size_t lda, int m_valid, const float* __restrict__ B, size_t ldb, int n_valid, int K, GemmSmem& s, float (&acc)[8][8]
) {
    gemm_tile_nt_ex<true, false>(A, lda, m_valid, nullptr, B, ldb, n_valid, K, s, acc);
}

} // namespace skmb
