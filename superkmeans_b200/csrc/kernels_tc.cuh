// Tensor-core (tcgen05 + TMA) variants of the dense kernels; see kernels_tc.cu.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace skmb {
namespace tc {

// Process-wide switch (on by default); off routes every dense kernel to the SIMT implementation.
void set_enabled(bool on);
bool enabled();

// The TMA path needs 16-byte aligned bases and row pitches.
bool eligible(const float* x, size_t ldx, const float* y, size_t ldy);

// top2_scratch: n entries of device scratch (candidate pairs handed from the tensor-core pass to the
// fp32 refinement).
// y_split (2 * k * d floats of scratch, optional): the centroids are split into their tf32 hi and lo parts once, in
// global memory, instead of in shared memory for every tile that uses them.
void launch_assign_full(const float* x, const float* y, size_t n, size_t k, size_t d, const float* norms_x, const float* norms_y, uint32_t* out_knn, float* out_dist,
                        uint2* top2_scratch, cudaStream_t stream, float* y_split = nullptr);
// y_split[0 .. rows*ld) = tf32(y), y_split[rows*ld .. 2*rows*ld) = tf32(y - tf32(y))
void launch_presplit(const float* y, size_t rows, size_t ld, float* y_split, cudaStream_t stream);
// Same two kernels, but the word that a kernel sets when one of its bounded waits runs out is supplied by
// the caller (device memory, zero on entry) instead of coming from this file's lazily allocated per-device word.
void launch_assign_full_flagged(const float* x, const float* y, size_t n, size_t k, size_t d, const float* norms_x, const float* norms_y, uint32_t* out_knn, float* out_dist,
                                uint2* top2_scratch, int* error_word, cudaStream_t stream);
void launch_gemm_nt(const float* a, size_t lda, const float* b, size_t ldb, float* out, size_t ldo, size_t n, size_t n_out, size_t k_dim, cudaStream_t stream);
// out[n][n_out] = a[n][k_dim] * b[n_out][k_dim]^T with the accumulation cut into four chains that are summed in fp32
// registers (kernels_tc_rotate.cu): the rotation and un-rotation GEMM.  out_sqnorms (optional): squared norm of every output row.
void launch_rotate(const float* a, size_t lda, const float* b, size_t ldb, float* out, size_t ldo, size_t n, size_t n_out, size_t k_dim, float* out_sqnorms,
                   cudaStream_t stream);

// First ADSampling test on the tensor cores for the row tiles [tile0, tile0 + n_tiles) of 128 points: partial
// distances over the first partial_d dimensions of every (point, centroid) pair, tested against
// best_in * ratio_first.  Pairs that pass go to one of eight lists per row tile (list h * 4 + q: rows 32q..32q+31,
// columns 128h..128h+127 of every 256-centroid tile) as {centroid << 5 | row in the 32-row group, partial
// distance}, at most cap_group entries per list, in centroid-tile order; list_offs receives, per list, the number
// of entries before every 1024-centroid chunk and the total (which exceeds cap_group on overflow).
void launch_first_test(const float* x, const float* y, size_t n, size_t k, size_t d, uint32_t partial_d, const float* norms_x, const float* norms_y, const float* best_in,
                       const uint32_t* skip, float ratio_first, size_t tile0, size_t n_tiles, uint2* lists, uint32_t* list_offs, uint32_t cap_group, cudaStream_t stream,
                       const float* y_split = nullptr,   // y already split by launch_presplit, optional
                       const uint32_t* tile_map = nullptr);   // optional: entry t of the range stands for row tile tile_map[t]; lists stay indexed by t

// The same first test (threshold widened by 1e-4 relative) for the row tiles tile_map[0 .. n_tiles), keeping only its
// footprint: bit c of union_bits[t * union_words + c / 32] is set (atomic OR into zeroed memory) when some row of tile t
// passes the test against centroid c.  y_split: the centroids split by launch_presplit.
// Counts, for every row of x (n x d, only the first partial_d dimensions are read), the centroids whose partial distance
// is below thr_rows[row * thr_chunks + chunk], chunk = the centroid's block of 1024: the first ADSampling test with a
// threshold per point and chunk.  count_out is zeroed by the call.
void launch_count_first_test(const float* x, size_t n, size_t k, size_t d, uint32_t partial_d, const float* norms_x, const float* norms_y, const float* thr_rows,
                             uint32_t thr_chunks, uint32_t* count_out, const float* y_split, cudaStream_t stream);

void launch_union(const float* x, size_t n, size_t k, size_t d, uint32_t partial_d, const float* norms_x, const float* norms_y, const float* best_in, float ratio_first,
                  const uint32_t* tile_map, size_t n_tiles, uint32_t* union_bits, uint32_t union_words, const float* y_split, cudaStream_t stream);

// Pruned assignment of the row tiles tile_map[0 .. n_tiles) as a chain over the centroids their union bits name
// (kernels_tc_sparse.cu).  For every listed tile and 1024-centroid chunk, cols[t * cols_stride + chunk * 1024 ..] holds
// the col_counts[t * n_chunks + chunk] local indices (ascending) of the chunk's centroids that can pass the first test for
// some row of the tile; all other centroids are skipped, which cannot change the result.  Other arguments as for
// launch_chain; y_split must already hold the split centroids.  Rows of listed tiles whose every chunk is empty keep
// what knn / dist / not_pruned / top2 held on entry.
void launch_sparse_chain(const float* x, size_t n, size_t k, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, const float* chain_norms_x,
                         const float* chain_norms_y, const float* ratios, const float* best_in, uint32_t* knn, float* dist, uint32_t* not_pruned, uint2* top2_scratch,
                         const float* y_split, const uint32_t* tile_map, size_t n_tiles, const uint16_t* cols, const uint32_t* col_counts, size_t cols_stride,
                         cudaStream_t stream, uint32_t* dirty = nullptr, uint32_t* cand = nullptr, uint32_t* cand_meta = nullptr, uint32_t cand_cap = 0);
// With `dirty` the call is the OPTIMISTIC pass instead: cols holds ONE ascending list of global centroid indices per tile
// (launch_build_flat_cols; col_counts = the list lengths, cols_stride >= k <= 65536) and every threshold comes from
// best_in alone, as if no point's best candidate changed during the search.  Written: not_pruned (first-test survivors)
// and dirty (1 = some centroid other than the previous one survived every test and ended below best_in; such a point
// must be redone by the exact call, all others keep their assignment and distance).  knn is only read.
void launch_build_flat_cols(const uint32_t* union_bits, uint32_t union_words, size_t n_tiles, size_t k, uint16_t* cols, uint32_t* totals, size_t cols_stride,
                            unsigned long long* total_cols, cudaStream_t stream);
// Profiling aid: cycles the roles of the gathered chain spent waiting, summed over CTAs since the last call (see kernels_tc_sparse.cu).
void role_cycles(unsigned long long out[16]);
// cols / col_counts from union bits: one warp per (tile, chunk); *total_cols += columns listed (rounded up to the 16 the
// tensor cores process), for work accounting.
void launch_build_cols(const uint32_t* union_bits, uint32_t union_words, size_t n_tiles, size_t k, uint16_t* cols, uint32_t* col_counts, size_t cols_stride,
                       unsigned long long* total_cols, cudaStream_t stream);
// Exact fp32 refinement of the chain's winner and runner-ups (see launch_chain) for the rows of the listed tiles only.
void launch_refine_chain_tiles(const float* x, const float* y, size_t n, size_t k, size_t d, const uint2* top2, uint32_t* knn, float* dist, const uint32_t* tile_map,
                               size_t n_tiles, cudaStream_t stream);

// Pruned assignment for all n points as a dense ADSampling chain on the tensor cores.  chain_norms_x /
// chain_norms_y hold, per row, the cumulative squared norm after each of the chain's checkpoints
// (launch_chain_norms; point norms row-major, centroid norms checkpoint-major); best_in the exact distance to the previous centroid; knn the previous
// assignment on entry and the new one on return.  The winner is settled, and its distance recomputed, in
// fp32 among the chain's winner and its two runner-ups (top2_scratch: n entries).
void launch_chain(const float* x, const float* y, size_t n, size_t k, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, const float* chain_norms_x,
                  const float* chain_norms_y, const float* ratios, const float* best_in, uint32_t* knn, float* dist, uint32_t* not_pruned, uint2* top2_scratch,
                  float* y_split, cudaStream_t stream);   // y_split: 2 * k * d floats of scratch for the tf32 parts of the centroids

// SM cycles after which a wait inside a tensor-core kernel gives up (about two seconds unless a test shortened it).
long long wait_limit();

// Test hook for the bounded waits: every wait of the tensor-core kernels gives up after
// wait_limit_cycles SM cycles (0 restores the default of about two seconds), and the TMA producer of the exact
// assignment kernel stops after producer_stops_after_kblocks k-blocks (0 = never), so that the other roles wait
// for tiles that never arrive.  The kernel then returns with an error code that fetch_error reports.
void set_debug_wait_injection(long long wait_limit_cycles, uint32_t producer_stops_after_kblocks);

// The per-device word (device memory) in which a tensor-core kernel records that one of its waits ran out; kernels that
// consume such a kernel's output read it first and do nothing when it is set.
int* error_word();

// Error code (0 = none) recorded by a kernel whose bounded wait expired; clears it.  Synchronises.
int fetch_error(cudaStream_t stream);

} // namespace tc
} // namespace skmb
