// Shared declarations of the CUDA side: error handling, launch parameter structs and the
// launcher prototypes implemented in kernels.cu and used by engine.cu.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace skmb {

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char* what, const char* file, int line) {
    if (e != cudaSuccess) {
        throw CudaError(std::string(what) + ": " + cudaGetErrorString(e) + " (" + file + ":" + std::to_string(line) + ")");
    }
}
#define SKM_CUDA(x) ::skmb::cuda_check((x), #x, __FILE__, __LINE__)

unsigned long long kernel_launch_count();
void note_kernel_launch();
// Device and pinned-host allocations made by this library in the calling process so far (every cudaMalloc /
// cudaMallocHost goes through DeviceBuffer, PinnedBuffer or a site that calls note_device_alloc).
unsigned long long device_alloc_count();
void note_device_alloc();

// Device memory of DeviceBuffer.  With the workspace cache switched on (off by default), blocks of 32 MB and more are
// kept when released and handed out again to later requests of about the same size on the same device, so that
// repeated Train calls of one shape do not pay cudaMalloc / cudaFree (both synchronise the device, and both take
// tens of milliseconds at tens of gigabytes) every time.  The price: the memory stays with this library until
// release_cached_memory() or the end of the process.
void* device_alloc(size_t bytes);
void device_free(void* p, size_t bytes);
void set_workspace_cache(bool on);
bool workspace_cache_enabled();
void release_cached_memory();
size_t cached_memory_bytes();
// wall-clock milliseconds this thread has spent inside cudaMalloc / cudaFree through device_alloc / device_free
double alloc_free_ms();
// After every kernel launch: count it and surface launch-configuration errors.
#define SKM_LAUNCH_CHECK()                                                                         \
    do {                                                                                           \
        ::skmb::note_kernel_launch();                                                              \
        SKM_CUDA(cudaGetLastError());                                                              \
    } while (0)

constexpr int kTileM = 128;        // points per CTA tile
constexpr int kTileN = 128;        // centroids per GEMM sub-tile (SIMT path)
constexpr int kChunk = 1024;       // centroids per pruning chunk (reference VECTOR_CHUNK_SIZE)
constexpr int kHBlock = 64;        // dimensions per horizontal block (reference H_DIM_SIZE)
constexpr int kUpdateTile = 1024;  // sorted points per segmented-sum tile

// ---------------------------------------------------------------------------------------------
// Launchers (all asynchronous on `stream`; pointers are device pointers unless stated otherwise)
// ---------------------------------------------------------------------------------------------

// In-place exclusive scan of n uint32 values; totals_tmp needs n / 2048 + 1 entries of scratch.
void exclusive_scan_u32(uint32_t* data, size_t n, uint32_t* totals_tmp, cudaStream_t stream);

// out[i] = sum_{j < upto} x[i*ld + j]^2
void launch_row_sqnorms(const float* x, size_t n, size_t ld, size_t upto, float* out, cudaStream_t stream);

// out[n x n_out] = a[n x k_dim] * b[n_out x k_dim]^T, all row-major with leading dimensions lda,
// ldb, ldo (NT GEMM).  Used for rotation (b = M) and un-rotation (b = M^T).
void launch_gemm_nt(const float* a, size_t lda, const float* b, size_t ldb, float* out, size_t ldo, size_t n, size_t n_out, size_t k_dim, cudaStream_t stream);

// out[j*n + i] = in[i*n + j]
void launch_transpose_square(const float* in, float* out, size_t n, cudaStream_t stream);

// Exact nearest centroid: dist = ||x||^2 + ||y||^2 - 2 x.y over all d dims, first minimum inside a
// 1024-centroid batch, strict < across batches, clamped at 0 when stored.
// top2_scratch (n entries, may be null) enables the tensor-core path: tcgen05 pass for the two best
// candidates per row, then an fp32 refinement; without it the fp32 SIMT kernel runs.
// y_split (2 * k * d floats, optional): scratch in which the tensor-core path keeps the centroids split into tf32 parts.
void launch_assign_full(const float* x, const float* y, size_t n, size_t k, size_t d, const float* norms_x, const float* norms_y, uint32_t* out_knn, float* out_dist, uint2* top2_scratch, cudaStream_t stream, float* y_split = nullptr);

struct PrunedParams {
    const float* x;             // n x d rotated points
    const float* y;             // k x d rotated centroids, row-major
    const float* y_pdx;         // k x d PDX-blocked copy of y
    const float* y_aux;         // k x vertical_d row-major copy of the first vertical_d dims
    const float* norms_x;       // partial norms (first partial_d dims)
    const float* norms_y;       // partial norms (first partial_d dims)
    const float* ratios;        // d + 1 ADSampling ratios
    uint32_t* knn;              // in: previous assignment, out: new assignment
    float* dist;                // out: distance to the new assignment
    uint32_t* not_pruned;       // out: per-point count of first-test survivors (added)
    uint2* scratch;             // candidate lists, pruned_scratch_elems() entries
    size_t n, k, d;
    uint32_t partial_d, vertical_d, horizontal_d;
    const float* best_in = nullptr;     // optional: exact distance to the previous centroid, per point
    const uint32_t* skip = nullptr;     // optional: 1 = leave this point to the dense kernel
};

// Work split of one pruned pass.  Points whose ADSampling test would keep a large share of the
// centroids alive (their current centroid is far away, so every threshold is loose) cost one gathered
// 64-dimension block per surviving pair and step in the candidate-list kernel; they are cheaper to
// treat densely.  pruned_prepare computes the exact distance to the previous centroid for every point
// and flags the expensive ones from the survival rate on a sample of 128 centroids;
// assign_pruned_dense runs the same test chain for the flagged points with a tile GEMM over all
// dimensions (no candidate lists).  The split changes only where the work is done, never the result.
struct PruneSplitWorkspace {
    float* best = nullptr;          // n
    uint32_t* flags = nullptr;      // n   (1 = dense)
    uint32_t* positions = nullptr;  // n + scan scratch  (exclusive scan of flags)
    uint32_t* hard_idx = nullptr;   // n
    float* sample = nullptr;        // 128 x d sampled centroid rows
    float* sample_norms = nullptr;  // 128
    float* chain_norms_y = nullptr; // k x n_checkpoints
    uint32_t* n_hard_dev = nullptr; // 1
    unsigned long long* alive_total = nullptr;  // 1: sampled pairs passing the first test
    int n_sample = 128;
    float ratio_first = 1.0f;       // ratios[partial_d], host copy
    uint32_t flag_mult = 16;        // a point is flagged when survivors * flag_mult >= n_sample
};
size_t prune_split_positions_elems(size_t n);
uint32_t prune_chain_checkpoints(uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d);
// out[i] = ||x_i - y_{knn[i]}||^2 accumulated directly in fp32 (no norm trick)
void launch_exact_dist(const float* x, const float* y, const uint32_t* knn, size_t n, size_t d, float* out, cudaStream_t stream);
// Cumulative squared norm of every row of m after each checkpoint of the chain: out[row][j], or
// out[j][row] when `transposed`.
void launch_chain_norms(const float* m, size_t rows, size_t d, uint32_t partial_d, uint32_t vertical_d, uint32_t horizontal_d, bool transposed, float* out,
                        cudaStream_t stream);
// Fills ws.best and ws.flags / ws.hard_idx / *ws.n_hard_dev.
void launch_pruned_prepare(const PrunedParams& p, PruneSplitWorkspace& ws, cudaStream_t stream);
// Runs the dense chain for the n_hard points listed in ws.hard_idx.
void launch_assign_pruned_dense(const PrunedParams& p, PruneSplitWorkspace& ws, size_t n_hard, cudaStream_t stream);

// Replay of the pruned search for the points listed in idx[0 .. n_listed) (rows of x) from the candidates the optimistic
// chain pass recorded for them (kernels_replay.cu).
struct ReplayParams {
    const float* x;              // rows, row-major, d floats each
    const float* y;              // row-major centroids
    const float* ratios;
    const float* best_in;        // per row: exact distance to the previous centroid
    const uint32_t* prev;        // per row: previous centroid
    const uint32_t* idx;         // listed rows
    const uint32_t* cand;        // per row two lists of `cap` centroid indices
    const uint32_t* meta;        // per row: list lengths (bits 0..7, 8..15) and the overflow bit (16)
    uint32_t* knn;               // per row, written when the point moves
    float* dist;
    float* thr;                  // per listed point and chunk of 1024 centroids: best at the chunk's start * ratio[partial_d]
    uint32_t* overflow;          // per listed point: 1 when its lists overflowed (nothing else is decided for it)
    size_t n_listed;
    size_t k;
    uint32_t d;
    uint32_t partial_d;
    uint32_t vertical_d;
    uint32_t horizontal_d;
    uint32_t cap;
};
void launch_replay_candidates(const ReplayParams& p, cudaStream_t stream);
void launch_scatter_u32(const uint32_t* idx, const uint32_t* in, uint32_t* out, size_t n, cudaStream_t stream);       // out[idx[i]] = in[i]
void launch_compose_u32(const uint32_t* outer, const uint32_t* inner, uint32_t* out, size_t n, cudaStream_t stream);  // out[i] = outer[inner[i]]

// Pruned assignment with candidate lists made by the tensor-core first test (kernels_tc.cu) and walked by
// walk_lists_kernel (kernels_walk.cu), for the row tiles [tile0, tile0 + n_tiles) of 128 points.
struct WalkParams {
    const float* x;
    const float* y;              // row-major centroids
    const float* norms_x;        // squared norms of the points over the first partial_d dimensions
    const float* y_pdx;
    const float* y_aux;
    const float* ratios;
    const uint2* lists;          // n_tiles * 8 lists of cap_group entries (see tc::launch_first_test)
    const uint32_t* list_offs;   // n_tiles * 8 * (n_chunks + 1)
    uint32_t cap_group;
    size_t n, k, d;
    uint32_t partial_d, vertical_d, horizontal_d;
    size_t tile0, n_tiles;
    const uint32_t* tile_map = nullptr;   // optional: entry t of the range stands for row tile tile_map[t] (lists stay indexed by t)
    const float* best_in;        // exact distance to the previous centroid
    const uint32_t* skip;        // may be null
    uint32_t* knn;
    float* dist;
    uint32_t* not_pruned;
    uint32_t* redo;              // set to 1 for points whose group list overflowed
    uint32_t* redo_count;
    unsigned long long* pair_steps;            // += pairs advanced by one 64-dimension block
    uint32_t rebalance_mask = 0x22;            // bit b: even the runs out after block b (here: after the 2nd and the 6th)
    const int* upstream_error = nullptr;       // set when the kernel that wrote the lists gave up on a wait: the lists are then not read
};
void launch_walk_lists(const WalkParams& w, int device, cudaStream_t stream);
// hard_idx / *n_hard_dev from an arbitrary flag array (same buffers as launch_pruned_prepare fills)
void launch_compact_flags(const uint32_t* flags, size_t n, PruneSplitWorkspace& ws, cudaStream_t stream);

void launch_gather_listed(const float* x, const float* best, const uint32_t* knn, const uint32_t* idx, size_t n_listed, size_t d, float* x_out, float* best_out,
                          uint32_t* knn_out, cudaStream_t stream);
void launch_scatter_listed(const uint32_t* idx, size_t n_listed, const uint32_t* knn_in, const float* dist_in, const uint32_t* np_in, uint32_t* knn, float* dist,
                           uint32_t* not_pruned, cudaStream_t stream);

// The pass over the points in the order of their previous centroid: a batch of rows order[0 .. cnt) gathered with their
// previous assignment (twice: knn_b is overwritten by the kernels, prev_b is not) and partial norm; the results
// scattered back; per-tile flags from per-row flags; the starting state of the rows of listed tiles; and the sampled
// survival classification alone (ws.best must already hold the exact distances to the previous centroids).
void launch_gather_sorted(const float* x, const uint32_t* order, const uint32_t* knn, const float* norms_x, size_t cnt, size_t d, float* xb, uint32_t* knn_b, uint32_t* prev_b,
                          float* nx_b, cudaStream_t stream);
void launch_scatter_sorted(const uint32_t* order, size_t cnt, const uint32_t* knn_b, const float* dist_b, const uint32_t* np_b, uint32_t* knn, float* dist,
                           uint32_t* not_pruned, cudaStream_t stream);
void launch_tile_flags(const uint32_t* row_flags, size_t n, uint32_t threshold, uint32_t* tile_flags, cudaStream_t stream);
void launch_init_chain_rows(const uint32_t* tile_map, size_t n_tiles, size_t n, const uint32_t* prev, const float* best, uint32_t* knn, float* dist, uint32_t* not_pruned,
                            uint2* top2, cudaStream_t stream);
void launch_classify(const PrunedParams& p, PruneSplitWorkspace& ws, cudaStream_t stream);
void launch_iota_u32(uint32_t* out, size_t n, cudaStream_t stream);   // out[i] = i

// k nearest rows of y for every row of q by ||q||^2 + ||y||^2 - 2 q.y (BatchComputer::FindKNearestNeighbors,
// batch_computers.h:191-274): out_idx / out_dist are n_q x k, ascending by (distance, index); dots_scratch needs
// topk_scratch_floats(n_q) floats, state n_q * k 64-bit words; k <= topk_max_k().
size_t topk_scratch_floats(size_t n_q);
size_t topk_max_k();
void launch_topk_nn(const float* q, const float* y, size_t n_q, size_t n_y, size_t d, const float* norms_q, const float* norms_y, uint32_t k, uint32_t* out_idx,
                    float* out_dist, float* dots_scratch, unsigned long long* state, cudaStream_t stream);
// found[q] = |{j < objective_k : assignments[gt[q][j]] is one of promising[q][0 .. n_explore)}| (superkmeans.h:1063-1086)
void launch_recall_count(const uint32_t* gt, uint32_t objective_k, const uint32_t* promising, uint32_t n_explore, const uint32_t* assignments, size_t n_assignments,
                         size_t n_q, uint32_t* found, cudaStream_t stream);

int pruned_grid_size(int device);
size_t pruned_scratch_elems(int grid);
void launch_assign_pruned(const PrunedParams& p, int grid, cudaStream_t stream);

// Centroid update -------------------------------------------------------------------------------
struct UpdateWorkspace {
    uint32_t* keys_a = nullptr;   // n
    uint32_t* keys_b = nullptr;   // n
    uint32_t* vals_a = nullptr;   // n
    uint32_t* vals_b = nullptr;   // n
    uint32_t* digit_table = nullptr;  // 256 * n_units
    uint32_t* seg_offsets = nullptr;  // k + 1
    float* tile_partials = nullptr;   // n_tiles * 2 * d
    double* block_sums = nullptr;     // reduction partials (>= 1024)
    size_t n_cap = 0, k_cap = 0, d = 0;
};
size_t update_sort_units(size_t n);
size_t update_tiles(size_t n);

// Stable sort of the indices 0 .. n-1 by keys[i] (< k): *sorted_keys_out / *order_out point into the workspace's key and
// value buffers (keys_a/b, vals_a/b, digit_table must be allocated for n).
void launch_sort_by_key(const uint32_t* keys, size_t n, size_t k, UpdateWorkspace& ws, const uint32_t** sorted_keys_out, const uint32_t** order_out, cudaStream_t stream);

// counts[c] = |{i : assign[i] == c}|, sums[c] = sum of x rows assigned to c (deterministic order),
// *wcss = sum_i dist[i] (double), *not_pruned_total = sum_i not_pruned[i] (may be null).
void launch_update(const float* x, const uint32_t* assign, const float* dist, const uint32_t* not_pruned, size_t n, size_t k, size_t d, UpdateWorkspace& ws, float* sums, uint32_t* counts, double* wcss, unsigned long long* not_pruned_total, cudaStream_t stream);

// c[i][:] *= 1/counts[i] for non-empty clusters
void launch_scale_by_counts(float* c, const uint32_t* counts, size_t k, size_t d, cudaStream_t stream);

struct SplitOpDev {
    uint32_t dst, src, kind;
    float wc;
};
void launch_apply_split_ops(float* c, size_t d, const SplitOpDev* ops, size_t n_ops, cudaStream_t stream);
void launch_normalize_rows(float* c, size_t k, size_t d, cudaStream_t stream);

// PDX-blocked copy and first-vertical_d copy of a row-major k x d matrix
void launch_pdxify(const float* c, float* pdx, float* aux, size_t k, size_t d, size_t vertical_d, cudaStream_t stream);

// *out = sum_c ||a[c] - b[c]||^2
void launch_shift(const float* a, const float* b, size_t k, size_t d, double* block_sums, double* out, cudaStream_t stream);

// out[i][:] = in[idx[i]][:]; an index of all ones gives a row of zeros
void launch_gather_rows(const float* in, const uint64_t* idx, float* out, size_t n_out, size_t d, cudaStream_t stream);
void launch_gather_f32(const float* in, const uint64_t* idx, float* out, size_t n_out, cudaStream_t stream);
// out[idx[i]] = in[i] + offset
void launch_scatter_u32_offset(const uint32_t* in, const uint64_t* idx, uint32_t* out, size_t n, uint32_t offset, cudaStream_t stream);

} // namespace skmb
