/*
 * C ABI of the B200 k-means engine (libskm_b200.so).
 *
 * Plain pointers and sizes only; every entry point returns a status code and never throws.  The
 * drop-in C++ classes in include/superkmeans/ and the Python package are thin layers over exactly
 * these functions.  Each declaration names the reference interface it stands in for, by path
 * inside the SuperKMeans repository.
 *
 * Unless a parameter says otherwise, matrices are row-major float32 and live in HOST memory; the
 * `*_on_device` flags switch an argument to device memory of the handle's GPU.
 */
#ifndef SKM_B200_H
#define SKM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct skm_handle skm_handle;

typedef enum skm_status {
    SKM_OK = 0,
    SKM_INVALID_ARGUMENT = 1, /* maps to std::invalid_argument / ValueError */
    SKM_RUNTIME_ERROR = 2,    /* maps to std::runtime_error / RuntimeError */
    SKM_CUDA_ERROR = 3,
    SKM_COMM_ERROR = 4
} skm_status;

/* Field-for-field mirror of SuperKMeansConfig (include/superkmeans/superkmeans.h:23-55) followed by
 * the three fields HierarchicalSuperKMeansConfig adds (include/superkmeans/hierarchical_superkmeans.h:11-17).
 * n_threads is accepted and ignored (there are no CPU worker threads). */
typedef struct skm_config {
    uint32_t iters;
    float sampling_fraction;
    uint32_t max_points_per_cluster;
    uint32_t n_threads;
    uint32_t seed;
    int32_t use_blas_only;
    float tol;
    float recall_tol;
    int32_t early_termination;
    int32_t sample_queries;
    uint64_t objective_k;
    float ann_explore_fraction;
    float min_not_pruned_pct;
    float max_not_pruned_pct;
    float adjustment_factor_for_partial_d;
    int32_t unrotate_centroids;
    int32_t verbose;
    int32_t angular;
    int32_t suppress_warnings;
    int32_t data_already_rotated;
    uint32_t iters_mesoclustering;
    uint32_t iters_fineclustering;
    uint32_t iters_refinement;
} skm_config;

/* Mirror of SuperKMeansIterationStats (superkmeans.h:60-72). */
typedef struct skm_iter_stats {
    uint64_t iteration;
    float objective;
    float shift;
    uint64_t split;
    float recall;
    float not_pruned_pct;
    uint32_t partial_d;
    int32_t is_gemm_only;
} skm_iter_stats;

/* Which list of statistics: SuperKMeans::iteration_stats (superkmeans.h:1492) or one of the three
 * lists of HierarchicalSuperKMeansIterationStats (hierarchical_superkmeans.h:22-26). */
typedef enum skm_stats_phase { SKM_STATS_FLAT = 0, SKM_STATS_MESO = 1, SKM_STATS_FINE = 2, SKM_STATS_REFINE = 3 } skm_stats_phase;

/* Sum-all-reduce of `count` elements at device pointer `buf` across the ranks of a sharded run.
 * dtype: 0 = float32, 1 = float64, 2 = int32.  Must return 0 on success, after the reduced values
 * are visible to work submitted later on any stream of the device. */
typedef int (*skm_allreduce_fn)(void* user, void* buf, uint64_t count, int dtype);

/* Defaults of SuperKMeansConfig{} / HierarchicalSuperKMeansConfig{}. */
void skm_default_config(skm_config* cfg, int hierarchical);

/* Message of the last failure on `h`; with h == NULL, of the last failed skm_create on this thread. */
const char* skm_last_error(const skm_handle* h);

/* SuperKMeans::SuperKMeans / HierarchicalSuperKMeans::HierarchicalSuperKMeans
 * (superkmeans.h:123-140, hierarchical_superkmeans.h:43-66): same validation, same exception
 * classes through the status code.  `device` is the CUDA device ordinal (-1 = current device). */
skm_status skm_create(const skm_config* cfg, uint64_t n_clusters, uint64_t dimensionality, int hierarchical, int device, skm_handle** out);
void skm_destroy(skm_handle* h);

/* The d x d rotation matrix M of ADSamplingPruner (include/superkmeans/pdx/adsampling.h:76-85);
 * Rotate computes X * M^T (:191-215).  Setting it replaces the matrix generated from the seed. */
skm_status skm_set_rotation(skm_handle* h, const float* m);
skm_status skm_get_rotation(skm_handle* h, float* m_out);
/* Replaces the matrix by the rotation of ADSamplingPruner's DCT branch (adsampling.h:53-73, :169-188: random sign
 * flips from the seed, then an orthonormal DCT-II), which the reference uses instead of the QR matrix when it is
 * built with FFTW and d is a power of two >= 512.  Applied as a matrix product here (same values up to fp32
 * rounding, not the O(d log d) cost).  Call before skm_train. */
skm_status skm_use_dct_rotation(skm_handle* h);

/* SuperKMeans::Train / HierarchicalSuperKMeans::Train (superkmeans.h:162-332,
 * hierarchical_superkmeans.h:84-541).  centroids_out: n_clusters x d, host.  data: n x d row-major, host
 * memory, or device memory of the handle's GPU when data_on_device != 0.  queries: n_queries x d in HOST
 * memory, or NULL with n_queries > 0 when config.sample_queries is set (queries are then drawn from the training
 * rows); with queries every iteration's statistics carry recall@objective_k (superkmeans.h:1044-1087) and early
 * termination also watches it (:1315-1331).  Flat algorithm only; objective_k and
 * n_clusters * ann_explore_fraction up to 1536. */
skm_status skm_train(skm_handle* h, const float* data, uint64_t n, int data_on_device, const float* queries, uint64_t n_queries, float* centroids_out);

/* SuperKMeans::Assign (superkmeans.h:346-382).  out: n entries, host (device if *_on_device). */
skm_status skm_assign(skm_handle* h, const float* vectors, const float* centroids, uint64_t n, uint64_t n_centroids, int on_device, uint32_t* out);

/* SuperKMeans::AssignTrainingPoints (superkmeans.h:397-564). */
skm_status skm_assign_training_points(skm_handle* h, const float* vectors, const float* centroids, uint64_t n, uint64_t n_centroids, int on_device, uint32_t* out);

/* GetNClusters, IsTrained, GetSamplingFraction (superkmeans.h:567-573); n_mesoclusters
 * (hierarchical_superkmeans.h:817). */
uint64_t skm_n_clusters(const skm_handle* h);
int skm_is_trained(const skm_handle* h);
float skm_sampling_fraction(const skm_handle* h);
uint64_t skm_n_mesoclusters(const skm_handle* h);

/* How many rows the training state covers: n_samples of Train (superkmeans.h:184, :1269-1277; the reference fills
 * assignments[0 .. n_samples) and distances[0 .. n_samples), :202-207), or n after an AssignTrainingPoints over all
 * rows of a model trained with sampling_fraction = 1.  0 before training. */
uint64_t skm_get_n_samples(const skm_handle* h);

/* iteration_stats / hierarchical_iteration_stats.  Writes at most `cap` entries; *count receives
 * the number available. */
skm_status skm_get_iteration_stats(const skm_handle* h, int phase, skm_iter_stats* out, uint64_t cap, uint64_t* count);

/* Public member `assignments` (superkmeans.h:1491) and GetDistancesPointer (:576): state left by
 * the last training pass, n <= skm_get_n_samples(h) entries each, copied to host. */
skm_status skm_get_assignments(skm_handle* h, uint32_t* out, uint64_t n);
skm_status skm_get_distances(skm_handle* h, float* out, uint64_t n);
/* horizontal_centroids after training: rotated-space centroids, n_clusters x d. */
skm_status skm_get_rotated_centroids(skm_handle* h, float* out);
/* Which kernels the last pruned assignment pass used: 0 none yet, 1 candidate lists (+ dense SIMT chain for
 * flagged points), 3 tensor-core chain, 4 tensor-core first test + list walk (+ tensor-core chain for flagged
 * points), 6 points taken in the order of their previous centroid, every 128-point tile through first test + list
 * walk or through the chain over the centroids its rows can still reach. */
int skm_last_prune_path(const skm_handle* h);
/* Work done by the pruned passes of this handle so far: out3[0] rows sent through a dense chain, out3[1]
 * (pair, 64-dimension block) steps of the candidate-list walk (each reads 256 bytes of a centroid and of a
 * point), out3[2] rows whose candidate list overflowed and were redone densely.  For roofline accounting. */
skm_status skm_get_prune_counters(const skm_handle* h, uint64_t* out3);
/* Work of the chain over gathered centroids (prune path 6) so far: out4[0] rows of the tiles it processed, out4[1]
 * centroid columns its units held (each unit rounded up to a multiple of 16), summed over tiles, passes and
 * units - its tensor-core work is 2 * 128 * out4[1] * d flop, counted once -, out4[2] the points that the
 * optimistic pass flagged (their best candidate can move; they are settled by replaying the search over the
 * candidates the pass recorded) and out4[3] those of them whose candidate lists overflowed and that went through the
 * exact, chunk-by-chunk chain pass instead.  For roofline accounting. */
skm_status skm_get_chain_counters(const skm_handle* h, uint64_t* out4);
/* Objective of the last iteration accumulated in float64 (the reference sums float32). */
double skm_last_objective_f64(const skm_handle* h);

/* Optional per-iteration snapshots of the training state, for step-wise comparison with another
 * implementation: what RunIteration (superkmeans.h:786-879) leaves behind after each call.  Sizes:
 * centroids n_clusters x d (rotated space, after the split), assign / dist n_samples, sizes_pre /
 * sizes_post n_clusters (cluster_sizes before and after SplitClusters).  Any output may be NULL.
 * The reference exposes this state only to subclasses (protected members). */
skm_status skm_set_trace(skm_handle* h, int enabled);
uint64_t skm_trace_count(const skm_handle* h);
skm_status skm_trace_get(const skm_handle* h, uint64_t idx, uint64_t* n_samples, uint64_t* n_clusters, uint32_t* partial_d_next, float* centroids, uint32_t* assign, float* dist,
                         uint32_t* sizes_pre, uint32_t* sizes_post);

/* Device time per phase of the path, measured with CUDA events on the engine's stream and summed
 * since creation or the last reset.  Phases follow the reference profiler's sections
 * (include/superkmeans/profiler.h, SKM_PROFILE_SCOPE names): 0 rotator, 1 norms_calc,
 * 2 search/1st_blas (exact assignment), 3 search (pruned assignment), 4 update_centroids,
 * 5 consolidate, 6 shift, 7 whole Train call; parts of phase 3: 8 first ADSampling test on the tensor cores,
 * 9 candidate-list walk, 10 chains (union pass, chain over gathered centroids, dense chain, their refinement);
 * 11 device allocation and release (host wall clock), 12 initial centroids (Forgy shuffle, row gather, rotation),
 * 13 sums across shards (the span of the collective on the stream, which includes waiting for the slowest shard),
 * 14 reserved. */
skm_status skm_get_phase_time(const skm_handle* h, int phase, double* ms, uint64_t* calls);
skm_status skm_reset_phase_times(skm_handle* h);
/* Process-wide choice between the tcgen05 tensor-core kernels (1, default) and the fp32 SIMT kernels
 * (0) for the dense products; both give fp32-accurate results.  Meant for profiling and A/B checks.
 * No counterpart in the reference (it delegates to whatever BLAS is linked). */
void skm_set_tensor_cores(int enabled);
int skm_get_tensor_cores(void);
/* Which kernels a pruned assignment pass uses.  0 (default): with rows that TMA can address (d % 4 == 0) the share of
 * pairs that survive the first test is estimated on 128 sampled centroids; below 2.5 % (or with fewer than 32 points per cluster, or fewer than 262 144 points) every point takes the
 * tensor-core first test + list walk in the original order (points that keep many centroids alive go through the dense
 * chain instead: the choice of 9), otherwise (and k <= 65536) the points are taken in the order of their previous
 * centroid and every tile of 128 goes through the chain over the centroids its rows can still reach (the choice of
 * 10); SIMT candidate lists when TMA cannot address the rows.  1 SIMT candidate lists for all points; 2 dense SIMT
 * chain for all; 3 dense tensor-core chain for all; 4 tensor-core first test + list walk for all, original order; 5 as
 * 4 with a quarter of the list capacity, so that overflowing lists take their fallback; 6 ordered points, exact
 * gathered chain for every tile; 7 ordered points, first test + list walk for every tile; 8 as 7 with the small lists
 * of 5; 9 unordered: dense chain for all points when the sampled survival is high, else first test + list walk with
 * flagged points on the dense chain; 10 ordered points, every tile through the optimistic chain pass (all thresholds
 * from the distance to the previous centroid, the 1024-centroid chunks ignored) followed by the exact gathered chain
 * for the points whose best candidate moves; 11 ordered points, per tile either first test + list walk or (tiles with
 * many expensive points, and tiles whose lists overflow) the chain as in 10.  The results do not depend on the choice
 * (up to fp32 rounding); it exists for profiling and for testing each kernel on its own.  No counterpart in the
 * reference. */
void skm_set_prune_split(int mode);
int skm_get_prune_split(void);
/* Test hook for the failure path of the tensor-core kernels (current device).  Every wait inside those kernels is
 * bounded: when it runs out the kernel records a code, all of its roles leave their loops, tensor memory is released
 * and the kernel returns; the call that launched it then reports SKM_CUDA_ERROR and the context stays usable.  This
 * hook shortens the limit to wait_limit_cycles SM cycles (0 = back to the default of about two seconds) and makes the
 * TMA producer of the exact-assignment kernel stop after producer_stops_after_kblocks k-blocks (0 = never), so that
 * a test can watch that path without a fault or a hang.  No counterpart in the reference. */
skm_status skm_debug_wait_injection(uint64_t wait_limit_cycles, uint32_t producer_stops_after_kblocks);

/* Profiling aid for the chain over gathered centroids (current device): SM cycles its roles spent waiting, summed over
 * the CTAs of all launches since the last call, then cleared.  out16: [0] MMA thread waiting for the rows to hand an
 * accumulator back, [1] waiting for a stage, [2] its whole loop; [3] a row warp waiting for an accumulator, [4] fetching
 * centroid norms, [5] its whole loop, [6] waiting for its partner at chunk ends; [7] a gather thread waiting for a free
 * stage, [8] for its copies, [9] its whole loop; [10] an X splitter waiting for its tile; [11] the producer waiting for
 * a free stage; [12] (unit, segment) steps; [13] CTAs.  No counterpart in the reference. */
skm_status skm_debug_role_cycles(uint64_t* out16);

/* Kernels launched by this library in the calling process so far. */
uint64_t skm_kernel_launches(void);
/* Device and pinned-host allocations (cudaMalloc, cudaMallocHost) made by this library in the calling process so
 * far.  Lets a caller check that a code path allocates nothing.  No counterpart in the reference. */
uint64_t skm_device_allocations(void);

/* Sharded training: this handle holds rows [row_offset, row_offset + n_local) of a global data set
 * of n_global rows; per-iteration sums, counts and scalars are combined through `fn`.  The
 * reference has no counterpart (single process). */
skm_status skm_set_shard(skm_handle* h, uint64_t n_global, uint64_t row_offset, skm_allreduce_fn fn, void* user);

/* The same with the sums done by NCCL inside this library, on the engine's own stream and as one launch per
 * iteration (k x d sums, k counts and two scalars in one NCCL group): no callback, no host synchronisation around the
 * collective, no Python.  NCCL is opened at run time (libnccl.so.2 from the loader's search path or $SKM_NCCL_LIB);
 * there is no link-time dependency.  One rank calls skm_comm_unique_id and passes the 128 bytes to every rank by
 * whatever means the application has (MPI, a file, torch.distributed); every rank then calls skm_comm_create (a
 * collective) with the device it trains on.  skm_comm_wrap adopts an ncclComm_t that the application already owns.
 * A communicator outlives the handles that use it and is destroyed by the caller.  No counterpart in the reference. */
typedef struct skm_comm skm_comm;
#define SKM_COMM_ID_BYTES 128
skm_status skm_comm_unique_id(uint8_t* id_out);
skm_status skm_comm_create(const uint8_t* id, int rank, int world, int device, skm_comm** out);
skm_status skm_comm_wrap(void* nccl_comm, int rank, int world, skm_comm** out);
void skm_comm_destroy(skm_comm* comm);
skm_status skm_set_shard_comm(skm_handle* h, uint64_t n_global, uint64_t row_offset, skm_comm* comm);

/* Workspace cache (off by default).  When on, device buffers of 32 MB and more that a handle releases (the rotated
 * copy of the training rows, sort and list workspaces) are kept by the library and reused by later calls that need
 * about the same size on the same GPU, so that repeated Train calls of one shape do not pay cudaMalloc / cudaFree of
 * tens of gigabytes (both synchronise the device) every time.  The memory stays with the library until
 * skm_release_cached_memory, skm_set_workspace_cache(0) or the end of the process; an allocation that fails drops the
 * cache and retries.  No counterpart in the reference. */
void skm_set_workspace_cache(int enabled);
int skm_get_workspace_cache(void);
void skm_release_cached_memory(void);
uint64_t skm_cached_memory_bytes(void);

/* ---- single operators of the path, for callers that hold their own state and for parity tests.
 * All arguments in host memory; each call uploads, runs the kernels and downloads. ------------- */

/* ADSamplingPruner::Rotate, matrix branch (adsampling.h:191-215): out = x * m^T. */
skm_status skm_op_rotate(int device, const float* m, const float* x, uint64_t n, uint64_t d, float* out);
/* ADSamplingPruner::Unrotate, matrix branch (adsampling.h:273-298): out = x * m. */
skm_status skm_op_unrotate(int device, const float* m, const float* x, uint64_t n, uint64_t d, float* out);
/* BatchComputer::FindNearestNeighbor (include/superkmeans/distance_computers/batch_computers.h:104-171)
 * with the norms of SuperKMeans::Assign. */
skm_status skm_op_find_nearest(int device, const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, uint32_t* out_knn, float* out_dist);
/* BatchComputer::FindNearestNeighborWithPruning (batch_computers.h:297-409) on rotated inputs;
 * knn_io holds the previous assignment on entry.  not_pruned_out: per-point survivor counts. */
skm_status skm_op_find_nearest_pruned(int device, const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, float epsilon0, uint32_t partial_d,
                                      uint32_t* knn_io, float* dist_out, uint64_t* not_pruned_out);
/* SuperKMeans::UpdateCentroids + ComputeCost (superkmeans.h:729-765, :973-981): per-cluster row
 * sums and sizes, and the float64 sum of `dist` (dist and wcss_out may be NULL). */
skm_status skm_op_update_centroids(int device, const float* x, const uint32_t* assign, const float* dist, uint64_t n, uint64_t k, uint64_t d, float* sums_out,
                                   uint32_t* counts_out, double* wcss_out);
/* PDXLayout::PDXify<false> (include/superkmeans/pdx/layout.h:155-232). */
skm_status skm_op_pdxify(int device, const float* in, uint64_t n, uint64_t d, float* out);

/* Exact nearest-centroid assignment that allocates nothing.  No counterpart in the reference (which
 * allocates freely on the host); the result is that of skm_op_find_nearest.
 *
 * For callers that cannot call cudaMalloc: code running inside a process whose own pool took the GPU's
 * memory at start-up, and latency-critical loops that cannot afford the device-wide synchronisation an
 * allocation or a free implies.  x_dev [n][d], y_dev [k][d], out_knn_dev [n] and out_dist_dev [n] are DEVICE
 * memory of `device` (-1 = the current device) supplied by the caller; cuda_stream is a cudaStream_t (NULL =
 * the default stream).  The call returns after the outputs are written (it synchronises that stream).
 *
 * The intermediate data (norms, candidate pairs, a status word) live in one fixed array in the library's
 * device image, about 3.3 MiB, which every GPU that loads the library holds until the process exits.  Hence:
 *   - n <= SKM_NOALLOC_MAX_ROWS and k <= SKM_NOALLOC_MAX_CENTROIDS, else SKM_INVALID_ARGUMENT (split a
 *     larger batch of rows into several calls); d is not limited;
 *   - every call uses the same array: calls whose kernels can overlap on one GPU (two streams, two
 *     threads) race with each other and must be serialised by the caller;
 *   - the first call on a device looks the array's address up; make that call before any stream
 *     capture starts. */
#define SKM_NOALLOC_MAX_ROWS 262144
#define SKM_NOALLOC_MAX_CENTROIDS 65536
skm_status skm_op_find_nearest_noalloc(int device, const float* x_dev, const float* y_dev, uint64_t n, uint64_t k, uint64_t d, uint32_t* out_knn_dev, float* out_dist_dev,
                                       void* cuda_stream);

/* ---- host-side decisions of the path (no GPU needed) ---------------------------------------- */

/* PDXLayout::GetDimensionSplit (layout.h:115-140). */
void skm_host_dimension_split(uint64_t d, uint64_t* horizontal_d, uint64_t* vertical_d);
/* ADSamplingPruner::InitializeRatios (adsampling.h:93-99): d + 1 floats. */
void skm_host_ratios(uint64_t d, float epsilon0, float* out);
/* Forgy indices of GenerateCentroids (superkmeans.h:1110-1123): k indices. */
void skm_host_forgy_indices(uint64_t n_points, uint64_t k, uint32_t seed, uint64_t* out);
/* SplitClusters (superkmeans.h:890-928; hierarchical_superkmeans.h:579-678): updates sizes in
 * place, writes up to `cap` operations as (dst, src, kind) triples, returns n_split through
 * *n_split and the number of operations through *n_ops. */
skm_status skm_host_split_clusters(uint32_t* sizes, uint64_t n_samples, uint64_t n_clusters, uint32_t seed, int hierarchical, uint32_t* ops_out, uint64_t cap, uint64_t* n_ops,
                                   uint64_t* n_split);
/* TunePartialD (superkmeans.h:1230-1258): returns the new d'. */
uint32_t skm_host_tune_partial_d(double not_pruned_total, uint64_t n_samples, uint64_t n_y, uint32_t partial_d, uint32_t vertical_d, float min_pct, float max_pct,
                                 float adjustment, float* avg_out);
/* ArrangeFineClusters (hierarchical_superkmeans.h:718-761). */
void skm_host_arrange_fine_clusters(uint64_t n_clusters, uint64_t n_meso, uint64_t n_samples, const uint32_t* meso_sizes, uint64_t* out);
/* Offset of (row, dim) in the PDX-blocked copy (layout.h:155-232). */
uint64_t skm_host_pdx_offset(uint64_t row, uint64_t dim, uint64_t n, uint64_t d);
/* The seed-derived rotation matrix (adsampling.h:76-85), d x d row-major. */
void skm_host_rotation_matrix(uint64_t d, uint32_t seed, float* out);
/* The sign-flip + DCT-II rotation of the reference's FFTW branch as a matrix (adsampling.h:53-73, :169-188). */
void skm_host_dct_rotation_matrix(uint64_t d, uint32_t seed, float* out);

#ifdef __cplusplus
}
#endif

#endif /* SKM_B200_H */
