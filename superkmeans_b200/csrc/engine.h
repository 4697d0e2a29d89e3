// Host orchestration of the k-means hot path: owns the device state and drives the kernels in the
// same order as the reference's Train / RunIteration / Assign / AssignTrainingPoints.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <functional>
#include <vector>

#include "../../include/skm_b200.h"
#include "common.cuh"
#include "comm_nccl.h"
#include "host_logic.h"

namespace skmb {

template <class T>
class DeviceBuffer {
  public:
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { release(); }
    void release() {
        if (p_) device_free(p_, bytes_);
        p_ = nullptr;
        cap_ = 0;
        bytes_ = 0;
    }
    // Grows (never shrinks) to at least `count` elements; contents are not preserved on growth.
    T* ensure(size_t count) {
        if (count > cap_) {
            release();
            bytes_ = sizeof(T) * (count ? count : 1);
            p_ = static_cast<T*>(device_alloc(bytes_));
            cap_ = count;
        }
        return p_;
    }
    T* get() const { return p_; }
    size_t capacity() const { return cap_; }
    void swap(DeviceBuffer& o) {
        std::swap(p_, o.p_);
        std::swap(cap_, o.cap_);
        std::swap(bytes_, o.bytes_);
    }

  private:
    T* p_ = nullptr;
    size_t cap_ = 0;
    size_t bytes_ = 0;
};

template <class T>
class PinnedBuffer {
  public:
    PinnedBuffer() = default;
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    ~PinnedBuffer() { release(); }
    void release() {
        if (p_) cudaFreeHost(p_);
        p_ = nullptr;
        cap_ = 0;
    }
    T* ensure(size_t count) {
        if (count > cap_) {
            release();
            note_device_alloc();
            SKM_CUDA(cudaMallocHost(&p_, sizeof(T) * (count ? count : 1)));
            cap_ = count;
        }
        return p_;
    }
    T* get() const { return p_; }

  private:
    T* p_ = nullptr;
    size_t cap_ = 0;
};

// Accumulating per-phase device timers (CUDA events on the engine's stream); names follow the
// sections of the reference's profiler (profiler.h): rotator, norms_calc, search/1st_blas, search,
// update_centroids, consolidate, shift.
// The last three are parts of the pruned assignment: first ADSampling test on the tensor cores, candidate-list walk, dense chain.
// Then four spans that no kernel phase covers: device allocation and release (host wall clock), the initial centroids (Forgy
// shuffle on the host, row gather, their rotation), the per-iteration sum across shards (device span of the collective,
// which includes waiting for the slowest shard), and host-side work of an iteration between kernels (split decisions,
// statistics, synchronisation).
enum Phase { PH_ROTATE = 0, PH_NORMS, PH_ASSIGN_FULL, PH_ASSIGN_PRUNED, PH_UPDATE, PH_CONSOLIDATE, PH_SHIFT, PH_TRAIN_TOTAL, PH_PRUNE_FIRST_TEST, PH_PRUNE_WALK, PH_PRUNE_DENSE,
             PH_ALLOC_FREE, PH_INIT_CENTROIDS, PH_ALLREDUCE, PH_HOST_OTHER, PH_COUNT };

class PhaseTimers {
  public:
    ~PhaseTimers();
    void begin(int phase, cudaStream_t s);
    void end(cudaStream_t s);
    void flush();  // call only after the stream has been synchronised
    void reset();
    void add_host(int phase, double milliseconds) {
        ms[phase] += milliseconds;
        calls[phase] += 1;
    }
    double ms[PH_COUNT] = {};
    uint64_t calls[PH_COUNT] = {};

  private:
    struct Pending {
        int phase;
        cudaEvent_t a, b;
    };
    cudaEvent_t get();
    std::vector<Pending> pending_;
    std::vector<Pending> open_;
    std::vector<cudaEvent_t> pool_;
};

// Device buffers of one pruned assignment pass (candidate lists, work split) and the pass itself:
// preparation, candidate-list kernel for the cheap points, dense chain for the expensive ones.
struct PrunePassBuffers {
    DeviceBuffer<uint2> lists, top2;
    DeviceBuffer<float> best, sample, sample_norms, chain_norms_y;
    DeviceBuffer<float> chain_norms_x;
    DeviceBuffer<uint32_t> flags, positions, hard_idx, n_hard_dev;
    DeviceBuffer<uint2> tc_lists, listed_top2;
    DeviceBuffer<uint32_t> tc_list_offs, redo, listed_knn, listed_np;
    DeviceBuffer<float> listed_x, listed_best, listed_dist, listed_norms, y_split;
    DeviceBuffer<unsigned long long> alive_total;
    PinnedBuffer<unsigned long long> counters_host;
    double last_survival = 0;   // share of sampled (point, centroid) pairs that passed the first test in the last automatic choice
    int last_path = 0;   // 1 lists (+ dense for flagged points), 3 tensor-core chain, 4 tensor-core first test + list walk
    int grid = 0;
    size_t last_n_hard = 0;
    size_t last_n_redo = 0;   // points whose candidate list overflowed (path 4)
    // running totals since the buffers were created: rows sent through a dense chain, (pair, 64-dimension block)
    // steps of the list walk, rows whose list overflowed
    unsigned long long total_dense_rows = 0, total_pair_steps = 0, total_redo_rows = 0;
    DeviceBuffer<unsigned long long> pair_steps_dev;
    // the pass over the points in the order of their previous centroid (paths 6-8)
    UpdateWorkspace sort_ws;
    DeviceBuffer<uint32_t> sort_keys_a, sort_keys_b, sort_vals_a, sort_vals_b, sort_table;
    DeviceBuffer<float> xb, best_b, dist_b, nx_b;
    DeviceBuffer<uint32_t> knn_b, prev_b, np_b, flags_b, tile_flags, tile_map_dense, tile_map_lists, union_bits, col_counts, dirty_b, redo_prev, tile_iota;
    DeviceBuffer<float> redo_nx;
    DeviceBuffer<uint16_t> cols;
    DeviceBuffer<uint2> top2_b;
    DeviceBuffer<unsigned long long> sparse_cols_dev;
    PinnedBuffer<uint32_t> tile_flags_host, tile_map_host;
    // totals since creation: rows of tiles sent through the gathered chain, centroid columns (rounded to 16) its units
    // held, summed over tiles and chunks - the chain's tensor-core work is 2 * 128 * columns * d flop (counted once)
    unsigned long long total_sparse_rows = 0, total_sparse_cols = 0;
    unsigned long long total_redone_rows = 0;   // points the optimistic chain pass flagged (settled by the candidate replay)
    unsigned long long total_fallback_rows = 0; // ... of which the candidate lists overflowed: redone by the exact chain pass
    DeviceBuffer<uint32_t> cand, cand_meta, replay_ovf, replay_np, positions2, hard_idx2, hard_idx3, n_hard_dev2;
    DeviceBuffer<float> replay_thr;
};
// mode: 0 = automatic: with rows that TMA can address, the points are taken in the order of their previous centroid and
// every tile of 128 goes either through the first test + list walk or, when many of its points keep a large share of
// the centroids alive, through the chain over the centroids its rows can still reach; SIMT candidate lists otherwise.
// 1 = SIMT candidate lists for every point, 2 = dense SIMT chain for every point, 3 = dense tensor-core chain for every
// point, 4 = tensor-core first test + list walk for every point (original order), 5 = as 4 with the list capacity cut
// to a quarter so that the overflow route runs, 6 = ordered points, gathered chain for every tile, 7 = ordered points,
// first test + list walk for every tile (overflowing tiles through the gathered chain), 8 = as 7 with the small lists
// of mode 5, 9 = the automatic choice without ordering (dense chain for all points when the sampled survival rate is
// high, else first test + list walk with flagged points on the dense chain), 10 = ordered points, every tile through
// the optimistic chain pass with the exact gathered chain for the points it flags (mode 0 does the same for the tiles
// it sends to the chain; mode 6 uses the exact gathered chain alone).
void set_prune_split_mode(int mode);
int prune_split_mode();
void run_pruned_pass_on(PrunedParams p, PrunePassBuffers& b, float ratio_first, int device, cudaStream_t stream, PhaseTimers* timers = nullptr);

class Engine {
  public:
    Engine(const skm_config& cfg, size_t n_clusters, size_t d, bool hierarchical, int device);
    ~Engine();

    void set_rotation(const float* m_host);
    void get_rotation(float* m_out);
    void set_shard(size_t n_global, size_t row_offset, skm_allreduce_fn fn, void* user);
    void set_shard_nccl(size_t n_global, size_t row_offset, NcclComm* comm);

    void train(const float* data, size_t n, bool on_device, const float* queries, size_t n_queries, float* centroids_out);
    void assign(const float* vectors, const float* centroids, size_t n, size_t n_centroids, bool on_device, uint32_t* out);
    void assign_training_points(const float* vectors, const float* centroids, size_t n, size_t n_centroids, bool on_device, uint32_t* out);

    void get_assignments(uint32_t* out, size_t n);
    void get_distances(float* out, size_t n);
    void get_rotated_centroids(float* out);

    size_t n_clusters() const { return k_; }
    size_t dimensionality() const { return d_; }
    const skm_config& config() const { return cfg_; }
    bool trained() const { return trained_; }
    float sampling_fraction() const { return cfg_.sampling_fraction; }
    size_t n_mesoclusters_value() const { return n_meso_; }
    // rows whose assignment and distance the last training pass left behind (n_samples of Train; n after a full AssignTrainingPoints)
    size_t n_state_rows() const { return n_state_rows_; }
    double last_objective_f64() const { return last_cost_f64_; }
    int last_prune_path() const { return prune_bufs_.last_path; }
    void prune_counters(uint64_t out[3]) const {
        out[0] = prune_bufs_.total_dense_rows;
        out[1] = prune_bufs_.total_pair_steps;
        out[2] = prune_bufs_.total_redo_rows;
    }
    void chain_counters(uint64_t out[4]) const {
        out[0] = prune_bufs_.total_sparse_rows;
        out[1] = prune_bufs_.total_sparse_cols;
        out[2] = prune_bufs_.total_redone_rows;
        out[3] = prune_bufs_.total_fallback_rows;
    }
    const std::vector<skm_iter_stats>& stats(int phase) const;
    int device() const { return device_; }
    // Per-iteration snapshots for step-wise parity checks (what RunIteration leaves behind).
    struct Snapshot {
        uint64_t n_samples = 0, n_clusters = 0;
        uint32_t partial_d_next = 0;
        std::vector<float> centroids;
        std::vector<uint32_t> assign;
        std::vector<float> dist;
        std::vector<uint32_t> sizes_pre, sizes_post;
    };
    void set_trace(bool on) { trace_on_ = on; }
    const std::vector<Snapshot>& trace() const { return trace_; }
    const PhaseTimers& timers() const { return timers_; }
    void reset_timers() { timers_.reset(); }

    // Stateless operators (used by the skm_op_* entry points).
    static void op_rotate(int device, const float* m, const float* x, size_t n, size_t d, float* out, bool inverse);
    static void op_find_nearest(int device, const float* x, const float* y, size_t n, size_t k, size_t d, uint32_t* out_knn, float* out_dist);
    static void op_find_nearest_pruned(int device, const float* x, const float* y, size_t n, size_t k, size_t d, float eps0, uint32_t partial_d, uint32_t* knn_io, float* dist_out,
                                       uint64_t* not_pruned_out);
    static void op_update(int device, const float* x, const uint32_t* assign, const float* dist, size_t n, size_t k, size_t d, float* sums_out, uint32_t* counts_out, double* wcss_out);
    static void op_pdxify(int device, const float* in, size_t n, size_t d, float* out);

  private:
    struct IterationInput {
        const float* x;       // device, rotated, n_samples x d
        size_t n_samples;     // local rows
        size_t n_samples_global;
        size_t n_clusters;
        float* norms;         // device, full or partial norms of x (rewritten when d' changes)
    };

    void ensure_rotation();
    // after_rows(r0, cnt), if given, is called (host side, work enqueued on stream_) whenever rows [r0, r0 + cnt) of dst
    // have been enqueued, in order, in pieces of at least `piece` rows: lets the caller's kernels run between the
    // copies of a host source instead of after them.
    void rotate_to_device(const float* src, bool src_on_device, size_t n, float* dst, const std::function<void(size_t, size_t)>& after_rows = nullptr,
                          size_t piece = 0);
    void upload_rows(const float* src, bool src_on_device, size_t n, float* dst);
    void prepare_update_workspace(size_t n, size_t k);
    void run_iteration(bool gemm_only, const IterationInput& in, size_t iter_idx, bool is_first, std::vector<skm_iter_stats>& target);
    void run_pruned_pass(const float* x, size_t n, size_t k_cur, const float* y, const float* norms_x, const float* norms_y, uint32_t* knn, float* dist, uint32_t* not_pruned);
    void consolidate(size_t n_samples_global, size_t k_cur);
    // `precomputed`: the Forgy indices when the caller has already drawn them (on another thread, while buffers were allocated)
    void generate_centroids_from_host(const float* data, bool on_device, size_t n_points_global, size_t k_cur, bool rotate, const std::vector<size_t>* precomputed = nullptr);
    bool sharded_() const { return allreduce_fn_ != nullptr || comm_ != nullptr; }
    void generate_centroids_from_device_rows(const float* dev_rows, size_t n_points, size_t k_cur, const std::vector<size_t>* precomputed = nullptr);
    void train_flat(const float* data, size_t n, bool on_device, const float* queries, size_t n_queries, float* centroids_out);
    void prepare_recall(const float* queries, size_t n_queries, bool rotate);
    float compute_recall(size_t k_cur);
    void train_hierarchical(const float* data, size_t n, bool on_device, float* centroids_out);
    void output_centroids(float* out_host);
    void allreduce(void* buf, size_t count, int dtype);
    void allreduce_iteration(float* sums, size_t n_sums, uint32_t* counts, size_t n_counts, double* scalars, size_t n_scalars);
    void sync() {
        SKM_CUDA(cudaStreamSynchronize(stream_));
        timers_.flush();
    }
    struct PhaseScope {
        Engine& e;
        PhaseScope(Engine& eng, int phase) : e(eng) { e.timers_.begin(phase, e.stream_); }
        ~PhaseScope() { e.timers_.end(e.stream_); }
    };
    PhaseTimers timers_;
    bool trace_on_ = false;
    std::vector<Snapshot> trace_;

    skm_config cfg_;
    size_t k_, d_;
    bool hierarchical_;
    int device_;
    cudaStream_t stream_ = nullptr;
    cudaStream_t copy_stream_ = nullptr;

    // sharding
    size_t shard_n_global_ = 0, shard_row_offset_ = 0;
    skm_allreduce_fn allreduce_fn_ = nullptr;
    void* allreduce_user_ = nullptr;
    NcclComm* comm_ = nullptr;          // when set, the sums go through NCCL on the engine's stream (comm_nccl.h)
    DeviceBuffer<float> init_raw_;      // initial centroids before rotation
    DeviceBuffer<uint64_t> init_idx_dev_;
    PinnedBuffer<uint64_t> init_idx_host_;
    PinnedBuffer<float> init_rows_host_;

    // pruner state
    float epsilon0_;
    std::vector<float> rotation_host_;  // d x d, empty until needed
    bool rotation_ready_ = false;
    DeviceBuffer<float> m_dev_, mt_dev_, ratios_dev_;
    uint32_t vertical_d_ = 0, horizontal_d_ = 0, partial_d_ = 0;

    // iteration state
    bool trained_ = false;
    bool first_assign_done_ = false;   // the exact assignment of iteration 1 already ran, piecewise, during the upload
    size_t n_samples_ = 0;      // rows held locally
    size_t n_state_rows_ = 0;   // valid entries of assignments_ / distances_
    size_t n_split_ = 0;
    float prev_cost_ = 0.f, cost_ = 0.f, shift_ = 0.f;
    double last_cost_f64_ = 0.0;
    size_t n_meso_ = 0;

    DeviceBuffer<float> x_rot_;          // training rows (rotated)
    DeviceBuffer<float> data_norms_;     // full or partial norms of the training rows
    DeviceBuffer<float> c_cur_, c_prev_; // row-major centroids (horizontal_centroids / prev_centroids)
    DeviceBuffer<float> c_pdx_, c_aux_;  // PDX-blocked copy and first-vertical_d copy
    DeviceBuffer<float> centroid_norms_;
    DeviceBuffer<uint32_t> counts_;
    DeviceBuffer<uint32_t> assignments_, not_pruned_;
    DeviceBuffer<float> distances_;
    PrunePassBuffers prune_bufs_;
    std::vector<float> ratios_host_;
    DeviceBuffer<uint2> top2_;           // candidate pairs of the tensor-core exact assignment
    DeviceBuffer<float> y_split_;        // centroids split into tf32 hi / lo parts for the tensor-core kernels
    // training with query vectors (recall after every iteration)
    size_t n_queries_ = 0, centroids_to_explore_ = 0;
    DeviceBuffer<float> queries_rot_, query_norms_, topk_dots_;
    DeviceBuffer<uint32_t> gt_idx_, promising_, recall_found_;
    DeviceBuffer<unsigned long long> topk_state_;
    PinnedBuffer<uint32_t> recall_found_host_;
    float recall_ = 0.0f;
    DeviceBuffer<SplitOpDev> split_ops_dev_;
    DeviceBuffer<double> scalars_dev_;   // [0] wcss, [1] not-pruned total (as double), [2] shift
    DeviceBuffer<unsigned long long> np_total_dev_;
    PinnedBuffer<double> scalars_host_;
    PinnedBuffer<uint32_t> counts_host_;
    std::vector<uint32_t> sizes_host_;   // cluster_sizes after the last split

    // update workspace
    UpdateWorkspace ws_;
    DeviceBuffer<uint32_t> ws_keys_a_, ws_keys_b_, ws_vals_a_, ws_vals_b_, ws_table_, ws_offsets_;
    DeviceBuffer<float> ws_partials_;
    DeviceBuffer<double> ws_block_sums_;

    // hierarchical extras
    DeviceBuffer<float> full_norms_;      // immutable_data_norms
    DeviceBuffer<float> meso_buffer_;
    DeviceBuffer<float> meso_norms_;
    DeviceBuffer<uint64_t> meso_indices_dev_;
    DeviceBuffer<uint32_t> final_assignments_;
    DeviceBuffer<float> final_centroids_;

    // sampling
    std::vector<size_t> sampled_indices_;

    std::vector<skm_iter_stats> stats_flat_, stats_meso_, stats_fine_, stats_refine_;
};

} // namespace skmb
