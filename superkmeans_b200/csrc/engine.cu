// Host orchestration: see engine.h.  Every step cites the reference code it reproduces
// (paths relative to the SuperKMeans repository, include/superkmeans/...).
#include "engine.h"

#include <cstdlib>
#include "kernels_tc.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <future>
#include <thread>
#include <atomic>
#include <iostream>
#include <numeric>
#include <random>

namespace skmb {

namespace {

struct DeviceGuard {
    int prev = 0;
    explicit DeviceGuard(int dev) {
        SKM_CUDA(cudaGetDevice(&prev));
        if (prev != dev) SKM_CUDA(cudaSetDevice(dev));
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

__global__ void u64_to_f64_kernel(const unsigned long long* in, double* out) { *out = static_cast<double>(*in); }

__global__ void widen_u32_kernel(const uint32_t* __restrict__ in, uint64_t* __restrict__ out, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i];
}

// Rows per staging chunk when streaming a host matrix through the GPU.
size_t chunk_rows_for(size_t d, size_t n) {
    const size_t target_bytes = size_t{256} << 20;
    size_t rows = std::max<size_t>(1024, target_bytes / (d * sizeof(float)));
    rows = (rows / kTileM) * kTileM;
    return std::max<size_t>(kTileM, std::min(rows, std::max<size_t>(n, 1)));
}

void ensure_positive(bool ok, const char* name) {
    if (!ok) throw std::invalid_argument(std::string("Value must be positive: ") + name);
}

void check_tc_error(cudaStream_t stream) {
    const int code = tc::fetch_error(stream);
    if (code != 0) throw CudaError("a tensor-core kernel gave up waiting on a barrier (code " + std::to_string(code) + ")");
}

int sm_count_of(int device) {
    int sms = 0;
    SKM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    return std::max(sms, 1);
}

int resolve_device(int device) {
    if (device >= 0) return device;
    int cur = 0;
    SKM_CUDA(cudaGetDevice(&cur));
    return cur;
}

} // namespace

// -------------------------------------------------------------------------------------------------
// Phase timers
// -------------------------------------------------------------------------------------------------
PhaseTimers::~PhaseTimers() {
    for (auto& p : pending_) {
        cudaEventDestroy(p.a);
        cudaEventDestroy(p.b);
    }
    for (auto& p : open_) {
        cudaEventDestroy(p.a);
        cudaEventDestroy(p.b);
    }
    for (auto e : pool_) cudaEventDestroy(e);
}

cudaEvent_t PhaseTimers::get() {
    if (!pool_.empty()) {
        cudaEvent_t e = pool_.back();
        pool_.pop_back();
        return e;
    }
    cudaEvent_t e;
    SKM_CUDA(cudaEventCreate(&e));
    return e;
}

void PhaseTimers::begin(int phase, cudaStream_t s) {
    Pending p{phase, get(), get()};
    SKM_CUDA(cudaEventRecord(p.a, s));
    open_.push_back(p);
}

void PhaseTimers::end(cudaStream_t s) {
    if (open_.empty()) return;
    Pending p = open_.back();
    open_.pop_back();
    cudaEventRecord(p.b, s);
    pending_.push_back(p);
}

void PhaseTimers::flush() {
    for (auto& p : pending_) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, p.a, p.b) == cudaSuccess) {
            ms[p.phase] += t;
            calls[p.phase] += 1;
        }
        pool_.push_back(p.a);
        pool_.push_back(p.b);
    }
    pending_.clear();
}

void PhaseTimers::reset() {
    for (int i = 0; i < PH_COUNT; ++i) {
        ms[i] = 0.0;
        calls[i] = 0;
    }
}

// -------------------------------------------------------------------------------------------------
// Construction (superkmeans.h:123-140, hierarchical_superkmeans.h:43-66)
// -------------------------------------------------------------------------------------------------
Engine::Engine(const skm_config& cfg, size_t n_clusters, size_t d, bool hierarchical, int device)
    : cfg_(cfg), k_(n_clusters), d_(d), hierarchical_(hierarchical), device_(0) {
    ensure_positive(n_clusters > 0, "n_clusters");
    ensure_positive(d > 0, "dimensionality");
    ensure_positive(cfg.iters > 0, "config.iters");
    ensure_positive(cfg.sampling_fraction > 0, "config.sampling_fraction");
    if (cfg.sampling_fraction > 1.0) throw std::invalid_argument("sampling_fraction must be <= 1.0");
    if (hierarchical) {
        ensure_positive(cfg.iters_mesoclustering > 0, "config.iters_mesoclustering");
        ensure_positive(cfg.iters_fineclustering > 0, "config.iters_fineclustering");
    }
    if (cfg_.data_already_rotated) cfg_.unrotate_centroids = 0;
    epsilon0_ = hierarchical ? kHierarchicalPrunerInitialThreshold : kPrunerInitialThreshold;
    const DimensionSplit split = dimension_split(d);
    vertical_d_ = static_cast<uint32_t>(split.vertical_d);
    horizontal_d_ = static_cast<uint32_t>(split.horizontal_d);

    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        throw CudaError("no CUDA device is available: this engine has no CPU path");
    }
    device_ = resolve_device(device);
    if (device_ >= count) throw std::invalid_argument("device ordinal out of range");
    DeviceGuard guard(device_);
    SKM_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    SKM_CUDA(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
    ratios_host_ = make_ratios(d, epsilon0_);
    SKM_CUDA(cudaMemcpy(ratios_dev_.ensure(d + 1), ratios_host_.data(), sizeof(float) * (d + 1), cudaMemcpyHostToDevice));
    scalars_dev_.ensure(8);
    np_total_dev_.ensure(1);
    scalars_host_.ensure(8);
    if (hierarchical && n_clusters <= 128 && !cfg.suppress_warnings) {
        std::cout << "WARNING: n_clusters <= 128 is not recommended for HierarchicalSuperKMeans. "
                     "Consider using at least 128 clusters."
                  << std::endl;
    }
}

Engine::~Engine() {
    cudaSetDevice(device_);
    if (stream_) cudaStreamDestroy(stream_);
    if (copy_stream_) cudaStreamDestroy(copy_stream_);
}

const std::vector<skm_iter_stats>& Engine::stats(int phase) const {
    switch (phase) {
        case SKM_STATS_MESO: return stats_meso_;
        case SKM_STATS_FINE: return stats_fine_;
        case SKM_STATS_REFINE: return stats_refine_;
        default: return stats_flat_;
    }
}

// -------------------------------------------------------------------------------------------------
// Rotation (adsampling.h:76-85, :191-215, :273-298)
// -------------------------------------------------------------------------------------------------
void Engine::ensure_rotation() {
    if (rotation_ready_) return;
    if (rotation_host_.empty()) rotation_host_ = make_rotation_matrix(d_, cfg_.seed);
    SKM_CUDA(cudaMemcpyAsync(m_dev_.ensure(d_ * d_), rotation_host_.data(), sizeof(float) * d_ * d_, cudaMemcpyHostToDevice, stream_));
    mt_dev_.ensure(d_ * d_);
    launch_transpose_square(m_dev_.get(), mt_dev_.get(), d_, stream_);
    sync();
    rotation_ready_ = true;
}

void Engine::set_rotation(const float* m_host) {
    DeviceGuard guard(device_);
    rotation_host_.assign(m_host, m_host + d_ * d_);
    rotation_ready_ = false;
    ensure_rotation();
}

void Engine::get_rotation(float* m_out) {
    DeviceGuard guard(device_);
    ensure_rotation();
    std::memcpy(m_out, rotation_host_.data(), sizeof(float) * d_ * d_);
}

void Engine::set_shard(size_t n_global, size_t row_offset, skm_allreduce_fn fn, void* user) {
    shard_n_global_ = n_global;
    shard_row_offset_ = row_offset;
    allreduce_fn_ = fn;
    allreduce_user_ = user;
    comm_ = nullptr;
}

void Engine::set_shard_nccl(size_t n_global, size_t row_offset, NcclComm* comm) {
    shard_n_global_ = n_global;
    shard_row_offset_ = row_offset;
    allreduce_fn_ = nullptr;
    allreduce_user_ = nullptr;
    comm_ = comm;
}

// Sum of one buffer across the shards.  Through NCCL the sum is enqueued on the engine's stream and nothing waits on the
// host; through the callback the stream is drained first (the callback works on its own stream).
void Engine::allreduce(void* buf, size_t count, int dtype) {
    if (!sharded_()) return;
    PhaseScope ps(*this, PH_ALLREDUCE);
    if (comm_) {
        comm_->allreduce_group(dtype == 0 ? static_cast<float*>(buf) : nullptr, dtype == 0 ? count : 0, dtype == 2 ? static_cast<uint32_t*>(buf) : nullptr, dtype == 2 ? count : 0,
                               dtype == 1 ? static_cast<double*>(buf) : nullptr, dtype == 1 ? count : 0, stream_);
        return;
    }
    sync();
    if (allreduce_fn_(allreduce_user_, buf, count, dtype) != 0) {
        throw std::runtime_error("all-reduce callback reported a failure");
    }
}

// The per-iteration sum (superkmeans.h:729-765 run on every shard): k x d row sums, k counts and two scalars.  One NCCL
// group, hence one launch, when a communicator is set; three callback calls otherwise.
void Engine::allreduce_iteration(float* sums, size_t n_sums, uint32_t* counts, size_t n_counts, double* scalars, size_t n_scalars) {
    if (!sharded_()) return;
    if (comm_) {
        PhaseScope ps(*this, PH_ALLREDUCE);
        comm_->allreduce_group(sums, n_sums, counts, n_counts, scalars, n_scalars, stream_);
        return;
    }
    allreduce(sums, n_sums, 0);
    allreduce(counts, n_counts, 2);
    allreduce(scalars, n_scalars, 1);
}

// dst[n x d] (device) = rotate(src).  Host sources are streamed through two staging buffers so
// that the copy of chunk i+1 overlaps the rotation of chunk i.
void Engine::rotate_to_device(const float* src, bool src_on_device, size_t n, float* dst, const std::function<void(size_t, size_t)>& after_rows, size_t piece) {
    if (n == 0) return;
    ensure_rotation();
    if (src_on_device) {
        PhaseScope ps(*this, PH_ROTATE);
        launch_gemm_nt(src, d_, m_dev_.get(), d_, dst, d_, n, d_, d_, stream_);
        return;
    }
    PhaseScope ps_total(*this, PH_ROTATE);
    const size_t rows = chunk_rows_for(d_, n);
    DeviceBuffer<float> raw[2];
    raw[0].ensure(rows * d_);
    if (n > rows) raw[1].ensure(rows * d_);
    cudaEvent_t copied[2], consumed[2];
    for (int i = 0; i < 2; ++i) {
        SKM_CUDA(cudaEventCreateWithFlags(&copied[i], cudaEventDisableTiming));
        SKM_CUDA(cudaEventCreateWithFlags(&consumed[i], cudaEventDisableTiming));
    }
    size_t ci = 0, handed = 0;
    for (size_t r0 = 0; r0 < n; r0 += rows, ++ci) {
        const int b = static_cast<int>(ci & 1);
        const size_t cnt = std::min(rows, n - r0);
        if (ci >= 2) SKM_CUDA(cudaStreamWaitEvent(copy_stream_, consumed[b], 0));
        SKM_CUDA(cudaMemcpyAsync(raw[b].get(), src + r0 * d_, sizeof(float) * cnt * d_, cudaMemcpyHostToDevice, copy_stream_));
        SKM_CUDA(cudaEventRecord(copied[b], copy_stream_));
        SKM_CUDA(cudaStreamWaitEvent(stream_, copied[b], 0));
        launch_gemm_nt(raw[b].get(), d_, m_dev_.get(), d_, dst + r0 * d_, d_, cnt, d_, d_, stream_);
        SKM_CUDA(cudaEventRecord(consumed[b], stream_));
        const size_t done = r0 + cnt;
        if (after_rows && (done - handed >= piece || done == n)) {
            after_rows(handed, done - handed);
            handed = done;
        }
    }
    sync();
    for (int i = 0; i < 2; ++i) {
        cudaEventDestroy(copied[i]);
        cudaEventDestroy(consumed[i]);
    }
}

void Engine::upload_rows(const float* src, bool src_on_device, size_t n, float* dst) {
    if (n == 0) return;
    SKM_CUDA(cudaMemcpyAsync(dst, src, sizeof(float) * n * d_, src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream_));
    sync();
}

void Engine::prepare_update_workspace(size_t n, size_t k) {
    const size_t units = update_sort_units(n);
    const size_t tiles = update_tiles(n);
    ws_.keys_a = ws_keys_a_.ensure(n);
    ws_.keys_b = ws_keys_b_.ensure(n);
    ws_.vals_a = ws_vals_a_.ensure(n);
    ws_.vals_b = ws_vals_b_.ensure(n);
    ws_.digit_table = ws_table_.ensure(256 * units + (256 * units) / 2048 + 64);
    ws_.seg_offsets = ws_offsets_.ensure(k + 1);
    ws_.tile_partials = ws_partials_.ensure(tiles * 2 * d_);
    ws_.block_sums = ws_block_sums_.ensure(2048);
    ws_.n_cap = n;
    ws_.k_cap = k;
    ws_.d = d_;
}

// -------------------------------------------------------------------------------------------------
// Initial centroids (superkmeans.h:1100-1142): Forgy rows, optionally rotated, into c_prev_.
// -------------------------------------------------------------------------------------------------
void Engine::generate_centroids_from_host(const float* data, bool on_device, size_t n_points_global, size_t k_cur, bool rotate, const std::vector<size_t>* precomputed) {
    PhaseScope ps(*this, PH_INIT_CENTROIDS);
    std::vector<size_t> own;
    if (!precomputed) own = forgy_indices(n_points_global, k_cur, cfg_.seed);
    const std::vector<size_t>& idx = precomputed ? *precomputed : own;
    float* raw = init_raw_.ensure(k_cur * d_);
    const bool sharded = sharded_();
    const size_t n_local = n_samples_;
    if (on_device) {
        // Rows this shard holds are gathered by a kernel; rows of other shards stay zero and arrive through the sum.
        uint64_t* idx_host = init_idx_host_.ensure(k_cur);
        const uint64_t none = ~uint64_t{0};
        for (size_t i = 0; i < k_cur; ++i) {
            size_t g = idx[i];
            if (sharded) g = (g >= shard_row_offset_ && g < shard_row_offset_ + n_local) ? g - shard_row_offset_ : none;
            idx_host[i] = g;
        }
        SKM_CUDA(cudaMemcpyAsync(init_idx_dev_.ensure(k_cur), idx_host, sizeof(uint64_t) * k_cur, cudaMemcpyHostToDevice, stream_));
        launch_gather_rows(data, init_idx_dev_.get(), raw, k_cur, d_, stream_);
    } else {
        float* host = init_rows_host_.ensure(k_cur * d_);
#pragma omp parallel for
        for (size_t i = 0; i < k_cur; ++i) {
            size_t g = idx[i];
            const bool mine = !sharded || (g >= shard_row_offset_ && g < shard_row_offset_ + n_local);
            if (sharded) g -= shard_row_offset_;
            if (mine) std::memcpy(host + i * d_, data + g * d_, sizeof(float) * d_);
            else std::memset(host + i * d_, 0, sizeof(float) * d_);
        }
        SKM_CUDA(cudaMemcpyAsync(raw, host, sizeof(float) * k_cur * d_, cudaMemcpyHostToDevice, stream_));
    }
    if (sharded) allreduce(raw, k_cur * d_, 0);
    if (rotate) {
        ensure_rotation();
        launch_gemm_nt(raw, d_, m_dev_.get(), d_, c_prev_.get(), d_, k_cur, d_, d_, stream_);
    } else {
        SKM_CUDA(cudaMemcpyAsync(c_prev_.get(), raw, sizeof(float) * k_cur * d_, cudaMemcpyDeviceToDevice, stream_));
    }
}

// Fine-clustering variant (hierarchical_superkmeans.h:333-342): rows of an already rotated device
// buffer, no rotation.
void Engine::generate_centroids_from_device_rows(const float* dev_rows, size_t n_points, size_t k_cur, const std::vector<size_t>* precomputed) {
    std::vector<size_t> own;
    if (!precomputed) own = forgy_indices(n_points, k_cur, cfg_.seed);
    const std::vector<size_t>& idx = precomputed ? *precomputed : own;
    std::vector<uint64_t> idx64(idx.begin(), idx.end());
    DeviceBuffer<uint64_t> idx_dev;
    SKM_CUDA(cudaMemcpyAsync(idx_dev.ensure(k_cur), idx64.data(), sizeof(uint64_t) * k_cur, cudaMemcpyHostToDevice, stream_));
    launch_gather_rows(dev_rows, idx_dev.get(), c_prev_.get(), k_cur, d_, stream_);
    sync();
}

// -------------------------------------------------------------------------------------------------
// One pruned assignment pass (batch_computers.h:297-409)
// -------------------------------------------------------------------------------------------------
namespace {
int g_prune_split_mode = 0;

__global__ void fill_iota_kernel(uint32_t* idx, uint32_t* flags, size_t n, uint32_t flag_value) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        idx[i] = static_cast<uint32_t>(i);
        flags[i] = flag_value;
    }
}
} // namespace

void set_prune_split_mode(int mode) { g_prune_split_mode = mode; }
int prune_split_mode() { return g_prune_split_mode; }

namespace {

// The points listed in ws.hard_idx through the dense chain: on the tensor cores over a gathered copy of their
// rows when `on_tensor_cores`, else with the SIMT kernel in place.
void run_listed_dense(const PrunedParams& p, PruneSplitWorkspace& ws, PrunePassBuffers& b, size_t n_listed, bool on_tensor_cores, cudaStream_t stream) {
    if (n_listed == 0) return;
    if (!on_tensor_cores) {
        launch_assign_pruned_dense(p, ws, n_listed, stream);
        return;
    }
    const uint32_t n_ck = prune_chain_checkpoints(p.partial_d, p.vertical_d, p.horizontal_d);
    float* xl = b.listed_x.ensure(n_listed * p.d);
    float* bestl = b.listed_best.ensure(n_listed);
    uint32_t* knnl = b.listed_knn.ensure(n_listed);
    launch_gather_listed(p.x, ws.best, p.knn, ws.hard_idx, n_listed, p.d, xl, bestl, knnl, stream);
    launch_chain_norms(xl, n_listed, p.d, p.partial_d, p.vertical_d, p.horizontal_d, false, b.listed_norms.ensure(n_listed * n_ck), stream);
    launch_chain_norms(p.y, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, true, ws.chain_norms_y, stream);
    tc::launch_chain(xl, p.y, n_listed, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, b.listed_norms.get(), ws.chain_norms_y, p.ratios, bestl, knnl,
                     b.listed_dist.ensure(n_listed), b.listed_np.ensure(n_listed), b.listed_top2.ensure(n_listed), b.y_split.ensure(2 * p.k * p.d), stream);
    launch_scatter_listed(ws.hard_idx, n_listed, knnl, b.listed_dist.get(), b.listed_np.get(), p.knn, p.dist, p.not_pruned, stream);
}

} // namespace

namespace {

struct SubPhase {
    PhaseTimers* t;
    cudaStream_t s;
    SubPhase(PhaseTimers* t_, int phase, cudaStream_t s_) : t(t_), s(s_) {
        if (t) t->begin(phase, s);
    }
    ~SubPhase() {
        if (t) t->end(s);
    }
};

// Rows per batch of the ordered pass: about 8 GB of gathered rows, a whole number of 128-row tiles.
size_t sorted_batch_rows(size_t n, size_t d) {
    const size_t target = (size_t{8} << 30) / (d * sizeof(float));
    size_t rows = std::max<size_t>(target, 16 * kTileM);
    rows = (rows / kTileM) * kTileM;
    return std::min(rows, ((n + kTileM - 1) / kTileM) * kTileM);
}

// The pruned pass over the points in the order of their previous centroid (modes 6, 7, 8, 10, 11, and 0 when it picks it).  Points that share a
// previous centroid have nearly the same thresholds and the same neighbourhood of centroids, so a tile of 128 of them
// either has short candidate lists (first test + list walk) or keeps a common, limited set of centroids alive (chain
// over the centroids named by the tile's union bits).  The order changes where work is done, not what is computed.
void run_pruned_pass_sorted(const PrunedParams& p, PrunePassBuffers& b, float ratio_first, int device, cudaStream_t stream, PhaseTimers* timers, int mode) {
    const uint32_t n_ck = prune_chain_checkpoints(p.partial_d, p.vertical_d, p.horizontal_d);
    const size_t n_chunks = (p.k + kChunk - 1) / kChunk;
    const uint32_t union_words = static_cast<uint32_t>((p.k + 31) / 32);
    const size_t cols_stride = n_chunks * kChunk;

    // ---- order of the points by previous centroid
    const size_t units = update_sort_units(p.n);
    b.sort_ws.keys_a = b.sort_keys_a.ensure(p.n);
    b.sort_ws.keys_b = b.sort_keys_b.ensure(p.n);
    b.sort_ws.vals_a = b.sort_vals_a.ensure(p.n);
    b.sort_ws.vals_b = b.sort_vals_b.ensure(p.n);
    b.sort_ws.digit_table = b.sort_table.ensure(256 * units + (256 * units) / 2048 + 64);
    const uint32_t* sorted_keys = nullptr;
    const uint32_t* order = nullptr;
    launch_sort_by_key(p.knn, p.n, p.k, b.sort_ws, &sorted_keys, &order, stream);

    // ---- centroid side, once per pass
    float* y_split = b.y_split.ensure(2 * p.k * p.d);
    tc::launch_presplit(p.y, p.k, p.d, y_split, stream);
    float* chain_norms_y = b.chain_norms_y.ensure(p.k * n_ck);
    launch_chain_norms(p.y, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, true, chain_norms_y, stream);

    const size_t batch = sorted_batch_rows(p.n, p.d);
    const size_t batch_tiles = batch / kTileM;
    float* xb = b.xb.ensure(batch * p.d);
    uint32_t* knn_b = b.knn_b.ensure(batch);
    uint32_t* prev_b = b.prev_b.ensure(batch);
    float* best_b = b.best_b.ensure(batch);
    float* dist_b = b.dist_b.ensure(batch);
    float* nx_b = b.nx_b.ensure(batch);
    uint32_t* np_b = b.np_b.ensure(batch);
    uint32_t* flags_b = b.flags_b.ensure(batch);
    uint32_t* redo_b = b.redo.ensure(batch + 1);
    uint2* top2_b = b.top2_b.ensure(batch);
    uint32_t* tile_flags = b.tile_flags.ensure(batch_tiles);
    uint32_t* tile_flags_host = b.tile_flags_host.ensure(batch_tiles);
    uint32_t* map_dense = b.tile_map_dense.ensure(batch_tiles);
    uint32_t* map_lists = b.tile_map_lists.ensure(batch_tiles);
    uint32_t* map_host = b.tile_map_host.ensure(2 * batch_tiles);
    unsigned long long* pair_steps = b.pair_steps_dev.ensure(1);
    unsigned long long* sparse_cols = b.sparse_cols_dev.ensure(1);
    unsigned long long* counters_host = b.counters_host.ensure(2);
    SKM_CUDA(cudaMemsetAsync(pair_steps, 0, sizeof(unsigned long long), stream));
    SKM_CUDA(cudaMemsetAsync(sparse_cols, 0, sizeof(unsigned long long), stream));

    PruneSplitWorkspace ws;
    ws.sample = b.sample.ensure(128 * p.d);
    ws.sample_norms = b.sample_norms.ensure(128);
    ws.alive_total = b.alive_total.ensure(1);
    ws.ratio_first = ratio_first;
    ws.flag_mult = 22;   // a point is "expensive" from 6 of 128 sampled survivors up
    uint32_t dense_tile_rows = 16;   // a tile takes the chain when at least this many of its 128 points are expensive
    // (tuning aids: both thresholds can be overridden from the environment)
    if (const char* v = std::getenv("SKM_DENSE_FLAG_MULT")) ws.flag_mult = static_cast<uint32_t>(std::max(1, std::atoi(v)));
    if (const char* v = std::getenv("SKM_DENSE_TILE_ROWS")) dense_tile_rows = static_cast<uint32_t>(std::max(1, std::atoi(v)));

    // candidate lists: eight per tile, each with room for an eighth of its pairs (modes 5 / 8: a thirty-second)
    const uint32_t cap_group = static_cast<uint32_t>(std::max<size_t>(128, mode == 8 ? p.k / 2 : p.k * 2));
    const size_t list_tile_bytes = 8 * static_cast<size_t>(cap_group) * sizeof(uint2);
    const size_t lists_per_launch = std::max<size_t>(1, (static_cast<size_t>(6) << 30) / list_tile_bytes);
    // chain: at most ~1 GB of column lists per launch
    const size_t chain_per_launch = std::max<size_t>(1, (size_t{1} << 30) / (cols_stride * sizeof(uint16_t)));

    b.last_path = 6;
    b.last_n_hard = 0;
    b.last_n_redo = 0;

    // The exact chain (chunk by chunk) over the tiles map_dev[0 .. n_t) of the row set (x_rows, n_rows) with its per-row arrays.
    auto exact_chain = [&](const float* x_rows, size_t n_rows, const uint32_t* map_dev, size_t n_t, const float* nx, const float* best, uint32_t* knn, float* dist, uint32_t* np,
                           uint2* top2, const float* chain_nx) {
        const size_t per = std::min(n_t, chain_per_launch);
        uint32_t* ubits = b.union_bits.ensure(per * union_words);
        uint16_t* cols = b.cols.ensure(per * cols_stride);
        uint32_t* counts = b.col_counts.ensure(per * n_chunks);
        for (size_t t0 = 0; t0 < n_t; t0 += per) {
            const size_t nt = std::min(per, n_t - t0);
            SKM_CUDA(cudaMemsetAsync(ubits, 0, sizeof(uint32_t) * nt * union_words, stream));
            tc::launch_union(x_rows, n_rows, p.k, p.d, p.partial_d, nx, p.norms_y, best, ratio_first, map_dev + t0, nt, ubits, union_words, y_split, stream);
            tc::launch_build_cols(ubits, union_words, nt, p.k, cols, counts, cols_stride, sparse_cols, stream);
            tc::launch_sparse_chain(x_rows, n_rows, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, chain_nx, chain_norms_y, p.ratios, best, knn, dist, np, top2, y_split,
                                    map_dev + t0, nt, cols, counts, cols_stride, stream);
        }
        tc::launch_refine_chain_tiles(x_rows, p.y, n_rows, p.k, p.d, top2, knn, dist, map_dev, n_t, stream);
    };

    // The chain over the tiles listed in map_dev[0 .. n_t) of the current batch.  With `optimistic` every tile first takes
    // the pass that ignores the chunk structure and assumes that no point's best candidate changes; the points for which
    // that does not hold are gathered (their order kept) and redone exactly.
    const bool optimistic = (mode == 11 || mode == 10) && p.k <= 65536 && std::getenv("SKM_NO_OPTIMISTIC_CHAIN") == nullptr;
    auto run_chain_tiles = [&](const uint32_t* map_dev, size_t n_t, size_t rows_in_batch) {
        if (n_t == 0) return;
        SubPhase sub(timers, PH_PRUNE_DENSE, stream);
        float* chain_norms_xb = b.chain_norms_x.ensure(batch * n_ck);
        // cumulative norms for all rows of the batch are cheap next to what follows, and keep the indexing plain
        launch_chain_norms(xb, rows_in_batch, p.d, p.partial_d, p.vertical_d, p.horizontal_d, false, chain_norms_xb, stream);
        launch_init_chain_rows(map_dev, n_t, rows_in_batch, prev_b, best_b, knn_b, dist_b, np_b, top2_b, stream);
        b.total_sparse_rows += n_t * kTileM;
        b.total_dense_rows += n_t * kTileM;
        b.last_n_hard += n_t * kTileM;
        if (!optimistic) {
            exact_chain(xb, rows_in_batch, map_dev, n_t, nx_b, best_b, knn_b, dist_b, np_b, top2_b, chain_norms_xb);
            return;
        }
        uint32_t* dirty_b = b.dirty_b.ensure(batch);
        SKM_CUDA(cudaMemsetAsync(dirty_b, 0, sizeof(uint32_t) * rows_in_batch, stream));
        // candidates of the flagged points, for the replay: two lists of kCandCap per point
        constexpr uint32_t kCandCap = 16;
        const bool replay = std::getenv("SKM_NO_CANDIDATE_REPLAY") == nullptr;
        uint32_t* cand_b = replay ? b.cand.ensure(batch * 2 * kCandCap) : nullptr;
        uint32_t* meta_b = replay ? b.cand_meta.ensure(batch) : nullptr;
        {
            const size_t per = std::min(n_t, chain_per_launch);
            uint32_t* ubits = b.union_bits.ensure(per * union_words);
            uint16_t* cols = b.cols.ensure(per * cols_stride);
            uint32_t* totals = b.col_counts.ensure(per * n_chunks);
            for (size_t t0 = 0; t0 < n_t; t0 += per) {
                const size_t nt = std::min(per, n_t - t0);
                SKM_CUDA(cudaMemsetAsync(ubits, 0, sizeof(uint32_t) * nt * union_words, stream));
                tc::launch_union(xb, rows_in_batch, p.k, p.d, p.partial_d, nx_b, p.norms_y, best_b, ratio_first, map_dev + t0, nt, ubits, union_words, y_split, stream);
                tc::launch_build_flat_cols(ubits, union_words, nt, p.k, cols, totals, cols_stride, sparse_cols, stream);
                tc::launch_sparse_chain(xb, rows_in_batch, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, chain_norms_xb, chain_norms_y, p.ratios, best_b, knn_b, dist_b, np_b,
                                        top2_b, y_split, map_dev + t0, nt, cols, totals, cols_stride, stream, dirty_b, cand_b, meta_b, kCandCap);
            }
        }
        // the points whose best candidate can move, in order
        PruneSplitWorkspace cw;
        cw.positions = b.positions.ensure(prune_split_positions_elems(batch));
        cw.hard_idx = b.hard_idx.ensure(batch);
        cw.n_hard_dev = b.n_hard_dev.ensure(1);
        launch_compact_flags(dirty_b, rows_in_batch, cw, stream);
        SKM_CUDA(cudaMemcpyAsync(&counters_host[0], cw.n_hard_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaStreamSynchronize(stream));
        const size_t n_dirty = static_cast<size_t>(counters_host[0] & 0xFFFFFFFFull);
        b.total_redone_rows += n_dirty;
        if (n_dirty == 0) return;

        // The exact chain, chunk by chunk, for the points idx[0 .. cnt) of the batch (gathered, their order kept).
        auto exact_redo = [&](const uint32_t* idx, size_t cnt) {
            const size_t nt_d = (cnt + kTileM - 1) / kTileM;
            float* xd = b.listed_x.ensure(cnt * p.d);
            float* best_d = b.listed_best.ensure(cnt);
            uint32_t* knn_d = b.listed_knn.ensure(cnt);
            uint32_t* prev_d = b.redo_prev.ensure(cnt);
            float* dist_d = b.listed_dist.ensure(cnt);
            uint32_t* np_d = b.listed_np.ensure(cnt);
            float* nx_d = b.redo_nx.ensure(cnt);
            uint2* top2_d = b.listed_top2.ensure(cnt);
            float* chain_nd = b.listed_norms.ensure(cnt * n_ck);
            uint32_t* iota = b.tile_iota.ensure(nt_d);
            launch_gather_listed(xb, best_b, prev_b, idx, cnt, p.d, xd, best_d, knn_d, stream);
            SKM_CUDA(cudaMemcpyAsync(prev_d, knn_d, sizeof(uint32_t) * cnt, cudaMemcpyDeviceToDevice, stream));
            launch_row_sqnorms(xd, cnt, p.d, p.partial_d, nx_d, stream);
            launch_chain_norms(xd, cnt, p.d, p.partial_d, p.vertical_d, p.horizontal_d, false, chain_nd, stream);
            launch_iota_u32(iota, nt_d, stream);
            launch_init_chain_rows(iota, nt_d, cnt, prev_d, best_d, knn_d, dist_d, np_d, top2_d, stream);
            exact_chain(xd, cnt, iota, nt_d, nx_d, best_d, knn_d, dist_d, np_d, top2_d, chain_nd);
            launch_scatter_listed(idx, cnt, knn_d, dist_d, np_d, knn_b, dist_b, np_b, stream);
        };
        if (!replay) {
            b.total_fallback_rows += n_dirty;
            exact_redo(cw.hard_idx, n_dirty);
            return;
        }
        // Replay of the search over the recorded candidates (assignment, distance, per-chunk thresholds), then the
        // not-pruned counts from a first test with those thresholds.
        const uint32_t n_chunks32 = static_cast<uint32_t>(n_chunks);
        float* thr = b.replay_thr.ensure(n_dirty * n_chunks);
        uint32_t* ovf = b.replay_ovf.ensure(n_dirty);
        ReplayParams rp{};
        rp.x = xb;
        rp.y = p.y;
        rp.ratios = p.ratios;
        rp.best_in = best_b;
        rp.prev = prev_b;
        rp.idx = cw.hard_idx;
        rp.cand = cand_b;
        rp.meta = meta_b;
        rp.knn = knn_b;
        rp.dist = dist_b;
        rp.thr = thr;
        rp.overflow = ovf;
        rp.n_listed = n_dirty;
        rp.k = p.k;
        rp.d = static_cast<uint32_t>(p.d);
        rp.partial_d = p.partial_d;
        rp.vertical_d = p.vertical_d;
        rp.horizontal_d = p.horizontal_d;
        rp.cap = kCandCap;
        launch_replay_candidates(rp, stream);
        {
            float* xd = b.listed_x.ensure(n_dirty * p.d);
            float* best_d = b.listed_best.ensure(n_dirty);
            uint32_t* knn_d = b.listed_knn.ensure(n_dirty);
            float* nx_d = b.redo_nx.ensure(n_dirty);
            uint32_t* np_d = b.replay_np.ensure(n_dirty);
            launch_gather_listed(xb, best_b, prev_b, cw.hard_idx, n_dirty, p.d, xd, best_d, knn_d, stream);
            launch_row_sqnorms(xd, n_dirty, p.d, p.partial_d, nx_d, stream);
            tc::launch_count_first_test(xd, n_dirty, p.k, p.d, p.partial_d, nx_d, p.norms_y, thr, n_chunks32, np_d, y_split, stream);
            launch_scatter_u32(cw.hard_idx, np_d, np_b, n_dirty, stream);
        }
        // points with more candidates than the lists hold
        PruneSplitWorkspace cw2;
        cw2.positions = b.positions2.ensure(prune_split_positions_elems(n_dirty));
        cw2.hard_idx = b.hard_idx2.ensure(n_dirty);
        cw2.n_hard_dev = b.n_hard_dev2.ensure(1);
        launch_compact_flags(ovf, n_dirty, cw2, stream);
        SKM_CUDA(cudaMemcpyAsync(&counters_host[0], cw2.n_hard_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaStreamSynchronize(stream));
        const size_t n_over = static_cast<size_t>(counters_host[0] & 0xFFFFFFFFull);
        if (n_over == 0) return;
        b.total_fallback_rows += n_over;
        uint32_t* over_rows = b.hard_idx3.ensure(n_over);
        launch_compose_u32(cw.hard_idx, cw2.hard_idx, over_rows, n_over, stream);
        // their state is still the starting one: the replay leaves such points alone
        exact_redo(over_rows, n_over);
    };

    for (size_t b0 = 0; b0 < p.n; b0 += batch) {
        const size_t cnt = std::min(batch, p.n - b0);
        const size_t n_tiles = (cnt + kTileM - 1) / kTileM;
        launch_gather_sorted(p.x, order + b0, p.knn, p.norms_x, cnt, p.d, xb, knn_b, prev_b, nx_b, stream);
        launch_exact_dist(xb, p.y, knn_b, cnt, p.d, best_b, stream);

        // ---- which tiles take which route
        size_t n_dense = 0, n_lists = 0;
        if (mode == 11) {
            PrunedParams pb = p;
            pb.x = xb;
            pb.n = cnt;
            pb.norms_x = nx_b;
            ws.best = best_b;
            ws.flags = flags_b;
            launch_classify(pb, ws, stream);
            launch_tile_flags(flags_b, cnt, dense_tile_rows, tile_flags, stream);
            SKM_CUDA(cudaMemcpyAsync(tile_flags_host, tile_flags, sizeof(uint32_t) * n_tiles, cudaMemcpyDeviceToHost, stream));
            SKM_CUDA(cudaStreamSynchronize(stream));
            for (size_t t = 0; t < n_tiles; ++t) {
                if (tile_flags_host[t]) map_host[n_dense++] = static_cast<uint32_t>(t);
                else map_host[batch_tiles + n_lists++] = static_cast<uint32_t>(t);
            }
        } else if (mode == 6 || mode == 10) {
            for (size_t t = 0; t < n_tiles; ++t) map_host[n_dense++] = static_cast<uint32_t>(t);
        } else {
            for (size_t t = 0; t < n_tiles; ++t) map_host[batch_tiles + n_lists++] = static_cast<uint32_t>(t);
        }
        if (n_dense) SKM_CUDA(cudaMemcpyAsync(map_dense, map_host, sizeof(uint32_t) * n_dense, cudaMemcpyHostToDevice, stream));
        if (n_lists) SKM_CUDA(cudaMemcpyAsync(map_lists, map_host + batch_tiles, sizeof(uint32_t) * n_lists, cudaMemcpyHostToDevice, stream));

        // ---- first test + list walk
        if (n_lists) {
            uint32_t* redo_count = redo_b + batch;
            SKM_CUDA(cudaMemsetAsync(redo_b, 0, sizeof(uint32_t) * (batch + 1), stream));
            const size_t per = std::min(n_lists, lists_per_launch);
            uint2* lists = b.tc_lists.ensure(per * 8 * cap_group);
            uint32_t* offs = b.tc_list_offs.ensure(per * 8 * (n_chunks + 1));
            for (size_t t0 = 0; t0 < n_lists; t0 += per) {
                const size_t nt = std::min(per, n_lists - t0);
                {
                    SubPhase sub(timers, PH_PRUNE_FIRST_TEST, stream);
                    tc::launch_first_test(xb, p.y, cnt, p.k, p.d, p.partial_d, nx_b, p.norms_y, best_b, nullptr, ratio_first, 0, nt, lists, offs, cap_group, stream, y_split,
                                          map_lists + t0);
                }
                WalkParams w{};
                w.x = xb;
                w.y = p.y;
                w.norms_x = nx_b;
                w.y_pdx = p.y_pdx;
                w.y_aux = p.y_aux;
                w.ratios = p.ratios;
                w.lists = lists;
                w.list_offs = offs;
                w.cap_group = cap_group;
                w.n = cnt;
                w.k = p.k;
                w.d = p.d;
                w.partial_d = p.partial_d;
                w.vertical_d = p.vertical_d;
                w.horizontal_d = p.horizontal_d;
                w.tile0 = 0;
                w.n_tiles = nt;
                w.tile_map = map_lists + t0;
                w.best_in = best_b;
                w.skip = nullptr;
                w.knn = knn_b;
                w.dist = dist_b;
                w.not_pruned = np_b;
                w.redo = redo_b;
                w.redo_count = redo_count;
                w.pair_steps = pair_steps;
                w.upstream_error = tc::error_word();
                SubPhase sub(timers, PH_PRUNE_WALK, stream);
                launch_walk_lists(w, device, stream);
            }
            // tiles with a list that overflowed: the whole tile goes through the chain, from its starting state
            launch_tile_flags(redo_b, cnt, 1, tile_flags, stream);
            SKM_CUDA(cudaMemcpyAsync(tile_flags_host, tile_flags, sizeof(uint32_t) * n_tiles, cudaMemcpyDeviceToHost, stream));
            SKM_CUDA(cudaMemcpyAsync(&counters_host[0], redo_count, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
            SKM_CUDA(cudaStreamSynchronize(stream));
            const size_t n_redo_rows = static_cast<size_t>(counters_host[0] & 0xFFFFFFFFull);
            if (n_redo_rows) {
                for (size_t t = 0; t < n_tiles; ++t)
                    if (tile_flags_host[t]) map_host[n_dense++] = static_cast<uint32_t>(t);
                SKM_CUDA(cudaMemcpyAsync(map_dense, map_host, sizeof(uint32_t) * n_dense, cudaMemcpyHostToDevice, stream));
                b.last_n_redo += n_redo_rows;
                b.total_redo_rows += n_redo_rows;
            }
        }

        // ---- chain over the centroids the tile can still reach
        run_chain_tiles(map_dense, n_dense, cnt);

        launch_scatter_sorted(order + b0, cnt, knn_b, dist_b, np_b, p.knn, p.dist, p.not_pruned, stream);
        // map_host / tile_flags_host are reused by the next batch: the copies above must have been consumed
        SKM_CUDA(cudaStreamSynchronize(stream));
    }
    SKM_CUDA(cudaMemcpyAsync(&counters_host[0], pair_steps, sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream));
    SKM_CUDA(cudaMemcpyAsync(&counters_host[1], sparse_cols, sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream));
    SKM_CUDA(cudaStreamSynchronize(stream));
    b.total_pair_steps += counters_host[0];
    b.total_sparse_cols += counters_host[1];
}

} // namespace

// Share of (point, sampled centroid) pairs passing the first test from which the automatic choice takes the ordered chain
// (a tuning aid: SKM_AUTO_CHAIN_SURVIVAL overrides it).
static double auto_chain_survival() {
    if (const char* v = std::getenv("SKM_AUTO_CHAIN_SURVIVAL")) return std::atof(v);
    return 0.025;
}

void run_pruned_pass_on(PrunedParams p, PrunePassBuffers& b, float ratio_first, int device, cudaStream_t stream, PhaseTimers* timers) {
    struct Sub {
        PhaseTimers* t;
        cudaStream_t s;
        Sub(PhaseTimers* t_, int phase, cudaStream_t s_) : t(t_), s(s_) {
            if (t) t->begin(phase, s);
        }
        ~Sub() {
            if (t) t->end(s);
        }
    };
    if (p.n == 0) return;
    int mode = g_prune_split_mode;
    const bool auto_mode = mode == 0;
    if (((mode >= 6 && mode <= 8) || mode == 10 || mode == 11) && tc::eligible(p.x, p.d, p.y, p.d)) {
        run_pruned_pass_sorted(p, b, ratio_first, device, stream, timers, mode);
        return;
    }
    if ((mode >= 6 && mode <= 8) || mode == 10 || mode == 11) throw std::invalid_argument("the ordered pruned pass needs 16-byte aligned rows (d % 4 == 0) and the tensor-core kernels switched on");
    if (mode == 9) mode = 0;
    if (b.grid == 0) b.grid = pruned_grid_size(device);
    const uint32_t n_ck = prune_chain_checkpoints(p.partial_d, p.vertical_d, p.horizontal_d);
    PruneSplitWorkspace ws;
    ws.best = b.best.ensure(p.n);
    ws.flags = b.flags.ensure(p.n);
    ws.positions = b.positions.ensure(prune_split_positions_elems(p.n));
    ws.hard_idx = b.hard_idx.ensure(p.n);
    ws.sample = b.sample.ensure(128 * p.d);
    ws.sample_norms = b.sample_norms.ensure(128);
    ws.chain_norms_y = b.chain_norms_y.ensure(p.k * n_ck);
    ws.n_hard_dev = b.n_hard_dev.ensure(1);
    ws.ratio_first = ratio_first;
    ws.alive_total = b.alive_total.ensure(1);
    // with the tensor-core chain available, points from 6 of 128 sampled survivors up are cheaper there
    if (tc::eligible(p.x, p.d, p.y, p.d) && (mode == 0)) ws.flag_mult = 22;
    launch_pruned_prepare(p, ws, stream);
    const int n_sample = static_cast<int>(std::min<size_t>(p.k, 128));
    const bool tc_ok = tc::eligible(p.x, p.d, p.y, p.d);
    size_t n_hard = 0;
    bool use_chain = false, use_tc_lists = false;
    if (mode == 0) {
        unsigned long long* host = b.counters_host.ensure(2);
        host[0] = 0;
        host[1] = 0;
        SKM_CUDA(cudaMemcpyAsync(&host[0], ws.alive_total, sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaMemcpyAsync(&host[1], ws.n_hard_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaStreamSynchronize(stream));
        n_hard = static_cast<size_t>(host[1] & 0xFFFFFFFFull);
        // Candidate lists cost one gathered block per surviving pair and step; the tensor-core chain costs a
        // full product whatever survives.  Past roughly 0.8 % of surviving pairs the chain is cheaper.
        const double survival = static_cast<double>(host[0]) / (static_cast<double>(p.n) * n_sample);
        b.last_survival = survival;
        // Which family of routes: candidate lists cost one gathered 64-dimension block per surviving pair and step, so
        // they win while few pairs survive the first test; past ~2.5 % of surviving pairs, and with at least 32 points
        // per cluster (so that a tile of 128 ordered points spans few clusters), the points go, in the order of their
        // previous centroid, through the chain over each tile's reachable centroids (whose cost follows the union of
        // the tile's survivors, not their number).
        // Measured on one B200, 10 iterations: 10M x 1024, k = 10 000 (survival 3.3 - 4.2 %): 5.0 s against 7.3 s;
        // 1M x 1536, k = 4096 (2.2 %, then below 0.1 %): lists 0.22 s against 0.39 s; a shard of 1.25M x 1024 of the
        // first workload (125 points per cluster): 0.58 s against 0.99 s.  Below 2^18 points the fixed costs of the
        // ordered route (sort, batches, host round trips) outweigh it: 100k x 768, k = 1000: 23.5 ms against 16.9 ms.
        if (auto_mode && tc_ok && p.k <= 65536 && survival >= auto_chain_survival() && p.n >= 32 * p.k && p.n >= (size_t{1} << 18)) {
            run_pruned_pass_sorted(p, b, ratio_first, device, stream, timers, 10);
            return;
        }
        // The chain costs a full product whatever survives; lists cost a partial product plus one gathered
        // block per surviving pair and step, and their capacity is an eighth of all pairs.
        use_chain = tc_ok && (survival > 0.08 || n_hard * 2 > p.n);
        use_tc_lists = tc_ok && !use_chain;
    } else if (mode == 3) {
        if (!tc_ok) throw std::invalid_argument("the tensor-core chain needs 16-byte aligned rows (d % 4 == 0)");
        use_chain = true;
    } else {
        const bool dense = mode == 2;
        use_tc_lists = mode == 4 || mode == 5;
        if (use_tc_lists && !tc_ok) throw std::invalid_argument("the tensor-core first test needs 16-byte aligned rows (d % 4 == 0)");
        fill_iota_kernel<<<static_cast<unsigned>((p.n + 255) / 256), 256, 0, stream>>>(ws.hard_idx, ws.flags, p.n, dense ? 1u : 0u);
        note_kernel_launch();
        SKM_CUDA(cudaGetLastError());
        n_hard = dense ? p.n : 0;
    }
    if (use_chain) {
        b.last_path = 3;
        b.last_n_hard = p.n;
        b.total_dense_rows += p.n;
        Sub sub(timers, PH_PRUNE_DENSE, stream);
        launch_chain_norms(p.x, p.n, p.d, p.partial_d, p.vertical_d, p.horizontal_d, false, b.chain_norms_x.ensure(p.n * n_ck), stream);
        launch_chain_norms(p.y, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, true, ws.chain_norms_y, stream);
        tc::launch_chain(p.x, p.y, p.n, p.k, p.d, p.partial_d, p.vertical_d, p.horizontal_d, b.chain_norms_x.get(), ws.chain_norms_y, p.ratios, ws.best, p.knn, p.dist,
                         p.not_pruned, b.top2.ensure(p.n), b.y_split.ensure(2 * p.k * p.d), stream);
        return;
    }
    p.best_in = ws.best;
    p.skip = ws.flags;
    if (use_tc_lists) {
        b.last_path = 4;
        b.last_n_hard = n_hard;
        uint32_t* redo = b.redo.ensure(p.n + 1);
        uint32_t* redo_count = redo + p.n;
        SKM_CUDA(cudaMemsetAsync(redo, 0, sizeof(uint32_t) * (p.n + 1), stream));
        unsigned long long* pair_steps = b.pair_steps_dev.ensure(1);
        SKM_CUDA(cudaMemsetAsync(pair_steps, 0, sizeof(unsigned long long), stream));
        if (n_hard < p.n) {
            const size_t n_chunks = (p.k + kChunk - 1) / kChunk;
            // eight lists per tile of 128 points, each with room for an eighth of its pairs (32 points x half the
            // centroids); mode 5: a thirty-second, so that lists overflow
            const uint32_t cap_group = static_cast<uint32_t>(std::max<size_t>(128, mode == 5 ? p.k / 2 : p.k * 2));
            const size_t tile_bytes = 8 * static_cast<size_t>(cap_group) * sizeof(uint2);
            const size_t n_tiles = (p.n + kTileM - 1) / kTileM;
            const size_t list_bytes_cap = static_cast<size_t>(6) << 30;
            // at least one tile per batch; when even one tile's lists exceed the cap (k in the millions) the batch is that one tile
            const size_t per_batch = std::min(n_tiles, std::max<size_t>(1, list_bytes_cap / tile_bytes));
            uint2* lists = b.tc_lists.ensure(per_batch * 8 * cap_group);
            uint32_t* offs = b.tc_list_offs.ensure(per_batch * 8 * (n_chunks + 1));
            float* y_split = b.y_split.ensure(2 * p.k * p.d);
            tc::launch_presplit(p.y, p.k, p.d, y_split, stream);
            for (size_t t0 = 0; t0 < n_tiles; t0 += per_batch) {
                const size_t nt = std::min(per_batch, n_tiles - t0);
                {
                    Sub sub(timers, PH_PRUNE_FIRST_TEST, stream);
                    tc::launch_first_test(p.x, p.y, p.n, p.k, p.d, p.partial_d, p.norms_x, p.norms_y, ws.best, ws.flags, ratio_first, t0, nt, lists, offs, cap_group, stream, y_split);
                }
                WalkParams w{};
                w.x = p.x;
                w.y = p.y;
                w.norms_x = p.norms_x;
                w.y_pdx = p.y_pdx;
                w.y_aux = p.y_aux;
                w.ratios = p.ratios;
                w.lists = lists;
                w.list_offs = offs;
                w.cap_group = cap_group;
                w.n = p.n;
                w.k = p.k;
                w.d = p.d;
                w.partial_d = p.partial_d;
                w.vertical_d = p.vertical_d;
                w.horizontal_d = p.horizontal_d;
                w.tile0 = t0;
                w.n_tiles = nt;
                w.best_in = ws.best;
                w.skip = ws.flags;
                w.knn = p.knn;
                w.dist = p.dist;
                w.not_pruned = p.not_pruned;
                w.redo = redo;
                w.redo_count = redo_count;
                w.pair_steps = pair_steps;
                w.upstream_error = tc::error_word();
                Sub sub(timers, PH_PRUNE_WALK, stream);
                launch_walk_lists(w, device, stream);
            }
        }
        {
            Sub sub(timers, PH_PRUNE_DENSE, stream);
            run_listed_dense(p, ws, b, n_hard, true, stream);
        }
        // points of groups whose list overflowed
        unsigned long long* host = b.counters_host.ensure(2);
        host[0] = 0;
        host[1] = 0;
        SKM_CUDA(cudaMemcpyAsync(&host[0], redo_count, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaMemcpyAsync(&host[1], pair_steps, sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream));
        SKM_CUDA(cudaStreamSynchronize(stream));
        const size_t n_redo = static_cast<size_t>(host[0] & 0xFFFFFFFFull);
        b.last_n_redo = n_redo;
        b.total_pair_steps += host[1];
        b.total_dense_rows += n_hard + n_redo;
        b.total_redo_rows += n_redo;
        if (n_redo != 0) {
            Sub sub(timers, PH_PRUNE_DENSE, stream);
            launch_compact_flags(redo, p.n, ws, stream);
            run_listed_dense(p, ws, b, n_redo, true, stream);
        }
        return;
    }
    b.last_path = 1;
    b.last_n_hard = n_hard;
    if (n_hard < p.n) {
        p.scratch = b.lists.ensure(pruned_scratch_elems(b.grid));
        launch_assign_pruned(p, b.grid, stream);
    }
    launch_assign_pruned_dense(p, ws, n_hard, stream);
}

void Engine::run_pruned_pass(const float* x, size_t n, size_t k_cur, const float* y, const float* norms_x, const float* norms_y, uint32_t* knn, float* dist, uint32_t* not_pruned) {
    PrunedParams p{};
    p.x = x;
    p.y = y;
    p.y_pdx = c_pdx_.get();
    p.y_aux = c_aux_.get();
    p.norms_x = norms_x;
    p.norms_y = norms_y;
    p.ratios = ratios_dev_.get();
    p.knn = knn;
    p.dist = dist;
    p.not_pruned = not_pruned;
    p.n = n;
    p.k = k_cur;
    p.d = d_;
    p.partial_d = partial_d_;
    p.vertical_d = vertical_d_;
    p.horizontal_d = horizontal_d_;
    run_pruned_pass_on(p, prune_bufs_, ratios_host_[partial_d_], device_, stream_, &timers_);
}

// -------------------------------------------------------------------------------------------------
// ConsolidateCentroids (superkmeans.h:936-968): mean, split, optional normalisation, PDX copies.
// counts_host_ holds this iteration's (globally reduced) cluster sizes.
// -------------------------------------------------------------------------------------------------
void Engine::consolidate(size_t n_samples_global, size_t k_cur) {
    launch_scale_by_counts(c_cur_.get(), counts_.get(), k_cur, d_, stream_);
    sizes_host_.assign(counts_host_.get(), counts_host_.get() + k_cur);
    if (!split_can_terminate(sizes_host_, n_samples_global, k_cur)) {
        throw std::runtime_error("cannot repopulate empty clusters: no cluster holds more than one point");
    }
    std::vector<SplitOp> ops;
    n_split_ = hierarchical_ ? split_clusters_hierarchical(sizes_host_, n_samples_global, k_cur, cfg_.seed, ops)
                             : split_clusters_flat(sizes_host_, n_samples_global, k_cur, cfg_.seed, ops);
    if (!ops.empty()) {
        static_assert(sizeof(SplitOp) == sizeof(SplitOpDev), "layout");
        SKM_CUDA(cudaMemcpyAsync(split_ops_dev_.ensure(ops.size()), ops.data(), sizeof(SplitOp) * ops.size(), cudaMemcpyHostToDevice, stream_));
        launch_apply_split_ops(c_cur_.get(), d_, split_ops_dev_.get(), ops.size(), stream_);
        sync();  // `ops` must outlive the asynchronous copy
    }
    if (cfg_.angular) launch_normalize_rows(c_cur_.get(), k_cur, d_, stream_);
    launch_pdxify(c_cur_.get(), c_pdx_.get(), c_aux_.get(), k_cur, d_, vertical_d_, stream_);
}

// -------------------------------------------------------------------------------------------------
// RunIteration<GEMM_ONLY> (superkmeans.h:786-879)
// -------------------------------------------------------------------------------------------------
void Engine::run_iteration(bool gemm_only, const IterationInput& in, size_t iter_idx, bool is_first, std::vector<skm_iter_stats>& target) {
    if (!is_first) c_cur_.swap(c_prev_);
    const size_t n = in.n_samples, k_cur = in.n_clusters;
    float* norms = in.norms;
    if (gemm_only) {
        launch_row_sqnorms(c_prev_.get(), k_cur, d_, d_, centroid_norms_.get(), stream_);
        PhaseScope ps(*this, PH_ASSIGN_FULL);
        if (is_first && first_assign_done_) {
            first_assign_done_ = false;   // done during the upload (train_flat)
        } else {
            launch_assign_full(in.x, c_prev_.get(), n, k_cur, d_, norms, centroid_norms_.get(), assignments_.get(), distances_.get(), top2_.ensure(n), stream_,
                               y_split_.ensure(2 * k_cur * d_));
        }
    } else {
        launch_row_sqnorms(c_prev_.get(), k_cur, d_, partial_d_, centroid_norms_.get(), stream_);
        PhaseScope ps(*this, PH_ASSIGN_PRUNED);
        run_pruned_pass(in.x, n, k_cur, c_prev_.get(), norms, centroid_norms_.get(), assignments_.get(), distances_.get(), not_pruned_.get());
    }
    // UpdateCentroids + ComputeCost (superkmeans.h:729-765, :973-981)
    {
        PhaseScope ps(*this, PH_UPDATE);
        launch_update(in.x, assignments_.get(), distances_.get(), gemm_only ? nullptr : not_pruned_.get(), n, k_cur, d_, ws_, c_cur_.get(), counts_.get(), scalars_dev_.get(),
                      gemm_only ? nullptr : np_total_dev_.get(), stream_);
        if (!gemm_only) {
            u64_to_f64_kernel<<<1, 1, 0, stream_>>>(np_total_dev_.get(), scalars_dev_.get() + 1);
            note_kernel_launch();
            SKM_CUDA(cudaGetLastError());
        }
    }
    allreduce_iteration(c_cur_.get(), k_cur * d_, counts_.get(), k_cur, scalars_dev_.get(), 2);
    SKM_CUDA(cudaMemcpyAsync(counts_host_.ensure(k_), counts_.get(), sizeof(uint32_t) * k_cur, cudaMemcpyDeviceToHost, stream_));
    SKM_CUDA(cudaMemcpyAsync(scalars_host_.get(), scalars_dev_.get(), sizeof(double) * 2, cudaMemcpyDeviceToHost, stream_));
    sync();
    check_tc_error(stream_);
    const double wcss = scalars_host_.get()[0];

    float avg_not_pruned = -1.0f;
    const uint32_t old_partial_d = partial_d_;
    if (!gemm_only) {
        const TuneResult t = tune_partial_d(scalars_host_.get()[1], in.n_samples_global, k_cur, partial_d_, vertical_d_, cfg_.min_not_pruned_pct, cfg_.max_not_pruned_pct,
                                            cfg_.adjustment_factor_for_partial_d);
        avg_not_pruned = t.avg_not_pruned_pct;
        partial_d_ = t.new_partial_d;
        if (t.changed) {
            PhaseScope ps(*this, PH_NORMS);
            launch_row_sqnorms(in.x, n, d_, partial_d_, norms, stream_);
        }
    }
    {
        PhaseScope ps(*this, PH_CONSOLIDATE);
        consolidate(in.n_samples_global, k_cur);
    }

    prev_cost_ = cost_;
    cost_ = static_cast<float>(wcss);
    last_cost_f64_ = wcss;
    // ComputeShift (superkmeans.h:988-998)
    {
        PhaseScope ps(*this, PH_SHIFT);
        launch_shift(c_cur_.get(), c_prev_.get(), k_cur, d_, ws_.block_sums, scalars_dev_.get() + 2, stream_);
    }
    SKM_CUDA(cudaMemcpyAsync(scalars_host_.get() + 2, scalars_dev_.get() + 2, sizeof(double), cudaMemcpyDeviceToHost, stream_));
    sync();
    shift_ = static_cast<float>(scalars_host_.get()[2]);

    if (trace_on_) {
        Snapshot snap;
        snap.n_samples = n;
        snap.n_clusters = k_cur;
        snap.partial_d_next = partial_d_;
        snap.centroids.resize(k_cur * d_);
        snap.assign.resize(n);
        snap.dist.resize(n);
        snap.sizes_pre.assign(counts_host_.get(), counts_host_.get() + k_cur);
        snap.sizes_post.assign(sizes_host_.begin(), sizes_host_.begin() + k_cur);
        SKM_CUDA(cudaMemcpyAsync(snap.centroids.data(), c_cur_.get(), sizeof(float) * k_cur * d_, cudaMemcpyDeviceToHost, stream_));
        SKM_CUDA(cudaMemcpyAsync(snap.assign.data(), assignments_.get(), sizeof(uint32_t) * n, cudaMemcpyDeviceToHost, stream_));
        SKM_CUDA(cudaMemcpyAsync(snap.dist.data(), distances_.get(), sizeof(float) * n, cudaMemcpyDeviceToHost, stream_));
        sync();
        trace_.push_back(std::move(snap));
    }

    // superkmeans.h:848-851
    recall_ = (n_queries_ > 0 && &target == &stats_flat_) ? compute_recall(k_cur) : 0.0f;

    skm_iter_stats s{};
    s.iteration = iter_idx + 1;
    s.objective = cost_;
    s.shift = shift_;
    s.split = n_split_;
    s.recall = recall_;
    s.is_gemm_only = gemm_only ? 1 : 0;
    s.not_pruned_pct = gemm_only ? -1.0f : avg_not_pruned;
    s.partial_d = gemm_only ? 0u : old_partial_d;
    target.push_back(s);
    if (cfg_.verbose) {
        std::cout << "Iteration " << iter_idx + 1 << " | Objective: " << cost_ << " | Shift: " << shift_ << " | Split: " << n_split_ << " | Recall: " << recall_;
        if (gemm_only) std::cout << " [GEMM-only]";
        else std::cout << " | Not Pruned %: " << avg_not_pruned * 100.0f << " | d': " << old_partial_d << " -> " << partial_d_;
        std::cout << std::endl;
    }
}

// -------------------------------------------------------------------------------------------------
// Train
// -------------------------------------------------------------------------------------------------
void Engine::train(const float* data, size_t n, bool on_device, const float* queries, size_t n_queries, float* centroids_out) {
    DeviceGuard guard(device_);
    ensure_positive(n > 0, "n");
    if (trained_) throw std::runtime_error("The clustering has already been trained");
    const size_t n_global = sharded_() ? shard_n_global_ : n;
    if (hierarchical_) {
        if (n_queries > 0 && !cfg_.suppress_warnings) {
            std::cout << "WARNING: Early Termination by Recall is not supported in HierarchicalSuperKMeans" << std::endl;
        }
    }
    if (n_global < k_) throw std::runtime_error("The number of points should be at least as large as the number of clusters");
    if (!hierarchical_) {
        if (n_queries > 0 && queries == nullptr && !cfg_.sample_queries) {
            throw std::invalid_argument("Queries must be provided if n_queries > 0 and sample_queries is false");
        }
        if (n_queries > 0 && sharded_()) throw std::runtime_error("training with queries is not available for sharded training");
    }
    if (sharded_() && cfg_.sampling_fraction != 1.0f) {
        throw std::runtime_error("sharded training requires sampling_fraction == 1.0");
    }
    if (sharded_() && hierarchical_) {
        throw std::runtime_error("sharded training is available for the flat algorithm only");
    }
    const double alloc_ms0 = alloc_free_ms();
    timers_.begin(PH_TRAIN_TOTAL, stream_);
    try {
        if (hierarchical_) train_hierarchical(data, n, on_device, centroids_out);
        else train_flat(data, n, on_device, queries, n_queries, centroids_out);
    } catch (...) {
        timers_.end(stream_);
        throw;
    }
    timers_.end(stream_);
    sync();
    timers_.add_host(PH_ALLOC_FREE, alloc_free_ms() - alloc_ms0);
}

// Copies (and rotates unless the data is pre-rotated) the training rows into x_rot_; with sampling
// the rows are the first n_samples entries of the shuffle (superkmeans.h:1385-1443).
static void gather_host_rows(const float* data, const size_t* idx, size_t cnt, size_t d, float* out) {
#pragma omp parallel for
    for (size_t i = 0; i < cnt; ++i) std::memcpy(out + i * d, data + idx[i] * d, sizeof(float) * d);
}

void Engine::train_flat(const float* data, size_t n, bool on_device, const float* queries, size_t n_queries, float* centroids_out) {
    stats_flat_.clear();
    n_queries_ = 0;
    first_assign_done_ = false;
    const size_t n_global = sharded_() ? shard_n_global_ : n;
    const size_t n_samples_global = n_vectors_to_sample(n_global, k_, cfg_.sampling_fraction, cfg_.max_points_per_cluster, false);
    if (n_samples_global < k_) {
        throw std::runtime_error("Not enough samples to train. Try increasing the sampling_fraction or max_points_per_cluster");
    }
    n_samples_ = sharded_() ? n : n_samples_global;
    const bool rotate = !cfg_.data_already_rotated;
    partial_d_ = initial_partial_d(vertical_d_);
    // The Forgy shuffle runs over all n_samples indices with std::mt19937 (a tenth of a second at 1e7): on a thread of
    // its own, while this one allocates the buffers and starts the rotation.
    std::future<std::vector<size_t>> forgy = std::async(std::launch::async, [n_samples_global, k = k_, seed = cfg_.seed] { return forgy_indices(n_samples_global, k, seed); });
    bool centroids_ready = false;
    auto make_centroids = [&] {
        if (centroids_ready) return;
        const std::vector<size_t> idx = forgy.get();
        generate_centroids_from_host(data, on_device, n_samples_global, k_, rotate, &idx);
        centroids_ready = true;
    };

    c_cur_.ensure(k_ * d_);
    c_prev_.ensure(k_ * d_);
    c_pdx_.ensure(k_ * d_);
    c_aux_.ensure(k_ * static_cast<size_t>(vertical_d_) + 1);
    centroid_norms_.ensure(k_);
    counts_.ensure(k_);
    counts_host_.ensure(k_);
    assignments_.ensure(n_samples_);
    distances_.ensure(n_samples_);
    not_pruned_.ensure(n_samples_);
    data_norms_.ensure(n_samples_);
    x_rot_.ensure(n_samples_ * d_);
    SKM_CUDA(cudaMemsetAsync(assignments_.get(), 0, sizeof(uint32_t) * n_samples_, stream_));
    prepare_update_workspace(n_samples_, k_);

    // GenerateCentroids picks among the first n_samples rows of the caller's data (:221-222).
    if (n_samples_global < n_global) {
        make_centroids();
        sampled_indices_ = sampling_permutation(n, cfg_.seed);
        const size_t rows = chunk_rows_for(d_, n_samples_);
        if (on_device) {
            DeviceBuffer<uint64_t> idx_dev;
            DeviceBuffer<float> raw;
            idx_dev.ensure(rows);
            raw.ensure(rows * d_);
            std::vector<uint64_t> idx64(rows);
            for (size_t r0 = 0; r0 < n_samples_; r0 += rows) {
                const size_t cnt = std::min(rows, n_samples_ - r0);
                for (size_t i = 0; i < cnt; ++i) idx64[i] = sampled_indices_[r0 + i];
                SKM_CUDA(cudaMemcpyAsync(idx_dev.get(), idx64.data(), sizeof(uint64_t) * cnt, cudaMemcpyHostToDevice, stream_));
                float* dst = rotate ? raw.get() : x_rot_.get() + r0 * d_;
                launch_gather_rows(data, idx_dev.get(), dst, cnt, d_, stream_);
                if (rotate) rotate_to_device(raw.get(), true, cnt, x_rot_.get() + r0 * d_);
                sync();
            }
        } else {
            std::vector<float> staged(rows * d_);
            for (size_t r0 = 0; r0 < n_samples_; r0 += rows) {
                const size_t cnt = std::min(rows, n_samples_ - r0);
                gather_host_rows(data, sampled_indices_.data() + r0, cnt, d_, staged.data());
                if (rotate) rotate_to_device(staged.data(), false, cnt, x_rot_.get() + r0 * d_);
                else upload_rows(staged.data(), false, cnt, x_rot_.get() + r0 * d_);
            }
        }
    } else {
        if (rotate && !on_device) {
            // Host input: the exact assignment of iteration 1 needs nothing but the rotated rows and the initial
            // centroids, so it runs piece by piece between the uploads instead of after the last one.
            uint2* top2 = top2_.ensure(n_samples_);
            float* y_split = y_split_.ensure(2 * k_ * d_);
            rotate_to_device(
                data, false, n_samples_, x_rot_.get(),
                [&](size_t r0, size_t cnt) {
                    if (!centroids_ready) {
                        make_centroids();
                        launch_row_sqnorms(c_prev_.get(), k_, d_, d_, centroid_norms_.get(), stream_);
                    }
                    launch_row_sqnorms(x_rot_.get() + r0 * d_, cnt, d_, d_, data_norms_.get() + r0, stream_);
                    launch_assign_full(x_rot_.get() + r0 * d_, c_prev_.get(), cnt, k_, d_, data_norms_.get() + r0, centroid_norms_.get(), assignments_.get() + r0,
                                       distances_.get() + r0, top2 + r0, stream_, y_split);
                },
                static_cast<size_t>(sm_count_of(device_)) * kTileM * 14);   // ~14 waves of row tiles (one per SM) per piece
            first_assign_done_ = true;
        } else if (rotate) {
            rotate_to_device(data, on_device, n_samples_, x_rot_.get());
        } else {
            upload_rows(data, on_device, n_samples_, x_rot_.get());
        }
    }
    make_centroids();
    sync();

    {
        PhaseScope ps(*this, PH_NORMS);
        launch_row_sqnorms(x_rot_.get(), n_samples_, d_, d_, data_norms_.get(), stream_);
    }

    // Ground truth for the recall figure (superkmeans.h:243-274): needs the full norms computed just above.
    if (n_queries > 0) prepare_recall(queries, n_queries, rotate);

    const bool always_gemm_only = d_ < kDimensionThresholdForPruning || cfg_.use_blas_only || k_ <= kNClustersThresholdForPruning;
    bool partial_norms_computed = false;
    float best_recall = 0.0f;
    size_t iters_without_improvement = 0;
    IterationInput in{x_rot_.get(), n_samples_, n_samples_global, k_, data_norms_.get()};
    for (size_t iter = 0; iter < cfg_.iters; ++iter) {
        const bool gemm_only = (iter == 0) || always_gemm_only;
        if (!gemm_only && !partial_norms_computed) {
            PhaseScope ps(*this, PH_NORMS);
            launch_row_sqnorms(x_rot_.get(), n_samples_, d_, partial_d_, data_norms_.get(), stream_);
            partial_norms_computed = true;
        }
        run_iteration(gemm_only, in, iter, iter == 0, stats_flat_);
        if (cfg_.early_termination &&
            should_stop_early(shift_, cost_, prev_cost_, cfg_.tol, iter, n_queries_ > 0, recall_, cfg_.recall_tol, &best_recall, &iters_without_improvement)) {
            break;
        }
    }
    queries_rot_.release();
    topk_dots_.release();
    n_state_rows_ = n_samples_;
    trained_ = true;
    output_centroids(centroids_out);
    check_tc_error(stream_);
    x_rot_.release();
    ws_partials_.release();
}

// Query side of Train (superkmeans.h:243-274): rotated queries (or a sample of the rotated training rows), their
// norms, and the objective_k nearest training rows of every query.
void Engine::prepare_recall(const float* queries, size_t n_queries, bool rotate) {
    centroids_to_explore_ = std::max<size_t>(static_cast<size_t>(static_cast<float>(k_) * cfg_.ann_explore_fraction), 1);
    if (cfg_.verbose) {
        std::cout << "Centroids to explore: " << centroids_to_explore_ << " (" << cfg_.ann_explore_fraction * 100.0f << "% of " << k_ << ")" << std::endl;
    }
    const size_t objective_k = cfg_.objective_k;
    if (objective_k == 0 || objective_k > topk_max_k() || centroids_to_explore_ > topk_max_k()) {
        throw std::runtime_error("objective_k and the number of centroids to explore must lie in [1, " + std::to_string(topk_max_k()) + "]");
    }
    float* qr = queries_rot_.ensure(n_queries * d_);
    if (cfg_.sample_queries) {
        // SampleAndRotateVectors(data_to_cluster, ..., n_samples, n_queries, false): the first n_queries entries of a
        // shuffle of the training rows, already rotated
        if (n_queries >= n_samples_) throw std::runtime_error("sample_queries needs fewer queries than training points");
        std::cout << "Sampling queries from data..." << std::endl;   // printed unconditionally by the reference (superkmeans.h:263)
        const std::vector<size_t> perm = sampling_permutation(n_samples_, cfg_.seed);
        std::vector<uint64_t> idx(perm.begin(), perm.begin() + n_queries);
        DeviceBuffer<uint64_t> idx_dev;
        SKM_CUDA(cudaMemcpyAsync(idx_dev.ensure(n_queries), idx.data(), sizeof(uint64_t) * n_queries, cudaMemcpyHostToDevice, stream_));
        launch_gather_rows(x_rot_.get(), idx_dev.get(), qr, n_queries, d_, stream_);
        sync();
    } else if (rotate) {
        rotate_to_device(queries, false, n_queries, qr);
    } else {
        upload_rows(queries, false, n_queries, qr);
    }
    launch_row_sqnorms(qr, n_queries, d_, d_, query_norms_.ensure(n_queries), stream_);
    const size_t kmax = std::max(objective_k, centroids_to_explore_);
    launch_topk_nn(qr, x_rot_.get(), n_queries, n_samples_, d_, query_norms_.get(), data_norms_.get(), static_cast<uint32_t>(objective_k), gt_idx_.ensure(n_queries * objective_k),
                   nullptr, topk_dots_.ensure(topk_scratch_floats(n_queries)), topk_state_.ensure(n_queries * kmax), stream_);
    promising_.ensure(n_queries * centroids_to_explore_);
    recall_found_.ensure(n_queries);
    recall_found_host_.ensure(n_queries);
    n_queries_ = n_queries;
    sync();
}

// ComputeRecall (superkmeans.h:1044-1087) on the consolidated centroids of this iteration.
float Engine::compute_recall(size_t k_cur) {
    launch_row_sqnorms(c_cur_.get(), k_cur, d_, d_, centroid_norms_.get(), stream_);
    launch_topk_nn(queries_rot_.get(), c_cur_.get(), n_queries_, k_cur, d_, query_norms_.get(), centroid_norms_.get(), static_cast<uint32_t>(centroids_to_explore_),
                   promising_.get(), nullptr, topk_dots_.get(), topk_state_.get(), stream_);
    launch_recall_count(gt_idx_.get(), static_cast<uint32_t>(cfg_.objective_k), promising_.get(), static_cast<uint32_t>(centroids_to_explore_), assignments_.get(), n_samples_,
                        n_queries_, recall_found_.get(), stream_);
    SKM_CUDA(cudaMemcpyAsync(recall_found_host_.get(), recall_found_.get(), sizeof(uint32_t) * n_queries_, cudaMemcpyDeviceToHost, stream_));
    sync();
    float sum_recall = 0.0f;
    for (size_t i = 0; i < n_queries_; ++i) sum_recall += static_cast<float>(recall_found_host_.get()[i]) / static_cast<float>(cfg_.objective_k);
    return sum_recall / static_cast<float>(n_queries_);
}

// GetOutputCentroids (superkmeans.h:1341-1351)
void Engine::output_centroids(float* out_host) {
    PhaseScope ps(*this, PH_ROTATE);   // the reference's profiler books Unrotate under "rotator" too
    if (cfg_.unrotate_centroids) {
        ensure_rotation();
        DeviceBuffer<float> tmp;
        tmp.ensure(k_ * d_);
        launch_gemm_nt(c_cur_.get(), d_, mt_dev_.get(), d_, tmp.get(), d_, k_, d_, d_, stream_);
        SKM_CUDA(cudaMemcpyAsync(out_host, tmp.get(), sizeof(float) * k_ * d_, cudaMemcpyDeviceToHost, stream_));
        sync();
    } else {
        SKM_CUDA(cudaMemcpyAsync(out_host, c_cur_.get(), sizeof(float) * k_ * d_, cudaMemcpyDeviceToHost, stream_));
        sync();
    }
}

// -------------------------------------------------------------------------------------------------
// HierarchicalSuperKMeans::Train (hierarchical_superkmeans.h:84-541)
// -------------------------------------------------------------------------------------------------
void Engine::train_hierarchical(const float* data, size_t n, bool on_device, float* centroids_out) {
    stats_meso_.clear();
    stats_fine_.clear();
    stats_refine_.clear();
    n_meso_ = n_mesoclusters(k_);
    n_samples_ = n_vectors_to_sample(n, k_, cfg_.sampling_fraction, cfg_.max_points_per_cluster, true);
    if (n_samples_ < k_) {
        throw std::runtime_error("Not enough samples to train. Try increasing the sampling_fraction or max_points_per_cluster");
    }
    const size_t n_all = n_samples_;
    const bool rotate = !cfg_.data_already_rotated;
    partial_d_ = initial_partial_d(vertical_d_);
    const uint32_t initial_pd = partial_d_;

    c_cur_.ensure(k_ * d_);
    c_prev_.ensure(k_ * d_);
    c_pdx_.ensure(k_ * d_);
    c_aux_.ensure(k_ * static_cast<size_t>(vertical_d_) + 1);
    centroid_norms_.ensure(k_);
    counts_.ensure(k_);
    counts_host_.ensure(k_);
    assignments_.ensure(n);
    distances_.ensure(n);
    not_pruned_.ensure(n_all);
    data_norms_.ensure(n_all);
    full_norms_.ensure(n_all);
    final_assignments_.ensure(n_all);
    final_centroids_.ensure(k_ * d_);
    x_rot_.ensure(n_all * d_);
    SKM_CUDA(cudaMemsetAsync(assignments_.get(), 0, sizeof(uint32_t) * n, stream_));
    // Points that no mesocluster's index range covers (possible only when the last mesoclustering iteration split clusters,
    // see the partition below) keep cluster 0, as with the reference's freshly mapped array (hierarchical_superkmeans.h:121).
    SKM_CUDA(cudaMemsetAsync(final_assignments_.get(), 0, sizeof(uint32_t) * n_all, stream_));
    prepare_update_workspace(n_all, k_);

    // ---- phase 1: mesoclustering (:161-257)
    generate_centroids_from_host(data, on_device, n_all, n_meso_, rotate);
    if (n_all < n) {
        sampled_indices_ = sampling_permutation(n, cfg_.seed);
        const size_t rows = chunk_rows_for(d_, n_all);
        std::vector<float> staged;
        DeviceBuffer<uint64_t> idx_dev;
        DeviceBuffer<float> raw;
        std::vector<uint64_t> idx64;
        if (on_device) {
            idx_dev.ensure(rows);
            raw.ensure(rows * d_);
            idx64.resize(rows);
        } else {
            staged.resize(rows * d_);
        }
        for (size_t r0 = 0; r0 < n_all; r0 += rows) {
            const size_t cnt = std::min(rows, n_all - r0);
            if (on_device) {
                for (size_t i = 0; i < cnt; ++i) idx64[i] = sampled_indices_[r0 + i];
                SKM_CUDA(cudaMemcpyAsync(idx_dev.get(), idx64.data(), sizeof(uint64_t) * cnt, cudaMemcpyHostToDevice, stream_));
                float* dst = rotate ? raw.get() : x_rot_.get() + r0 * d_;
                launch_gather_rows(data, idx_dev.get(), dst, cnt, d_, stream_);
                if (rotate) rotate_to_device(raw.get(), true, cnt, x_rot_.get() + r0 * d_);
                sync();
            } else {
                gather_host_rows(data, sampled_indices_.data() + r0, cnt, d_, staged.data());
                if (rotate) rotate_to_device(staged.data(), false, cnt, x_rot_.get() + r0 * d_);
                else upload_rows(staged.data(), false, cnt, x_rot_.get() + r0 * d_);
            }
        }
    } else {
        if (rotate) rotate_to_device(data, on_device, n_all, x_rot_.get());
        else upload_rows(data, on_device, n_all, x_rot_.get());
    }
    sync();
    launch_row_sqnorms(x_rot_.get(), n_all, d_, d_, data_norms_.get(), stream_);
    SKM_CUDA(cudaMemcpyAsync(full_norms_.get(), data_norms_.get(), sizeof(float) * n_all, cudaMemcpyDeviceToDevice, stream_));

    {
        const bool always_gemm_only = d_ < kDimensionThresholdForPruning || cfg_.use_blas_only || n_meso_ <= kNClustersThresholdForPruning;
        bool partial_norms_computed = false;
        IterationInput in{x_rot_.get(), n_all, n_all, n_meso_, data_norms_.get()};
        for (size_t iter = 0; iter < cfg_.iters_mesoclustering; ++iter) {
            const bool gemm_only = (iter == 0) || always_gemm_only;
            if (!gemm_only && !partial_norms_computed) {
                launch_row_sqnorms(x_rot_.get(), n_all, d_, partial_d_, data_norms_.get(), stream_);
                partial_norms_computed = true;
            }
            run_iteration(gemm_only, in, iter, iter == 0, stats_meso_);
            if (cfg_.early_termination && should_stop_early(shift_, cost_, prev_cost_, cfg_.tol, iter)) break;
        }
    }

    // ---- partition the points by mesocluster (:260-286).  The sizes are cluster_sizes as left by
    // the last split, exactly as in the reference; writes that would leave the index array (possible
    // only when that split moved sizes around) are dropped.
    const std::vector<uint32_t> meso_sizes(sizes_host_.begin(), sizes_host_.begin() + n_meso_);
    std::vector<size_t> offsets(n_meso_ + 1, 0);
    for (size_t m = 0; m < n_meso_; ++m) offsets[m + 1] = offsets[m] + meso_sizes[m];
    meso_indices_dev_.ensure(n_all);
    if (n_split_ == 0 && offsets[n_meso_] == n_all) {
        // No split in the last mesoclustering iteration: the sizes are the actual counts, and the partition is the stable
        // sort of the point indices by mesocluster - on the device, with the update's radix sort.
        const uint32_t* sorted_keys = nullptr;
        const uint32_t* order = nullptr;
        launch_sort_by_key(assignments_.get(), n_all, n_meso_, ws_, &sorted_keys, &order, stream_);
        widen_u32_kernel<<<static_cast<unsigned>((n_all + 255) / 256), 256, 0, stream_>>>(order, meso_indices_dev_.get(), n_all);
        note_kernel_launch();
        SKM_CUDA(cudaGetLastError());
    } else {
        std::vector<uint32_t> meso_assign(n_all);
        SKM_CUDA(cudaMemcpyAsync(meso_assign.data(), assignments_.get(), sizeof(uint32_t) * n_all, cudaMemcpyDeviceToHost, stream_));
        sync();
        std::vector<uint64_t> flat(n_all, 0);
        std::vector<size_t> next = offsets;
        for (size_t i = 0; i < n_all; ++i) {
            const size_t pos = next[meso_assign[i]]++;
            if (pos < n_all) flat[pos] = i;
        }
        SKM_CUDA(cudaMemcpyAsync(meso_indices_dev_.get(), flat.data(), sizeof(uint64_t) * n_all, cudaMemcpyHostToDevice, stream_));
        sync();
    }

    // ---- phase 2: fine clustering, one mesocluster after the other (:301-425)
    const std::vector<size_t> fine_nums = arrange_fine_clusters(k_, n_meso_, n_all, meso_sizes);
    const size_t max_meso = *std::max_element(meso_sizes.begin(), meso_sizes.end());
    meso_buffer_.ensure(std::max<size_t>(max_meso, 1) * d_);
    meso_norms_.ensure(std::max<size_t>(max_meso, 1));
    // The Forgy rows of every mesocluster (a shuffle of its member positions each) are drawn ahead by a host thread.
    auto meso_rows = [&](size_t m) { return std::min<size_t>(meso_sizes[m], n_all - std::min(offsets[m], n_all)); };
    std::vector<std::vector<size_t>> forgy(n_meso_);
    std::atomic<size_t> forgy_done{0};
    std::thread forgy_thread([&, seed = cfg_.seed] {
        for (size_t m = 0; m < n_meso_; ++m) {
            if (fine_nums[m] != 0) forgy[m] = forgy_indices(meso_rows(m), fine_nums[m], seed);
            forgy_done.store(m + 1, std::memory_order_release);
        }
    });
    struct Joiner {
        std::thread& t;
        ~Joiner() {
            if (t.joinable()) t.join();
        }
    } joiner{forgy_thread};
    size_t fine_offset = 0;
    for (size_t m = 0; m < n_meso_; ++m) {
        const size_t n_fine = fine_nums[m];
        if (n_fine == 0) continue;
        partial_d_ = initial_pd;
        const size_t msize = meso_rows(m);
        n_samples_ = msize;
        if (msize < n_fine) {
            throw std::runtime_error("a mesocluster holds fewer points than the fine clusters allotted to it");
        }
        const uint64_t* idx = meso_indices_dev_.get() + offsets[m];
        launch_gather_rows(x_rot_.get(), idx, meso_buffer_.get(), msize, d_, stream_);      // CompactMesoclusterToBuffer (:685-704)
        launch_gather_f32(full_norms_.get(), idx, meso_norms_.get(), msize, stream_);
        while (forgy_done.load(std::memory_order_acquire) <= m) std::this_thread::yield();
        generate_centroids_from_device_rows(meso_buffer_.get(), msize, n_fine, &forgy[m]);

        const bool always_gemm_only = d_ < kDimensionThresholdForPruning || cfg_.use_blas_only || n_fine <= kNClustersThresholdForPruning;
        bool partial_norms_computed = false;
        IterationInput in{meso_buffer_.get(), msize, msize, n_fine, meso_norms_.get()};
        for (size_t iter = 0; iter < cfg_.iters_fineclustering; ++iter) {
            const bool gemm_only = (iter == 0) || always_gemm_only;
            if (!gemm_only && !partial_norms_computed) {
                launch_row_sqnorms(meso_buffer_.get(), msize, d_, partial_d_, meso_norms_.get(), stream_);
                partial_norms_computed = true;
            }
            run_iteration(gemm_only, in, iter, iter == 0, stats_fine_);
            if (cfg_.early_termination && should_stop_early(shift_, cost_, prev_cost_, cfg_.tol, iter)) break;
        }
        // GetTrueAssignmentsFromIndirectionBuffer (:763-779) and the centroid copy (:416-423)
        launch_scatter_u32_offset(assignments_.get(), idx, final_assignments_.get(), msize, static_cast<uint32_t>(fine_offset), stream_);
        SKM_CUDA(cudaMemcpyAsync(final_centroids_.get() + fine_offset * d_, c_cur_.get(), sizeof(float) * n_fine * d_, cudaMemcpyDeviceToDevice, stream_));
        fine_offset += n_fine;
    }

    // ---- phase 3: refinement over all clusters (:434-516)
    n_samples_ = n_all;
    partial_d_ = std::max<uint32_t>(kMinPartialD, vertical_d_ / 3);
    SKM_CUDA(cudaMemcpyAsync(c_cur_.get(), final_centroids_.get(), sizeof(float) * k_ * d_, cudaMemcpyDeviceToDevice, stream_));   // SetupCentroids (:788-815)
    launch_pdxify(c_cur_.get(), c_pdx_.get(), c_aux_.get(), k_, d_, vertical_d_, stream_);
    SKM_CUDA(cudaMemcpyAsync(c_prev_.get(), final_centroids_.get(), sizeof(float) * k_ * d_, cudaMemcpyDeviceToDevice, stream_));
    SKM_CUDA(cudaMemcpyAsync(assignments_.get(), final_assignments_.get(), sizeof(uint32_t) * n_all, cudaMemcpyDeviceToDevice, stream_));
    {
        const bool always_gemm_only = d_ < kDimensionThresholdForPruning || k_ <= kNClustersThresholdForPruning;
        bool partial_norms_computed = false;
        IterationInput in{x_rot_.get(), n_all, n_all, k_, data_norms_.get()};
        for (size_t iter = 0; iter < cfg_.iters_refinement; ++iter) {
            if (!always_gemm_only && !partial_norms_computed) {
                launch_row_sqnorms(x_rot_.get(), n_all, d_, partial_d_, data_norms_.get(), stream_);
                partial_norms_computed = true;
            } else if (always_gemm_only && !partial_norms_computed) {
                // data_norms_ still holds whatever the mesoclustering left; GEMM-only needs full norms.
                SKM_CUDA(cudaMemcpyAsync(data_norms_.get(), full_norms_.get(), sizeof(float) * n_all, cudaMemcpyDeviceToDevice, stream_));
                partial_norms_computed = true;
            }
            run_iteration(always_gemm_only, in, iter, false, stats_refine_);
        }
    }
    sync();
    n_state_rows_ = n_all;
    trained_ = true;
    output_centroids(centroids_out);
    x_rot_.release();
    meso_buffer_.release();
    ws_partials_.release();
}

// -------------------------------------------------------------------------------------------------
// Assign (superkmeans.h:346-382): stateless brute force in the caller's domain, streamed in row
// chunks so that host inputs of any size fit.
// -------------------------------------------------------------------------------------------------
void Engine::assign(const float* vectors, const float* centroids, size_t n, size_t n_centroids, bool on_device, uint32_t* out) {
    DeviceGuard guard(device_);
    if (n == 0) return;
    if (n_centroids == 0) throw std::invalid_argument("Value must be positive: n_centroids");
    DeviceBuffer<float> c_dev_own, cn;
    const float* c_dev = centroids;
    if (!on_device) {
        SKM_CUDA(cudaMemcpyAsync(c_dev_own.ensure(n_centroids * d_), centroids, sizeof(float) * n_centroids * d_, cudaMemcpyHostToDevice, stream_));
        c_dev = c_dev_own.get();
    }
    launch_row_sqnorms(c_dev, n_centroids, d_, d_, cn.ensure(n_centroids), stream_);
    if (on_device) {
        DeviceBuffer<float> xn, dist;
        xn.ensure(n);
        dist.ensure(n);
        top2_.ensure(n);
        y_split_.ensure(2 * n_centroids * d_);
        {
            PhaseScope ps(*this, PH_ASSIGN_FULL);
            launch_row_sqnorms(vectors, n, d_, d_, xn.get(), stream_);
            launch_assign_full(vectors, c_dev, n, n_centroids, d_, xn.get(), cn.get(), out, dist.get(), top2_.get(), stream_, y_split_.get());
        }
        sync();
        check_tc_error(stream_);
        return;
    }
    const size_t rows = chunk_rows_for(d_, n);
    DeviceBuffer<float> xb[2], xn[2], dist[2];
    DeviceBuffer<uint32_t> knn[2];
    cudaEvent_t copied[2], consumed[2];
    for (int i = 0; i < 2; ++i) {
        xb[i].ensure(rows * d_);
        xn[i].ensure(rows);
        dist[i].ensure(rows);
        knn[i].ensure(rows);
        SKM_CUDA(cudaEventCreateWithFlags(&copied[i], cudaEventDisableTiming));
        SKM_CUDA(cudaEventCreateWithFlags(&consumed[i], cudaEventDisableTiming));
    }
    size_t ci = 0;
    top2_.ensure(rows);
    y_split_.ensure(2 * n_centroids * d_);
    timers_.begin(PH_ASSIGN_FULL, stream_);
    for (size_t r0 = 0; r0 < n; r0 += rows, ++ci) {
        const int b = static_cast<int>(ci & 1);
        const size_t cnt = std::min(rows, n - r0);
        if (ci >= 2) SKM_CUDA(cudaStreamWaitEvent(copy_stream_, consumed[b], 0));
        SKM_CUDA(cudaMemcpyAsync(xb[b].get(), vectors + r0 * d_, sizeof(float) * cnt * d_, cudaMemcpyHostToDevice, copy_stream_));
        SKM_CUDA(cudaEventRecord(copied[b], copy_stream_));
        SKM_CUDA(cudaStreamWaitEvent(stream_, copied[b], 0));
        launch_row_sqnorms(xb[b].get(), cnt, d_, d_, xn[b].get(), stream_);
        launch_assign_full(xb[b].get(), c_dev, cnt, n_centroids, d_, xn[b].get(), cn.get(), knn[b].get(), dist[b].get(), top2_.ensure(rows), stream_, y_split_.ensure(2 * n_centroids * d_));
        SKM_CUDA(cudaMemcpyAsync(out + r0, knn[b].get(), sizeof(uint32_t) * cnt, cudaMemcpyDeviceToHost, stream_));
        SKM_CUDA(cudaEventRecord(consumed[b], stream_));
    }
    timers_.end(stream_);
    sync();
    for (int i = 0; i < 2; ++i) {
        cudaEventDestroy(copied[i]);
        cudaEventDestroy(consumed[i]);
    }
    check_tc_error(stream_);
}

// -------------------------------------------------------------------------------------------------
// AssignTrainingPoints (superkmeans.h:397-564)
// -------------------------------------------------------------------------------------------------
void Engine::assign_training_points(const float* vectors, const float* centroids, size_t n, size_t n_centroids, bool on_device, uint32_t* out) {
    DeviceGuard guard(device_);
    if (!trained_) throw std::runtime_error("AssignTrainingPoints requires SuperKMeans to be trained first");
    if (cfg_.use_blas_only || d_ < kDimensionThresholdForPruning || k_ <= kNClustersThresholdForPruning) {
        if (!cfg_.suppress_warnings) {
            std::cout << "WARNING: AssignTrainingPoints cannot use pruning, falling back to brute force Assign" << std::endl;
        }
        assign(vectors, centroids, n, n_centroids, on_device, out);
        return;
    }
    if (n == 0) return;
    partial_d_ = initial_partial_d(vertical_d_);
    launch_row_sqnorms(c_cur_.get(), k_, d_, partial_d_, centroid_norms_.get(), stream_);

    // Seeds: one starting centroid per vector.
    std::vector<uint32_t> seeds(n);
    const bool store_state = (cfg_.sampling_fraction == 1.0f);
    if (cfg_.sampling_fraction == 1.0f) {
        if (n > assignments_.capacity()) throw std::runtime_error("AssignTrainingPoints needs the vectors used in Train()");
        SKM_CUDA(cudaMemcpyAsync(seeds.data(), assignments_.get(), sizeof(uint32_t) * n, cudaMemcpyDeviceToHost, stream_));
        sync();
    } else {
        if (sampled_indices_.size() != n) throw std::runtime_error("AssignTrainingPoints needs the vectors used in Train()");
        std::vector<uint32_t> trained_assign(n_samples_);
        SKM_CUDA(cudaMemcpyAsync(trained_assign.data(), assignments_.get(), sizeof(uint32_t) * n_samples_, cudaMemcpyDeviceToHost, stream_));
        sync();
        size_t cur = 0;
        for (; cur < n_samples_; ++cur) seeds[sampled_indices_[cur]] = trained_assign[cur];
        if (cfg_.sampling_fraction <= 0.8f && on_device) {
            throw std::runtime_error("AssignTrainingPoints with sampling_fraction <= 0.8 needs host vectors");
        }
        if (cfg_.sampling_fraction > 0.8f) {
            // Size-proportional random seeds (:477-484).
            std::mt19937 rng(cfg_.seed + 1);
            std::discrete_distribution<uint32_t> cluster_dist(sizes_host_.begin(), sizes_host_.begin() + k_);
            for (; cur < n; ++cur) seeds[sampled_indices_[cur]] = cluster_dist(rng);
        } else {
            // Two-level seeds (:505-542): cluster the centroids into sqrt(k) groups and start every
            // unsampled vector at one representative centroid of its group.
            std::vector<float> cent_host(n_centroids * d_), vec_host_own;
            if (on_device) {
                SKM_CUDA(cudaMemcpy(cent_host.data(), centroids, sizeof(float) * n_centroids * d_, cudaMemcpyDeviceToHost));
            } else {
                std::memcpy(cent_host.data(), centroids, sizeof(float) * n_centroids * d_);
            }
            skm_config tmp{};
            skm_default_config(&tmp, 0);
            tmp.iters = 10;
            tmp.sampling_fraction = 1.0f;
            tmp.use_blas_only = 0;
            tmp.verbose = cfg_.verbose;
            tmp.suppress_warnings = cfg_.suppress_warnings;
            tmp.seed = cfg_.seed;
            tmp.angular = cfg_.angular;
            tmp.data_already_rotated = cfg_.data_already_rotated;
            const size_t n_meso = static_cast<size_t>(std::sqrt(n_centroids));
            Engine nested(tmp, n_meso, d_, false, device_);
            if (!rotation_host_.empty()) nested.set_rotation(rotation_host_.data());
            std::vector<float> meso_centroids(n_meso * d_);
            nested.train(cent_host.data(), n_centroids, false, nullptr, 0, meso_centroids.data());
            std::vector<uint32_t> meso_assign(n), cent_to_meso(n_centroids);
            nested.assign(vectors, meso_centroids.data(), n, n_meso, false, meso_assign.data());
            nested.assign(cent_host.data(), meso_centroids.data(), n_centroids, n_meso, false, cent_to_meso.data());
            std::vector<uint32_t> meso_to_original(n_meso, 0);
            for (size_t c = 0; c < n_centroids; ++c) meso_to_original[cent_to_meso[c]] = static_cast<uint32_t>(c);
            for (; cur < n; ++cur) {
                const size_t orig = sampled_indices_[cur];
                seeds[orig] = meso_to_original[meso_assign[orig]];
            }
        }
    }

    if (store_state) {
        assignments_.ensure(n);
        distances_.ensure(n);
        n_state_rows_ = n;
    }
    const size_t rows = chunk_rows_for(d_, n);
    DeviceBuffer<float> xr, xn, dist;
    DeviceBuffer<uint32_t> knn, np;
    xr.ensure(rows * d_);
    xn.ensure(rows);
    dist.ensure(rows);
    knn.ensure(rows);
    np.ensure(rows);
    for (size_t r0 = 0; r0 < n; r0 += rows) {
        const size_t cnt = std::min(rows, n - r0);
        if (cfg_.data_already_rotated) upload_rows(vectors + r0 * d_, on_device, cnt, xr.get());
        else rotate_to_device(vectors + r0 * d_, on_device, cnt, xr.get());
        launch_row_sqnorms(xr.get(), cnt, d_, partial_d_, xn.get(), stream_);
        SKM_CUDA(cudaMemcpyAsync(knn.get(), seeds.data() + r0, sizeof(uint32_t) * cnt, cudaMemcpyHostToDevice, stream_));
        run_pruned_pass(xr.get(), cnt, k_, c_cur_.get(), xn.get(), centroid_norms_.get(), knn.get(), dist.get(), np.get());
        SKM_CUDA(cudaMemcpyAsync(out + r0, knn.get(), sizeof(uint32_t) * cnt, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, stream_));
        if (store_state) {
            SKM_CUDA(cudaMemcpyAsync(assignments_.get() + r0, knn.get(), sizeof(uint32_t) * cnt, cudaMemcpyDeviceToDevice, stream_));
            SKM_CUDA(cudaMemcpyAsync(distances_.get() + r0, dist.get(), sizeof(float) * cnt, cudaMemcpyDeviceToDevice, stream_));
        }
        sync();
    }
}

void Engine::get_assignments(uint32_t* out, size_t n) {
    DeviceGuard guard(device_);
    if (n > n_state_rows_ || n > assignments_.capacity()) throw std::invalid_argument("more assignments requested than the engine holds");
    SKM_CUDA(cudaMemcpy(out, assignments_.get(), sizeof(uint32_t) * n, cudaMemcpyDeviceToHost));
}

void Engine::get_distances(float* out, size_t n) {
    DeviceGuard guard(device_);
    if (n > n_state_rows_ || n > distances_.capacity()) throw std::invalid_argument("more distances requested than the engine holds");
    SKM_CUDA(cudaMemcpy(out, distances_.get(), sizeof(float) * n, cudaMemcpyDeviceToHost));
}

void Engine::get_rotated_centroids(float* out) {
    DeviceGuard guard(device_);
    if (!trained_) throw std::runtime_error("the model has not been trained");
    SKM_CUDA(cudaMemcpy(out, c_cur_.get(), sizeof(float) * k_ * d_, cudaMemcpyDeviceToHost));
}

// -------------------------------------------------------------------------------------------------
// Stateless operators
// -------------------------------------------------------------------------------------------------
namespace {
struct OpContext {
    DeviceGuard guard;
    cudaStream_t stream = nullptr;
    explicit OpContext(int device) : guard(resolve_device(device)) { SKM_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking)); }
    ~OpContext() {
        if (stream) cudaStreamDestroy(stream);
    }
    template <class T>
    T* upload(DeviceBuffer<T>& buf, const T* host, size_t count) {
        T* p = buf.ensure(count);
        if (count) SKM_CUDA(cudaMemcpyAsync(p, host, sizeof(T) * count, cudaMemcpyHostToDevice, stream));
        return p;
    }
    template <class T>
    void download(T* host, const T* dev, size_t count) {
        if (count) SKM_CUDA(cudaMemcpyAsync(host, dev, sizeof(T) * count, cudaMemcpyDeviceToHost, stream));
    }
    void sync() { SKM_CUDA(cudaStreamSynchronize(stream)); }
};
} // namespace

void Engine::op_rotate(int device, const float* m, const float* x, size_t n, size_t d, float* out, bool inverse) {
    OpContext ctx(device);
    DeviceBuffer<float> md, mtd, xd, od;
    ctx.upload(md, m, d * d);
    const float* b = md.get();
    if (inverse) {
        launch_transpose_square(md.get(), mtd.ensure(d * d), d, ctx.stream);
        b = mtd.get();
    }
    ctx.upload(xd, x, n * d);
    launch_gemm_nt(xd.get(), d, b, d, od.ensure(n * d), d, n, d, d, ctx.stream);
    ctx.download(out, od.get(), n * d);
    ctx.sync();
    check_tc_error(ctx.stream);
}

void Engine::op_find_nearest(int device, const float* x, const float* y, size_t n, size_t k, size_t d, uint32_t* out_knn, float* out_dist) {
    OpContext ctx(device);
    DeviceBuffer<float> xd, yd, nx, ny, dist;
    DeviceBuffer<uint32_t> knn;
    ctx.upload(xd, x, n * d);
    ctx.upload(yd, y, k * d);
    launch_row_sqnorms(xd.get(), n, d, d, nx.ensure(n), ctx.stream);
    launch_row_sqnorms(yd.get(), k, d, d, ny.ensure(k), ctx.stream);
    DeviceBuffer<uint2> top2;
    DeviceBuffer<float> ysplit;
    launch_assign_full(xd.get(), yd.get(), n, k, d, nx.get(), ny.get(), knn.ensure(n), dist.ensure(n), top2.ensure(n), ctx.stream, ysplit.ensure(2 * k * d));
    ctx.download(out_knn, knn.get(), n);
    ctx.download(out_dist, dist.get(), n);
    ctx.sync();
    check_tc_error(ctx.stream);
}

void Engine::op_find_nearest_pruned(int device, const float* x, const float* y, size_t n, size_t k, size_t d, float eps0, uint32_t partial_d, uint32_t* knn_io, float* dist_out,
                                    uint64_t* not_pruned_out) {
    const DimensionSplit split = dimension_split(d);
    if (split.horizontal_d == 0) throw std::invalid_argument("the pruned search needs d > 64");
    if (partial_d == 0 || partial_d > split.vertical_d) throw std::invalid_argument("partial_d must be in [1, vertical_d]");
    for (size_t i = 0; i < n; ++i)
        if (knn_io[i] >= k) throw std::invalid_argument("previous assignment out of range");
    OpContext ctx(device);
    DeviceBuffer<float> xd, yd, nx, ny, pdx, aux, dist, ratios_d;
    DeviceBuffer<uint32_t> knn, np;
    const std::vector<float> ratios = make_ratios(d, eps0);
    ctx.upload(xd, x, n * d);
    ctx.upload(yd, y, k * d);
    ctx.upload(ratios_d, ratios.data(), d + 1);
    ctx.upload(knn, knn_io, n);
    launch_row_sqnorms(xd.get(), n, d, partial_d, nx.ensure(n), ctx.stream);
    launch_row_sqnorms(yd.get(), k, d, partial_d, ny.ensure(k), ctx.stream);
    launch_pdxify(yd.get(), pdx.ensure(k * d), aux.ensure(k * split.vertical_d + 1), k, d, split.vertical_d, ctx.stream);
    int dev = 0;
    SKM_CUDA(cudaGetDevice(&dev));
    PrunedParams p{};
    p.x = xd.get();
    p.y = yd.get();
    p.y_pdx = pdx.get();
    p.y_aux = aux.get();
    p.norms_x = nx.get();
    p.norms_y = ny.get();
    p.ratios = ratios_d.get();
    p.knn = knn.get();
    p.dist = dist.ensure(n);
    p.not_pruned = np.ensure(n);
    p.n = n;
    p.k = k;
    p.d = d;
    p.partial_d = partial_d;
    p.vertical_d = static_cast<uint32_t>(split.vertical_d);
    p.horizontal_d = static_cast<uint32_t>(split.horizontal_d);
    PrunePassBuffers bufs;
    run_pruned_pass_on(p, bufs, ratios[partial_d], dev, ctx.stream);
    std::vector<uint32_t> np_host(n);
    ctx.download(knn_io, knn.get(), n);
    ctx.download(dist_out, dist.get(), n);
    ctx.download(np_host.data(), np.get(), n);
    ctx.sync();
    for (size_t i = 0; i < n; ++i) not_pruned_out[i] = np_host[i];
}

void Engine::op_update(int device, const float* x, const uint32_t* assign, const float* dist, size_t n, size_t k, size_t d, float* sums_out, uint32_t* counts_out, double* wcss_out) {
    for (size_t i = 0; i < n; ++i)
        if (assign[i] >= k) throw std::invalid_argument("assignment out of range");
    OpContext ctx(device);
    DeviceBuffer<float> xd, dd, sums, partials;
    DeviceBuffer<uint32_t> ad, counts, ka, kb, va, vb, table, offs;
    DeviceBuffer<double> block_sums, wcss;
    ctx.upload(xd, x, n * d);
    ctx.upload(ad, assign, n);
    std::vector<float> zeros;
    if (dist) ctx.upload(dd, dist, n);
    else {
        zeros.assign(n, 0.f);
        ctx.upload(dd, zeros.data(), n);
    }
    UpdateWorkspace ws;
    const size_t units = update_sort_units(n), tiles = update_tiles(n);
    ws.keys_a = ka.ensure(n);
    ws.keys_b = kb.ensure(n);
    ws.vals_a = va.ensure(n);
    ws.vals_b = vb.ensure(n);
    ws.digit_table = table.ensure(256 * units + (256 * units) / 2048 + 64);
    ws.seg_offsets = offs.ensure(k + 1);
    ws.tile_partials = partials.ensure(std::max<size_t>(tiles, 1) * 2 * d);
    ws.block_sums = block_sums.ensure(2048);
    launch_update(xd.get(), ad.get(), dd.get(), nullptr, n, k, d, ws, sums.ensure(k * d), counts.ensure(k), wcss.ensure(1), nullptr, ctx.stream);
    ctx.download(sums_out, sums.get(), k * d);
    ctx.download(counts_out, counts.get(), k);
    double w = 0.0;
    ctx.download(&w, wcss.get(), 1);
    ctx.sync();
    if (wcss_out) *wcss_out = w;
}

void Engine::op_pdxify(int device, const float* in, size_t n, size_t d, float* out) {
    OpContext ctx(device);
    DeviceBuffer<float> id, od;
    ctx.upload(id, in, n * d);
    launch_pdxify(id.get(), od.ensure(n * d), nullptr, n, d, dimension_split(d).vertical_d, ctx.stream);
    ctx.download(out, od.get(), n * d);
    ctx.sync();
}

} // namespace skmb
