// extern "C" surface of libskm_b200.so (declared in include/skm_b200.h): translates between the C
// ABI and the Engine class, and between C++ exceptions and status codes.
#include <cstring>
#include <memory>
#include <new>
#include <string>

#include "engine.h"
#include "noalloc.h"
#include "kernels_tc.cuh"

using skmb::Engine;

struct skm_comm {
    std::unique_ptr<skmb::NcclComm> comm;
};

struct skm_handle {
    std::unique_ptr<Engine> engine;
    mutable std::string err;
};

namespace {

thread_local std::string g_create_error;

template <class F>
skm_status guarded(std::string& err, F&& f) {
    try {
        f();
        return SKM_OK;
    } catch (const std::invalid_argument& e) {
        err = e.what();
        return SKM_INVALID_ARGUMENT;
    } catch (const skmb::CudaError& e) {
        err = e.what();
        return SKM_CUDA_ERROR;
    } catch (const std::runtime_error& e) {
        err = e.what();
        return SKM_RUNTIME_ERROR;
    } catch (const std::bad_alloc&) {
        err = "out of host memory";
        return SKM_RUNTIME_ERROR;
    } catch (const std::exception& e) {
        err = e.what();
        return SKM_RUNTIME_ERROR;
    }
}

thread_local std::string g_op_error;

} // namespace

extern "C" {

void skm_default_config(skm_config* c, int hierarchical) {
    c->iters = 10;
    c->sampling_fraction = hierarchical ? 1.0f : 0.3f;
    c->max_points_per_cluster = 256;
    c->n_threads = 0;
    c->seed = 42;
    c->use_blas_only = 0;
    c->tol = 1e-4f;
    c->recall_tol = 0.005f;
    c->early_termination = 1;
    c->sample_queries = 0;
    c->objective_k = 100;
    c->ann_explore_fraction = 0.01f;
    c->min_not_pruned_pct = 0.03f;
    c->max_not_pruned_pct = 0.05f;
    c->adjustment_factor_for_partial_d = 0.20f;
    c->unrotate_centroids = 1;
    c->verbose = 0;
    c->angular = 0;
    c->suppress_warnings = 0;
    c->data_already_rotated = 0;
    c->iters_mesoclustering = 3;
    c->iters_fineclustering = 5;
    c->iters_refinement = 0;
}

const char* skm_last_error(const skm_handle* h) {
    if (!h) return g_create_error.empty() ? g_op_error.c_str() : g_create_error.c_str();
    return h->err.c_str();
}

skm_status skm_create(const skm_config* cfg, uint64_t n_clusters, uint64_t dimensionality, int hierarchical, int device, skm_handle** out) {
    g_create_error.clear();
    if (!out) {
        g_create_error = "out must not be NULL";
        return SKM_INVALID_ARGUMENT;
    }
    *out = nullptr;
    skm_config local;
    if (cfg) local = *cfg;
    else skm_default_config(&local, hierarchical);
    auto h = std::make_unique<skm_handle>();
    const skm_status st = guarded(g_create_error, [&] { h->engine = std::make_unique<Engine>(local, n_clusters, dimensionality, hierarchical != 0, device); });
    if (st == SKM_OK) *out = h.release();
    return st;
}

void skm_destroy(skm_handle* h) { delete h; }

#define SKM_NEED(h)                                                                                \
    if (!(h) || !(h)->engine) return SKM_INVALID_ARGUMENT

skm_status skm_set_rotation(skm_handle* h, const float* m) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->set_rotation(m); });
}

skm_status skm_use_dct_rotation(skm_handle* h) {
    SKM_NEED(h);
    return guarded(h->err, [&] {
        const std::vector<float> m = skmb::make_dct_rotation_matrix(h->engine->dimensionality(), h->engine->config().seed);
        h->engine->set_rotation(m.data());
    });
}

skm_status skm_get_rotation(skm_handle* h, float* m_out) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->get_rotation(m_out); });
}

skm_status skm_train(skm_handle* h, const float* data, uint64_t n, int data_on_device, const float* queries, uint64_t n_queries, float* centroids_out) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->train(data, n, data_on_device != 0, queries, n_queries, centroids_out); });
}

skm_status skm_assign(skm_handle* h, const float* vectors, const float* centroids, uint64_t n, uint64_t n_centroids, int on_device, uint32_t* out) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->assign(vectors, centroids, n, n_centroids, on_device != 0, out); });
}

skm_status skm_assign_training_points(skm_handle* h, const float* vectors, const float* centroids, uint64_t n, uint64_t n_centroids, int on_device, uint32_t* out) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->assign_training_points(vectors, centroids, n, n_centroids, on_device != 0, out); });
}

uint64_t skm_n_clusters(const skm_handle* h) { return (h && h->engine) ? h->engine->n_clusters() : 0; }
int skm_is_trained(const skm_handle* h) { return (h && h->engine) ? (h->engine->trained() ? 1 : 0) : 0; }
float skm_sampling_fraction(const skm_handle* h) { return (h && h->engine) ? h->engine->sampling_fraction() : 0.f; }
uint64_t skm_n_mesoclusters(const skm_handle* h) { return (h && h->engine) ? h->engine->n_mesoclusters_value() : 0; }
uint64_t skm_get_n_samples(const skm_handle* h) { return (h && h->engine) ? h->engine->n_state_rows() : 0; }
int skm_last_prune_path(const skm_handle* h) { return (h && h->engine) ? h->engine->last_prune_path() : 0; }

skm_status skm_get_prune_counters(const skm_handle* h, uint64_t* out3) {
    SKM_NEED(h);
    if (!out3) return SKM_INVALID_ARGUMENT;
    h->engine->prune_counters(out3);
    return SKM_OK;
}
skm_status skm_get_chain_counters(const skm_handle* h, uint64_t* out4) {
    SKM_NEED(h);
    if (!out4) return SKM_INVALID_ARGUMENT;
    h->engine->chain_counters(out4);
    return SKM_OK;
}
double skm_last_objective_f64(const skm_handle* h) { return (h && h->engine) ? h->engine->last_objective_f64() : 0.0; }

skm_status skm_get_iteration_stats(const skm_handle* h, int phase, skm_iter_stats* out, uint64_t cap, uint64_t* count) {
    SKM_NEED(h);
    const auto& v = h->engine->stats(phase);
    if (count) *count = v.size();
    for (uint64_t i = 0; i < v.size() && i < cap && out; ++i) out[i] = v[i];
    return SKM_OK;
}

skm_status skm_get_assignments(skm_handle* h, uint32_t* out, uint64_t n) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->get_assignments(out, n); });
}

skm_status skm_get_distances(skm_handle* h, float* out, uint64_t n) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->get_distances(out, n); });
}

skm_status skm_get_rotated_centroids(skm_handle* h, float* out) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->get_rotated_centroids(out); });
}

skm_status skm_get_phase_time(const skm_handle* h, int phase, double* ms, uint64_t* calls) {
    SKM_NEED(h);
    if (phase < 0 || phase >= skmb::PH_COUNT) return SKM_INVALID_ARGUMENT;
    if (ms) *ms = h->engine->timers().ms[phase];
    if (calls) *calls = h->engine->timers().calls[phase];
    return SKM_OK;
}

skm_status skm_reset_phase_times(skm_handle* h) {
    SKM_NEED(h);
    h->engine->reset_timers();
    return SKM_OK;
}

skm_status skm_set_trace(skm_handle* h, int enabled) {
    SKM_NEED(h);
    h->engine->set_trace(enabled != 0);
    return SKM_OK;
}

uint64_t skm_trace_count(const skm_handle* h) { return (h && h->engine) ? h->engine->trace().size() : 0; }

skm_status skm_trace_get(const skm_handle* h, uint64_t idx, uint64_t* n_samples, uint64_t* n_clusters, uint32_t* partial_d_next, float* centroids, uint32_t* assign, float* dist,
                         uint32_t* sizes_pre, uint32_t* sizes_post) {
    SKM_NEED(h);
    const auto& tr = h->engine->trace();
    if (idx >= tr.size()) return SKM_INVALID_ARGUMENT;
    const auto& s = tr[idx];
    if (n_samples) *n_samples = s.n_samples;
    if (n_clusters) *n_clusters = s.n_clusters;
    if (partial_d_next) *partial_d_next = s.partial_d_next;
    if (centroids) std::memcpy(centroids, s.centroids.data(), sizeof(float) * s.centroids.size());
    if (assign) std::memcpy(assign, s.assign.data(), sizeof(uint32_t) * s.assign.size());
    if (dist) std::memcpy(dist, s.dist.data(), sizeof(float) * s.dist.size());
    if (sizes_pre) std::memcpy(sizes_pre, s.sizes_pre.data(), sizeof(uint32_t) * s.sizes_pre.size());
    if (sizes_post) std::memcpy(sizes_post, s.sizes_post.data(), sizeof(uint32_t) * s.sizes_post.size());
    return SKM_OK;
}

void skm_set_tensor_cores(int enabled) { skmb::tc::set_enabled(enabled != 0); }
int skm_get_tensor_cores(void) { return skmb::tc::enabled() ? 1 : 0; }

void skm_set_prune_split(int mode) { skmb::set_prune_split_mode(mode); }
int skm_get_prune_split(void) { return skmb::prune_split_mode(); }

skm_status skm_debug_wait_injection(uint64_t wait_limit_cycles, uint32_t producer_stops_after_kblocks) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { skmb::tc::set_debug_wait_injection(static_cast<long long>(wait_limit_cycles), producer_stops_after_kblocks); });
}

skm_status skm_debug_role_cycles(uint64_t* out16) {
    g_create_error.clear();
    if (!out16) return SKM_INVALID_ARGUMENT;
    return guarded(g_op_error, [&] {
        unsigned long long tmp[16];
        skmb::tc::role_cycles(tmp);
        for (int i = 0; i < 16; ++i) out16[i] = tmp[i];
    });
}

uint64_t skm_kernel_launches(void) { return skmb::kernel_launch_count(); }
uint64_t skm_device_allocations(void) { return skmb::device_alloc_count(); }

skm_status skm_set_shard(skm_handle* h, uint64_t n_global, uint64_t row_offset, skm_allreduce_fn fn, void* user) {
    SKM_NEED(h);
    return guarded(h->err, [&] { h->engine->set_shard(n_global, row_offset, fn, user); });
}

skm_status skm_comm_unique_id(uint8_t* id_out) {
    g_create_error.clear();
    if (!id_out) return SKM_INVALID_ARGUMENT;
    return guarded(g_op_error, [&] { skmb::NcclComm::unique_id(id_out); });
}

skm_status skm_comm_create(const uint8_t* id, int rank, int world, int device, skm_comm** out) {
    g_create_error.clear();
    if (!id || !out) return SKM_INVALID_ARGUMENT;
    *out = nullptr;
    auto c = std::make_unique<skm_comm>();
    skm_status st = guarded(g_op_error, [&] { c->comm.reset(skmb::NcclComm::create(id, rank, world, device)); });
    if (st == SKM_RUNTIME_ERROR) st = SKM_COMM_ERROR;
    if (st == SKM_OK) *out = c.release();
    return st;
}

skm_status skm_comm_wrap(void* nccl_comm, int rank, int world, skm_comm** out) {
    g_create_error.clear();
    if (!out) return SKM_INVALID_ARGUMENT;
    *out = nullptr;
    auto c = std::make_unique<skm_comm>();
    skm_status st = guarded(g_op_error, [&] { c->comm.reset(skmb::NcclComm::wrap(nccl_comm, rank, world)); });
    if (st == SKM_RUNTIME_ERROR) st = SKM_COMM_ERROR;
    if (st == SKM_OK) *out = c.release();
    return st;
}

void skm_comm_destroy(skm_comm* comm) { delete comm; }

skm_status skm_set_shard_comm(skm_handle* h, uint64_t n_global, uint64_t row_offset, skm_comm* comm) {
    SKM_NEED(h);
    if (!comm || !comm->comm) return SKM_INVALID_ARGUMENT;
    return guarded(h->err, [&] { h->engine->set_shard_nccl(n_global, row_offset, comm->comm.get()); });
}

void skm_set_workspace_cache(int enabled) { skmb::set_workspace_cache(enabled != 0); }
int skm_get_workspace_cache(void) { return skmb::workspace_cache_enabled() ? 1 : 0; }
void skm_release_cached_memory(void) { skmb::release_cached_memory(); }
uint64_t skm_cached_memory_bytes(void) { return skmb::cached_memory_bytes(); }

// ---- operators ------------------------------------------------------------------------------
skm_status skm_op_rotate(int device, const float* m, const float* x, uint64_t n, uint64_t d, float* out) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { Engine::op_rotate(device, m, x, n, d, out, false); });
}

skm_status skm_op_unrotate(int device, const float* m, const float* x, uint64_t n, uint64_t d, float* out) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { Engine::op_rotate(device, m, x, n, d, out, true); });
}

skm_status skm_op_find_nearest(int device, const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, uint32_t* out_knn, float* out_dist) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { Engine::op_find_nearest(device, x, y, n, k, d, out_knn, out_dist); });
}

skm_status skm_op_find_nearest_pruned(int device, const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, float epsilon0, uint32_t partial_d, uint32_t* knn_io,
                                      float* dist_out, uint64_t* not_pruned_out) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { Engine::op_find_nearest_pruned(device, x, y, n, k, d, epsilon0, partial_d, knn_io, dist_out, not_pruned_out); });
}

skm_status skm_op_update_centroids(int device, const float* x, const uint32_t* assign, const float* dist, uint64_t n, uint64_t k, uint64_t d, float* sums_out, uint32_t* counts_out,
                                   double* wcss_out) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { Engine::op_update(device, x, assign, dist, n, k, d, sums_out, counts_out, wcss_out); });
}

skm_status skm_op_pdxify(int device, const float* in, uint64_t n, uint64_t d, float* out) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { Engine::op_pdxify(device, in, n, d, out); });
}

// ---- allocation-free operator (noalloc.cu) -----------------------------------------------------
skm_status skm_op_find_nearest_noalloc(int device, const float* x_dev, const float* y_dev, uint64_t n, uint64_t k, uint64_t d, uint32_t* out_knn_dev, float* out_dist_dev,
                                       void* cuda_stream) {
    g_create_error.clear();
    return guarded(g_op_error, [&] { skmb::noalloc::find_nearest(device, x_dev, y_dev, n, k, d, out_knn_dev, out_dist_dev, static_cast<cudaStream_t>(cuda_stream)); });
}

// ---- host-side decisions ---------------------------------------------------------------------
void skm_host_dimension_split(uint64_t d, uint64_t* horizontal_d, uint64_t* vertical_d) {
    const skmb::DimensionSplit s = skmb::dimension_split(d);
    *horizontal_d = s.horizontal_d;
    *vertical_d = s.vertical_d;
}

void skm_host_ratios(uint64_t d, float epsilon0, float* out) {
    const std::vector<float> r = skmb::make_ratios(d, epsilon0);
    std::memcpy(out, r.data(), sizeof(float) * r.size());
}

void skm_host_forgy_indices(uint64_t n_points, uint64_t k, uint32_t seed, uint64_t* out) {
    const std::vector<size_t> idx = skmb::forgy_indices(n_points, k, seed);
    for (size_t i = 0; i < idx.size(); ++i) out[i] = idx[i];
}

skm_status skm_host_split_clusters(uint32_t* sizes, uint64_t n_samples, uint64_t n_clusters, uint32_t seed, int hierarchical, uint32_t* ops_out, uint64_t cap, uint64_t* n_ops,
                                   uint64_t* n_split) {
    std::vector<uint32_t> s(sizes, sizes + n_clusters);
    if (!skmb::split_can_terminate(s, n_samples, n_clusters)) return SKM_RUNTIME_ERROR;
    std::vector<skmb::SplitOp> ops;
    const size_t ns = hierarchical ? skmb::split_clusters_hierarchical(s, n_samples, n_clusters, seed, ops) : skmb::split_clusters_flat(s, n_samples, n_clusters, seed, ops);
    std::memcpy(sizes, s.data(), sizeof(uint32_t) * n_clusters);
    for (size_t i = 0; i < ops.size() && i < cap && ops_out; ++i) {
        ops_out[3 * i + 0] = ops[i].dst;
        ops_out[3 * i + 1] = ops[i].src;
        ops_out[3 * i + 2] = ops[i].kind;
    }
    if (n_ops) *n_ops = ops.size();
    if (n_split) *n_split = ns;
    return SKM_OK;
}

uint32_t skm_host_tune_partial_d(double not_pruned_total, uint64_t n_samples, uint64_t n_y, uint32_t partial_d, uint32_t vertical_d, float min_pct, float max_pct, float adjustment,
                                 float* avg_out) {
    const skmb::TuneResult t = skmb::tune_partial_d(not_pruned_total, n_samples, n_y, partial_d, vertical_d, min_pct, max_pct, adjustment);
    if (avg_out) *avg_out = t.avg_not_pruned_pct;
    return t.new_partial_d;
}

void skm_host_arrange_fine_clusters(uint64_t n_clusters, uint64_t n_meso, uint64_t n_samples, const uint32_t* meso_sizes, uint64_t* out) {
    const std::vector<uint32_t> sizes(meso_sizes, meso_sizes + n_meso);
    const std::vector<size_t> r = skmb::arrange_fine_clusters(n_clusters, n_meso, n_samples, sizes);
    for (size_t i = 0; i < r.size(); ++i) out[i] = r[i];
}

uint64_t skm_host_pdx_offset(uint64_t row, uint64_t dim, uint64_t n, uint64_t d) {
    return skmb::pdx_offset(row, dim, n, d, skmb::dimension_split(d).vertical_d);
}

void skm_host_rotation_matrix(uint64_t d, uint32_t seed, float* out) {
    const std::vector<float> m = skmb::make_rotation_matrix(d, seed);
    std::memcpy(out, m.data(), sizeof(float) * m.size());
}

void skm_host_dct_rotation_matrix(uint64_t d, uint32_t seed, float* out) {
    const std::vector<float> m = skmb::make_dct_rotation_matrix(d, seed);
    std::memcpy(out, m.data(), sizeof(float) * m.size());
}

} // extern "C"
