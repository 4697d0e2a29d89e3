// Drop-in for include/superkmeans/superkmeans.h of the SuperKMeans repository, backed by the B200
// engine: same namespace, class template, configuration and statistics structs, method signatures,
// public members and exception classes (reference: superkmeans.h:23-98, :123-149, :162-167, :346-351,
// :397-402, :567-590, :1490-1492).  Every method forwards to the C ABI in skm_b200.h; link with
// libskm_b200.so.  Inputs are row-major float32 host arrays, exactly as in the reference.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <iostream>
#include <memory>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "../skm_b200.h"
#include "common.h"

namespace skmeans {

struct SuperKMeansConfig {
    uint32_t iters = 10;
    float sampling_fraction = 0.3f;
    uint32_t max_points_per_cluster = 256;
    uint32_t n_threads = 0;  // accepted for compatibility; the engine has no CPU worker threads
    uint32_t seed = 42;
    bool use_blas_only = false;

    float tol = 1e-4f;
    float recall_tol = 0.005f;
    bool early_termination = true;
    bool sample_queries = false;
    size_t objective_k = 100;
    float ann_explore_fraction = 0.01f;

    float min_not_pruned_pct = 0.03f;
    float max_not_pruned_pct = 0.05f;
    float adjustment_factor_for_partial_d = 0.20f;

    bool unrotate_centroids = true;
    bool verbose = false;
    bool angular = false;
    bool suppress_warnings = false;

    bool data_already_rotated = false;
};

struct SuperKMeansIterationStats {
    size_t iteration = 0;
    float objective = 0.0f;
    float shift = 0.0f;
    size_t split = 0;
    float recall = 0.0f;
    float not_pruned_pct = -1.0f;
    uint32_t partial_d = 0;
    bool is_gemm_only = false;
};

struct ClusterBalanceStats {
    float mean = 0.0f;
    float geometric_mean = 0.0f;
    float stdev = 0.0f;
    float cv = 0.0f;
    size_t min = 0;
    size_t max = 0;

    std::string to_json() const {
        std::ostringstream oss;
        oss << "{\"mean\":" << mean << ",\"geometric_mean\":" << geometric_mean << ",\"stdev\":" << stdev << ",\"cv\":" << cv << ",\"min\":" << min << ",\"max\":" << max
            << "}";
        return oss.str();
    }
    void print() const {
        std::cout << "Cluster size stats: mean=" << mean << ", gmean=" << geometric_mean << ", std=" << stdev << ", CV=" << cv << ", min=" << min << ", max=" << max
                  << std::endl;
    }
};

namespace detail {

inline void raise(skm_status st, const skm_handle* h) {
    const char* msg = skm_last_error(h);
    const std::string text = (msg && *msg) ? msg : "skm_b200 call failed";
    if (st == SKM_INVALID_ARGUMENT) throw std::invalid_argument(text);
    throw std::runtime_error(text);
}

inline skm_config to_c(const SuperKMeansConfig& c, int hierarchical, uint32_t meso = 3, uint32_t fine = 5, uint32_t refine = 0) {
    skm_config o;
    skm_default_config(&o, hierarchical);
    o.iters = c.iters;
    o.sampling_fraction = c.sampling_fraction;
    o.max_points_per_cluster = c.max_points_per_cluster;
    o.n_threads = c.n_threads;
    o.seed = c.seed;
    o.use_blas_only = c.use_blas_only;
    o.tol = c.tol;
    o.recall_tol = c.recall_tol;
    o.early_termination = c.early_termination;
    o.sample_queries = c.sample_queries;
    o.objective_k = c.objective_k;
    o.ann_explore_fraction = c.ann_explore_fraction;
    o.min_not_pruned_pct = c.min_not_pruned_pct;
    o.max_not_pruned_pct = c.max_not_pruned_pct;
    o.adjustment_factor_for_partial_d = c.adjustment_factor_for_partial_d;
    o.unrotate_centroids = c.unrotate_centroids;
    o.verbose = c.verbose;
    o.angular = c.angular;
    o.suppress_warnings = c.suppress_warnings;
    o.data_already_rotated = c.data_already_rotated;
    o.iters_mesoclustering = meso;
    o.iters_fineclustering = fine;
    o.iters_refinement = refine;
    return o;
}

inline std::vector<SuperKMeansIterationStats> fetch_stats(const skm_handle* h, int phase) {
    uint64_t count = 0;
    skm_get_iteration_stats(h, phase, nullptr, 0, &count);
    std::vector<skm_iter_stats> raw(count);
    if (count) skm_get_iteration_stats(h, phase, raw.data(), count, &count);
    std::vector<SuperKMeansIterationStats> out(count);
    for (uint64_t i = 0; i < count; ++i) {
        out[i].iteration = raw[i].iteration;
        out[i].objective = raw[i].objective;
        out[i].shift = raw[i].shift;
        out[i].split = raw[i].split;
        out[i].recall = raw[i].recall;
        out[i].not_pruned_pct = raw[i].not_pruned_pct;
        out[i].partial_d = raw[i].partial_d;
        out[i].is_gemm_only = raw[i].is_gemm_only != 0;
    }
    return out;
}

struct HandleDeleter {
    void operator()(skm_handle* h) const { skm_destroy(h); }
};

} // namespace detail

template <Quantization q = Quantization::f32, DistanceFunction alpha = DistanceFunction::l2>
class SuperKMeans {
    static_assert(q == Quantization::f32 && alpha == DistanceFunction::l2, "only <f32, l2> is implemented (as in the reference)");

  public:
    using centroid_value_t = float;
    using vector_value_t = float;
    using distance_t = float;

    virtual ~SuperKMeans() = default;

    SuperKMeans(size_t n_clusters, size_t dimensionality, const SuperKMeansConfig& config) : SuperKMeans(n_clusters, dimensionality, config, 0, 3, 5, 0) {}
    SuperKMeans(size_t n_clusters, size_t dimensionality) : SuperKMeans(n_clusters, dimensionality, SuperKMeansConfig{}) {}

    virtual std::vector<centroid_value_t> Train(const vector_value_t* data, const size_t n, const vector_value_t* queries = nullptr, const size_t n_queries = 0) {
        std::vector<centroid_value_t> out(n_clusters * d);
        const skm_status st = skm_train(handle.get(), data, n, 0, queries, n_queries, out.data());
        if (st != SKM_OK) detail::raise(st, handle.get());
        AfterTrain(n);
        return out;
    }

    [[nodiscard]] std::vector<uint32_t> Assign(const vector_value_t* vectors, const vector_value_t* centroids, const size_t n_vectors, const size_t n_centroids) {
        std::vector<uint32_t> out(n_vectors);
        const skm_status st = skm_assign(handle.get(), vectors, centroids, n_vectors, n_centroids, 0, out.data());
        if (st != SKM_OK) detail::raise(st, handle.get());
        return out;
    }

    [[nodiscard]] std::vector<uint32_t> AssignTrainingPoints(const vector_value_t* vectors, const vector_value_t* centroids, const size_t n_vectors, const size_t n_centroids) {
        std::vector<uint32_t> out(n_vectors);
        const skm_status st = skm_assign_training_points(handle.get(), vectors, centroids, n_vectors, n_centroids, 0, out.data());
        if (st != SKM_OK) detail::raise(st, handle.get());
        return out;
    }

    [[nodiscard]] size_t GetNClusters() const noexcept { return n_clusters; }
    [[nodiscard]] bool IsTrained() const noexcept { return skm_is_trained(handle.get()) != 0; }
    [[nodiscard]] float GetSamplingFraction() const noexcept { return config.sampling_fraction; }
    [[nodiscard]] distance_t* GetDistancesPointer() { return distances.get(); }

    // superkmeans.h:586-628
    [[nodiscard]] static ClusterBalanceStats GetClustersBalanceStats(const uint32_t* assignments, size_t n_samples, size_t n_clusters) {
        ClusterBalanceStats stats;
        std::vector<size_t> sizes(n_clusters, 0);
        for (size_t i = 0; i < n_samples; ++i) sizes[assignments[i]]++;
        const size_t sum = std::accumulate(sizes.begin(), sizes.end(), size_t{0});
        stats.mean = static_cast<float>(sum) / static_cast<float>(sizes.size());
        float log_sum = 0.0f;
        size_t non_zero = 0;
        size_t sq_sum = 0;
        stats.min = sizes.empty() ? 0 : sizes[0];
        stats.max = stats.min;
        for (size_t s : sizes) {
            if (s > 0) {
                log_sum += std::log(static_cast<float>(s));
                non_zero++;
            }
            sq_sum += s * s;
            stats.min = s < stats.min ? s : stats.min;
            stats.max = s > stats.max ? s : stats.max;
        }
        stats.geometric_mean = non_zero ? std::exp(log_sum / static_cast<float>(non_zero)) : 0.0f;
        stats.stdev = std::sqrt(static_cast<float>(sq_sum) / static_cast<float>(sizes.size()) - stats.mean * stats.mean);
        stats.cv = stats.stdev / stats.mean;
        return stats;
    }

    // Not in the reference: direct access to the engine handle (e.g. to select a GPU, inject a rotation
    // matrix or read phase timings through skm_b200.h).
    skm_handle* Handle() const { return handle.get(); }

  protected:
    SuperKMeans(size_t n_clusters_, size_t dimensionality, const SuperKMeansConfig& config_, int hierarchical, uint32_t meso, uint32_t fine, uint32_t refine)
        : d(dimensionality), n_clusters(n_clusters_), config(config_) {
        if (config.data_already_rotated) config.unrotate_centroids = false;
        const skm_config c = detail::to_c(config, hierarchical, meso, fine, refine);
        skm_handle* h = nullptr;
        const skm_status st = skm_create(&c, n_clusters, dimensionality, hierarchical, -1, &h);
        if (st != SKM_OK) detail::raise(st, nullptr);
        handle.reset(h);
    }

    void AfterTrain(size_t n) {
        iteration_stats = detail::fetch_stats(handle.get(), SKM_STATS_FLAT);
        assignments.reset(new uint32_t[n]);
        distances.reset(new distance_t[n]);
        // The engine holds one entry per training row: n_samples <= n of them (superkmeans.h:184, :1269-1277).
        // The buffers have n entries and are filled up to n_samples, as in the reference (:202-207).
        const uint64_t held = std::min<uint64_t>(skm_get_n_samples(handle.get()), n);
        if (held) {
            skm_status st = skm_get_assignments(handle.get(), assignments.get(), held);
            if (st == SKM_OK) st = skm_get_distances(handle.get(), distances.get(), held);
            if (st != SKM_OK) detail::raise(st, handle.get());
        }
    }

    const size_t d;
    const size_t n_clusters;
    SuperKMeansConfig config;
    std::unique_ptr<skm_handle, detail::HandleDeleter> handle;
    std::unique_ptr<distance_t[]> distances;

  public:
    std::unique_ptr<uint32_t[]> assignments;
    std::vector<SuperKMeansIterationStats> iteration_stats;
};

} // namespace skmeans
