// Drop-in for include/superkmeans/hierarchical_superkmeans.h of the SuperKMeans repository
// (reference: hierarchical_superkmeans.h:11-26, :43-72, :84-89, :549-551, :817-825).
#pragma once

#include <cmath>

#include "superkmeans.h"

namespace skmeans {

struct HierarchicalSuperKMeansConfig : SuperKMeansConfig {
    uint32_t iters_mesoclustering = 3;
    uint32_t iters_fineclustering = 5;
    uint32_t iters_refinement = 0;

    HierarchicalSuperKMeansConfig() { sampling_fraction = 1.0f; }
};

struct HierarchicalSuperKMeansIterationStats {
    std::vector<SuperKMeansIterationStats> mesoclustering_iteration_stats;
    std::vector<SuperKMeansIterationStats> refinement_iteration_stats;
    std::vector<SuperKMeansIterationStats> fineclustering_iteration_stats;
};

template <Quantization q = Quantization::f32, DistanceFunction alpha = DistanceFunction::l2>
class HierarchicalSuperKMeans : public SuperKMeans<q, alpha> {
    using Base = SuperKMeans<q, alpha>;

  public:
    using typename Base::centroid_value_t;
    using typename Base::vector_value_t;

    HierarchicalSuperKMeans(size_t n_clusters, size_t dimensionality, const HierarchicalSuperKMeansConfig& config)
        : Base(n_clusters, dimensionality, config, 1, config.iters_mesoclustering, config.iters_fineclustering, config.iters_refinement), hierarchical_config(config) {
        static_cast<SuperKMeansConfig&>(hierarchical_config) = this->config;
        hierarchical_config.sampling_fraction = config.sampling_fraction;
    }
    HierarchicalSuperKMeans(size_t n_clusters, size_t dimensionality) : HierarchicalSuperKMeans(n_clusters, dimensionality, HierarchicalSuperKMeansConfig{}) {}

    std::vector<centroid_value_t> Train(const vector_value_t* data, const size_t n, const vector_value_t* queries = nullptr, const size_t n_queries = 0) override {
        std::vector<centroid_value_t> out = Base::Train(data, n, queries, n_queries);
        n_mesoclusters = skm_n_mesoclusters(this->handle.get());
        hierarchical_iteration_stats.mesoclustering_iteration_stats = detail::fetch_stats(this->handle.get(), SKM_STATS_MESO);
        hierarchical_iteration_stats.fineclustering_iteration_stats = detail::fetch_stats(this->handle.get(), SKM_STATS_FINE);
        hierarchical_iteration_stats.refinement_iteration_stats = detail::fetch_stats(this->handle.get(), SKM_STATS_REFINE);
        return out;
    }

    static size_t GetNMesoclusters(const size_t n_clusters) { return static_cast<size_t>(std::round(std::sqrt(n_clusters))); }

    size_t n_mesoclusters = 0;
    HierarchicalSuperKMeansConfig hierarchical_config;
    HierarchicalSuperKMeansIterationStats hierarchical_iteration_stats;
};

} // namespace skmeans
