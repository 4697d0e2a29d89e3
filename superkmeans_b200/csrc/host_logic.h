// Host-side pieces of the k-means hot path that must reproduce the reference bit for bit because
// they consume the random-number stream or take integer decisions: Forgy initialisation, cluster
// splitting, d' tuning, early stopping, dimension split, ADSampling ratios, fine-cluster
// allocation and the random orthogonal matrix.  Pure C++17, no CUDA: the same header is exercised
// by CPU-only tests through the skm_host_* entry points.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <numeric>
#include <random>
#include <vector>

namespace skmb {

// Constants of the reference (include/superkmeans/common.h:89-115).
constexpr float kProportionHorizontalDim = 0.75f;
constexpr size_t kHDimSize = 64;
constexpr uint32_t kMinPartialD = 16;
constexpr size_t kDimensionThresholdForPruning = 128;
constexpr size_t kNClustersThresholdForPruning = 256;
constexpr size_t kXBatchSize = 4096;
constexpr size_t kYBatchSize = 1024;
constexpr size_t kVectorChunkSize = kYBatchSize;
constexpr float kCentroidPerturbationEps = 1.0f / 1024.0f;
constexpr float kPrunerInitialThreshold = 1.5f;
constexpr float kHierarchicalPrunerInitialThreshold = 1.1f;

struct DimensionSplit {
    size_t horizontal_d = 0;
    size_t vertical_d = 0;
};

// PDXLayout::GetDimensionSplit (include/superkmeans/pdx/layout.h:115-140): 75 % of the dimensions
// (25 % when d <= 256) go to the horizontal part, rounded to a multiple of 64; never all of them;
// none when d <= 64.
inline DimensionSplit dimension_split(size_t d) {
    float proportion = kProportionHorizontalDim;
    if (d <= 256) proportion = 0.25f;
    size_t horizontal_d = static_cast<size_t>(static_cast<double>(d) * proportion);
    size_t vertical_d = d - horizontal_d;
    if (horizontal_d % kHDimSize > 0) {
        horizontal_d = static_cast<size_t>(std::lround(
                           static_cast<double>(horizontal_d) / static_cast<double>(kHDimSize))) *
                       kHDimSize;
        vertical_d = d - horizontal_d;
    }
    if (!vertical_d) {
        horizontal_d = kHDimSize;
        vertical_d = d - horizontal_d;
    }
    if (d <= kHDimSize) {
        horizontal_d = 0;
        vertical_d = d;
    }
    return {horizontal_d, vertical_d};
}

// ADSamplingPruner::GetRatio / InitializeRatios (include/superkmeans/pdx/adsampling.h:93-99,
// :315-327): ratio[v] = v/d * (1 + eps0/sqrt(v))^2 in double, rounded to float; ratio[0] =
// ratio[d] = 1.
inline std::vector<float> make_ratios(size_t d, float epsilon0) {
    std::vector<float> r(d + 1);
    for (size_t v = 0; v <= d; ++v) {
        if (v == 0 || v == d) {
            r[v] = 1.0f;
            continue;
        }
        const double dv = static_cast<double>(v);
        const double t = 1.0 + epsilon0 / std::sqrt(dv);
        r[v] = static_cast<float>(dv / static_cast<double>(d) * t * t);
    }
    return r;
}

// Initial d' (include/superkmeans/superkmeans.h:211-215): half of vertical_d, at least 16, at most
// vertical_d.
inline uint32_t initial_partial_d(uint32_t vertical_d, uint32_t divisor = 2) {
    uint32_t p = std::max<uint32_t>(kMinPartialD, vertical_d / divisor);
    if (p > vertical_d) p = vertical_d;
    return p;
}

// SuperKMeans::GetNVectorsToSample (superkmeans.h:1269-1277) and the hierarchical override
// (hierarchical_superkmeans.h:559-567).
inline size_t n_vectors_to_sample(size_t n, size_t k, float sampling_fraction, uint32_t max_points_per_cluster, bool hierarchical) {
    if (hierarchical) {
        if (sampling_fraction == 1.0) return n;
        return static_cast<size_t>(std::floor(static_cast<double>(n) * sampling_fraction));
    }
    if (sampling_fraction == 1.0) return n;
    const size_t by_clusters = k * max_points_per_cluster;
    const size_t by_n = static_cast<size_t>(std::floor(static_cast<float>(n) * sampling_fraction));
    return std::min(by_n, by_clusters);
}

// Forgy initialisation (superkmeans.h:1110-1123): the first k entries of std::shuffle applied to
// [0, n_points) with std::mt19937(seed).  std::shuffle is library-specific; this engine and the
// oracle are both built with libstdc++.
inline std::vector<size_t> forgy_indices(size_t n_points, size_t k, uint32_t seed) {
    std::mt19937 rng(seed);
    std::vector<size_t> indices(n_points);
    std::iota(indices.begin(), indices.end(), size_t{0});
    std::shuffle(indices.begin(), indices.end(), rng);
    indices.resize(std::min(k, n_points));
    return indices;
}

// Sampling permutation (superkmeans.h:1402-1407): a full shuffle of [0, n); the first n_samples
// entries are the sample.
inline std::vector<size_t> sampling_permutation(size_t n, uint32_t seed) {
    std::mt19937 rng(seed);
    std::vector<size_t> idx(n);
    std::iota(idx.begin(), idx.end(), size_t{0});
    std::shuffle(idx.begin(), idx.end(), rng);
    return idx;
}

// One row operation produced by the split logic, applied to the row-major centroid matrix in list
// order by a device kernel (each dimension independently).
//   kind 0: row[dst] = row[src]; then even dims: dst *= 1+eps, src *= 1-eps; odd dims the opposite
//           (superkmeans.h:905-920).
//   kind 1: row[dst] = (wc*row[dst] + 1*row[src]) / (wc + 1)   (hierarchical_superkmeans.h:665-673).
struct SplitOp {
    uint32_t dst;
    uint32_t src;
    uint32_t kind;
    float wc;
};

// SuperKMeans::SplitClusters (superkmeans.h:890-928).  `sizes` is updated in place exactly like
// cluster_sizes.  Returns n_split.
inline size_t split_clusters_flat(std::vector<uint32_t>& sizes, size_t n_samples, size_t n_clusters, uint32_t seed, std::vector<SplitOp>& ops) {
    size_t n_split = 0;
    std::mt19937 rng(seed);
    // The walk below draws ~n_clusters numbers per empty cluster (tens of millions when a thousand clusters are empty), so
    // the acceptance probabilities are tabulated - with the reference's own expression, double division rounded to
    // float - and refreshed for the two clusters a split changes; the draws and comparisons are the reference's.
    const float denom = (float) (n_samples - n_clusters);
    auto prob = [&](size_t c) -> float { return (sizes[c] - 1.0) / denom; };
    std::vector<float> p(n_clusters);
    for (size_t c = 0; c < n_clusters; ++c) p[c] = prob(c);
    std::uniform_real_distribution<float> uniform(0, 1);   // stateless: one object draws what a fresh one per call would
    for (size_t ci = 0; ci < n_clusters; ci++) {
        if (sizes[ci] == 0) {
            size_t cj = 0;
            while (!(uniform(rng) < p[cj])) cj = (cj + 1 == n_clusters) ? 0 : cj + 1;
            ops.push_back({static_cast<uint32_t>(ci), static_cast<uint32_t>(cj), 0u, 0.0f});
            sizes[ci] = sizes[cj] / 2;
            sizes[cj] -= sizes[ci];
            p[ci] = prob(ci);
            p[cj] = prob(cj);
            n_split++;
        }
    }
    return n_split;
}

// HierarchicalSuperKMeans::SplitClusters (hierarchical_superkmeans.h:579-678): the same
// empty-cluster split followed by a pull of every cluster not larger than 25 % of the average
// towards a large cluster picked with probability proportional to its excess size.
inline size_t split_clusters_hierarchical(std::vector<uint32_t>& sizes, size_t n_samples, size_t n_clusters, uint32_t seed, std::vector<SplitOp>& ops) {
    constexpr float kCenterAdjustmentWeight = 7.0f;
    constexpr float kBalancingThreshold = 0.25f;
    size_t n_split = 0;
    std::mt19937 rng(seed);
    const size_t average_size = n_samples / n_clusters;
    const size_t threshold_size = static_cast<size_t>(static_cast<float>(average_size) * kBalancingThreshold);
    {
        // tabulated acceptance probabilities, as in split_clusters_flat (here the reference divides in float)
        const float denom = static_cast<float>(n_samples - n_clusters);
        auto prob = [&](size_t c) -> float { return (sizes[c] - 1.0f) / denom; };
        std::vector<float> p(n_clusters);
        for (size_t c = 0; c < n_clusters; ++c) p[c] = prob(c);
        std::uniform_real_distribution<float> uniform(0, 1);
        for (size_t ci = 0; ci < n_clusters; ci++) {
            if (sizes[ci] == 0) {
                size_t cj = 0;
                while (!(uniform(rng) < p[cj])) cj = (cj + 1 == n_clusters) ? 0 : cj + 1;
                ops.push_back({static_cast<uint32_t>(ci), static_cast<uint32_t>(cj), 0u, 0.0f});
                sizes[ci] = sizes[cj] / 2;
                sizes[cj] -= sizes[ci];
                p[ci] = prob(ci);
                p[cj] = prob(cj);
                n_split++;
            }
        }
    }
    for (size_t ci = 0; ci < n_clusters; ci++) {
        const size_t csize = sizes[ci];
        if (csize == 0 || csize > threshold_size) continue;
        size_t large;
        for (large = 0; true; large = (large + 1) % n_clusters) {
            const size_t large_size = sizes[large];
            if (large_size < average_size) continue;
            float p = static_cast<float>(large_size - average_size + 1) /
                      static_cast<float>(n_samples - average_size * n_clusters + n_clusters);
            float r = std::uniform_real_distribution<float>(0, 1)(rng);
            if (r < p) break;
        }
        const float wc = std::min(static_cast<float>(csize), kCenterAdjustmentWeight);
        ops.push_back({static_cast<uint32_t>(ci), static_cast<uint32_t>(large), 1u, wc});
        n_split++;
    }
    return n_split;
}

// The empty-cluster loop above never ends when no cluster has more than one point (every p <= 0).
// The reference has the same property; the engine reports it instead of spinning.
inline bool split_can_terminate(const std::vector<uint32_t>& sizes, size_t n_samples, size_t n_clusters) {
    bool any_empty = false;
    uint32_t max_size = 0;
    for (size_t c = 0; c < n_clusters; ++c) {
        any_empty |= sizes[c] == 0;
        max_size = std::max(max_size, sizes[c]);
    }
    if (!any_empty) return true;
    return max_size > 1 && n_samples > n_clusters;
}

struct TuneResult {
    float avg_not_pruned_pct;
    uint32_t new_partial_d;
    bool changed;
};

// SuperKMeans::TunePartialD (superkmeans.h:1230-1258).  The reference accumulates the per-point
// counts in a float; the engine passes the exact integer total.
inline TuneResult tune_partial_d(double not_pruned_total, size_t n_samples, size_t n_y, uint32_t partial_d, uint32_t vertical_d, float min_pct, float max_pct, float adjustment) {
    float avg = static_cast<float>(not_pruned_total);
    avg /= static_cast<float>(n_samples * n_y);
    uint32_t nd = partial_d;
    if (avg > max_pct) {
        auto increase = static_cast<uint32_t>(partial_d * adjustment * 2);
        nd = std::min(partial_d + std::max(increase, 1u), vertical_d);
    } else if (avg < min_pct) {
        auto decrease = static_cast<uint32_t>(partial_d * adjustment);
        nd = std::max(partial_d - std::max(decrease, 1u), kMinPartialD);
    }
    return {avg, nd, nd != partial_d};
}

// SuperKMeans::ShouldStopEarly (superkmeans.h:1294-1333).  With tracking_recall, best_recall and
// iters_without_improvement carry the recall history from call to call.
constexpr size_t kRecallConvergencePatience = 2;   // RECALL_CONVERGENCE_PATIENCE (common.h:111)
inline bool should_stop_early(float shift, float cost, float prev_cost, float tol, size_t iter_idx, bool tracking_recall = false, float recall = 0.0f,
                              float recall_tol = 0.0f, float* best_recall = nullptr, size_t* iters_without_improvement = nullptr) {
    if (shift < tol) return true;
    if (iter_idx > 0) {
        const float cost_delta = cost / prev_cost;
        if (cost_delta > 1 - tol) return true;
    }
    if (tracking_recall) {
        const float improvement = recall - *best_recall;
        if (improvement > recall_tol) {
            *best_recall = recall;
            *iters_without_improvement = 0;
        } else {
            ++*iters_without_improvement;
            if (*iters_without_improvement >= kRecallConvergencePatience) return true;
        }
    }
    return false;
}

// HierarchicalSuperKMeans::GetNMesoclusters (hierarchical_superkmeans.h:549-551).
inline size_t n_mesoclusters(size_t n_clusters) {
    return static_cast<size_t>(std::round(std::sqrt(n_clusters)));
}

// HierarchicalSuperKMeans::ArrangeFineClusters (hierarchical_superkmeans.h:718-761).
inline std::vector<size_t> arrange_fine_clusters(size_t n_clusters, size_t n_meso, size_t n_samples, const std::vector<uint32_t>& meso_sizes) {
    std::vector<size_t> out(n_meso);
    size_t clusters_remaining = n_clusters;
    size_t nonempty_remaining = 0;
    for (size_t i = 0; i < n_meso; ++i)
        if (meso_sizes[i] > 0) nonempty_remaining++;
    size_t samples_remaining = n_samples;
    for (size_t i = 0; i < n_meso; ++i) {
        if (i < n_meso - 1) {
            if (meso_sizes[i] == 0) {
                out[i] = 0;
            } else {
                nonempty_remaining--;
                const double proportion = static_cast<double>(clusters_remaining * meso_sizes[i]) /
                                          static_cast<double>(samples_remaining);
                size_t allocated = static_cast<size_t>(std::lround(proportion));
                allocated = std::min(allocated, clusters_remaining - nonempty_remaining);
                out[i] = std::max(allocated, size_t{1});
            }
        } else {
            out[i] = clusters_remaining;
        }
        clusters_remaining -= out[i];
        samples_remaining -= meso_sizes[i];
    }
    return out;
}

// Random orthogonal matrix of the ADSampling rotation (adsampling.h:76-85): a d x d matrix of
// N(0,1) draws from std::mt19937(seed), filled row by row, whose Householder-QR factor Q is the
// rotation.  Sign convention: each reflector maps its column to -sign(x0)*||x|| e1, as in the usual
// LAPACK/Eigen formulation, so Q agrees with the reference's up to floating-point rounding.
// Computed in double, rounded once to float.  Output row-major d x d.
// The rotation of ADSamplingPruner's DCT branch (adsampling.h:53-73, :169-188) as an explicit matrix: a random sign
// per input dimension, then the orthonormal DCT-II (FFTW's REDFT10, 2 * sum_j x_j cos(pi (j + 1/2) k / d), scaled by
// sqrt(1 / 4d) for k = 0 and sqrt(1 / 2d) otherwise).  M[k][j] = scale_k * 2 cos(pi (j + 1/2) k / d) * sign_j, so that
// X * M^T is what a reference built with FFTW computes for power-of-two d >= 512.
inline std::vector<float> make_dct_rotation_matrix(size_t d, uint32_t seed) {
    std::mt19937 gen(seed);
    std::uniform_int_distribution<int> dist(0, 1);
    std::vector<double> sign(d);
    for (size_t j = 0; j < d; ++j) sign[j] = dist(gen) ? 1.0 : -1.0;
    std::vector<float> m(d * d);
    const double pi = 3.14159265358979323846;
    const double s0 = std::sqrt(1.0 / (4.0 * static_cast<double>(d))), s = std::sqrt(1.0 / (2.0 * static_cast<double>(d)));
    for (size_t k = 0; k < d; ++k) {
        const double scale = (k == 0 ? s0 : s) * 2.0;
        for (size_t j = 0; j < d; ++j) {
            m[k * d + j] = static_cast<float>(scale * std::cos(pi * (static_cast<double>(j) + 0.5) * static_cast<double>(k) / static_cast<double>(d)) * sign[j]);
        }
    }
    return m;
}

inline std::vector<float> make_rotation_matrix(size_t d, uint32_t seed) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    std::vector<double> a(d * d);
    for (size_t i = 0; i < d; ++i)
        for (size_t j = 0; j < d; ++j) a[i * d + j] = static_cast<double>(dist(gen));
    std::vector<double> beta(d, 0.0), w(d);
    for (size_t k = 0; k < d; ++k) {
        double norm2 = 0.0;
        for (size_t i = k; i < d; ++i) norm2 += a[i * d + k] * a[i * d + k];
        const double x0 = a[k * d + k];
        const double tail2 = norm2 - x0 * x0;
        if (tail2 <= 0.0 || k == d - 1) continue;
        const double alpha = (x0 >= 0.0) ? -std::sqrt(norm2) : std::sqrt(norm2);
        const double v0 = x0 - alpha;
        for (size_t i = k + 1; i < d; ++i) a[i * d + k] /= v0;
        beta[k] = -v0 / alpha;
        a[k * d + k] = alpha;
        const size_t m = d - k - 1;
        for (size_t j = 0; j < m; ++j) w[j] = a[k * d + k + 1 + j];
        for (size_t i = k + 1; i < d; ++i) {
            const double vi = a[i * d + k];
            const double* row = &a[i * d + k + 1];
            for (size_t j = 0; j < m; ++j) w[j] += vi * row[j];
        }
        const double b = beta[k];
        for (size_t j = 0; j < m; ++j) a[k * d + k + 1 + j] -= b * w[j];
#pragma omp parallel for if (m > 256)
        for (size_t i = k + 1; i < d; ++i) {
            const double vi = b * a[i * d + k];
            double* row = &a[i * d + k + 1];
            for (size_t j = 0; j < m; ++j) row[j] -= vi * w[j];
        }
    }
    std::vector<double> q(d * d, 0.0);
    for (size_t i = 0; i < d; ++i) q[i * d + i] = 1.0;
    for (size_t kk = d; kk-- > 0;) {
        const double b = beta[kk];
        if (b == 0.0) continue;
        const size_t m = d - kk;
        for (size_t j = 0; j < m; ++j) w[j] = q[kk * d + kk + j];
        for (size_t i = kk + 1; i < d; ++i) {
            const double vi = a[i * d + kk];
            const double* row = &q[i * d + kk];
            for (size_t j = 0; j < m; ++j) w[j] += vi * row[j];
        }
        for (size_t j = 0; j < m; ++j) q[kk * d + kk + j] -= b * w[j];
#pragma omp parallel for if (m > 256)
        for (size_t i = kk + 1; i < d; ++i) {
            const double vi = b * a[i * d + kk];
            double* row = &q[i * d + kk];
            for (size_t j = 0; j < m; ++j) row[j] -= vi * w[j];
        }
    }
    std::vector<float> out(d * d);
    for (size_t i = 0; i < d * d; ++i) out[i] = static_cast<float>(q[i]);
    return out;
}

// Offset of element (row, dim) inside the PDX-blocked copy of a row-major n x d matrix
// (layout.h:155-232): rows are grouped in chunks of 1024; inside a chunk of `cs` rows the first
// vertical_d dimensions are stored dimension-major ([vertical_d][cs]) and the remaining ones as
// consecutive blocks of 64 dimensions, each block row-major ([cs][64]).  The last chunk uses its
// own, smaller cs.
inline size_t pdx_offset(size_t row, size_t dim, size_t n, size_t d, size_t vertical_d) {
    const size_t chunk = row / kVectorChunkSize;
    const size_t v = row % kVectorChunkSize;
    const size_t cs = std::min(kVectorChunkSize, n - chunk * kVectorChunkSize);
    const size_t base = chunk * kVectorChunkSize * d;
    if (dim < vertical_d) return base + dim * cs + v;
    const size_t h = dim - vertical_d;
    return base + vertical_d * cs + (h / kHDimSize) * cs * kHDimSize + v * kHDimSize + (h % kHDimSize);
}

} // namespace skmb
