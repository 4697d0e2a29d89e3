// TEST INFRASTRUCTURE ONLY (never part of the shipped engine).
//
// C-ABI harness around the UNMODIFIED SuperKMeans reference headers.  It is compiled by
// oracle/Makefile from the reference sources where they lie (include path given on the command
// line) together with oracle/eigen_shim, and linked against the OpenBLAS that ships inside SciPy.
// The result (oracle/_ref/libskm_ref*.so) is the real reference algorithm, used
//   * to pin the independent restatement in oracle/skm_oracle.cpp,
//   * as the parity checker of the CUDA engine in tests/,
//   * as the timed CPU baseline of bench.py.
//
// Per-iteration state is captured without touching the reference: SplitClusters() is virtual and is
// called exactly once per RunIteration (superkmeans.h:952), after assignment, update and d' tuning,
// so an override can snapshot everything an iteration produced.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "superkmeans/hierarchical_superkmeans.h"
#include "superkmeans/superkmeans.h"

// The reference declares Fortran sgemm_ (common.h:7-23); SciPy's OpenBLAS exports it with a prefix.
extern "C" int scipy_sgemm_(
    const char*, const char*, int*, int*, int*, const float*, const float*, int*, const float*,
    int*, float*, float*, int*
);
extern "C" void scipy_openblas_set_num_threads(int);
extern "C" int scipy_openblas_get_num_threads(void);

extern "C" int sgemm_(
    const char* ta, const char* tb, int* m, int* n, int* k, const float* alpha, const float* a,
    int* lda, const float* b, int* ldb, float* beta, float* c, int* ldc
) {
    return scipy_sgemm_(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

namespace {

using Flat = skmeans::SuperKMeans<skmeans::Quantization::f32, skmeans::DistanceFunction::l2>;
using Hier =
    skmeans::HierarchicalSuperKMeans<skmeans::Quantization::f32, skmeans::DistanceFunction::l2>;
using Batch = skmeans::BatchComputer<skmeans::DistanceFunction::l2, skmeans::Quantization::f32>;
using Layout = skmeans::PDXLayout<skmeans::Quantization::f32, skmeans::DistanceFunction::l2>;
using Pruner = skmeans::ADSamplingPruner<skmeans::Quantization::f32>;

struct Snapshot {
    uint64_t n_samples = 0;
    uint64_t n_clusters = 0;
    uint32_t partial_d_next = 0;
    std::vector<float> centroids;    // rotated, row-major, after split (what the next iteration reads)
    std::vector<uint32_t> assign;    // this iteration's assignments
    std::vector<float> dist;         // this iteration's distances
    std::vector<uint32_t> sizes_pre; // before SplitClusters
    std::vector<uint32_t> sizes_post;
};

struct Trace {
    bool enabled = false;
    std::vector<Snapshot> snaps;
};

template <class Base>
class Probe : public Base {
  public:
    using Base::Base;
    Trace trace;

    void SplitClusters(const size_t n_samples, const size_t n_clusters) override {
        Snapshot s;
        if (trace.enabled) {
            s.n_samples = n_samples;
            s.n_clusters = n_clusters;
            s.partial_d_next = this->partial_d;
            s.sizes_pre.assign(this->cluster_sizes.get(), this->cluster_sizes.get() + n_clusters);
            s.assign.assign(this->assignments.get(), this->assignments.get() + n_samples);
            s.dist.assign(this->distances.get(), this->distances.get() + n_samples);
        }
        Base::SplitClusters(n_samples, n_clusters);
        if (trace.enabled) {
            s.sizes_post.assign(this->cluster_sizes.get(), this->cluster_sizes.get() + n_clusters);
            s.centroids.assign(
                this->horizontal_centroids.get(),
                this->horizontal_centroids.get() + n_clusters * this->d
            );
            trace.snaps.push_back(std::move(s));
        }
    }

    void RotationMatrix(float* out_m) {
        // Rotate(I) = I * M^T, so transposing gives M (adsampling.h:191-215).
        const size_t dd = this->d;
        std::vector<float> eye(dd * dd, 0.0f), rt(dd * dd);
        for (size_t i = 0; i < dd; ++i) eye[i * dd + i] = 1.0f;
        this->pruner->Rotate(eye.data(), rt.data(), static_cast<uint32_t>(dd));
        for (size_t i = 0; i < dd; ++i)
            for (size_t j = 0; j < dd; ++j) out_m[i * dd + j] = rt[j * dd + i];
    }
    void Ratios(float* out) {
        std::memcpy(out, this->pruner->ratios.data(), sizeof(float) * (this->d + 1));
    }
    const float* RotatedCentroids() { return this->horizontal_centroids.get(); }
    const uint32_t* Sizes() { return this->cluster_sizes.get(); }
    uint32_t PartialD() { return this->partial_d; }
    uint32_t VerticalD() { return this->vertical_d; }
};

class HierProbe : public Probe<Hier> {
  public:
    using Probe<Hier>::Probe;
    const uint32_t* FinalAssignments() { return this->final_assignments.get(); }
    const std::vector<uint32_t>& MesoSizes() { return this->mesoclusters_sizes; }
    const std::vector<uint32_t>& MesoAssignments() { return this->mesoclusters_assignments; }
};

struct Handle {
    bool hierarchical = false;
    uint64_t k = 0, d = 0, n_trained = 0;
    std::unique_ptr<Probe<Flat>> flat;
    std::unique_ptr<HierProbe> hier;
    std::string err;
    Trace& trace() { return hierarchical ? hier->trace : flat->trace; }
};

} // namespace

extern "C" {

struct ref_config {
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
};

struct ref_iter_stats {
    uint64_t iteration;
    float objective;
    float shift;
    uint64_t split;
    float recall;
    float not_pruned_pct;
    uint32_t partial_d;
    int32_t is_gemm_only;
};

static void fill_base(skmeans::SuperKMeansConfig& c, const ref_config* in) {
    c.iters = in->iters;
    c.sampling_fraction = in->sampling_fraction;
    c.max_points_per_cluster = in->max_points_per_cluster;
    c.n_threads = in->n_threads;
    c.seed = in->seed;
    c.use_blas_only = in->use_blas_only != 0;
    c.tol = in->tol;
    c.recall_tol = in->recall_tol;
    c.early_termination = in->early_termination != 0;
    c.sample_queries = in->sample_queries != 0;
    c.objective_k = in->objective_k;
    c.ann_explore_fraction = in->ann_explore_fraction;
    c.min_not_pruned_pct = in->min_not_pruned_pct;
    c.max_not_pruned_pct = in->max_not_pruned_pct;
    c.adjustment_factor_for_partial_d = in->adjustment_factor_for_partial_d;
    c.unrotate_centroids = in->unrotate_centroids != 0;
    c.verbose = in->verbose != 0;
    c.angular = in->angular != 0;
    c.suppress_warnings = in->suppress_warnings != 0;
    c.data_already_rotated = in->data_already_rotated != 0;
}

// Fills *cfg with the reference's own defaults (superkmeans.h:23-55,
// hierarchical_superkmeans.h:11-17).
void ref_default_config(ref_config* cfg, int hierarchical) {
    skmeans::HierarchicalSuperKMeansConfig h;
    skmeans::SuperKMeansConfig f;
    const skmeans::SuperKMeansConfig& c = hierarchical ? static_cast<skmeans::SuperKMeansConfig&>(h) : f;
    cfg->iters = c.iters;
    cfg->sampling_fraction = c.sampling_fraction;
    cfg->max_points_per_cluster = c.max_points_per_cluster;
    cfg->n_threads = c.n_threads;
    cfg->seed = c.seed;
    cfg->use_blas_only = c.use_blas_only;
    cfg->tol = c.tol;
    cfg->recall_tol = c.recall_tol;
    cfg->early_termination = c.early_termination;
    cfg->sample_queries = c.sample_queries;
    cfg->objective_k = c.objective_k;
    cfg->ann_explore_fraction = c.ann_explore_fraction;
    cfg->min_not_pruned_pct = c.min_not_pruned_pct;
    cfg->max_not_pruned_pct = c.max_not_pruned_pct;
    cfg->adjustment_factor_for_partial_d = c.adjustment_factor_for_partial_d;
    cfg->unrotate_centroids = c.unrotate_centroids;
    cfg->verbose = c.verbose;
    cfg->angular = c.angular;
    cfg->suppress_warnings = c.suppress_warnings;
    cfg->data_already_rotated = c.data_already_rotated;
    cfg->iters_mesoclustering = h.iters_mesoclustering;
    cfg->iters_fineclustering = h.iters_fineclustering;
    cfg->iters_refinement = h.iters_refinement;
}

void ref_set_blas_threads(int n) { scipy_openblas_set_num_threads(n); }
int ref_get_blas_threads(void) { return scipy_openblas_get_num_threads(); }
int ref_get_omp_threads(void) { return omp_get_max_threads(); }

static thread_local std::string g_err;
const char* ref_last_error(void) { return g_err.c_str(); }

// Status: 0 ok, 1 std::invalid_argument, 2 std::runtime_error, 3 other.
#define REF_GUARD(...)                                                                             \
    try {                                                                                          \
        __VA_ARGS__;                                                                               \
        return 0;                                                                                  \
    } catch (const std::invalid_argument& e) {                                                     \
        g_err = e.what();                                                                          \
        return 1;                                                                                  \
    } catch (const std::runtime_error& e) {                                                        \
        g_err = e.what();                                                                          \
        return 2;                                                                                  \
    } catch (const std::exception& e) {                                                            \
        g_err = e.what();                                                                          \
        return 3;                                                                                  \
    }

int ref_create(uint64_t k, uint64_t d, const ref_config* cfg, int hierarchical, int trace, void** out) {
    REF_GUARD({
        auto h = std::make_unique<Handle>();
        h->hierarchical = hierarchical != 0;
        h->k = k;
        h->d = d;
        if (hierarchical) {
            skmeans::HierarchicalSuperKMeansConfig c;
            fill_base(c, cfg);
            c.iters_mesoclustering = cfg->iters_mesoclustering;
            c.iters_fineclustering = cfg->iters_fineclustering;
            c.iters_refinement = cfg->iters_refinement;
            h->hier = std::make_unique<HierProbe>(k, d, c);
        } else {
            skmeans::SuperKMeansConfig c;
            fill_base(c, cfg);
            h->flat = std::make_unique<Probe<Flat>>(k, d, c);
        }
        h->trace().enabled = trace != 0;
        *out = h.release();
    })
}

void ref_destroy(void* hv) { delete static_cast<Handle*>(hv); }

int ref_train(void* hv, const float* data, uint64_t n, const float* queries, uint64_t nq, float* out_centroids) {
    auto* h = static_cast<Handle*>(hv);
    REF_GUARD({
        std::vector<float> c = h->hierarchical ? h->hier->Train(data, n, queries, nq)
                                               : h->flat->Train(data, n, queries, nq);
        h->n_trained = n;
        std::memcpy(out_centroids, c.data(), sizeof(float) * c.size());
    })
}

int ref_assign(void* hv, const float* vectors, const float* centroids, uint64_t n, uint64_t k, uint32_t* out) {
    auto* h = static_cast<Handle*>(hv);
    REF_GUARD({
        std::vector<uint32_t> a = h->hierarchical ? h->hier->Assign(vectors, centroids, n, k)
                                                  : h->flat->Assign(vectors, centroids, n, k);
        std::memcpy(out, a.data(), sizeof(uint32_t) * a.size());
    })
}

int ref_assign_training_points(void* hv, const float* vectors, const float* centroids, uint64_t n, uint64_t k, uint32_t* out) {
    auto* h = static_cast<Handle*>(hv);
    REF_GUARD({
        std::vector<uint32_t> a = h->hierarchical
                                      ? h->hier->AssignTrainingPoints(vectors, centroids, n, k)
                                      : h->flat->AssignTrainingPoints(vectors, centroids, n, k);
        std::memcpy(out, a.data(), sizeof(uint32_t) * a.size());
    })
}

int ref_is_trained(void* hv) {
    auto* h = static_cast<Handle*>(hv);
    return h->hierarchical ? h->hier->IsTrained() : h->flat->IsTrained();
}

void ref_rotation_matrix(void* hv, float* out_m) {
    auto* h = static_cast<Handle*>(hv);
    if (h->hierarchical) h->hier->RotationMatrix(out_m); else h->flat->RotationMatrix(out_m);
}

void ref_ratios(void* hv, float* out) {
    auto* h = static_cast<Handle*>(hv);
    if (h->hierarchical) h->hier->Ratios(out); else h->flat->Ratios(out);
}

// Public `assignments` member (superkmeans.h:1491) and GetDistancesPointer (:576).
void ref_get_assignments(void* hv, uint32_t* out, uint64_t n) {
    auto* h = static_cast<Handle*>(hv);
    const uint32_t* p = h->hierarchical ? h->hier->assignments.get() : h->flat->assignments.get();
    std::memcpy(out, p, sizeof(uint32_t) * n);
}
void ref_get_distances(void* hv, float* out, uint64_t n) {
    auto* h = static_cast<Handle*>(hv);
    const float* p = h->hierarchical ? h->hier->GetDistancesPointer() : h->flat->GetDistancesPointer();
    std::memcpy(out, p, sizeof(float) * n);
}
void ref_get_rotated_centroids(void* hv, float* out) {
    auto* h = static_cast<Handle*>(hv);
    const float* p = h->hierarchical ? h->hier->RotatedCentroids() : h->flat->RotatedCentroids();
    std::memcpy(out, p, sizeof(float) * h->k * h->d);
}
void ref_get_final_assignments(void* hv, uint32_t* out, uint64_t n) { // hierarchical only
    auto* h = static_cast<Handle*>(hv);
    std::memcpy(out, h->hier->FinalAssignments(), sizeof(uint32_t) * n);
}
uint64_t ref_n_mesoclusters(void* hv) { return static_cast<Handle*>(hv)->hier->n_mesoclusters; }

// phase: 0 flat `iteration_stats`, 1 meso, 2 fine, 3 refinement.
uint64_t ref_get_stats(void* hv, int phase, ref_iter_stats* out, uint64_t cap) {
    auto* h = static_cast<Handle*>(hv);
    const std::vector<skmeans::SuperKMeansIterationStats>* v = nullptr;
    if (phase == 0) {
        v = h->hierarchical ? &h->hier->iteration_stats : &h->flat->iteration_stats;
    } else {
        auto& hs = h->hier->hierarchical_iteration_stats;
        v = phase == 1 ? &hs.mesoclustering_iteration_stats
                       : (phase == 2 ? &hs.fineclustering_iteration_stats : &hs.refinement_iteration_stats);
    }
    for (uint64_t i = 0; i < v->size() && i < cap; ++i) {
        const auto& s = (*v)[i];
        out[i].iteration = s.iteration;
        out[i].objective = s.objective;
        out[i].shift = s.shift;
        out[i].split = s.split;
        out[i].recall = s.recall;
        out[i].not_pruned_pct = s.not_pruned_pct;
        out[i].partial_d = s.partial_d;
        out[i].is_gemm_only = s.is_gemm_only;
    }
    return v->size();
}

uint64_t ref_trace_count(void* hv) { return static_cast<Handle*>(hv)->trace().snaps.size(); }

// Any output pointer may be null.  Sizes: centroids n_clusters*d, assign/dist n_samples,
// sizes_* n_clusters.
void ref_trace_get(
    void* hv, uint64_t idx, uint64_t* n_samples, uint64_t* n_clusters, uint32_t* partial_d_next,
    float* centroids, uint32_t* assign, float* dist, uint32_t* sizes_pre, uint32_t* sizes_post
) {
    const Snapshot& s = static_cast<Handle*>(hv)->trace().snaps[idx];
    if (n_samples) *n_samples = s.n_samples;
    if (n_clusters) *n_clusters = s.n_clusters;
    if (partial_d_next) *partial_d_next = s.partial_d_next;
    if (centroids) std::memcpy(centroids, s.centroids.data(), sizeof(float) * s.centroids.size());
    if (assign) std::memcpy(assign, s.assign.data(), sizeof(uint32_t) * s.assign.size());
    if (dist) std::memcpy(dist, s.dist.data(), sizeof(float) * s.dist.size());
    if (sizes_pre) std::memcpy(sizes_pre, s.sizes_pre.data(), sizeof(uint32_t) * s.sizes_pre.size());
    if (sizes_post) std::memcpy(sizes_post, s.sizes_post.data(), sizeof(uint32_t) * s.sizes_post.size());
}

// ---- free-standing pieces of the path (micro known-answers) ---------------------------------

void ref_dimension_split(uint64_t d, uint64_t* horizontal_d, uint64_t* vertical_d) {
    auto s = Layout::GetDimensionSplit(d);
    *horizontal_d = s.horizontal_d;
    *vertical_d = s.vertical_d;
}

void ref_pdxify(const float* in, float* out, uint64_t n, uint64_t d) {
    Layout::PDXify<false>(in, out, n, d);
}

float ref_horizontal(const float* a, const float* b, uint64_t n) {
    return skmeans::DistanceComputer<skmeans::DistanceFunction::l2, skmeans::Quantization::f32>::
        Horizontal(a, b, n);
}

static void row_norms(const float* x, uint64_t n, uint64_t d, uint64_t upto, float* out) {
    using MatrixR = Eigen::Matrix<float, Eigen::Dynamic, Eigen::Dynamic, Eigen::RowMajor>;
    Eigen::Map<const MatrixR> m(x, n, d);
    Eigen::Map<Eigen::VectorXf> o(out, n);
    o.noalias() = m.leftCols(upto).rowwise().squaredNorm();
}

// BatchComputer::FindNearestNeighbor (batch_computers.h:104-171) with norms computed the way
// SuperKMeans::Assign does (superkmeans.h:360-366).
void ref_find_nearest(const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, int n_threads, uint32_t* out_knn, float* out_dist) {
    skmeans::g_n_threads = n_threads > 0 ? n_threads : omp_get_max_threads();
    std::vector<float> nx(n), ny(k), tmp(skmeans::X_BATCH_SIZE * skmeans::Y_BATCH_SIZE);
    row_norms(x, n, d, d, nx.data());
    row_norms(y, k, d, d, ny.data());
    Batch::FindNearestNeighbor(x, y, n, k, d, nx.data(), ny.data(), out_knn, out_dist, tmp.data());
}

// One pruned assignment pass (batch_computers.h:297-409) from explicit inputs: rotated points x,
// rotated row-major centroids y, previous assignments in knn_io.  Builds the PDX copy and the
// auxiliary first-vertical_d copy exactly like ConsolidateCentroids (superkmeans.h:961-967).
void ref_find_nearest_pruned(
    const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, float epsilon0,
    uint32_t partial_d, int n_threads, uint32_t* knn_io, float* dist_out, uint64_t* not_pruned_out
) {
    skmeans::g_n_threads = n_threads > 0 ? n_threads : omp_get_max_threads();
    static std::unique_ptr<Pruner> pruner;
    static uint64_t pruner_d = 0;
    static float pruner_eps = 0;
    if (!pruner || pruner_d != d || pruner_eps != epsilon0) {
        pruner = std::make_unique<Pruner>(static_cast<uint32_t>(d), epsilon0, 42);
        pruner_d = d;
        pruner_eps = epsilon0;
    }
    const uint64_t vertical_d = Layout::GetDimensionSplit(d).vertical_d;
    std::vector<float> nx(n), ny(k), tmp(skmeans::X_BATCH_SIZE * skmeans::Y_BATCH_SIZE);
    std::vector<float> pdx(k * d), aux(k * vertical_d);
    row_norms(x, n, d, partial_d, nx.data());
    row_norms(y, k, d, partial_d, ny.data());
    Layout::PDXify<false>(y, pdx.data(), k, d);
    for (uint64_t c = 0; c < k; ++c)
        std::memcpy(&aux[c * vertical_d], &y[c * d], sizeof(float) * vertical_d);
    Layout layout(pdx.data(), *pruner, k, d, aux.data());
    std::vector<size_t> np(n, 0);
    Batch::FindNearestNeighborWithPruning(
        x, y, n, k, d, nx.data(), ny.data(), knn_io, dist_out, tmp.data(), layout, partial_d, np.data()
    );
    for (uint64_t i = 0; i < n; ++i) not_pruned_out[i] = np[i];
}

// Test-data helper of the reference (pdx/utils.h:74-123); note it seeds one RNG per OpenMP thread.
void ref_make_blobs(uint64_t n, uint64_t d, uint64_t centers, int normalize, float std_, float spread, uint32_t seed, float* out) {
    auto v = skmeans::MakeBlobs(n, d, centers, normalize != 0, std_, spread, seed);
    std::memcpy(out, v.data(), sizeof(float) * v.size());
}

} // extern "C"
