// TEST INFRASTRUCTURE ONLY (never part of the shipped engine; only tests/, the smoke check and
// bench.py's CPU-baseline leg may load it).
//
// Independent CPU restatement of the SuperKMeans flat k-means hot path, one plain function per step,
// each citing the reference code it follows (paths inside the SuperKMeans repository).  It needs no
// reference sources to build.  The only borrowed arithmetic is SGEMM, which the reference itself
// delegates to an external BLAS (include/superkmeans/common.h:7-23): this file calls the same
// OpenBLAS build that ships inside SciPy, with the same argument shapes, so dot products agree bit
// for bit with the compiled reference on the same host.
//
// Parity status: PINNED.  tests/test_oracle_pins.py checks every function here against the compiled
// reference (oracle/_ref, built from the unmodified headers) when it is present, and against golden
// vectors generated from it (tests/golden/) otherwise.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <random>
#include <vector>

extern "C" int scipy_sgemm_(const char*, const char*, int*, int*, int*, const float*, const float*, int*, const float*, int*, float*, float*, int*);

namespace {

constexpr size_t X_BATCH = 4096;   // common.h:105
constexpr size_t Y_BATCH = 1024;   // common.h:106 (= VECTOR_CHUNK_SIZE, :109)
constexpr size_t H_DIM = 64;       // common.h:91
constexpr uint32_t MIN_PARTIAL_D = 16;  // common.h:93

// distances[r * by + c] = x_r . y_c over the first kdim dimensions
// (BatchComputer::BlasMatrixMultiplication, distance_computers/batch_computers.h:47-83).
void dot_tile(const float* x, const float* y, size_t bx, size_t by, size_t d, size_t kdim, float* out) {
    const char ta = 'T', tb = 'N';
    int m = static_cast<int>(by), n = static_cast<int>(bx), k = static_cast<int>(kdim);
    int lda = static_cast<int>(d), ldb = static_cast<int>(d), ldc = static_cast<int>(by);
    float alpha = 1.0f, beta = 0.0f;
    scipy_sgemm_(&ta, &tb, &m, &n, &k, &alpha, y, &lda, x, &ldb, &beta, out, &ldc);
}

// Sum of squared differences with the summation order of the AVX-512 kernel
// (distance_computers/avx512_computers.h:80-111): sixteen interleaved fused accumulators, then the
// fold 16 -> 8 -> 4 -> pairwise.
float horizontal(const float* a, const float* b, size_t len) {
    float lane[16] = {0};
    size_t i = 0;
    for (; i + 16 <= len; i += 16)
        for (int l = 0; l < 16; ++l) {
            const float t = a[i + l] - b[i + l];
            lane[l] = std::fmaf(t, t, lane[l]);
        }
    for (int l = 0; i + l < len; ++l) {
        const float t = a[i + l] - b[i + l];
        lane[l] = std::fmaf(t, t, lane[l]);
    }
    float y[8], z[4];
    for (int l = 0; l < 8; ++l) y[l] = lane[l] + lane[l + 8];
    for (int l = 0; l < 4; ++l) z[l] = y[l] + y[l + 4];
    return (z[0] + z[1]) + (z[2] + z[3]);
}

} // namespace

extern "C" {

// PDXLayout::GetDimensionSplit (pdx/layout.h:115-140).
void orc_dimension_split(uint64_t d, uint64_t* horizontal_d, uint64_t* vertical_d) {
    double share = (d <= 256) ? 0.25 : 0.75;
    uint64_t h = static_cast<uint64_t>(static_cast<double>(d) * share);
    if (h % H_DIM) h = static_cast<uint64_t>(std::lround(static_cast<double>(h) / H_DIM)) * H_DIM;
    if (h == d) h = H_DIM;
    if (d <= H_DIM) h = 0;
    *horizontal_d = h;
    *vertical_d = d - h;
}

// ADSamplingPruner::GetRatio (pdx/adsampling.h:315-327).
void orc_ratios(uint64_t d, float eps0, float* out) {
    for (uint64_t v = 0; v <= d; ++v) {
        if (v == 0 || v == d) {
            out[v] = 1.0f;
        } else {
            const double s = 1.0 + eps0 / std::sqrt(static_cast<double>(v));
            out[v] = static_cast<float>(static_cast<double>(v) / static_cast<double>(d) * s * s);
        }
    }
}

// ADSamplingPruner::Rotate, matrix branch (pdx/adsampling.h:191-215): out = x * m^T.
void orc_rotate(const float* m, const float* x, uint64_t n, uint64_t d, float* out) {
    const char ta = 'T', tb = 'N';
    int mm = static_cast<int>(d), nn = static_cast<int>(n), kk = static_cast<int>(d), ld = static_cast<int>(d);
    float alpha = 1.0f, beta = 0.0f;
    scipy_sgemm_(&ta, &tb, &mm, &nn, &kk, &alpha, m, &ld, x, &ld, &beta, out, &ld);
}

// ADSamplingPruner::Unrotate, matrix branch (pdx/adsampling.h:273-298): out = x * m.
void orc_unrotate(const float* m, const float* x, uint64_t n, uint64_t d, float* out) {
    const char ta = 'N', tb = 'N';
    int mm = static_cast<int>(d), nn = static_cast<int>(n), kk = static_cast<int>(d), ld = static_cast<int>(d);
    float alpha = 1.0f, beta = 0.0f;
    scipy_sgemm_(&ta, &tb, &mm, &nn, &kk, &alpha, m, &ld, x, &ld, &beta, out, &ld);
}

// GetL2NormsRowMajor / GetPartialL2NormsRowMajor (superkmeans.h:1147-1171).
void orc_row_norms(const float* x, uint64_t n, uint64_t d, uint64_t upto, float* out) {
#pragma omp parallel for
    for (uint64_t i = 0; i < n; ++i) {
        const float* r = x + i * d;
        float acc = 0.f;
        for (uint64_t j = 0; j < upto; ++j) acc += r[j] * r[j];
        out[i] = acc;
    }
}

float orc_horizontal(const float* a, const float* b, uint64_t len) { return horizontal(a, b, len); }

// PDXLayout::PDXify<false> (pdx/layout.h:155-232): per chunk of 1024 rows (the last chunk with its
// own size cs): [vertical_d][cs] dimension-major, then for each 64-dimension block [cs][64].
void orc_pdxify(const float* in, float* out, uint64_t n, uint64_t d) {
    uint64_t hd, vd;
    orc_dimension_split(d, &hd, &vd);
    for (uint64_t c0 = 0; c0 < n; c0 += Y_BATCH) {
        const uint64_t cs = std::min<uint64_t>(Y_BATCH, n - c0);
        const float* src = in + c0 * d;
        float* dst = out + c0 * d;
        for (uint64_t j = 0; j < vd; ++j)
            for (uint64_t v = 0; v < cs; ++v) dst[j * cs + v] = src[v * d + j];
        dst += vd * cs;
        for (uint64_t h = 0; h < hd; h += H_DIM) {
            for (uint64_t v = 0; v < cs; ++v) std::memcpy(dst + v * H_DIM, src + v * d + vd + h, sizeof(float) * H_DIM);
            dst += cs * H_DIM;
        }
    }
}

// BatchComputer::FindNearestNeighbor (distance_computers/batch_computers.h:104-171).
void orc_find_nearest(const float* x, const float* y, uint64_t n, uint64_t k, uint64_t d, const float* nx, const float* ny, uint32_t* out_knn, float* out_dist) {
    std::vector<float> tile(X_BATCH * Y_BATCH);
    std::fill_n(out_dist, n, std::numeric_limits<float>::max());
    for (uint64_t i = 0; i < n; i += X_BATCH) {
        const uint64_t bx = std::min<uint64_t>(X_BATCH, n - i);
        for (uint64_t j = 0; j < k; j += Y_BATCH) {
            const uint64_t by = std::min<uint64_t>(Y_BATCH, k - j);
            dot_tile(x + i * d, y + j * d, bx, by, d, d, tile.data());
#pragma omp parallel for
            for (uint64_t r = 0; r < bx; ++r) {
                float* row = tile.data() + r * by;
                float best = std::numeric_limits<float>::max();
                uint32_t bi = 0;
                for (uint64_t c = 0; c < by; ++c) {
                    const float v = -2.0f * row[c] + nx[i + r] + ny[j + c];
                    if (c == 0 || v < best) {  // first minimum of the batch
                        best = v;
                        bi = static_cast<uint32_t>(c);
                    }
                }
                if (best < out_dist[i + r]) {  // a later batch must be strictly better
                    out_dist[i + r] = std::max(0.0f, best);
                    out_knn[i + r] = static_cast<uint32_t>(j) + bi;
                }
            }
        }
    }
}

// BatchComputer::FindNearestNeighborWithPruning (batch_computers.h:297-409) with
// PDXearch::Top1PartialSearchWithThresholdAndPartialDistances / Prune / SetBestCandidate
// (pdx/pdxearch.h:118-327) inlined for one 1024-centroid chunk per call of the inner block.
//   y      : row-major centroids (GEMM operand and exact distance to the previous centroid)
//   y_pdx  : PDX-blocked copy of y (horizontal blocks are read from here)
//   y_aux  : first vertical_d dimensions of y, row-major (dimensions [d', vertical_d) come from here)
void orc_find_nearest_pruned(
    const float* x, const float* y, const float* y_pdx, const float* y_aux, uint64_t n, uint64_t k, uint64_t d, const float* nx_partial, const float* ny_partial,
    const float* ratios, uint32_t partial_d, uint32_t* knn_io, float* dist_io, uint64_t* not_pruned
) {
    uint64_t hd, vd;
    orc_dimension_split(d, &hd, &vd);
    std::vector<float> tile(X_BATCH * Y_BATCH);
    for (uint64_t i = 0; i < n; i += X_BATCH) {
        const uint64_t bx = std::min<uint64_t>(X_BATCH, n - i);
        for (uint64_t j = 0; j < k; j += Y_BATCH) {
            const uint64_t cs = std::min<uint64_t>(Y_BATCH, k - j);
            dot_tile(x + i * d, y + j * d, bx, cs, d, partial_d, tile.data());
            const float* chunk_pdx = y_pdx + j * d;       // chunk offset is the same in both layouts
            const float* chunk_aux = y_aux + j * vd;
#pragma omp parallel for
            for (uint64_t r = 0; r < bx; ++r) {
                const uint64_t p = i + r;
                const float* q = x + p * d;
                float* pd = tile.data() + r * cs;
                for (uint64_t c = 0; c < cs; ++c) pd[c] = -2.0f * pd[c] + nx_partial[p] + ny_partial[j + c];
                const uint32_t prev = knn_io[p];
                // threshold: exact distance to the previous centroid at the first chunk, running best later
                float best = (j == 0) ? horizontal(y + static_cast<uint64_t>(prev) * d, q, d) : dist_io[p];
                uint32_t best_idx = prev;
                // first ADSampling test at d' dimensions
                uint32_t pos[Y_BATCH];
                size_t alive = 0;
                float thr = best * ratios[partial_d];
                for (uint64_t c = 0; c < cs; ++c)
                    if (pd[c] < thr) pos[alive++] = static_cast<uint32_t>(c);
                not_pruned[p] += alive;
                const bool only_previous = (alive == 1 && j + pos[0] == prev);
                if (!only_previous && alive) {
                    uint32_t dims = partial_d;
                    for (uint64_t h = 0; h < hd && alive; h += H_DIM) {
                        const float* blk = chunk_pdx + vd * cs + h * cs;
                        for (size_t s = 0; s < alive; ++s) pd[pos[s]] += horizontal(q + vd + h, blk + static_cast<uint64_t>(pos[s]) * H_DIM, H_DIM);
                        dims += H_DIM;
                        thr = best * ratios[dims];
                        size_t kept = 0;
                        for (size_t s = 0; s < alive; ++s)
                            if (pd[pos[s]] < thr) pos[kept++] = pos[s];
                        alive = kept;
                    }
                    if (alive && partial_d < vd) {
                        for (size_t s = 0; s < alive; ++s)
                            pd[pos[s]] += horizontal(q + partial_d, chunk_aux + static_cast<uint64_t>(pos[s]) * vd + partial_d, vd - partial_d);
                        thr = best * ratios[d];
                        size_t kept = 0;
                        for (size_t s = 0; s < alive; ++s)
                            if (pd[pos[s]] < thr) pos[kept++] = pos[s];
                        alive = kept;
                    }
                    for (size_t s = 0; s < alive; ++s)
                        if (pd[pos[s]] < best) {
                            best = pd[pos[s]];
                            best_idx = static_cast<uint32_t>(j) + pos[s];
                        }
                }
                knn_io[p] = best_idx;
                dist_io[p] = best;
            }
        }
    }
}

// UpdateCentroids (superkmeans.h:729-765): sums in point order.
void orc_update(const float* x, const uint32_t* assign, uint64_t n, uint64_t k, uint64_t d, float* sums, uint32_t* sizes) {
    std::fill_n(sums, k * d, 0.0f);
    std::fill_n(sizes, k, 0u);
    for (uint64_t i = 0; i < n; ++i) {
        const uint32_t c = assign[i];
        sizes[c] += 1;
        float* dst = sums + static_cast<uint64_t>(c) * d;
        const float* src = x + i * d;
        for (uint64_t j = 0; j < d; ++j) dst[j] += src[j];
    }
}

// ConsolidateCentroids, first half (superkmeans.h:936-953): mean, then SplitClusters (:890-928).
// Returns n_split.
uint64_t orc_mean_and_split(float* c, uint32_t* sizes, uint64_t n_samples, uint64_t k, uint64_t d, uint32_t seed) {
    for (uint64_t i = 0; i < k; ++i) {
        if (!sizes[i]) continue;
        const float mult = static_cast<float>(1.0 / sizes[i]);
        for (uint64_t j = 0; j < d; ++j) c[i * d + j] *= mult;
    }
    uint64_t n_split = 0;
    std::mt19937 rng(seed);
    const float eps = 1.0f / 1024.0f;
    for (uint64_t ci = 0; ci < k; ++ci) {
        if (sizes[ci]) continue;
        uint64_t cj = 0;
        for (;; cj = (cj + 1) % k) {
            const float p = static_cast<float>((sizes[cj] - 1.0) / static_cast<float>(n_samples - k));
            const float r = std::uniform_real_distribution<float>(0, 1)(rng);
            if (r < p) break;
        }
        for (uint64_t j = 0; j < d; ++j) {
            const float v = c[cj * d + j];
            const float up = v * (1 + eps), down = v * (1 - eps);
            c[ci * d + j] = (j % 2 == 0) ? up : down;
            c[cj * d + j] = (j % 2 == 0) ? down : up;
        }
        sizes[ci] = sizes[cj] / 2;
        sizes[cj] -= sizes[ci];
        ++n_split;
    }
    return n_split;
}

// TunePartialD (superkmeans.h:1230-1258).
uint32_t orc_tune_partial_d(const uint64_t* not_pruned, uint64_t n, uint64_t k, uint32_t partial_d, uint32_t vertical_d, float min_pct, float max_pct, float adj, float* avg_out) {
    float avg = 0.f;
    for (uint64_t i = 0; i < n; ++i) avg += static_cast<float>(not_pruned[i]);
    avg /= static_cast<float>(n * k);
    *avg_out = avg;
    if (avg > max_pct) {
        const uint32_t inc = static_cast<uint32_t>(partial_d * adj * 2);
        return std::min(partial_d + std::max(inc, 1u), vertical_d);
    }
    if (avg < min_pct) {
        const uint32_t dec = static_cast<uint32_t>(partial_d * adj);
        return std::max(partial_d - std::max(dec, 1u), MIN_PARTIAL_D);
    }
    return partial_d;
}

struct orc_stats {
    uint64_t iteration;
    float objective, shift;
    uint64_t split;
    float not_pruned_pct;
    uint32_t partial_d;
    int32_t is_gemm_only;
};

// SuperKMeans::Train for sampling_fraction == 1, no queries, early_termination off
// (superkmeans.h:162-332, RunIteration :786-879).  `m` is the rotation matrix (d x d); `rows_lo`,
// `rows_hi` restrict assignment and accumulation to a row range and `reduce` (may be null) is called
// on the per-iteration partial results, which is how a sharded run is emulated on the CPU:
//   reduce(user, buf, count, dtype)   dtype 0 = float32, 1 = float64, 2 = int32; sums in place.
typedef int (*orc_reduce_fn)(void* user, void* buf, uint64_t count, int dtype);

int orc_train_flat(
    const float* data, uint64_t n, uint64_t d, uint64_t k, const float* m, uint32_t iters, uint32_t seed, int use_blas_only, float eps0, uint64_t rows_lo, uint64_t rows_hi,
    orc_reduce_fn reduce, void* user, float* centroids_out /* k*d, unrotated */, float* rotated_centroids_out /* k*d or null */, uint32_t* assign_out /* rows_hi-rows_lo */,
    orc_stats* stats_out /* iters */
) {
    if (n < k) return 2;
    const uint64_t nl = rows_hi - rows_lo;
    uint64_t hd, vd;
    orc_dimension_split(d, &hd, &vd);
    uint32_t partial_d = std::max<uint32_t>(MIN_PARTIAL_D, static_cast<uint32_t>(vd) / 2);
    if (partial_d > vd) partial_d = static_cast<uint32_t>(vd);
    std::vector<float> ratios(d + 1);
    orc_ratios(d, eps0, ratios.data());

    // GenerateCentroids (:1100-1142): first k entries of a shuffle of [0, n)
    std::vector<size_t> idx(n);
    std::iota(idx.begin(), idx.end(), size_t{0});
    std::mt19937 rng(seed);
    std::shuffle(idx.begin(), idx.end(), rng);
    std::vector<float> init(k * d), prev(k * d), cur(k * d), pdx(k * d), aux(k * vd + 1);
    for (uint64_t c = 0; c < k; ++c) std::memcpy(&init[c * d], data + idx[c] * d, sizeof(float) * d);
    orc_rotate(m, init.data(), k, d, prev.data());

    std::vector<float> xr(nl * d), nx(nl), ny(k), dist(nl, 0.f);
    orc_rotate(m, data + rows_lo * d, nl, d, xr.data());
    orc_row_norms(xr.data(), nl, d, d, nx.data());
    std::vector<uint32_t> assign(nl, 0), sizes(k);
    std::vector<uint64_t> np(nl);
    const bool always_gemm = d < 128 || use_blas_only || k <= 256;  // :276-277
    bool partial_norms = false;
    float cost = 0.f;
    for (uint32_t it = 0; it < iters; ++it) {
        const bool gemm_only = it == 0 || always_gemm;
        if (!gemm_only && !partial_norms) {
            orc_row_norms(xr.data(), nl, d, partial_d, nx.data());
            partial_norms = true;
        }
        if (it > 0) std::swap(cur, prev);
        if (gemm_only) {
            orc_row_norms(prev.data(), k, d, d, ny.data());
            orc_find_nearest(xr.data(), prev.data(), nl, k, d, nx.data(), ny.data(), assign.data(), dist.data());
        } else {
            orc_row_norms(prev.data(), k, d, partial_d, ny.data());
            std::fill(np.begin(), np.end(), 0);
            orc_find_nearest_pruned(xr.data(), prev.data(), pdx.data(), aux.data(), nl, k, d, nx.data(), ny.data(), ratios.data(), partial_d, assign.data(), dist.data(), np.data());
        }
        orc_update(xr.data(), assign.data(), nl, k, d, cur.data(), sizes.data());
        double scal[2] = {0.0, 0.0};
        for (uint64_t i = 0; i < nl; ++i) {
            scal[0] += dist[i];
            scal[1] += static_cast<double>(np[i]);
        }
        if (reduce) {
            std::vector<int32_t> s32(sizes.begin(), sizes.end());
            if (reduce(user, cur.data(), k * d, 0) || reduce(user, s32.data(), k, 2) || reduce(user, scal, 2, 1)) return 4;
            for (uint64_t c = 0; c < k; ++c) sizes[c] = static_cast<uint32_t>(s32[c]);
        }
        float avg = -1.f;
        const uint32_t old_pd = partial_d;
        if (!gemm_only) {
            avg = static_cast<float>(scal[1]) / static_cast<float>(n * k);
            uint32_t nd = partial_d;
            if (avg > 0.05f) nd = std::min(partial_d + std::max(static_cast<uint32_t>(partial_d * 0.20f * 2), 1u), static_cast<uint32_t>(vd));
            else if (avg < 0.03f) nd = std::max(partial_d - std::max(static_cast<uint32_t>(partial_d * 0.20f), 1u), MIN_PARTIAL_D);
            if (nd != partial_d) {
                partial_d = nd;
                orc_row_norms(xr.data(), nl, d, partial_d, nx.data());
            }
        }
        const uint64_t n_split = orc_mean_and_split(cur.data(), sizes.data(), n, k, d, seed);
        orc_pdxify(cur.data(), pdx.data(), k, d);                                          // :961-965
        for (uint64_t c = 0; c < k; ++c) std::memcpy(&aux[c * vd], &cur[c * d], sizeof(float) * vd);  // :1206-1212
        cost = static_cast<float>(scal[0]);
        double shift = 0.0;
        for (uint64_t c = 0; c < k; ++c) {
            float s = 0.f;
            for (uint64_t j = 0; j < d; ++j) {
                const float t = cur[c * d + j] - prev[c * d + j];
                s += t * t;
            }
            shift += s;
        }
        if (stats_out) stats_out[it] = {it + 1, cost, static_cast<float>(shift), n_split, avg, gemm_only ? 0u : old_pd, gemm_only ? 1 : 0};
    }
    orc_unrotate(m, cur.data(), k, d, centroids_out);
    if (rotated_centroids_out) std::memcpy(rotated_centroids_out, cur.data(), sizeof(float) * k * d);
    if (assign_out) std::memcpy(assign_out, assign.data(), sizeof(uint32_t) * nl);
    return 0;
}

} // extern "C"
