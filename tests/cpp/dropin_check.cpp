// Compile-and-run check of the drop-in C++ headers.  Mirrors the usage in the reference's
// examples/simple_clustering.cpp and the exception tests of tests/test_superkmeans.cpp:91-211.
// Prints one line per check; exit code 0 when all pass.  With argument "gpu" it also trains.
#include <cstdio>
#include <cstring>
#include <string>
#include <random>
#include <vector>

#include "superkmeans/hierarchical_superkmeans.h"
#include "superkmeans/superkmeans.h"

static int failures = 0;
#define CHECK(cond)                                                                                \
    do {                                                                                           \
        if (!(cond)) {                                                                             \
            std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond);                             \
            ++failures;                                                                            \
        }                                                                                          \
    } while (0)

template <class Ex, class F>
static bool throws(F&& f) {
    try {
        f();
    } catch (const Ex&) {
        return true;
    } catch (...) {
        return false;
    }
    return false;
}

int main(int argc, char** argv) {
    const bool gpu = argc > 1 && std::strcmp(argv[1], "gpu") == 0;
    // constructor validation (std::invalid_argument, superkmeans.h:125-131)
    CHECK(throws<std::invalid_argument>([] { skmeans::SuperKMeans<> k(0, 16); }));
    CHECK(throws<std::invalid_argument>([] { skmeans::SuperKMeans<> k(16, 0); }));
    {
        skmeans::SuperKMeansConfig c;
        c.iters = 0;
        CHECK(throws<std::invalid_argument>([&] { skmeans::SuperKMeans<> k(8, 16, c); }));
        c.iters = 5;
        c.sampling_fraction = 1.5f;
        CHECK(throws<std::invalid_argument>([&] { skmeans::SuperKMeans<> k(8, 16, c); }));
    }
    {
        skmeans::HierarchicalSuperKMeansConfig c;
        CHECK(c.sampling_fraction == 1.0f);
        c.iters_fineclustering = 0;
        CHECK(throws<std::invalid_argument>([&] { skmeans::HierarchicalSuperKMeans<> k(8, 16, c); }));
    }
    CHECK(skmeans::HierarchicalSuperKMeans<>::GetNMesoclusters(65536) == 256);
    if (!gpu) {
        // no device: construction with valid arguments reports a runtime error instead of falling back
        CHECK(throws<std::runtime_error>([] { skmeans::SuperKMeans<> k(8, 16); }));
        std::printf(failures ? "FAILED\n" : "OK (cpu)\n");
        return failures ? 1 : 0;
    }
    const size_t n = 6000, d = 64, k = 40;
    std::mt19937 rng(1);
    std::normal_distribution<float> g(0.f, 1.f);
    std::vector<float> data(n * d);
    for (auto& v : data) v = g(rng);
    skmeans::SuperKMeansConfig cfg;
    cfg.sampling_fraction = 1.0f;
    cfg.iters = 5;
    skmeans::SuperKMeans km(k, d, cfg);
    CHECK(!km.IsTrained());
    CHECK(throws<std::runtime_error>([&] { (void) km.AssignTrainingPoints(data.data(), data.data(), n, k); }));
    std::vector<float> cent = km.Train(data.data(), n);
    CHECK(cent.size() == k * d);
    CHECK(km.IsTrained() && km.GetNClusters() == k);
    CHECK(km.iteration_stats.size() >= 1 && km.iteration_stats[0].is_gemm_only);
    CHECK(throws<std::runtime_error>([&] { km.Train(data.data(), n); }));
    std::vector<uint32_t> a = km.Assign(data.data(), cent.data(), n, k);
    CHECK(a.size() == n);
    size_t same = 0;
    for (size_t i = 0; i < n; ++i) same += (a[i] == km.assignments[i]);
    CHECK(same >= n * 9 / 10);
    auto bal = skmeans::SuperKMeans<>::GetClustersBalanceStats(a.data(), n, k);
    CHECK(bal.mean == static_cast<float>(n) / k);
    {
        skmeans::SuperKMeans<> small(100, d, cfg);
        CHECK(throws<std::runtime_error>([&] { small.Train(data.data(), 50); }));
    }
    {
        // Default sampling (sampling_fraction 0.3): assignments / distances are filled for the n_samples training rows
        // (superkmeans.h:202-207) and agree with what the engine holds.
        skmeans::SuperKMeansConfig sc;
        sc.iters = 4;
        sc.early_termination = false;
        skmeans::SuperKMeans<> sk(k, d, sc);
        (void) sk.Train(data.data(), n);
        const uint64_t held = skm_get_n_samples(sk.Handle());
        CHECK(held == 1800);   // floor(6000 * 0.3), below k * max_points_per_cluster
        std::vector<uint32_t> own(held);
        std::vector<float> own_d(held);
        CHECK(skm_get_assignments(sk.Handle(), own.data(), held) == SKM_OK);
        CHECK(skm_get_distances(sk.Handle(), own_d.data(), held) == SKM_OK);
        size_t eq = 0;
        for (uint64_t i = 0; i < held; ++i) eq += (own[i] == sk.assignments[i] && own[i] < k && own_d[i] == sk.GetDistancesPointer()[i]);
        CHECK(eq == held);
        CHECK(skm_get_assignments(sk.Handle(), own.data(), held + 1) == SKM_INVALID_ARGUMENT);
        CHECK(std::string(skm_last_error(sk.Handle())).find("more assignments") != std::string::npos);
    }
    skmeans::HierarchicalSuperKMeansConfig hc;
    hc.suppress_warnings = true;
    skmeans::HierarchicalSuperKMeans hk(64, d, hc);
    std::vector<float> hcent = hk.Train(data.data(), n);
    CHECK(hcent.size() == 64 * d && hk.n_mesoclusters == 8);
    CHECK(hk.hierarchical_iteration_stats.fineclustering_iteration_stats.size() == 8 * 5 || hc.early_termination);
    std::printf(failures ? "FAILED\n" : "OK (gpu)\n");
    return failures ? 1 : 0;
}
