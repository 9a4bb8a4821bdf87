// test_facade.cpp -- the reference's own integration tests, restated against the C++ facade (vq_b200/cpp/vq.hpp).
// Each case names the reference test it mirrors.  Built and run by tests/test_gpu_cpp_facade.py on a GPU machine.
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>

#include "../../vq_b200/cpp/vq.hpp"

using namespace vq;

static int g_failed = 0;
#define CHECK(cond)                                                            \
    do {                                                                       \
        if (!(cond)) {                                                         \
            std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond);        \
            ++g_failed;                                                        \
        }                                                                      \
    } while (0)

template <typename F> static bool panics_with(F &&f, const std::string &needle)
{
    try {
        f();
    } catch (const VqError &e) {
        return std::string(e.what()).find(needle) != std::string::npos;
    }
    return false;
}

// tests/utils.rs:8-25: n vectors of `dim` values in [-1000, 1000) (seeded; stand-in generator)
static std::vector<Vector<float>> generate_test_data(size_t n, size_t dim, uint64_t seed = 42)
{
    detail::StandInRng rng(seed);
    std::vector<Vector<float>> out(n);
    for (auto &v : out) {
        v.data.resize(dim);
        for (auto &x : v.data) x = -1000.0f + 2000.0f * (float)((rng.next() >> 40) * (1.0 / 16777216.0));
    }
    return out;
}

static bool approx_eq(float a, float b, float eps) { return std::fabs(a - b) < eps; }

int main()
{
    // tests/test_distances.rs (a selection; the full table is checked from Python against the same entry point)
    CHECK(approx_eq(Distance::SquaredEuclidean().compute({1, 2, 3}, {4, 6, 8}), 50.0f, 1e-6f));
    CHECK(approx_eq(Distance::Euclidean().compute({1, 2, 3}, {4, 6, 8}), std::sqrt(50.0f), 1e-6f));
    CHECK(approx_eq(Distance::CosineDistance().compute({1, 0}, {0, 1}), 1.0f, 1e-6f));
    CHECK(approx_eq(Distance::Manhattan().compute({1, 2, 3}, {4, 6, 8}), 12.0f, 1e-6f));
    CHECK(approx_eq(Distance::Chebyshev().compute({1, 5, 3}, {4, 2, 9}), 6.0f, 1e-6f));
    CHECK(approx_eq(Distance::Minkowski(3.0).compute({1, 2, 3}, {4, 6, 8}), 6.0f, 1e-5f));
    CHECK(approx_eq(Distance::Hamming().compute({1, 2, 3, 4}, {1, 0, 3, 0}), 2.0f, 1e-6f));
    CHECK(panics_with([] { Distance::Euclidean().compute({1, 2}, {1}); }, "Dimension mismatch")); // test_distances.rs:206-213

    // src/utils.rs:126-160
    {
        std::vector<Vector<float>> data = {Vector<float>({1, 2}), Vector<float>({2, 3}), Vector<float>({3, 4}), Vector<float>({4, 5})};
        CHECK(lbg_quantize(data, 2, 10, 42).size() == 2);
        CHECK(lbg_quantize(data, 2, 100, 42).size() == 2);
        CHECK(panics_with([&] { lbg_quantize({Vector<float>({1, 2}), Vector<float>({2, 3})}, 0, 10, 42); }, "k must be greater than 0"));
        CHECK(panics_with([&] { lbg_quantize({Vector<float>({1, 2})}, 2, 10, 42); }, "Not enough data points for k clusters"));
        auto one = lbg_quantize({Vector<float>({1, 2})}, 1, 10, 42);
        CHECK(one.size() == 1 && one[0] == Vector<float>({1, 2}));
    }

    // tests/test_pq.rs:10-45
    {
        auto training = generate_test_data(1000, 10);
        auto pq = ProductQuantizer::fit(training, 2, 2, 50, Distance::SquaredEuclidean(), 42);
        auto q = pq.quantize(training[0]);
        CHECK(q.len() == 10);
        for (auto h : q.data) CHECK(std::isfinite(h.to_f32()));
        auto all = pq.quantize_batch(training);
        CHECK(all.size() == 1000 && all[0].data.size() == 10);
        for (size_t i = 0; i < 10; ++i) CHECK(all[0].data[i].bits == q.data[i].bits);
        CHECK(panics_with([&] { pq.quantize(Vector<float>({1, 2, 3})); }, "Dimension mismatch: expected 10, got 3"));
        CHECK(panics_with([&] { ProductQuantizer::fit({}, 2, 2, 5, Distance::Euclidean(), 0); }, "Empty input"));
        CHECK(panics_with([&] { ProductQuantizer::fit(training, 20, 2, 5, Distance::Euclidean(), 0); }, "Data dimension must be at least m"));
        CHECK(panics_with([&] { ProductQuantizer::fit(training, 3, 2, 5, Distance::Euclidean(), 0); }, "Data dimension must be divisible by m"));
    }

    // tests/test_rvq.rs:10-62
    {
        auto training = generate_test_data(1000, 10);
        auto rvq = ResidualQuantizer::fit(training, 2, 2, 50, 1e-6f, Distance::SquaredEuclidean(), 42);
        auto q = rvq.quantize(training[0]);
        CHECK(q.len() == 10);
        for (auto h : q.data) CHECK(std::isfinite(h.to_f32()));
        for (size_t i = 0; i < 20; ++i) CHECK(rvq.quantize(training[i]).len() == 10);
    }

    // tests/test_opq.rs:10-80
    {
        auto training = generate_test_data(1000, 10);
        auto opq = OptimizedProductQuantizer::fit(training, 2, 2, 50, 5, Distance::SquaredEuclidean(), 42);
        auto q = opq.quantize(training[0]);
        CHECK(q.len() == 10);
        for (auto h : q.data) CHECK(std::isfinite(h.to_f32()));
        CHECK(panics_with([&] { OptimizedProductQuantizer::fit(training, 3, 2, 5, 2, Distance::Euclidean(), 0); }, "Dimension must be divisible by m"));
        auto none = OptimizedProductQuantizer::fit(training, 2, 2, 5, 0, Distance::Euclidean(), 0); // opq.rs:119-124,197-204
        CHECK(none.quantize(training[0]).len() == 0);
    }

    // tests/test_sq.rs:9-33 and 36-77
    {
        auto sq = ScalarQuantizer::fit(-1.0f, 1.0f, 5);
        for (float x : {-1.2f, -1.0f, -0.8f, -0.3f, 0.0f, 0.3f, 0.6f, 1.0f, 1.2f}) {
            auto idx = sq.quantize(Vector<float>({x}));
            CHECK(idx.len() == 1);
            float recon = sq.min + idx.data[0] * sq.step, clamped = x < -1.0f ? -1.0f : (x > 1.0f ? 1.0f : x);
            CHECK(std::fabs(recon - clamped) <= sq.step / 2.0f + 1e-6f);
        }
        auto data = generate_test_data(100, 1024);
        auto big = ScalarQuantizer::fit(-1000.0f, 1000.0f, 256);
        for (const auto &v : data) {
            auto idx = big.quantize(v);
            CHECK(idx.len() == 1024);
            for (size_t i = 0; i < 1024; ++i) {
                float recon = big.min + idx.data[i] * big.step;
                CHECK(std::fabs(v.data[i] - recon) <= big.step / 2.0f + 2e-4f); // two ulps of 1000 on top of step/2
            }
        }
        CHECK(panics_with([] { ScalarQuantizer::fit(1.0f, 1.0f, 4); }, "max must be greater than min"));
        CHECK(panics_with([] { ScalarQuantizer::fit(0.0f, 1.0f, 1); }, "levels must be at least 2"));
        CHECK(panics_with([] { ScalarQuantizer::fit(0.0f, 1.0f, 257); }, "levels must be no more than 256"));
    }

    // tests/test_bq.rs:9-32 and the doc example src/bq.rs:12-20
    {
        auto v = generate_test_data(1, 1024)[0];
        auto bq = BinaryQuantizer::fit(0.0f, 0, 1);
        auto q = bq.quantize(v);
        CHECK(q.len() == 1024);
        for (size_t i = 0; i < 1024; ++i) CHECK(q.data[i] == (v.data[i] >= 0.0f ? 1 : 0));
        auto d = bq.quantize(Vector<float>({-1.0f, 0.0f, 1.0f}));
        CHECK(d.data[0] == 0 && d.data[1] == 1 && d.data[2] == 1);
        CHECK(panics_with([] { BinaryQuantizer::fit(0.0f, 1, 1); }, "Low quantization level must be less than high quantization level"));
    }

    // tests/test_tsvq.rs:11-22: ten copies of one vector, depth 3: the quantized vector equals it within 1e-6
    {
        Vector<float> v({1, 2, 3, 4, 5});
        std::vector<Vector<float>> data(10, v);
        TSVQ tsvq(data, 3, Distance::SquaredEuclidean());
        Vector<f16> q = tsvq.quantize(v);
        CHECK(q.len() == v.len());
        for (size_t i = 0; i < v.len(); ++i) CHECK(approx_eq(q.data[i].to_f32(), v.data[i], 1e-6f));
        CHECK(panics_with([&] { tsvq.quantize(Vector<float>({1, 2, 3})); }, "Dimension mismatch: expected 5, got 3"));
        CHECK(panics_with([] { TSVQ(std::vector<Vector<float>>{}, 3, Distance::Euclidean()); }, "Empty input"));
    }
    // tests/test_tsvq.rs:24-43: 1000 random vectors of width 10, depth 3: every output has the input's length and is finite
    {
        auto data = generate_test_data(1000, 10);
        TSVQ tsvq(data, 3, Distance::SquaredEuclidean());
        bool ok = true;
        for (size_t i = 0; i < data.size(); i += 37) {
            Vector<f16> q = tsvq.quantize(data[i]);
            ok = ok && q.len() == data[i].len();
            for (size_t t = 0; t < q.len(); ++t) ok = ok && std::isfinite(q.data[t].to_f32());
        }
        CHECK(ok);
    }
    // tests/test_tsvq.rs:11-22 pins f16 exactness on representable values; same property through PQ's f16 output
    {
        std::vector<Vector<float>> same(10, Vector<float>({1, 2, 3, 4, 5, 6}));
        auto pq = ProductQuantizer::fit(same, 2, 1, 5, Distance::Euclidean(), 0);
        auto q = pq.quantize(same[0]);
        for (size_t i = 0; i < 6; ++i) CHECK(approx_eq(q.data[i].to_f32(), same[0].data[i], 1e-6f));
    }

    std::printf(g_failed ? "%d check(s) failed\n" : "all facade checks passed\n", g_failed);
    return g_failed ? 1 : 0;
}
