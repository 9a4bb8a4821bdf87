// vq.hpp -- C++ host facade over libvqb.so with the names and behaviour of the Rust crate `vq`.
//
// The reference's public API (src/lib.rs:1-11) is mirrored one to one:
//   vq::Vector<T>                      <- vector::Vector<T>                 (src/vector.rs:149-176)
//   vq::Distance                       <- distances::Distance               (src/distances.rs:73-88)
//   vq::ProductQuantizer::fit/quantize <- pq::ProductQuantizer              (src/pq.rs:79-187)
//   vq::ResidualQuantizer              <- rvq::ResidualQuantizer            (src/rvq.rs:87-215)
//   vq::OptimizedProductQuantizer      <- opq::OptimizedProductQuantizer    (src/opq.rs:90-264)
//   vq::ScalarQuantizer, BinaryQuantizer <- sq::, bq::                      (src/sq.rs, src/bq.rs)
//   vq::VqError                        <- exceptions::VqError               (src/exceptions.rs:9-25)
// Where the reference panics, these functions throw vq::VqError whose what() is the reference's Display text.
// Seeded sampling uses the documented SplitMix64 stand-in (see seeding.py): the reference's StdRng draws cannot be
// reproduced without the `rand` crate, and the library takes row indices from its host for exactly that reason.
#pragma once
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/vqb.h"

namespace vq {

struct VqError : std::runtime_error {
    enum Kind { DimensionMismatch = 3, EmptyInput = 1, InvalidParameter = 2, InvalidMetricParameter = 4, Backend = 100 };
    Kind kind;
    int code;
    VqError(int c, const std::string &msg)
        : std::runtime_error(msg), kind(c >= 1 && c <= 4 ? static_cast<Kind>(c) : Backend), code(c)
    {
    }
};

// IEEE binary16 value as the reference's half::f16 (bits + conversion back to f32).
struct f16 {
    uint16_t bits = 0;
    float to_f32() const
    {
        uint32_t sign = (uint32_t)(bits & 0x8000u) << 16, e = (bits >> 10) & 0x1f, m = bits & 0x3ffu, out;
        if (e == 0) {
            if (m == 0) out = sign;
            else {
                int sh = 0;
                while (!(m & 0x400u)) {
                    m <<= 1;
                    ++sh;
                }
                out = sign | ((uint32_t)(113 - sh) << 23) | ((m & 0x3ffu) << 13);
            }
        } else if (e == 0x1f) out = sign | 0x7f800000u | (m << 13);
        else out = sign | ((e + 112u) << 23) | (m << 13);
        float f;
        std::memcpy(&f, &out, 4);
        return f;
    }
};

template <typename T> struct Vector {
    std::vector<T> data;
    Vector() {}
    explicit Vector(std::vector<T> d) : data(std::move(d)) {}
    size_t len() const { return data.size(); }
    bool is_empty() const { return data.empty(); }
    bool operator==(const Vector &o) const { return data == o.data; }
};

struct Distance {
    int metric;
    double p;
    static Distance SquaredEuclidean() { return {VQB_SQUARED_EUCLIDEAN, 0.0}; }
    static Distance Euclidean() { return {VQB_EUCLIDEAN, 0.0}; }
    static Distance CosineDistance() { return {VQB_COSINE, 0.0}; }
    static Distance Manhattan() { return {VQB_MANHATTAN, 0.0}; }
    static Distance Chebyshev() { return {VQB_CHEBYSHEV, 0.0}; }
    static Distance Minkowski(double p) { return {VQB_MINKOWSKI, p}; }
    static Distance Hamming() { return {VQB_HAMMING, 0.0}; }
    inline float compute(const std::vector<float> &a, const std::vector<float> &b) const;
};

namespace detail {

inline void check(int rc, vqb_ctx *ctx)
{
    if (rc != VQB_OK) throw VqError(rc, vqb_last_error(ctx));
}

// One context per process and device 0 unless set_device() was called before first use.
inline int &device_index()
{
    static int d = 0;
    return d;
}
inline vqb_ctx *context()
{
    struct Holder {
        vqb_ctx *c = nullptr;
        Holder() { check(vqb_ctx_create(device_index(), &c), nullptr); }
        ~Holder() { vqb_ctx_destroy(c); }
    };
    static Holder h;
    return h.c;
}

inline std::vector<float> pack_rows(const std::vector<Vector<float>> &rows, size_t *dim)
{
    *dim = rows.empty() ? 0 : rows[0].len();
    std::vector<float> flat;
    flat.reserve(rows.size() * *dim);
    for (const auto &r : rows) {
        if (r.len() != *dim) throw VqError(3, "Dimension mismatch: expected " + std::to_string(*dim) + ", got " + std::to_string(r.len()));
        flat.insert(flat.end(), r.data.begin(), r.data.end());
    }
    return flat;
}

// SplitMix64 stand-in for the reference's StdRng (same definition as vq_b200/seeding.py).
struct StandInRng {
    uint64_t state;
    explicit StandInRng(uint64_t seed) : state(seed) {}
    uint64_t next()
    {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    uint64_t below(uint64_t n) { return (uint64_t)(((unsigned __int128)next() * n) >> 64); }
    std::vector<uint64_t> choose_multiple(uint64_t n, size_t k)
    {
        std::unordered_map<uint64_t, uint64_t> swapped;
        std::vector<uint64_t> out(k);
        for (size_t i = 0; i < k; ++i) {
            uint64_t j = i + below(n - i);
            uint64_t vi = swapped.count(i) ? swapped[i] : i, vj = swapped.count(j) ? swapped[j] : j;
            swapped[i] = vj;
            swapped[j] = vi;
            out[i] = vj;
        }
        return out;
    }
};

// One stream per LBG call, seeded seed + stream (src/pq.rs:119, src/rvq.rs:107, src/opq.rs:140).
struct Seeder {
    uint64_t seed;
    size_t m = 0, k = 0;
    uint64_t n = 0;
    std::unordered_map<size_t, StandInRng> rngs;
    explicit Seeder(uint64_t s) : seed(s) {}
    std::vector<uint64_t> init(size_t stream, uint64_t nn, size_t kk)
    {
        rngs.erase(stream);
        auto it = rngs.emplace(stream, StandInRng(seed + stream)).first;
        return it->second.choose_multiple(nn, kk);
    }
    uint64_t draw(size_t stream, uint64_t nn)
    {
        auto it = rngs.find(stream);
        if (it == rngs.end()) it = rngs.emplace(stream, StandInRng(seed + stream)).first;
        return it->second.below(nn);
    }
    static uint64_t draw_cb(void *user, size_t stream, uint64_t nn) { return static_cast<Seeder *>(user)->draw(stream, nn); }
    static void init_cb(void *user, size_t stage, uint64_t nn, size_t kk, uint64_t *out)
    {
        auto v = static_cast<Seeder *>(user)->init(stage, nn, kk);
        std::memcpy(out, v.data(), kk * sizeof(uint64_t));
    }
    static void restart_cb(void *user)
    {
        Seeder *s = static_cast<Seeder *>(user);
        s->rngs.clear();
        for (size_t i = 0; i < s->m; ++i) s->init(i, s->n, s->k);
    }
};

inline Vector<f16> to_f16(const std::vector<uint16_t> &bits)
{
    Vector<f16> v;
    v.data.resize(bits.size());
    for (size_t i = 0; i < bits.size(); ++i) v.data[i].bits = bits[i];
    return v;
}

} // namespace detail

inline void set_device(int device) { detail::device_index() = device; }

inline float Distance::compute(const std::vector<float> &a, const std::vector<float> &b) const
{
    float out = 0.0f;
    vqb_ctx *c = detail::context();
    detail::check(vqb_distance_rows(c, metric, p, a.data(), a.size(), b.data(), b.size(), 1, &out), c);
    return out;
}

class ProductQuantizer {
  public:
    static ProductQuantizer fit(const std::vector<Vector<float>> &training_data, size_t m, size_t k, size_t max_iters,
                                Distance distance, uint64_t seed)
    {
        vqb_ctx *c = detail::context();
        size_t dim = 0;
        std::vector<float> flat = detail::pack_rows(training_data, &dim);
        const size_t n = training_data.size();
        detail::Seeder seeder(seed);
        std::vector<uint64_t> init(m * (k ? k : 1), 0);
        if (m && k && k <= n)
            for (size_t i = 0; i < m; ++i) {
                auto v = seeder.init(i, n, k);
                std::memcpy(&init[i * k], v.data(), k * sizeof(uint64_t));
            }
        vqb_pq *h = nullptr;
        detail::check(vqb_pq_fit(c, flat.data(), n, dim, m, k, max_iters, distance.metric, distance.p, init.data(),
                                 detail::Seeder::draw_cb, &seeder, VQB_ACCUM_AUTO, &h), c);
        return ProductQuantizer(h);
    }
    Vector<f16> quantize(const Vector<float> &vector) const
    {
        std::vector<uint16_t> out(vector.len());
        detail::check(vqb_pq_quantize(h_.get(), vector.data.data(), 1, vector.len(), out.data(), nullptr), detail::context());
        return detail::to_f16(out);
    }
    // All rows in one call (replaces the per-vector loop of src/bin/eval_pq.rs:51-59).
    std::vector<Vector<f16>> quantize_batch(const std::vector<Vector<float>> &rows) const
    {
        size_t dim = 0;
        std::vector<float> flat = detail::pack_rows(rows, &dim);
        std::vector<uint16_t> out(flat.size());
        detail::check(vqb_pq_quantize(h_.get(), flat.data(), rows.size(), dim, out.data(), nullptr), detail::context());
        std::vector<Vector<f16>> res(rows.size());
        for (size_t r = 0; r < rows.size(); ++r)
            res[r] = detail::to_f16(std::vector<uint16_t>(out.begin() + r * dim, out.begin() + (r + 1) * dim));
        return res;
    }

  private:
    explicit ProductQuantizer(vqb_pq *h) : h_(h, vqb_pq_destroy) {}
    std::shared_ptr<vqb_pq> h_;
};

class ResidualQuantizer {
  public:
    static ResidualQuantizer fit(const std::vector<Vector<float>> &training_data, size_t stages, size_t k, size_t max_iters,
                                 float epsilon, Distance distance, uint64_t seed)
    {
        vqb_ctx *c = detail::context();
        size_t dim = 0;
        std::vector<float> flat = detail::pack_rows(training_data, &dim);
        detail::Seeder seeder(seed);
        vqb_rvq *h = nullptr;
        detail::check(vqb_rvq_fit(c, flat.data(), training_data.size(), dim, stages, k, max_iters, epsilon, distance.metric,
                                  distance.p, detail::Seeder::init_cb, detail::Seeder::draw_cb, &seeder, VQB_ACCUM_AUTO, &h), c);
        return ResidualQuantizer(h);
    }
    Vector<f16> quantize(const Vector<float> &vector) const
    {
        std::vector<uint16_t> out(vector.len());
        detail::check(vqb_rvq_quantize(h_.get(), vector.data.data(), 1, vector.len(), out.data(), nullptr), detail::context());
        return detail::to_f16(out);
    }

  private:
    explicit ResidualQuantizer(vqb_rvq *h) : h_(h, vqb_rvq_destroy) {}
    std::shared_ptr<vqb_rvq> h_;
};

class OptimizedProductQuantizer {
  public:
    static OptimizedProductQuantizer fit(const std::vector<Vector<float>> &training_data, size_t m, size_t k, size_t max_iters,
                                         size_t opq_iters, Distance distance, uint64_t seed)
    {
        vqb_ctx *c = detail::context();
        size_t dim = 0;
        std::vector<float> flat = detail::pack_rows(training_data, &dim);
        const size_t n = training_data.size();
        detail::Seeder seeder(seed);
        seeder.m = (m && k && k <= n) ? m : 0;
        seeder.k = k;
        seeder.n = n;
        std::vector<uint64_t> init(m * (k ? k : 1), 0);
        for (size_t i = 0; i < seeder.m; ++i) {
            auto v = seeder.init(i, n, k);
            std::memcpy(&init[i * k], v.data(), k * sizeof(uint64_t));
        }
        vqb_opq *h = nullptr;
        detail::check(vqb_opq_fit(c, flat.data(), n, dim, m, k, max_iters, opq_iters, distance.metric, distance.p, init.data(),
                                  detail::Seeder::draw_cb, detail::Seeder::restart_cb, &seeder, VQB_ACCUM_AUTO, &h), c);
        return OptimizedProductQuantizer(h);
    }
    Vector<f16> quantize(const Vector<float> &vector) const
    {
        size_t m = 0;
        vqb_opq_shape(h_.get(), &m, nullptr, nullptr);
        std::vector<uint16_t> out(m ? vector.len() : 0); // no codebooks (opq_iters == 0): empty result, as the reference
        detail::check(vqb_opq_quantize(h_.get(), vector.data.data(), 1, vector.len(), out.empty() ? nullptr : out.data(), nullptr),
                      detail::context());
        return detail::to_f16(out);
    }

  private:
    explicit OptimizedProductQuantizer(vqb_opq *h) : h_(h, vqb_opq_destroy) {}
    std::shared_ptr<vqb_opq> h_;
};

// TSVQ (src/tsvq.rs:189-250)
class TSVQ {
  public:
    TSVQ(const std::vector<Vector<float>> &training_data, size_t max_depth, Distance distance_) : distance(distance_)
    {
        vqb_ctx *c = detail::context();
        size_t dim = 0;
        std::vector<float> flat = detail::pack_rows(training_data, &dim);
        vqb_tsvq *h = nullptr;
        detail::check(vqb_tsvq_fit(c, flat.data(), training_data.size(), dim, max_depth, distance.metric, distance.p, &h), c);
        h_ = std::shared_ptr<vqb_tsvq>(h, vqb_tsvq_destroy);
    }
    Vector<f16> quantize(const Vector<float> &vector) const
    {
        std::vector<uint16_t> out(vector.len());
        detail::check(vqb_tsvq_quantize(h_.get(), vector.data.data(), 1, vector.len(), out.data(), nullptr), detail::context());
        return detail::to_f16(out);
    }
    Distance distance;

  private:
    std::shared_ptr<vqb_tsvq> h_;
};

struct ScalarQuantizer {
    float min, max;
    size_t levels;
    float step;
    static ScalarQuantizer fit(float min, float max, size_t levels)
    {
        float step = 0.0f;
        detail::check(vqb_sq_fit(min, max, levels, &step), nullptr);
        return ScalarQuantizer{min, max, levels, step};
    }
    Vector<uint8_t> quantize(const Vector<float> &vector) const
    {
        Vector<uint8_t> out;
        out.data.resize(vector.len());
        vqb_ctx *c = detail::context();
        detail::check(vqb_sq_quantize(c, min, max, levels, step, vector.data.data(), vector.len(), out.data.data()), c);
        return out;
    }
};

struct BinaryQuantizer {
    float threshold;
    uint8_t low, high;
    static BinaryQuantizer fit(float threshold, uint8_t low, uint8_t high)
    {
        detail::check(vqb_bq_fit(threshold, low, high), nullptr);
        return BinaryQuantizer{threshold, low, high};
    }
    Vector<uint8_t> quantize(const Vector<float> &vector) const
    {
        Vector<uint8_t> out;
        out.data.resize(vector.len());
        vqb_ctx *c = detail::context();
        detail::check(vqb_bq_quantize(c, threshold, low, high, vector.data.data(), vector.len(), out.data.data()), c);
        return out;
    }
};

// lbg_quantize (src/utils.rs:32-109); crate-private in the reference, exposed here because its unit tests are part
// of the parity suite.
inline std::vector<Vector<float>> lbg_quantize(const std::vector<Vector<float>> &data, size_t k, size_t max_iters, uint64_t seed)
{
    vqb_ctx *c = detail::context();
    size_t dim = 0;
    std::vector<float> flat = detail::pack_rows(data, &dim);
    detail::Seeder seeder(seed);
    std::vector<uint64_t> init(k ? k : 1, 0);
    if (k && k <= data.size()) init = seeder.init(0, data.size(), k);
    std::vector<float> cent(k * dim);
    detail::check(vqb_lbg_fit(c, flat.data(), data.size(), dim, k, max_iters, init.data(), detail::Seeder::draw_cb, &seeder,
                              VQB_ACCUM_AUTO, cent.empty() ? nullptr : cent.data(), nullptr), c);
    std::vector<Vector<float>> out(k);
    for (size_t j = 0; j < k; ++j) out[j] = Vector<float>(std::vector<float>(cent.begin() + j * dim, cent.begin() + (j + 1) * dim));
    return out;
}

} // namespace vq
