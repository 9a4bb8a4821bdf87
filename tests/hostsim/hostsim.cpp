// hostsim.cpp -- TEST INFRASTRUCTURE: runs the product's host training loops (vq_b200/csrc/driver.cpp) on CPU ranks.
//
// The shipped library implements vqb::Device with CUDA kernels and vqb::Comm with NCCL.  To exercise the multi-rank
// protocol of the loops (shard offsets, row patches by max-reduce, all-reduce of sums/counts/flags, replicated draw
// callbacks, per-subspace retirement) without GPUs, this file implements Device with plain loops over host memory
// and Comm with callbacks that the Python test backs with torch.distributed (gloo).  It is built only by the test
// suite, is never part of libvqb.so, and is not a fallback of the product.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../vq_b200/csrc/backend.hpp"

using namespace vqb;

extern "C" {
// kind: 0 sum f32, 1 sum f64, 2 sum u32, 3 max u32, 4 sum u64; in place over `n` elements of host memory
typedef void (*hs_allreduce_fn)(void *user, int kind, void *buf, size_t n);
}

namespace {

class CallbackComm : public Comm {
  public:
    CallbackComm(hs_allreduce_fn f, void *u, int r, int w) : fn_(f), user_(u), rank_(r), world_(w) {}
    int rank() const override { return rank_; }
    int world() const override { return world_; }
    void allreduce_sum_f32(float *b, size_t n) override { fn_(user_, 0, b, n); }
    void allreduce_sum_f64(double *b, size_t n) override { fn_(user_, 1, b, n); }
    void allreduce_sum_u32(uint32_t *b, size_t n) override { fn_(user_, 2, b, n); }
    void allreduce_max_u32(uint32_t *b, size_t n) override { fn_(user_, 3, b, n); }
    void allreduce_sum_u64(uint64_t *b, size_t n) override { fn_(user_, 4, b, n); }

  private:
    hs_allreduce_fn fn_;
    void *user_;
    int rank_, world_;
};

float dist2(const float *a, const float *b, size_t d)
{
    float acc = 0.0f;
    for (size_t i = 0; i < d; ++i) {
        float diff = a[i] - b[i];
        float prod = diff * diff;
        acc = acc + prod;
    }
    return acc;
}

class HostDevice : public Device {
  public:
    void *alloc(size_t bytes) override { return std::malloc(bytes ? bytes : 1); }
    void release(void *p) override { std::free(p); }
    void upload(void *d, const void *s, size_t b) override { std::memcpy(d, s, b); }
    void download(void *d, const void *s, size_t b) override { std::memcpy(d, s, b); }
    void copy(void *d, const void *s, size_t b) override { std::memcpy(d, s, b); }
    void zero(void *d, size_t b) override { std::memset(d, 0, b); }
    size_t code_bytes(size_t) const override { return 4; }

    void patch_centroids(const Shape &sh, const float *x, uint64_t row_begin, const RowPatch *patches, size_t n, float *centroids,
                         Comm *comm) override
    {
        std::vector<uint32_t> stage(n * sh.sd, 0u);
        for (size_t p = 0; p < n; ++p) {
            const RowPatch &pt = patches[p];
            if (pt.row >= row_begin && pt.row - row_begin < sh.n_local)
                std::memcpy(&stage[p * sh.sd], x + (pt.row - row_begin) * sh.ld + pt.subspace * sh.sd, sh.sd * sizeof(float));
        }
        if (comm && comm->world() > 1) comm->allreduce_max_u32(stage.data(), stage.size());
        for (size_t p = 0; p < n; ++p)
            std::memcpy(centroids + ((size_t)patches[p].subspace * sh.k + patches[p].cluster) * sh.sd, &stage[p * sh.sd],
                        sh.sd * sizeof(float));
    }
    void assign_train(const Shape &sh, const float *x, const float *centroids, void *codes_v, const uint32_t *active,
                      const IterBuffers &buf) override
    {
        uint32_t *codes = (uint32_t *)codes_v;
        for (size_t s = 0; s < sh.m; ++s) {
            if (active && !active[s]) continue;
            for (size_t i = 0; i < sh.n_local; ++i) {
                const float *v = x + i * sh.ld + s * sh.sd;
                uint32_t best = 0;
                float bd = dist2(v, centroids + s * sh.k * sh.sd, sh.sd);
                for (size_t j = 1; j < sh.k; ++j) {
                    float d = dist2(v, centroids + (s * sh.k + j) * sh.sd, sh.sd);
                    if (d < bd) {
                        bd = d;
                        best = (uint32_t)j;
                    }
                }
                if (codes[i * sh.m + s] != best) buf.moved[s] |= 0x3F800000u; // the bits of 1.0f, as the kernels write them
                codes[i * sh.m + s] = best;
            }
        }
    }
    static void add_count(const IterBuffers &buf, size_t at)
    {
        if (buf.counts_f32) {
            float c;
            std::memcpy(&c, &buf.counts[at], 4);
            c += 1.0f;
            std::memcpy(&buf.counts[at], &c, 4);
        } else {
            buf.counts[at]++;
        }
    }
    void accumulate(const Shape &sh, const float *x, const void *codes_v, const uint32_t *active, bool, const IterBuffers &buf) override
    {
        const uint32_t *codes = (const uint32_t *)codes_v;
        for (size_t s = 0; s < sh.m; ++s) {
            if (active && !active[s]) continue;
            for (size_t i = 0; i < sh.n_local; ++i) {
                size_t j = codes[i * sh.m + s];
                float *dst = buf.sums + (s * sh.k + j) * sh.sd;
                const float *v = x + i * sh.ld + s * sh.sd;
                for (size_t c = 0; c < sh.sd; ++c) dst[c] = dst[c] + v[c];
                add_count(buf, s * sh.k + j);
            }
        }
    }
    // the running totals follow the rows whose code changed (the driver's short cut after the first iteration)
    bool accumulate_moved(const Shape &sh, const float *x, void *prev_v, const void *codes_v, const uint32_t *active, const IterBuffers &local) override
    {
        uint32_t *prev = (uint32_t *)prev_v;
        const uint32_t *codes = (const uint32_t *)codes_v;
        ++moved_passes;
        for (size_t s = 0; s < sh.m; ++s) {
            if (active && !active[s]) continue;
            for (size_t i = 0; i < sh.n_local; ++i) {
                const size_t was = prev[i * sh.m + s], now = codes[i * sh.m + s];
                if (was == now) continue;
                prev[i * sh.m + s] = (uint32_t)now; // the contract: equal to codes on return
                const float *v = x + i * sh.ld + s * sh.sd;
                float *add = local.sums + (s * sh.k + now) * sh.sd, *sub = local.sums + (s * sh.k + was) * sh.sd;
                for (size_t c = 0; c < sh.sd; ++c) add[c] = add[c] + v[c], sub[c] = sub[c] - v[c];
                if (local.counts_f32) {
                    float a, b;
                    std::memcpy(&a, &local.counts[s * sh.k + now], 4), std::memcpy(&b, &local.counts[s * sh.k + was], 4);
                    a += 1.0f, b -= 1.0f;
                    std::memcpy(&local.counts[s * sh.k + now], &a, 4), std::memcpy(&local.counts[s * sh.k + was], &b, 4);
                } else {
                    local.counts[s * sh.k + now]++, local.counts[s * sh.k + was]--;
                }
            }
        }
        return true;
    }
    size_t moved_passes = 0;
    // rows that "arrive" in pieces (Device::arriving_pieces): nothing is in flight on the host, the first iteration simply has
    // to walk the pieces and come out with the same result
    const float *arriving_x = nullptr;
    size_t arriving_n = 0, pieces = 0, awaited = 0, pieces_walked = 0;
    size_t arriving_pieces(const float *x) override { return (pieces && x == arriving_x && awaited == 0) ? pieces : 0; }
    size_t await_piece(const float *x, size_t i) override
    {
        if (x != arriving_x || i != awaited || i >= pieces) throw Error(2, "pieces awaited out of order");
        awaited = i + 1;
        ++pieces_walked;
        const size_t per = (arriving_n + pieces - 1) / pieces;
        return std::min(arriving_n, (i + 1) * per);
    }
    void update_centroids(const Shape &sh, const IterBuffers &buf, const uint32_t *active, float *centroids, IterStatus &st, const PeerExchange * = nullptr) override
    {
        const size_t wps = (sh.k + 31) / 32;
        st.moved.assign(sh.m, 0);
        st.has_empty.assign(sh.m, 0);
        st.empty_bits.assign(sh.m * wps, 0u);
        for (size_t s = 0; s < sh.m; ++s) {
            const bool act = !active || active[s];
            st.moved[s] = act && buf.moved[s] != 0;
            buf.moved[s] = 0;
            if (!act) continue;
            for (size_t j = 0; j < sh.k; ++j) {
                float cf;
                if (buf.counts_f32) std::memcpy(&cf, &buf.counts[s * sh.k + j], 4);
                else cf = (float)buf.counts[s * sh.k + j];
                if (cf == 0.0f) {
                    st.empty_bits[s * wps + j / 32] |= 1u << (j % 32);
                    st.has_empty[s] = 1;
                    continue;
                }
                for (size_t t = 0; t < sh.sd; ++t) {
                    centroids[(s * sh.k + j) * sh.sd + t] = buf.sums[(s * sh.k + j) * sh.sd + t] / cf;
                    buf.sums[(s * sh.k + j) * sh.sd + t] = 0.0f;
                }
                buf.counts[s * sh.k + j] = 0;
            }
        }
    }
    void rvq_update(float *res, size_t n, size_t dim, const float *cb, size_t k, int, double, double *norm_sum) override
    {
        for (size_t i = 0; i < n; ++i) {
            float *r = res + i * dim;
            size_t best = 0;
            float bd = std::sqrt(dist2(r, cb, dim));
            for (size_t j = 1; j < k; ++j) {
                float d = std::sqrt(dist2(r, cb + j * dim, dim));
                if (d < bd) {
                    bd = d;
                    best = j;
                }
            }
            float nsq = 0.0f;
            for (size_t t = 0; t < dim; ++t) {
                r[t] = r[t] - cb[best * dim + t];
                float v = r[t] * r[t];
                nsq = nsq + v;
            }
            *norm_sum += (double)std::sqrt(nsq);
        }
    }
    void pq_encode(const Shape &sh, const float *x, const float *cb, int, double, uint16_t *, uint32_t *, float *out_f32) override
    {
        for (size_t i = 0; i < sh.n_local; ++i)
            for (size_t s = 0; s < sh.m; ++s) {
                const float *v = x + i * sh.ld + s * sh.sd;
                size_t best = 0;
                float bd = std::sqrt(dist2(v, cb + s * sh.k * sh.sd, sh.sd));
                for (size_t j = 1; j < sh.k; ++j) {
                    float d = std::sqrt(dist2(v, cb + (s * sh.k + j) * sh.sd, sh.sd));
                    if (d < bd) {
                        bd = d;
                        best = j;
                    }
                }
                if (out_f32) std::memcpy(out_f32 + i * sh.m * sh.sd + s * sh.sd, cb + (s * sh.k + best) * sh.sd, sh.sd * sizeof(float));
            }
    }
    void rotate_rows(const float *rot, size_t dim, const float *x, size_t n, float *y) override
    {
        for (size_t r = 0; r < n; ++r)
            for (size_t i = 0; i < dim; ++i) {
                float acc = 0.0f;
                for (size_t j = 0; j < dim; ++j) acc += rot[i * dim + j] * x[r * dim + j];
                y[r * dim + i] = acc;
            }
    }
    void cross_cov(const float *y, const float *x, size_t n, size_t dim, double *a) override
    {
        std::memset(a, 0, sizeof(double) * dim * dim);
        for (size_t r = 0; r < n; ++r)
            for (size_t i = 0; i < dim; ++i)
                for (size_t j = 0; j < dim; ++j) a[i * dim + j] += (double)y[r * dim + i] * (double)x[r * dim + j];
    }
};

thread_local std::string g_err;

} // namespace

static size_t g_moved_passes = 0, g_pieces_walked = 0;

extern "C" {

const char *hs_last_error(void) { return g_err.c_str(); }

// vqb_pq_fit with a host Device; x = this rank's rows.  Euclidean metric (2 = error code for InvalidParameter etc.).
size_t hs_moved_passes() { return g_moved_passes; }
size_t hs_pieces_walked() { return g_pieces_walked; }

int hs_pq_fit(const float *x, size_t n_local, size_t dim, size_t m, size_t k, size_t max_iters, const uint64_t *init_idx,
              DrawFn draw, void *user, hs_allreduce_fn ar, void *ar_user, int rank, int world, float *codebooks, size_t *iterations)
{
    try {
        HostDevice dev;
        CallbackComm comm(ar, ar_user, rank, world);
        Shape sh;
        sh.n_local = n_local;
        sh.ld = dim;
        sh.m = m;
        sh.sd = dim / m;
        sh.k = k;
        // accumulation mode: ordered (1) unless the test asks for the unordered one (2), whose later iterations only move changed rows
        const char *mode = std::getenv("HOSTSIM_ACCUM");
        if (const char *pc = std::getenv("HOSTSIM_PIECES")) { // the rows count as still arriving, in that many pieces
            dev.arriving_x = x;
            dev.arriving_n = n_local;
            dev.pieces = std::min<size_t>((size_t)std::atoi(pc), n_local);
        }
        lbg_fit(dev, world > 1 ? &comm : nullptr, sh, x, max_iters, init_idx, draw, user, 0, mode ? std::atoi(mode) : 1, codebooks, iterations);
        g_moved_passes = dev.moved_passes;
        g_pieces_walked = dev.pieces_walked;
        return 0;
    } catch (const Error &e) {
        g_err = e.what();
        return e.code;
    }
}

int hs_rvq_fit(const float *x, size_t n_local, size_t dim, size_t stages, size_t k, size_t max_iters, float epsilon, InitFn init,
               DrawFn draw, void *user, hs_allreduce_fn ar, void *ar_user, int rank, int world, float *codebooks, size_t *stages_out)
{
    try {
        HostDevice dev;
        CallbackComm comm(ar, ar_user, rank, world);
        std::vector<float> res(x, x + n_local * dim);
        *stages_out = rvq_fit(dev, world > 1 ? &comm : nullptr, res.data(), n_local, dim, stages, k, max_iters, epsilon, 1, 0.0, init,
                              draw, user, 1, codebooks);
        return 0;
    } catch (const Error &e) {
        g_err = e.what();
        return e.code;
    }
}

int hs_opq_fit(const float *x, size_t n_local, size_t dim, size_t m, size_t k, size_t max_iters, size_t opq_iters,
               const uint64_t *init_idx, DrawFn draw, RestartFn restart, void *user, hs_allreduce_fn ar, void *ar_user, int rank,
               int world, float *rotation, float *codebooks)
{
    try {
        HostDevice dev;
        CallbackComm comm(ar, ar_user, rank, world);
        opq_fit(dev, world > 1 ? &comm : nullptr, x, n_local, dim, m, k, max_iters, opq_iters, 1, 0.0, init_idx, draw, restart, user, 1,
                rotation, codebooks);
        return 0;
    } catch (const Error &e) {
        g_err = e.what();
        return e.code;
    }
}

void hs_jacobi_svd(const double *a, size_t n, double *u, double *s, double *v) { jacobi_svd(a, n, u, s, v); }

} // extern "C"
