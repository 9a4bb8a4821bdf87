// driver.cpp -- host control flow of codebook training, written against Device/Comm (backend.hpp).
//
// Follows the reference's loops step for step:
//   lbg_fit  <- lbg_quantize                      src/utils.rs:32-109  (batched over PQ subspaces, src/pq.rs:106-121)
//   rvq_fit  <- ResidualQuantizer::fit            src/rvq.rs:87-154
//   opq_fit  <- OptimizedProductQuantizer::fit    src/opq.rs:90-205
// Everything that touches rows of data is a Device call; every exchange between ranks is a Comm call.
#include "backend.hpp"

#include <cmath>
#include <cstring>
#include <vector>

#include "../../include/vqb.h"

namespace vqb {

namespace {

struct DevBuf {
    Device &dev;
    void *p = nullptr;
    DevBuf(Device &d, size_t bytes) : dev(d) { p = dev.alloc(bytes ? bytes : 1); }
    ~DevBuf() { dev.release(p); }
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
    template <typename T> T *as() const { return static_cast<T *>(p); }
};

// Total rows over all ranks and the global index of this rank's first row (shards are contiguous
// blocks in rank order).
void global_rows(Device &dev, Comm *comm, size_t n_local, uint64_t *n_global, uint64_t *row_begin)
{
    *n_global = n_local;
    *row_begin = 0;
    if (!comm || comm->world() <= 1) return;
    const int w = comm->world();
    std::vector<uint64_t> per(w, 0);
    per[comm->rank()] = n_local;
    DevBuf buf(dev, sizeof(uint64_t) * w);
    dev.upload(buf.p, per.data(), sizeof(uint64_t) * w);
    comm->allreduce_sum_u64(buf.as<uint64_t>(), w);
    dev.download(per.data(), buf.p, sizeof(uint64_t) * w);
    uint64_t total = 0;
    for (int r = 0; r < w; ++r) {
        if (r == comm->rank()) *row_begin = total;
        total += per[r];
    }
    *n_global = total;
}

// Closes an NCCL group when the scope is left, also by an exception.
struct GroupGuard {
    Comm *c;
    bool open = true;
    explicit GroupGuard(Comm *comm) : c(comm) { c->group_begin(); }
    void close() // the normal path: errors of the group's collectives surface here
    {
        open = false;
        c->group_end();
    }
    ~GroupGuard()
    {
        if (!open) return;
        try {
            c->group_end();
        } catch (...) {
        }
    }
};

bool use_ordered(int flags, uint64_t n_global)
{
    if (flags == VQB_ACCUM_ORDERED) return true;
    if (flags == VQB_ACCUM_FAST) return false;
    return n_global <= 65536;
}

} // namespace

void lbg_fit(Device &dev, Comm *comm, const Shape &sh, const float *x, size_t max_iters, const uint64_t *init_idx,
             DrawFn draw, void *user, size_t stream0, int flags, float *centroids, size_t *iterations)
{
    const size_t m = sh.m, k = sh.k, sd = sh.sd;
    uint64_t n_global = 0, row_begin = 0;
    global_rows(dev, comm, sh.n_local, &n_global, &row_begin);
    if (k == 0) // src/utils.rs:39-44
        throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: k must be greater than 0");
    if (n_global < k) // src/utils.rs:45-50
        throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: Not enough data points for k clusters");
    if (n_global >= (1ull << 32)) throw Error(VQB_ERR_UNSUPPORTED, "2^32 or more rows: cluster counts are 32-bit");
    if (!init_idx) throw Error(VQB_ERR_BAD_ARGUMENT, "init_idx is NULL");
    const bool multi = comm && comm->world() > 1;
    const bool ordered = use_ordered(flags, n_global);

    // initial sample: k rows per subspace (src/utils.rs:52-54)
    std::vector<RowPatch> patches;
    patches.reserve(m * k);
    for (size_t s = 0; s < m; ++s)
        for (size_t j = 0; j < k; ++j) {
            uint64_t r = init_idx[s * k + j];
            if (r >= n_global) throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: initial row index out of range");
            patches.push_back(RowPatch{(uint32_t)s, (uint32_t)j, r});
        }
    dev.patch_centroids(sh, x, row_begin, patches.data(), patches.size(), centroids, comm);
    if (iterations)
        for (size_t s = 0; s < m; ++s) iterations[s] = 0;
    if (max_iters == 0) return; // src/utils.rs:57 never runs

    dev.prepare_rows(sh, x);
    const size_t cb = dev.code_bytes(k);
    DevBuf codes(dev, sh.n_local * m * cb);
    dev.zero(codes.p, sh.n_local * m * cb); // src/utils.rs:55: previous assignments start at 0
    // sums | counts | moved flags of one iteration, one allocation, cleared here once and then by every centroid update
    IterBuffers buf;
    const size_t words = buf.words(sh);
    auto lay_out = [&](IterBuffers &b, uint32_t *base) {
        b.sums = reinterpret_cast<float *>(base);
        b.counts = base + m * k * sd;
        b.moved = b.counts + m * k;
    };
    // Ranks that can map each other's memory gather into two alternating buffers of a shared window and the update kernel
    // adds the parts itself; otherwise one buffer and an all-reduce.  (Every rank comes here after the collective in
    // global_rows, i.e. after all kernels of an earlier fit on every rank: nobody reads the window's buffers any more.)
    uint32_t *window[2] = {nullptr, nullptr};
    const bool direct = multi && comm->peer_window(words, window);
    IterBuffers pair[2];
    DevBuf iter(dev, direct ? 0 : sizeof(float) * words);
    if (direct) {
        lay_out(pair[0], window[0]);
        lay_out(pair[1], window[1]);
    } else {
        dev.zero(iter.p, sizeof(float) * words);
        lay_out(buf, iter.as<uint32_t>());
    }
    // below 2^24 rows every count is exact in f32, and sums, counts and flags then cross the ranks as ONE f32 all-reduce
    buf.counts_f32 = multi && !direct && n_global < (1ull << 24);
    if (multi && !direct && !buf.counts_f32 && comm->world() > 256)
        throw Error(VQB_ERR_UNSUPPORTED, "more than 256 ranks with 2^24 or more rows are not supported");
    DevBuf act(dev, sizeof(uint32_t) * m);
    std::vector<uint32_t> active(m, 1);
    bool active_dirty = true;
    IterStatus status;
    const size_t wps = (k + 31) / 32;
    // Unordered accumulation keeps this rank's sums and counts from one iteration to the next and, from the second
    // iteration on, only moves the rows whose assignment changed (Device::accumulate_moved); the exchange buffer gets a copy.
    bool incremental = !ordered;
    const size_t sum_words = m * k * sd + m * k;
    DevBuf codes_prev(dev, incremental ? sh.n_local * m * cb : 0), local_mem(dev, incremental ? sizeof(uint32_t) * sum_words : 0);
    IterBuffers local;
    lay_out(local, local_mem.as<uint32_t>());
    local.moved = nullptr;
    bool local_valid = false;
    bool prev_current = false; // codes_prev already equals codes (accumulate_moved leaves it so)

    for (size_t it = 0; it < max_iters; ++it) {
        bool any = false;
        for (size_t s = 0; s < m; ++s) any = any || active[s];
        if (!any) break;
        if (active_dirty) { // the mask only changes when a subspace retires
            dev.upload(act.p, active.data(), sizeof(uint32_t) * m);
            active_dirty = false;
        }
        if (direct) buf = pair[it & 1];
        const bool moved_only = incremental && local_valid;
        const size_t pieces = it == 0 ? dev.arriving_pieces(x) : 0;
        if (pieces) {
            // The rows are still on their way from the host: assignment (59-80) and, where no order is asked for, the sums
            // (83-92) follow the copies piece by piece, so that all but the last piece's work hides behind the transfer.
            if (incremental) {
                local.counts_f32 = buf.counts_f32;
                dev.zero(local_mem.p, sizeof(uint32_t) * sum_words);
            }
            size_t r0 = 0;
            for (size_t i = 0; i < pieces; ++i) {
                const size_t r1 = dev.await_piece(x, i);
                if (r1 <= r0 || r1 > sh.n_local) throw Error(VQB_ERR_BAD_ARGUMENT, "rows arrive out of order");
                Shape part = sh;
                part.n_local = r1 - r0;
                const float *xp = x + r0 * sh.ld;
                void *cp = static_cast<char *>(codes.p) + r0 * m * cb;
                dev.assign_train(part, xp, centroids, cp, act.as<uint32_t>(), buf);
                if (!ordered) dev.accumulate(part, xp, cp, act.as<uint32_t>(), false, incremental ? local : buf);
                r0 = r1;
            }
            if (r0 != sh.n_local) throw Error(VQB_ERR_BAD_ARGUMENT, "not all rows arrived");
            if (ordered) dev.accumulate(sh, x, codes.p, act.as<uint32_t>(), true, buf);
            if (incremental) {
                local_valid = true;
                dev.copy(buf.sums, local.sums, sizeof(uint32_t) * sum_words);
            }
        } else {
            if (moved_only && !prev_current) dev.copy(codes_prev.p, codes.p, sh.n_local * m * cb);
            dev.assign_train(sh, x, centroids, codes.p, act.as<uint32_t>(), buf);          // 59-80
            if (incremental) {                                                             // 83-92
                local.counts_f32 = buf.counts_f32;
                if (moved_only) {
                    prev_current = dev.accumulate_moved(sh, x, codes_prev.p, codes.p, act.as<uint32_t>(), local);
                    if (!prev_current) incremental = false;
                }
                if (incremental && !moved_only) {
                    dev.zero(local_mem.p, sizeof(uint32_t) * sum_words);
                    dev.accumulate(sh, x, codes.p, act.as<uint32_t>(), false, local);
                    local_valid = true;
                }
                if (incremental) dev.copy(buf.sums, local.sums, sizeof(uint32_t) * sum_words); // the moved flags are already in buf
            }
            if (!incremental) dev.accumulate(sh, x, codes.p, act.as<uint32_t>(), ordered, buf);
        }
        PeerExchange px;
        if (direct) {
            px = comm->peer_exchange((int)(it & 1));
        } else if (multi) { // the only exchange of an iteration, ~144 KiB
            if (buf.counts_f32) {
                comm->allreduce_sum_f32(buf.sums, words);
            } else {
                GroupGuard gg(comm);
                comm->allreduce_sum_f32(buf.sums, m * k * sd);
                comm->allreduce_sum_u32(buf.counts, m * k + m);
                gg.close();
            }
        }
        dev.update_centroids(sh, buf, act.as<uint32_t>(), centroids, status, direct ? &px : nullptr); // 95-99; flags on the host when it returns
        patches.clear();
        for (size_t s = 0; s < m; ++s) {
            if (!active[s]) continue;
            if (iterations) iterations[s] += 1;
            if (!status.has_empty[s]) continue;
            for (size_t j = 0; j < k; ++j) // ascending j, one draw per empty cluster (95-101)
                if (status.empty_bits[s * wps + j / 32] >> (j % 32) & 1u) {
                    if (!draw) throw Error(VQB_ERR_CALLBACK, "an empty cluster needs a draw callback");
                    uint64_t r = draw(user, stream0 + s, n_global);
                    if (r >= n_global) throw Error(VQB_ERR_CALLBACK, "draw callback returned a row index out of range");
                    patches.push_back(RowPatch{(uint32_t)s, (uint32_t)j, r});
                }
        }
        if (!patches.empty())
            dev.patch_centroids(sh, x, row_begin, patches.data(), patches.size(), centroids, comm);
        for (size_t s = 0; s < m; ++s)
            if (active[s] && !status.moved[s]) { // 104-106: stop after the update
                active[s] = 0;
                active_dirty = true;
            }
    }
}

size_t rvq_fit(Device &dev, Comm *comm, float *res, size_t n_local, size_t dim, size_t stages, size_t k,
               size_t max_iters, float epsilon, int metric, double p, InitFn init, DrawFn draw, void *user,
               int flags, float *codebooks)
{
    uint64_t n_global = 0, row_begin = 0;
    global_rows(dev, comm, n_local, &n_global, &row_begin);
    const bool multi = comm && comm->world() > 1;
    Shape sh;
    sh.n_local = n_local;
    sh.ld = dim;
    sh.m = 1;
    sh.sd = dim;
    sh.k = k;
    DevBuf norm(dev, sizeof(double));
    std::vector<uint64_t> idx(k ? k : 1, 0);
    size_t done = 0;
    for (size_t stage = 0; stage < stages; ++stage) { // src/rvq.rs:105
        float *cb = codebooks + stage * k * dim;
        if (k > 0 && n_global >= k) {
            if (!init) throw Error(VQB_ERR_BAD_ARGUMENT, "init callback is NULL");
            init(user, stage, n_global, k, idx.data());
        }
        lbg_fit(dev, comm, sh, res, max_iters, idx.data(), draw, user, stage, flags, cb, nullptr); // 107
        ++done;
        if (k >= 2 && metric == VQB_MINKOWSKI && p <= 0.0) // first distance.compute call (rvq.rs:118)
            throw Error(VQB_ERR_INVALID_METRIC_PARAMETER, "Invalid metric parameter for Minkowski: p must be positive");
        dev.zero(norm.p, sizeof(double));
        dev.rvq_update(res, n_local, dim, cb, k, metric, p, norm.as<double>()); // 111-138
        if (multi) comm->allreduce_sum_f64(norm.as<double>(), 1);
        double total = 0.0;
        dev.download(&total, norm.p, sizeof(double));
        float avg = (float)(total / (double)n_global);
        if (avg < epsilon) break; // 139-141
    }
    return done; // 145
}

bool opq_fit(Device &dev, Comm *comm, const float *x, size_t n_local, size_t dim, size_t m, size_t k,
             size_t max_iters, size_t opq_iters, int metric, double p, const uint64_t *init_idx, DrawFn draw,
             RestartFn restart, void *user, int flags, float *rotation_host, float *codebooks)
{
    for (size_t i = 0; i < dim; ++i)
        for (size_t j = 0; j < dim; ++j) rotation_host[i * dim + j] = (i == j) ? 1.0f : 0.0f; // src/opq.rs:119
    if (opq_iters == 0) return false;
    const bool multi = comm && comm->world() > 1;
    Shape sh;
    sh.n_local = n_local;
    sh.ld = dim;
    sh.m = m;
    sh.sd = dim / m;
    sh.k = k;
    const size_t bytes = sizeof(float) * n_local * dim;
    DevBuf rotated(dev, bytes), rec(dev, bytes);
    DevBuf a_d(dev, sizeof(double) * dim * dim), rot_d(dev, sizeof(float) * dim * dim);
    dev.copy(rotated.p, x, bytes); // src/opq.rs:121
    std::vector<double> a(dim * dim), u(dim * dim), sv(dim), v(dim * dim);
    bool have_v = false; // v holds the previous outer iteration's right singular vectors
    for (size_t it = 0; it < opq_iters; ++it) { // 124
        if (restart) restart(user);             // the reference builds fresh StdRng(seed + i) here (140)
        lbg_fit(dev, comm, sh, rotated.as<float>(), max_iters, init_idx, draw, user, 0, flags, codebooks, nullptr);
        if (k >= 2 && metric == VQB_MINKOWSKI && p <= 0.0)
            throw Error(VQB_ERR_INVALID_METRIC_PARAMETER, "Invalid metric parameter for Minkowski: p must be positive");
        dev.pq_encode(sh, rotated.as<float>(), codebooks, metric, p, nullptr, nullptr, rec.as<float>()); // 146-168
        dev.cross_cov(rec.as<float>(), rotated.as<float>(), n_local, dim, a_d.as<double>());            // 172-179
        if (multi) comm->allreduce_sum_f64(a_d.as<double>(), dim * dim);
        // 180-183: rotation = V U^T.  On the device as the polar factor of A^T when that converges (full-rank A), else the SVD.
        if (dev.polar_rotation(a_d.as<double>(), dim, rot_d.as<float>())) {
            dev.download(rotation_host, rot_d.p, sizeof(float) * dim * dim);
            have_v = false;
        } else {
            dev.download(a.data(), a_d.p, sizeof(double) * dim * dim);
            // The rotation moves little from one outer iteration to the next, so the sweeps start from the previous V: G = A V
            // then has nearly orthogonal columns and two or three sweeps suffice.  V U^T (the orthogonal polar factor of A^T)
            // does not depend on where the sweeps start.
            jacobi_svd(a.data(), dim, u.data(), sv.data(), v.data(), &dev, have_v ? v.data() : nullptr); // 180-182
            have_v = true;
            for (size_t i = 0; i < dim; ++i)                          // rotation = V * U^T (183)
                for (size_t j = 0; j < dim; ++j) {
                    double acc = 0.0;
                    for (size_t t = 0; t < dim; ++t) acc += v[i * dim + t] * u[j * dim + t];
                    rotation_host[i * dim + j] = (float)acc;
                }
            dev.upload(rot_d.p, rotation_host, sizeof(float) * dim * dim);
        }
        dev.rotate_rows(rot_d.as<float>(), dim, x, n_local, rotated.as<float>()); // 186-194, from the ORIGINAL rows
    }
    return true;
}

// One-sided (Hestenes) Jacobi SVD in f64.  Columns with a vanishing singular value get an orthonormal
// completion so that U stays orthogonal (V * U^T must be a rotation even for rank-deficient input).
void jacobi_svd(const double *a, size_t n, double *u, double *s, double *v, Device *dev, const double *v0)
{
    // gt / vt hold the working matrices TRANSPOSED (row p = column p of g = a * v), so that each plane rotation
    // streams two contiguous rows.
    std::vector<double> gt(n * n), vt(n * n, 0.0);
    if (v0) { // start from G = A V0, V = V0 (v0 may alias v: it is consumed before v is written)
        for (size_t i = 0; i < n; ++i)
            for (size_t j = 0; j < n; ++j) vt[j * n + i] = v0[i * n + j];
        for (size_t j = 0; j < n; ++j)     // column j of G = A * (column j of V0) = A * (row j of vt)
            for (size_t i = 0; i < n; ++i) {
                double acc = 0.0;
                for (size_t t = 0; t < n; ++t) acc += a[i * n + t] * vt[j * n + t];
                gt[j * n + i] = acc;
            }
    } else {
        for (size_t i = 0; i < n; ++i)
            for (size_t j = 0; j < n; ++j) gt[j * n + i] = a[i * n + j];
        for (size_t i = 0; i < n; ++i) vt[i * n + i] = 1.0;
    }
    const double eps = 1e-15;
    const bool on_device = dev && dev->svd_sweeps(gt.data(), vt.data(), n);
    for (int sweep = 0; !on_device && sweep < 60; ++sweep) {
        bool rotated = false;
        for (size_t p = 0; p + 1 < n; ++p)
            for (size_t q = p + 1; q < n; ++q) {
                double *gp = &gt[p * n], *gq = &gt[q * n];
                double alpha = 0, beta = 0, gamma = 0;
                for (size_t i = 0; i < n; ++i) {
                    alpha += gp[i] * gp[i];
                    beta += gq[i] * gq[i];
                    gamma += gp[i] * gq[i];
                }
                if (std::fabs(gamma) <= eps * std::sqrt(alpha * beta) || gamma == 0.0) continue;
                rotated = true;
                double zeta = (beta - alpha) / (2.0 * gamma);
                double t = (zeta >= 0 ? 1.0 : -1.0) / (std::fabs(zeta) + std::sqrt(1.0 + zeta * zeta));
                double c = 1.0 / std::sqrt(1.0 + t * t), sn = c * t;
                double *vp = &vt[p * n], *vq = &vt[q * n];
                for (size_t i = 0; i < n; ++i) {
                    double a0 = gp[i], b0 = gq[i];
                    gp[i] = c * a0 - sn * b0;
                    gq[i] = sn * a0 + c * b0;
                    double a1 = vp[i], b1 = vq[i];
                    vp[i] = c * a1 - sn * b1;
                    vq[i] = sn * a1 + c * b1;
                }
            }
        if (!rotated) break;
    }
    std::vector<double> g(n * n);
    for (size_t i = 0; i < n; ++i)
        for (size_t j = 0; j < n; ++j) {
            g[i * n + j] = gt[j * n + i];
            v[i * n + j] = vt[j * n + i];
        }
    double smax = 0.0;
    for (size_t j = 0; j < n; ++j) {
        double nn = 0;
        for (size_t i = 0; i < n; ++i) nn += g[i * n + j] * g[i * n + j];
        s[j] = std::sqrt(nn);
        if (s[j] > smax) smax = s[j];
    }
    std::vector<char> filled(n, 0);
    for (size_t j = 0; j < n; ++j)
        if (s[j] > smax * 1e-13 && s[j] > 0.0) {
            for (size_t i = 0; i < n; ++i) u[i * n + j] = g[i * n + j] / s[j];
            filled[j] = 1;
        }
    for (size_t j = 0; j < n; ++j) { // complete the null space, Gram-Schmidt over unit vectors
        if (filled[j]) continue;
        s[j] = 0.0;
        for (size_t e = 0; e < n; ++e) {
            std::vector<double> w(n, 0.0);
            w[e] = 1.0;
            for (int pass = 0; pass < 2; ++pass)
                for (size_t c = 0; c < n; ++c) {
                    if (!filled[c]) continue;
                    double d = 0;
                    for (size_t i = 0; i < n; ++i) d += w[i] * u[i * n + c];
                    for (size_t i = 0; i < n; ++i) w[i] -= d * u[i * n + c];
                }
            double nn = 0;
            for (size_t i = 0; i < n; ++i) nn += w[i] * w[i];
            if (nn > 1e-6) {
                nn = std::sqrt(nn);
                for (size_t i = 0; i < n; ++i) u[i * n + j] = w[i] / nn;
                filled[j] = 1;
                break;
            }
        }
    }
}

} // namespace vqb
