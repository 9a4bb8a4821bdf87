// api.cpp -- the extern "C" surface declared in include/vqb.h.
//
// Validation follows the reference's order and wording (src/pq.rs:87-102,147-156; src/opq.rs:99-114;
// src/rvq.rs:96-98; src/sq.rs:51-68; src/bq.rs:47-54; src/exceptions.rs).  Host pointers are staged
// through device buffers; device pointers are used in place.
#include <algorithm>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/vqb.h"
#include "cuda_device.hpp"
#include "opq_parts.hpp"
#include "tsvq.hpp"

namespace vqb {
void nccl_unique_id(uint8_t *out128);
Comm *make_nccl_comm(CudaDevice &dev, const uint8_t *id_bytes, int rank, int world);
} // namespace vqb

using namespace vqb;

struct vqb_ctx {
    std::unique_ptr<CudaDevice> dev;
    std::unique_ptr<Comm> comm;
    std::mutex mu;
    std::string err;
};

struct vqb_pq {
    vqb_ctx *ctx;
    size_t m, k, sd;
    int metric;
    double p;
    float *codebooks; // device
    std::vector<size_t> iters;
};

struct vqb_rvq {
    vqb_ctx *ctx;
    size_t stages, k, dim;
    float epsilon;
    int metric;
    double p;
    float *codebooks; // device, stages x k x dim
};

struct vqb_tsvq {
    vqb_ctx *ctx;
    int metric;
    double p;
    TsvqTree tree;
};

struct vqb_opq {
    vqb_ctx *ctx;
    size_t m, k, sd, dim;
    int metric;
    double p;
    bool empty; // opq_iters == 0: identity rotation, no codebooks (src/opq.rs:119-124,197-204)
    std::vector<float> rotation; // host copy, dim x dim row-major
    float *rotation_d;
    float *codebooks;
};

namespace {

thread_local std::string g_err;

int set_err(vqb_ctx *ctx, int code, const std::string &msg)
{
    if (ctx) ctx->err = msg;
    g_err = msg;
    return code;
}

template <typename F> int guarded(vqb_ctx *ctx, F &&f)
{
    try {
        if (ctx) ctx->dev->make_current();
        f();
        return VQB_OK;
    } catch (const Error &e) {
        return set_err(ctx, e.code, e.what());
    } catch (const std::bad_alloc &) {
        return set_err(ctx, VQB_ERR_CUDA, "out of host memory");
    } catch (const std::exception &e) {
        return set_err(ctx, VQB_ERR_BAD_ARGUMENT, e.what());
    } catch (...) {
        return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "unknown error");
    }
}

bool metric_ok(int m) { return m >= 0 && m <= 6; }

// A read-only input that lives on the device for the duration of a call.
struct In {
    CudaDevice &dev;
    const void *d = nullptr;
    void *owned = nullptr;
    In(CudaDevice &dv, const void *p, size_t bytes) : dev(dv)
    {
        if (bytes == 0 || dev.is_device_pointer(p)) {
            d = p;
        } else {
            owned = dev.alloc(bytes);
            VQB_CUDA_CHECK(cudaMemcpyAsync(owned, p, bytes, cudaMemcpyHostToDevice, dev.stream()));
            d = owned;
        }
    }
    ~In() { dev.release(owned); }
    template <typename T> const T *as() const { return static_cast<const T *>(d); }
};

// The rows of a fit.  A large host buffer is copied in pieces on a helper stream and announced to the device, so that
// the first iteration can follow the copy (CudaDevice::begin_arrival); everything else behaves like In.
struct RowsIn {
    CudaDevice &dev;
    const float *d = nullptr;
    void *owned = nullptr;
    RowsIn(CudaDevice &dv, const float *p, size_t n, size_t ld) : dev(dv)
    {
        const size_t bytes = sizeof(float) * n * ld;
        if (bytes == 0 || dev.is_device_pointer(p)) {
            d = p;
            return;
        }
        owned = dev.alloc(bytes);
        d = static_cast<const float *>(owned);
        try {
            if (!dev.begin_arrival(static_cast<float *>(owned), p, n, ld))
                VQB_CUDA_CHECK(cudaMemcpyAsync(owned, p, bytes, cudaMemcpyHostToDevice, dev.stream()));
        } catch (...) {
            dev.end_arrival();
            dev.release(owned);
            throw;
        }
    }
    ~RowsIn()
    {
        dev.end_arrival(); // no copy from the caller's buffer is left running
        dev.release(owned);
    }
    RowsIn(const RowsIn &) = delete;
    RowsIn &operator=(const RowsIn &) = delete;
};

// An output that is produced on the device and, when the caller's pointer is host memory, copied back.
struct Out {
    CudaDevice &dev;
    void *d = nullptr;
    void *host = nullptr;
    size_t bytes = 0;
    Out(CudaDevice &dv, void *p, size_t b) : dev(dv), bytes(b)
    {
        if (!p) return;
        if (b == 0 || dev.is_device_pointer(p)) {
            d = p;
        } else {
            host = p;
            d = dev.alloc(b);
        }
    }
    void finish()
    {
        if (host) {
            dev.download(host, d, bytes);
            dev.release(d);
            host = nullptr;
            d = nullptr;
        }
    }
    ~Out()
    {
        if (host) dev.release(d);
    }
    template <typename T> T *as() const { return static_cast<T *>(d); }
};

// Host buffers in, host buffers out: the items are cut into chunks and walked through a two-slot pipeline so that the
// upload of chunk i+1, the kernels of chunk i and the download of chunk i-1 overlap (PCIe is full duplex).
//   in_bytes / out_bytes[k]: bytes per item;  run(dev_in, items, dev_out[]) launches the kernels of one chunk on dev.stream().
struct HostPipeline {
    static constexpr int MAX_OUT = 2;
    CudaDevice &dev;
    size_t chunk_items;
    HostPipeline(CudaDevice &d, size_t items_per_chunk) : dev(d), chunk_items(items_per_chunk) {}

    template <typename Run>
    void go(const void *host_in, size_t n_items, size_t in_bytes, void *const host_out[MAX_OUT], const size_t out_bytes[MAX_OUT], Run &&run)
    {
        cudaStream_t s_in = dev.aux_stream(0), s_out = dev.aux_stream(1), s_run = dev.stream();
        void *din[2] = {nullptr, nullptr}, *dout[2][MAX_OUT] = {{nullptr, nullptr}, {nullptr, nullptr}};
        cudaEvent_t in_done[2], run_done[2], out_done[2], start;
        for (int b = 0; b < 2; ++b) {
            din[b] = dev.alloc(chunk_items * in_bytes);
            for (int k = 0; k < MAX_OUT; ++k)
                if (host_out[k]) dout[b][k] = dev.alloc(chunk_items * out_bytes[k]);
            VQB_CUDA_CHECK(cudaEventCreateWithFlags(&in_done[b], cudaEventDisableTiming));
            VQB_CUDA_CHECK(cudaEventCreateWithFlags(&run_done[b], cudaEventDisableTiming));
            VQB_CUDA_CHECK(cudaEventCreateWithFlags(&out_done[b], cudaEventDisableTiming));
        }
        VQB_CUDA_CHECK(cudaEventCreateWithFlags(&start, cudaEventDisableTiming));
        VQB_CUDA_CHECK(cudaEventRecord(start, s_run)); // the buffers were allocated in s_run's order
        VQB_CUDA_CHECK(cudaStreamWaitEvent(s_in, start, 0));
        VQB_CUDA_CHECK(cudaStreamWaitEvent(s_out, start, 0));
        size_t c = 0;
        for (size_t off = 0; off < n_items; off += chunk_items, ++c) {
            const int b = (int)(c & 1);
            const size_t items = std::min(chunk_items, n_items - off);
            if (c >= 2) VQB_CUDA_CHECK(cudaStreamWaitEvent(s_in, run_done[b], 0)); // slot b's input was consumed
            VQB_CUDA_CHECK(cudaMemcpyAsync(din[b], (const char *)host_in + off * in_bytes, items * in_bytes, cudaMemcpyHostToDevice, s_in));
            VQB_CUDA_CHECK(cudaEventRecord(in_done[b], s_in));
            VQB_CUDA_CHECK(cudaStreamWaitEvent(s_run, in_done[b], 0));
            if (c >= 2) VQB_CUDA_CHECK(cudaStreamWaitEvent(s_run, out_done[b], 0)); // slot b's outputs were downloaded
            void *outs[MAX_OUT] = {dout[b][0], dout[b][1]};
            run(din[b], items, outs);
            VQB_CUDA_CHECK(cudaEventRecord(run_done[b], s_run));
            VQB_CUDA_CHECK(cudaStreamWaitEvent(s_out, run_done[b], 0));
            for (int k = 0; k < MAX_OUT; ++k)
                if (host_out[k])
                    VQB_CUDA_CHECK(cudaMemcpyAsync((char *)host_out[k] + off * out_bytes[k], dout[b][k], items * out_bytes[k],
                                                   cudaMemcpyDeviceToHost, s_out));
            VQB_CUDA_CHECK(cudaEventRecord(out_done[b], s_out));
        }
        // everything the caller waits for goes through s_run: it joins the copy streams, then the host waits once
        for (int b = 0; b < 2; ++b) {
            if (c > (size_t)b) VQB_CUDA_CHECK(cudaStreamWaitEvent(s_run, out_done[b], 0));
        }
        VQB_CUDA_CHECK(cudaStreamSynchronize(s_run));
        for (int b = 0; b < 2; ++b) {
            dev.release(din[b]);
            for (int k = 0; k < MAX_OUT; ++k) dev.release(dout[b][k]);
            cudaEventDestroy(in_done[b]);
            cudaEventDestroy(run_done[b]);
            cudaEventDestroy(out_done[b]);
        }
        cudaEventDestroy(start);
    }
};

void check_minkowski(int metric, double p)
{
    if (metric == VQB_MINKOWSKI && p <= 0.0) // src/distances.rs:155-163
        throw Error(VQB_ERR_INVALID_METRIC_PARAMETER, "Invalid metric parameter for Minkowski: p must be positive");
}

std::string dim_mismatch(size_t expected, size_t found)
{
    return "Dimension mismatch: expected " + std::to_string(expected) + ", got " + std::to_string(found);
}

} // namespace

namespace vqb {
OpqParts opq_parts(vqb_opq *oq)
{
    OpqParts v;
    v.dev = oq->ctx->dev.get();
    v.mu = &oq->ctx->mu;
    v.err = &oq->ctx->err;
    v.rotation = oq->rotation_d;
    v.codebooks = oq->codebooks;
    v.m = oq->m;
    v.k = oq->k;
    v.sd = oq->sd;
    v.dim = oq->dim;
    v.metric = oq->metric;
    v.p = oq->p;
    v.empty = oq->empty;
    return v;
}
} // namespace vqb

extern "C" {

const char *vqb_version(void) { return "vqb 0.1 (sm_100a)"; }

int vqb_ctx_create(int device, vqb_ctx **out)
{
    if (!out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "out is NULL");
    *out = nullptr;
    vqb_ctx *ctx = nullptr;
    int rc = guarded(nullptr, [&] {
        std::unique_ptr<vqb_ctx> c(new vqb_ctx);
        c->dev.reset(new CudaDevice(device));
        ctx = c.release();
    });
    if (rc == VQB_OK) *out = ctx;
    return rc;
}

int vqb_ctx_destroy(vqb_ctx *ctx)
{
    if (!ctx) return VQB_OK;
    try {
        ctx->dev->make_current();
        ctx->dev->synchronize();
    } catch (...) {
    }
    ctx->comm.reset();
    delete ctx;
    return VQB_OK;
}

const char *vqb_last_error(const vqb_ctx *ctx) { return ctx ? ctx->err.c_str() : g_err.c_str(); }

int vqb_ctx_set_stream(vqb_ctx *ctx, void *cuda_stream)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->dev->set_stream(static_cast<cudaStream_t>(cuda_stream));
    return VQB_OK;
}

int vqb_ctx_reset_stream(vqb_ctx *ctx)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->dev->reset_stream();
    return VQB_OK;
}

int vqb_ctx_synchronize(vqb_ctx *ctx)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] { ctx->dev->synchronize(); });
}

int vqb_ctx_launch_count(const vqb_ctx *ctx, uint64_t *out)
{
    if (!ctx || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = ctx->dev->launches();
    return VQB_OK;
}

int vqb_ctx_alloc_count(const vqb_ctx *ctx, uint64_t *out)
{
    if (!ctx || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = ctx->dev->device_allocs();
    return VQB_OK;
}

int vqb_ctx_timing(vqb_ctx *ctx, int enable)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] { ctx->dev->set_timing(enable != 0); });
}

int vqb_ctx_timing_report(vqb_ctx *ctx, char *buf, size_t cap)
{
    if (!ctx || !buf || cap == 0) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        std::string r = ctx->dev->timing_report();
        if (r.size() + 1 > cap) throw Error(VQB_ERR_BAD_ARGUMENT, "report buffer too small");
        std::memcpy(buf, r.c_str(), r.size() + 1);
    });
}

int vqb_comm_unique_id(uint8_t *out)
{
    if (!out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "out is NULL");
    return guarded(nullptr, [&] { nccl_unique_id(out); });
}

int vqb_comm_init(vqb_ctx *ctx, const uint8_t *unique_id, int rank, int world)
{
    if (!ctx || !unique_id) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    if (world < 1 || rank < 0 || rank >= world) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "rank/world out of range");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        ctx->comm.reset();
        ctx->comm.reset(make_nccl_comm(*ctx->dev, unique_id, rank, world));
    });
}

int vqb_comm_exchange_count(const vqb_ctx *ctx, uint64_t *out)
{
    if (!ctx || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = ctx->comm ? ctx->comm->peer_exchanges() : 0;
    return VQB_OK;
}

int vqb_comm_destroy(vqb_ctx *ctx)
{
    if (!ctx) return VQB_OK;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        ctx->dev->synchronize();
        ctx->comm.reset();
    });
}

int vqb_distance_rows(vqb_ctx *ctx, int metric, double p, const float *a, size_t da, const float *b, size_t db, size_t n,
                      float *out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        if (da != db) throw Error(VQB_ERR_DIMENSION_MISMATCH, dim_mismatch(da, db)); // src/distances.rs:119-127
        check_minkowski(metric, p);
        if (n == 0) return;
        if (!a || !b || !out) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL data pointer");
        CudaDevice &dev = *ctx->dev;
        In ia(dev, a, sizeof(float) * n * da), ib(dev, b, sizeof(float) * n * da);
        Out o(dev, out, sizeof(float) * n);
        dev.distance_rows(metric, p, ia.as<float>(), ib.as<float>(), da, n, o.as<float>());
        o.finish();
    });
}

int vqb_tsvq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t max_depth, int metric, double p, vqb_tsvq **out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!out) throw Error(VQB_ERR_BAD_ARGUMENT, "out is NULL");
        *out = nullptr;
        if (metric < 0 || metric > 6) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        if (n == 0 || dim == 0) throw Error(VQB_ERR_EMPTY_INPUT, "Empty input: at least one vector is required."); // src/tsvq.rs:206-208
        if (!x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        In ix(dev, x, sizeof(float) * n * dim);
        std::unique_ptr<vqb_tsvq> t(new vqb_tsvq{ctx, metric, p, TsvqTree{}});
        tsvq_fit(dev, ix.as<float>(), n, dim, max_depth, t->tree);
        *out = t.release();
    });
}

int vqb_tsvq_quantize(vqb_tsvq *t, const float *x, size_t n, size_t dim, uint16_t *out_f16, uint32_t *leaf_out)
{
    if (!t) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "tsvq is NULL");
    vqb_ctx *ctx = t->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (dim != t->tree.dim) throw Error(VQB_ERR_DIMENSION_MISMATCH, dim_mismatch(t->tree.dim, dim)); // src/tsvq.rs:232-240
        if (n == 0) return;
        if (!x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        check_minkowski(t->metric, t->p);
        CudaDevice &dev = *ctx->dev;
        In ix(dev, x, sizeof(float) * n * dim);
        Out of(dev, out_f16, sizeof(uint16_t) * n * dim), ol(dev, leaf_out, sizeof(uint32_t) * n);
        tsvq_quantize(dev, t->tree, t->metric, t->p, ix.as<float>(), n, of.as<uint16_t>(), ol.as<uint32_t>());
        of.finish();
        ol.finish();
    });
}

int vqb_tsvq_shape(const vqb_tsvq *t, size_t *nodes, size_t *dim)
{
    if (!t) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "tsvq is NULL");
    if (nodes) *nodes = t->tree.nodes;
    if (dim) *dim = t->tree.dim;
    return VQB_OK;
}

int vqb_tsvq_tree(const vqb_tsvq *t, float *centroids_out, int32_t *left_out, int32_t *right_out)
{
    if (!t) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "tsvq is NULL");
    vqb_ctx *ctx = t->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (centroids_out) {
            const size_t bytes = sizeof(float) * t->tree.nodes * t->tree.dim;
            if (ctx->dev->is_device_pointer(centroids_out)) ctx->dev->copy(centroids_out, t->tree.centroids, bytes);
            else ctx->dev->download(centroids_out, t->tree.centroids, bytes);
        }
        if (left_out) std::memcpy(left_out, t->tree.h_left.data(), sizeof(int32_t) * t->tree.nodes);
        if (right_out) std::memcpy(right_out, t->tree.h_right.data(), sizeof(int32_t) * t->tree.nodes);
    });
}

int vqb_tsvq_destroy(vqb_tsvq *t)
{
    if (!t) return VQB_OK;
    vqb_ctx *ctx = t->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    guarded(ctx, [&] { tsvq_release(*ctx->dev, t->tree); });
    delete t;
    return VQB_OK;
}

int vqb_evaluate_f16(vqb_ctx *ctx, const float *x, const uint16_t *q_f16, size_t n, size_t dim, size_t k, float *mse_out,
                     float *recall_out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!x || !q_f16 || !mse_out || !recall_out) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL argument");
        CudaDevice &dev = *ctx->dev;
        In ix(dev, x, sizeof(float) * n * dim), iq(dev, q_f16, sizeof(uint16_t) * n * dim);
        dev.evaluate_f16(ix.as<float>(), iq.as<uint16_t>(), n, dim, k, mse_out, recall_out);
    });
}

int vqb_dense_dots(vqb_ctx *ctx, const float *x, size_t n, size_t dim, const float *codebook, size_t k, float *dots_out,
                   unsigned long long *stats_out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!x || !codebook || !stats_out || n == 0) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL or empty argument");
        CudaDevice &dev = *ctx->dev;
        In ix(dev, x, sizeof(float) * n * dim), ic(dev, codebook, sizeof(float) * k * dim);
        Out od(dev, dots_out, sizeof(float) * n * 256);
        dev.dense_debug(ix.as<float>(), n, dim, ic.as<float>(), k, od.as<float>(), stats_out);
        od.finish();
    });
}

int vqb_pq_tensor_scores(vqb_ctx *ctx, const float *x, size_t n, size_t m, const float *codebooks, size_t k, float *scores_out,
                         uint32_t *codes_out, unsigned long long *marked_out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!x || !codebooks || !codes_out || !marked_out || n == 0) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL or empty argument");
        CudaDevice &dev = *ctx->dev;
        In ix(dev, x, sizeof(float) * n * m * 8), ic(dev, codebooks, sizeof(float) * m * k * 8);
        Out os(dev, scores_out, scores_out ? sizeof(float) * n * m * 256 : 0), oc(dev, codes_out, sizeof(uint32_t) * n * m);
        dev.pq_tensor_debug(ix.as<float>(), n, m, ic.as<float>(), k, scores_out ? os.as<float>() : nullptr, oc.as<uint32_t>(), marked_out);
        os.finish();
        oc.finish();
    });
}

int vqb_opq_rotate_rows(vqb_ctx *ctx, const float *rot, size_t dim, const float *x, size_t n, float *y_out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!rot || !x || !y_out || n == 0 || dim == 0) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL or empty argument");
        CudaDevice &dev = *ctx->dev;
        In ir(dev, rot, sizeof(float) * dim * dim), ix(dev, x, sizeof(float) * n * dim);
        Out oy(dev, y_out, sizeof(float) * n * dim);
        dev.rotate_rows(ir.as<float>(), dim, ix.as<float>(), n, oy.as<float>());
        oy.finish();
        dev.synchronize();
    });
}

int vqb_opq_cross_cov(vqb_ctx *ctx, const float *y, const float *x, size_t n, size_t dim, double *a_out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!y || !x || !a_out || n == 0 || dim == 0) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL or empty argument");
        CudaDevice &dev = *ctx->dev;
        In iy(dev, y, sizeof(float) * n * dim), ix(dev, x, sizeof(float) * n * dim);
        Out oa(dev, a_out, sizeof(double) * dim * dim);
        dev.cross_cov(iy.as<float>(), ix.as<float>(), n, dim, oa.as<double>());
        oa.finish();
        dev.synchronize();
    });
}

int vqb_lbg_fit(vqb_ctx *ctx, const float *x, size_t n, size_t d, size_t k, size_t max_iters, const uint64_t *init_idx,
                vqb_draw_fn draw, void *user, int flags, float *centroids_out, size_t *iterations_out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        CudaDevice &dev = *ctx->dev;
        if (n && !x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        In ix(dev, x, sizeof(float) * n * d);
        Shape sh;
        sh.n_local = n;
        sh.ld = d;
        sh.m = 1;
        sh.sd = d;
        sh.k = k;
        Out o(dev, centroids_out, sizeof(float) * k * d);
        float *cd = o.as<float>();
        void *tmp = nullptr;
        if (!cd) tmp = cd = (float *)dev.alloc(sizeof(float) * k * d);
        size_t it = 0;
        try {
            lbg_fit(dev, ctx->comm.get(), sh, ix.as<float>(), max_iters, init_idx, draw, user, 0, flags, cd, &it);
        } catch (...) {
            dev.release(tmp);
            throw;
        }
        dev.release(tmp);
        if (iterations_out) *iterations_out = it;
        o.finish();
    });
}

// ---- PQ ----------------------------------------------------------------------------------------

int vqb_pq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t m, size_t k, size_t max_iters, int metric,
               double p, const uint64_t *init_idx, vqb_draw_fn draw, void *user, int flags, vqb_pq **out)
{
    if (!ctx || !out) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        const bool multi = ctx->comm && ctx->comm->world() > 1;
        if (n == 0 && !multi) // src/pq.rs:87-89
            throw Error(VQB_ERR_EMPTY_INPUT, "Empty input: at least one vector is required.");
        if (m == 0) throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: m must be greater than 0");
        if (dim < m) // 91-96
            throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: Data dimension must be at least m");
        if (dim % m != 0) // 97-102
            throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: Data dimension must be divisible by m");
        if (n && !x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        std::unique_ptr<vqb_pq> pq(new vqb_pq);
        pq->ctx = ctx;
        pq->m = m;
        pq->k = k;
        pq->sd = dim / m;
        pq->metric = metric;
        pq->p = p;
        pq->iters.assign(m, 0);
        pq->codebooks = (float *)dev.alloc(sizeof(float) * m * k * pq->sd);
        try {
            RowsIn ix(dev, x, n, dim);
            Shape sh;
            sh.n_local = n;
            sh.ld = dim;
            sh.m = m;
            sh.sd = pq->sd;
            sh.k = k;
            lbg_fit(dev, ctx->comm.get(), sh, ix.d, max_iters, init_idx, draw, user, 0, flags, pq->codebooks,
                    pq->iters.data());
            dev.synchronize();
        } catch (...) {
            dev.release(pq->codebooks);
            throw;
        }
        *out = pq.release();
    });
}

int vqb_pq_from_codebooks(vqb_ctx *ctx, const float *codebooks, size_t m, size_t k, size_t sub_dim, int metric, double p,
                          vqb_pq **out)
{
    if (!ctx || !out) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        if (!codebooks || m == 0 || k == 0 || sub_dim == 0) throw Error(VQB_ERR_BAD_ARGUMENT, "empty codebooks");
        CudaDevice &dev = *ctx->dev;
        std::unique_ptr<vqb_pq> pq(new vqb_pq);
        pq->ctx = ctx;
        pq->m = m;
        pq->k = k;
        pq->sd = sub_dim;
        pq->metric = metric;
        pq->p = p;
        pq->iters.assign(m, 0);
        const size_t bytes = sizeof(float) * m * k * sub_dim;
        pq->codebooks = (float *)dev.alloc(bytes);
        if (dev.is_device_pointer(codebooks)) dev.copy(pq->codebooks, codebooks, bytes);
        else dev.upload(pq->codebooks, codebooks, bytes);
        dev.synchronize();
        *out = pq.release();
    });
}

int vqb_pq_quantize(vqb_pq *pq, const float *x, size_t n, size_t dim, uint16_t *out_f16, uint32_t *codes)
{
    if (!pq) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "pq is NULL");
    vqb_ctx *ctx = pq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        const size_t full = pq->m * pq->sd;
        if (dim != full) throw Error(VQB_ERR_DIMENSION_MISMATCH, dim_mismatch(full, dim)); // src/pq.rs:147-156
        check_minkowski(pq->metric, pq->p);
        if (n == 0) return;
        if (!x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        Shape sh;
        sh.n_local = n;
        sh.ld = dim;
        sh.m = pq->m;
        sh.sd = pq->sd;
        sh.k = pq->k;
        const size_t chunk_rows = 1u << 16;
        const bool all_host = !dev.is_device_pointer(x) && (!out_f16 || !dev.is_device_pointer(out_f16)) &&
                              (!codes || !dev.is_device_pointer(codes)) && (out_f16 || codes);
        if (all_host && n >= 2 * chunk_rows) {
            // large host batch (the loop of src/bin/eval_pq.rs:51-59 in one call): chunked copy / encode / copy pipeline
            HostPipeline pipe(dev, chunk_rows);
            void *const outs[2] = {out_f16, codes};
            const size_t ob[2] = {sizeof(uint16_t) * dim, sizeof(uint32_t) * pq->m};
            pipe.go(x, n, sizeof(float) * dim, outs, ob, [&](void *din, size_t rows, void *const *dout) {
                Shape c = sh;
                c.n_local = rows;
                dev.pq_encode(c, (const float *)din, pq->codebooks, pq->metric, pq->p, (uint16_t *)dout[0], (uint32_t *)dout[1], nullptr);
            });
            return;
        }
        In ix(dev, x, sizeof(float) * n * dim);
        Out of(dev, out_f16, sizeof(uint16_t) * n * dim), oc(dev, codes, sizeof(uint32_t) * n * pq->m);
        dev.pq_encode(sh, ix.as<float>(), pq->codebooks, pq->metric, pq->p, of.as<uint16_t>(), oc.as<uint32_t>(), nullptr);
        of.finish();
        oc.finish();
    });
}

int vqb_pq_shape(const vqb_pq *pq, size_t *m, size_t *k, size_t *sub_dim)
{
    if (!pq) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "pq is NULL");
    if (m) *m = pq->m;
    if (k) *k = pq->k;
    if (sub_dim) *sub_dim = pq->sd;
    return VQB_OK;
}

int vqb_pq_codebooks(const vqb_pq *pq, float *out)
{
    if (!pq || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    vqb_ctx *ctx = pq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        const size_t bytes = sizeof(float) * pq->m * pq->k * pq->sd;
        if (ctx->dev->is_device_pointer(out)) ctx->dev->copy(out, pq->codebooks, bytes);
        else ctx->dev->download(out, pq->codebooks, bytes);
    });
}

int vqb_pq_iterations(const vqb_pq *pq, size_t *out)
{
    if (!pq || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    for (size_t s = 0; s < pq->m; ++s) out[s] = pq->iters[s];
    return VQB_OK;
}

int vqb_pq_destroy(vqb_pq *pq)
{
    if (!pq) return VQB_OK;
    vqb_ctx *ctx = pq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    guarded(ctx, [&] { ctx->dev->release(pq->codebooks); });
    delete pq;
    return VQB_OK;
}

// ---- RVQ ---------------------------------------------------------------------------------------

int vqb_rvq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t stages, size_t k, size_t max_iters,
                float epsilon, int metric, double p, vqb_init_fn init, vqb_draw_fn draw, void *user, int flags,
                vqb_rvq **out)
{
    if (!ctx || !out) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        const bool multi = ctx->comm && ctx->comm->world() > 1;
        if (n == 0 && !multi) // src/rvq.rs:96-98
            throw Error(VQB_ERR_EMPTY_INPUT, "Empty input: at least one vector is required.");
        if (n && !x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        std::unique_ptr<vqb_rvq> rq(new vqb_rvq);
        rq->ctx = ctx;
        rq->stages = 0;
        rq->k = k;
        rq->dim = dim;
        rq->epsilon = epsilon;
        rq->metric = metric;
        rq->p = p;
        rq->codebooks = (float *)dev.alloc(sizeof(float) * stages * k * dim);
        float *res = (float *)dev.alloc(sizeof(float) * n * dim); // src/rvq.rs:103
        try {
            const size_t bytes = sizeof(float) * n * dim;
            if (bytes) {
                if (dev.is_device_pointer(x)) dev.copy(res, x, bytes);
                else dev.upload(res, x, bytes);
            }
            rq->stages = rvq_fit(dev, ctx->comm.get(), res, n, dim, stages, k, max_iters, epsilon, metric, p, init, draw,
                                 user, flags, rq->codebooks);
            dev.synchronize();
        } catch (...) {
            dev.release(res);
            dev.release(rq->codebooks);
            throw;
        }
        dev.release(res);
        *out = rq.release();
    });
}

int vqb_rvq_from_codebooks(vqb_ctx *ctx, const float *codebooks, size_t stages, size_t k, size_t dim, float epsilon,
                           int metric, double p, vqb_rvq **out)
{
    if (!ctx || !out) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        if (dim == 0 || (stages > 0 && (k == 0 || !codebooks))) throw Error(VQB_ERR_BAD_ARGUMENT, "empty codebooks");
        CudaDevice &dev = *ctx->dev;
        std::unique_ptr<vqb_rvq> rq(new vqb_rvq);
        rq->ctx = ctx;
        rq->stages = stages;
        rq->k = k;
        rq->dim = dim;
        rq->epsilon = epsilon;
        rq->metric = metric;
        rq->p = p;
        const size_t bytes = sizeof(float) * stages * k * dim;
        rq->codebooks = (float *)dev.alloc(bytes);
        if (bytes) {
            if (dev.is_device_pointer(codebooks)) dev.copy(rq->codebooks, codebooks, bytes);
            else dev.upload(rq->codebooks, codebooks, bytes);
        }
        dev.synchronize();
        *out = rq.release();
    });
}

int vqb_rvq_quantize(vqb_rvq *rq, const float *x, size_t n, size_t dim, uint16_t *out_f16, uint32_t *codes)
{
    if (!rq) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "rvq is NULL");
    vqb_ctx *ctx = rq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (dim != rq->dim) throw Error(VQB_ERR_DIMENSION_MISMATCH, dim_mismatch(rq->dim, dim)); // src/rvq.rs:172-180
        if (rq->stages > 0 && rq->k >= 2) check_minkowski(rq->metric, rq->p);
        if (n == 0) return;
        if (!x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        Out of(dev, out_f16, sizeof(uint16_t) * n * dim), oc(dev, codes, sizeof(uint32_t) * n * rq->stages);
        if (rq->stages == 0) { // no codebooks: the sum stays zero (src/rvq.rs:182-183,209-213)
            if (of.d) dev.zero(of.d, sizeof(uint16_t) * n * dim);
        } else {
            In ix(dev, x, sizeof(float) * n * dim);
            dev.rvq_quantize(ix.as<float>(), n, dim, rq->codebooks, rq->stages, rq->k, rq->epsilon, rq->metric, rq->p,
                             of.as<uint16_t>(), oc.as<uint32_t>());
        }
        of.finish();
        oc.finish();
    });
}

int vqb_rvq_shape(const vqb_rvq *rq, size_t *stages, size_t *k, size_t *dim)
{
    if (!rq) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "rvq is NULL");
    if (stages) *stages = rq->stages;
    if (k) *k = rq->k;
    if (dim) *dim = rq->dim;
    return VQB_OK;
}

int vqb_rvq_codebooks(const vqb_rvq *rq, float *out)
{
    if (!rq || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    vqb_ctx *ctx = rq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        const size_t bytes = sizeof(float) * rq->stages * rq->k * rq->dim;
        if (ctx->dev->is_device_pointer(out)) ctx->dev->copy(out, rq->codebooks, bytes);
        else ctx->dev->download(out, rq->codebooks, bytes);
    });
}

int vqb_rvq_destroy(vqb_rvq *rq)
{
    if (!rq) return VQB_OK;
    vqb_ctx *ctx = rq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    guarded(ctx, [&] { ctx->dev->release(rq->codebooks); });
    delete rq;
    return VQB_OK;
}

// ---- OPQ ---------------------------------------------------------------------------------------

int vqb_opq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t m, size_t k, size_t max_iters,
                size_t opq_iters, int metric, double p, const uint64_t *init_idx, vqb_draw_fn draw,
                vqb_restart_fn restart, void *user, int flags, vqb_opq **out)
{
    if (!ctx || !out) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        const bool multi = ctx->comm && ctx->comm->world() > 1;
        if (n == 0 && !multi) // src/opq.rs:99-101
            throw Error(VQB_ERR_EMPTY_INPUT, "Empty input: at least one vector is required.");
        if (m == 0) throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: m must be greater than 0");
        if (dim < m) // 103-108
            throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: Dimension must be at least m");
        if (dim % m != 0) // 109-114
            throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: Dimension must be divisible by m");
        if (n && !x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        std::unique_ptr<vqb_opq> oq(new vqb_opq);
        oq->ctx = ctx;
        oq->m = m;
        oq->k = k;
        oq->sd = dim / m;
        oq->dim = dim;
        oq->metric = metric;
        oq->p = p;
        oq->rotation.assign(dim * dim, 0.0f);
        oq->codebooks = (float *)dev.alloc(sizeof(float) * m * k * oq->sd);
        oq->rotation_d = (float *)dev.alloc(sizeof(float) * dim * dim);
        try {
            In ix(dev, x, sizeof(float) * n * dim);
            bool trained = opq_fit(dev, ctx->comm.get(), ix.as<float>(), n, dim, m, k, max_iters, opq_iters, metric, p,
                                   init_idx, draw, restart, user, flags, oq->rotation.data(), oq->codebooks);
            oq->empty = !trained;
            dev.upload(oq->rotation_d, oq->rotation.data(), sizeof(float) * dim * dim);
            dev.synchronize();
        } catch (...) {
            dev.release(oq->codebooks);
            dev.release(oq->rotation_d);
            throw;
        }
        *out = oq.release();
    });
}

int vqb_opq_from_parts(vqb_ctx *ctx, const float *rotation, const float *codebooks, size_t m, size_t k, size_t sub_dim,
                       int metric, double p, vqb_opq **out)
{
    if (!ctx || !out) return set_err(ctx, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (!metric_ok(metric)) throw Error(VQB_ERR_BAD_ARGUMENT, "unknown metric");
        if (!rotation || !codebooks || m == 0 || k == 0 || sub_dim == 0) throw Error(VQB_ERR_BAD_ARGUMENT, "empty parts");
        CudaDevice &dev = *ctx->dev;
        const size_t dim = m * sub_dim;
        std::unique_ptr<vqb_opq> oq(new vqb_opq);
        oq->ctx = ctx;
        oq->m = m;
        oq->k = k;
        oq->sd = sub_dim;
        oq->dim = dim;
        oq->metric = metric;
        oq->p = p;
        oq->empty = false;
        oq->rotation.assign(dim * dim, 0.0f);
        oq->codebooks = (float *)dev.alloc(sizeof(float) * m * k * sub_dim);
        oq->rotation_d = (float *)dev.alloc(sizeof(float) * dim * dim);
        if (dev.is_device_pointer(rotation)) dev.download(oq->rotation.data(), rotation, sizeof(float) * dim * dim);
        else std::memcpy(oq->rotation.data(), rotation, sizeof(float) * dim * dim);
        dev.upload(oq->rotation_d, oq->rotation.data(), sizeof(float) * dim * dim);
        const size_t bytes = sizeof(float) * m * k * sub_dim;
        if (dev.is_device_pointer(codebooks)) dev.copy(oq->codebooks, codebooks, bytes);
        else dev.upload(oq->codebooks, codebooks, bytes);
        dev.synchronize();
        *out = oq.release();
    });
}

int vqb_opq_quantize(vqb_opq *oq, const float *x, size_t n, size_t dim, uint16_t *out_f16, uint32_t *codes)
{
    if (!oq) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "opq is NULL");
    vqb_ctx *ctx = oq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (dim != oq->dim) throw Error(VQB_ERR_DIMENSION_MISMATCH, dim_mismatch(oq->dim, dim)); // src/opq.rs:223-231
        if (oq->empty) return; // no codebooks: the reference returns an empty vector (src/opq.rs:244-263)
        check_minkowski(oq->metric, oq->p);
        if (n == 0) return;
        if (!x) throw Error(VQB_ERR_BAD_ARGUMENT, "x is NULL");
        CudaDevice &dev = *ctx->dev;
        In ix(dev, x, sizeof(float) * n * dim);
        Out of(dev, out_f16, sizeof(uint16_t) * n * dim), oc(dev, codes, sizeof(uint32_t) * n * oq->m);
        float *y = (float *)dev.alloc(sizeof(float) * n * dim);
        try {
            dev.rotate_rows(oq->rotation_d, dim, ix.as<float>(), n, y); // 232-234
            Shape sh;
            sh.n_local = n;
            sh.ld = dim;
            sh.m = oq->m;
            sh.sd = oq->sd;
            sh.k = oq->k;
            dev.pq_encode(sh, y, oq->codebooks, oq->metric, oq->p, of.as<uint16_t>(), oc.as<uint32_t>(), nullptr);
        } catch (...) {
            dev.release(y);
            throw;
        }
        dev.release(y);
        of.finish();
        oc.finish();
    });
}

int vqb_opq_shape(const vqb_opq *oq, size_t *m, size_t *k, size_t *sub_dim)
{
    if (!oq) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "opq is NULL");
    if (m) *m = oq->empty ? 0 : oq->m;
    if (k) *k = oq->k;
    if (sub_dim) *sub_dim = oq->sd;
    return VQB_OK;
}

int vqb_opq_rotation(const vqb_opq *oq, float *out)
{
    if (!oq || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    vqb_ctx *ctx = oq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        const size_t bytes = sizeof(float) * oq->dim * oq->dim;
        if (ctx->dev->is_device_pointer(out)) ctx->dev->copy(out, oq->rotation_d, bytes);
        else std::memcpy(out, oq->rotation.data(), bytes);
    });
}

int vqb_opq_codebooks(const vqb_opq *oq, float *out)
{
    if (!oq || !out) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "NULL argument");
    vqb_ctx *ctx = oq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (oq->empty) return;
        const size_t bytes = sizeof(float) * oq->m * oq->k * oq->sd;
        if (ctx->dev->is_device_pointer(out)) ctx->dev->copy(out, oq->codebooks, bytes);
        else ctx->dev->download(out, oq->codebooks, bytes);
    });
}

int vqb_opq_destroy(vqb_opq *oq)
{
    if (!oq) return VQB_OK;
    vqb_ctx *ctx = oq->ctx;
    std::lock_guard<std::mutex> lk(ctx->mu);
    guarded(ctx, [&] {
        ctx->dev->release(oq->codebooks);
        ctx->dev->release(oq->rotation_d);
    });
    delete oq;
    return VQB_OK;
}

// ---- SQ / BQ -----------------------------------------------------------------------------------

int vqb_sq_fit(float min, float max, size_t levels, float *step_out)
{
    if (max <= min) return set_err(nullptr, VQB_ERR_INVALID_PARAMETER, "Invalid parameter: max must be greater than min");
    if (levels < 2) return set_err(nullptr, VQB_ERR_INVALID_PARAMETER, "Invalid parameter: levels must be at least 2");
    if (levels > 256) return set_err(nullptr, VQB_ERR_INVALID_PARAMETER, "Invalid parameter: levels must be no more than 256");
    if (step_out) *step_out = (max - min) / (float)(levels - 1); // src/sq.rs:69
    return VQB_OK;
}

int vqb_sq_quantize(vqb_ctx *ctx, float min, float max, size_t levels, float step, const float *x, size_t n_elems,
                    uint8_t *out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (levels < 2 || levels > 256) throw Error(VQB_ERR_INVALID_PARAMETER, "Invalid parameter: levels must be between 2 and 256");
        if (n_elems == 0) return;
        if (!x || !out) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL data pointer");
        CudaDevice &dev = *ctx->dev;
        const size_t chunk = 1u << 23; // 8 Mi values = 32 MiB in, 8 MiB out
        if (!dev.is_device_pointer(x) && !dev.is_device_pointer(out) && n_elems >= 2 * chunk) {
            HostPipeline pipe(dev, chunk);
            void *const outs[2] = {out, nullptr};
            const size_t ob[2] = {1, 0};
            pipe.go(x, n_elems, sizeof(float), outs, ob, [&](void *din, size_t items, void *const *dout) {
                dev.sq_quantize(min, max, levels, step, (const float *)din, items, (uint8_t *)dout[0]);
            });
            return;
        }
        In ix(dev, x, sizeof(float) * n_elems);
        Out o(dev, out, n_elems);
        dev.sq_quantize(min, max, levels, step, ix.as<float>(), n_elems, o.as<uint8_t>());
        o.finish();
    });
}

int vqb_bq_fit(float threshold, uint8_t low, uint8_t high)
{
    (void)threshold;
    if (low >= high)
        return set_err(nullptr, VQB_ERR_INVALID_PARAMETER,
                       "Invalid parameter: Low quantization level must be less than high quantization level");
    return VQB_OK;
}

int vqb_bq_quantize(vqb_ctx *ctx, float threshold, uint8_t low, uint8_t high, const float *x, size_t n_elems, uint8_t *out)
{
    if (!ctx) return set_err(nullptr, VQB_ERR_BAD_ARGUMENT, "ctx is NULL");
    std::lock_guard<std::mutex> lk(ctx->mu);
    return guarded(ctx, [&] {
        if (n_elems == 0) return;
        if (!x || !out) throw Error(VQB_ERR_BAD_ARGUMENT, "NULL data pointer");
        CudaDevice &dev = *ctx->dev;
        const size_t chunk = 1u << 23;
        if (!dev.is_device_pointer(x) && !dev.is_device_pointer(out) && n_elems >= 2 * chunk) {
            HostPipeline pipe(dev, chunk);
            void *const outs[2] = {out, nullptr};
            const size_t ob[2] = {1, 0};
            pipe.go(x, n_elems, sizeof(float), outs, ob, [&](void *din, size_t items, void *const *dout) {
                dev.bq_quantize(threshold, low, high, (const float *)din, items, (uint8_t *)dout[0]);
            });
            return;
        }
        In ix(dev, x, sizeof(float) * n_elems);
        Out o(dev, out, n_elems);
        dev.bq_quantize(threshold, low, high, ix.as<float>(), n_elems, o.as<uint8_t>());
        o.finish();
    });
}

} // extern "C"
