// cuda_device.cu -- sm_100a implementation of vqb::Device: centroid accumulation and update, row
// patches, rotation / cross-covariance for OPQ, row-wise distances and the element-wise quantizers.
// The nearest-centroid kernels live in assign_reg.cuh / assign_generic.cuh (launched from assign_launch.cu).
#include "cuda_device.hpp"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <vector>

#include <cstdlib>

#include "assign_generic.cuh"
#include "assign_reg.cuh"
#include "dense_tc.hpp"
#include "opq_tc.hpp"
#include "pq_tc.hpp"
#include "kernels_common.cuh"

namespace vqb {

// ------------------------------------------------------------------------------------------------
// context plumbing
// ------------------------------------------------------------------------------------------------
CudaDevice::CudaDevice(int device) : device_(device)
{
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        throw Error(102, std::string("no CUDA device available: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
    if (device < 0 || device >= count) throw Error(102, "CUDA device index out of range");
    VQB_CUDA_CHECK(cudaSetDevice(device));
    cudaDeviceProp prop;
    VQB_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        throw Error(102, std::string("this library contains sm_100a code only; device is ") + prop.name);
    sm_count_ = prop.multiProcessorCount;
    smem_limit_ = prop.sharedMemPerBlockOptin;
    VQB_CUDA_CHECK(cudaStreamCreateWithFlags(&own_stream_, cudaStreamNonBlocking));
    stream_ = own_stream_;
    ++device_allocs_;
    if (cudaHostAlloc(reinterpret_cast<void **>(&stage_), STAGE_BYTES, cudaHostAllocMapped) != cudaSuccess) {
        stage_ = nullptr; // pinned memory is an optimisation only
        cudaGetLastError();
    } else {
        VQB_CUDA_CHECK(cudaEventCreateWithFlags(&stage_event_, cudaEventDisableTiming));
        if (cudaHostGetDevicePointer(reinterpret_cast<void **>(&stage_dev_), stage_, 0) != cudaSuccess) {
            stage_dev_ = nullptr;
            cudaGetLastError();
        }
    }
    {
        const char *e = std::getenv("VQB_NO_TENSOR"); // VQB_NO_TENSOR=1: CUDA-core kernels only (A/B comparisons)
        tensor_enabled_ = !(e && *e && *e != '0');
        // The product quantizer's 8-wide sub-spaces run on the tcgen05 kernel of pq_tc.cu (about twice as fast as the
        // CUDA-core filter kernel); VQB_PQ_TENSOR=0 selects the filter kernel (A/B comparisons).
        const char *f = std::getenv("VQB_PQ_TENSOR");
        pq_tensor_enabled_ = tensor_enabled_ && !(f && *f == '0');
    }
    {
        const char *o = std::getenv("VQB_OPQ_TENSOR"); // 0: rotation and cross-covariance on the CUDA-core kernels (A/B comparisons)
        opq_tensor_enabled_ = tensor_enabled_ && !(o && *o == '0');
    }
    // the small fixed-size buffers of the tensor-core kernels exist from the start, so that no later call has to create them
    if (tensor_enabled_) ensure_tc_buffers(0);
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
        unsigned long long keep = ~0ull; // keep freed blocks cached; repeated fits reuse them
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
}

CudaDevice::~CudaDevice()
{
    if (own_stream_) {
        cudaSetDevice(device_);
        cudaStreamSynchronize(own_stream_);
        for (int i = 0; i < 2; ++i)
            if (aux_[i]) cudaStreamDestroy(aux_[i]);
        if (stage_event_) cudaEventDestroy(stage_event_);
        for (cudaEvent_t e : arrival_done_) cudaEventDestroy(e);
        if (arrival_fence_) cudaEventDestroy(arrival_fence_);
        if (stage_) cudaFreeHost(stage_);
        cudaFree(rownorm_);
        cudaFree(hn_scratch_);
        cudaFree(rot_split_);
        cudaFree(pq_scratch_);
        cudaFree(pq_marks_);
        cudaFree(cand_);
        cudaFree(list_);
        cudaFree(tc_stats_);
        cudaFree(tc_error_);
        if (status_host_) cudaFreeHost(status_host_);
        for (auto &sp : spans_) {
            event_pool_.push_back(sp.a);
            event_pool_.push_back(sp.b);
        }
        for (cudaEvent_t e : event_pool_) cudaEventDestroy(e);
        cudaStreamDestroy(own_stream_);
    }
}

void CudaDevice::set_timing(bool on)
{
    if (!on) {
        for (auto &sp : spans_) {
            event_pool_.push_back(sp.a);
            event_pool_.push_back(sp.b);
        }
        spans_.clear();
    }
    timing_ = on;
}

cudaEvent_t CudaDevice::take_event()
{
    if (!event_pool_.empty()) {
        cudaEvent_t e = event_pool_.back();
        event_pool_.pop_back();
        return e;
    }
    cudaEvent_t e;
    VQB_CUDA_CHECK(cudaEventCreate(&e));
    return e;
}

void CudaDevice::timing_begin(const char *name)
{
    Span sp;
    sp.name = name;
    sp.a = take_event();
    sp.b = take_event();
    VQB_CUDA_CHECK(cudaEventRecord(sp.a, stream_));
    spans_.push_back(sp);
}

void CudaDevice::timing_end()
{
    if (!spans_.empty()) cudaEventRecord(spans_.back().b, stream_);
}

std::string CudaDevice::timing_report()
{
    VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
    std::map<std::string, std::pair<uint64_t, double>> agg;
    for (auto &sp : spans_) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) {
            auto &e = agg[sp.name];
            e.first += 1;
            e.second += ms;
        }
        event_pool_.push_back(sp.a);
        event_pool_.push_back(sp.b);
    }
    spans_.clear();
    std::string out = "{";
    bool first = true;
    for (auto &kv : agg) {
        if (!first) out += ", ";
        first = false;
        out += "\"" + kv.first + "\": {\"launches\": " + std::to_string(kv.second.first) + ", \"ms\": " + std::to_string(kv.second.second) + "}";
    }
    return out + "}";
}

cudaStream_t CudaDevice::aux_stream(int i)
{
    if (!aux_[i]) VQB_CUDA_CHECK(cudaStreamCreateWithFlags(&aux_[i], cudaStreamNonBlocking));
    return aux_[i];
}

void CudaDevice::make_current() const { VQB_CUDA_CHECK(cudaSetDevice(device_)); }

// A tensor-core kernel whose bounded wait expired stops early and leaves a code in the error word; callers that pass device
// outputs never download anything, so this is where they learn of it.
void CudaDevice::synchronize()
{
    if (tc_error_) check_tc_error();
    else VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
}

bool CudaDevice::is_device_pointer(const void *p) const
{
    if (!p) return false;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

void *CudaDevice::alloc(size_t bytes)
{
    void *p = nullptr;
    ++device_allocs_;
    VQB_CUDA_CHECK(cudaMallocAsync(&p, bytes ? bytes : 1, stream_));
    return p;
}

void CudaDevice::release(void *p)
{
    if (p) cudaFreeAsync(p, stream_);
}

// Reads mapped host memory over the link; used for small uploads while a large copy occupies the copy engine.
__global__ void fetch_host_bytes_kernel(unsigned char *dst, const unsigned char *src, unsigned long long bytes)
{
    const unsigned long long t = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x;
    const bool words = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 3u) == 0;
    if (words) {
        if (4 * t + 4 <= bytes) reinterpret_cast<uint32_t *>(dst)[t] = reinterpret_cast<const uint32_t *>(src)[t];
        else
            for (unsigned long long b = 4 * t; b < bytes; ++b) dst[b] = src[b];
    } else {
        for (unsigned long long b = 4 * t; b < bytes && b < 4 * t + 4; ++b) dst[b] = src[b];
    }
}

void CudaDevice::upload(void *dst, const void *src, size_t bytes)
{
    if (!bytes) return;
    if (arrival_.dev && arrival_.awaited < arrival_.pieces && stage_dev_ && bytes <= STAGE_BYTES) {
        // Host-to-device copies run one after the other, so this one would wait for all the rows still arriving
        // (begin_arrival); a kernel fetches the bytes from the pinned staging buffer instead.
        std::memcpy(stage_, src, bytes);
        const unsigned long long threads = (bytes + 3) / 4;
        fetch_host_bytes_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream_>>>(static_cast<unsigned char *>(dst), stage_dev_, bytes);
        VQB_CUDA_CHECK(cudaGetLastError());
        VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
        return;
    }
    VQB_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream_));
    VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
}

// ------------------------------------------------------------------------------------------------
// Rows that arrive while the first iteration already works on them.  A fit that is handed a host buffer copies it in
// pieces on a helper stream; the first assignment pass waits piece by piece (lbg_fit), so that the copy, which takes about
// as long as nine iterations at PCIe speed, hides one of them.
// ------------------------------------------------------------------------------------------------
bool CudaDevice::begin_arrival(float *dst, const float *host, size_t n, size_t ld)
{
    end_arrival();
    static const bool whole = std::getenv("VQB_UPLOAD_WHOLE") != nullptr; // one copy ahead of everything, for comparison
    if (whole || n == 0 || ld == 0) return false;
    // at most 16 pieces, none below 8 MiB (a copy of that size still runs at the link's full rate), at least four of them
    const size_t min_rows = std::max<size_t>(1024, ((size_t(8) << 20) / (ld * sizeof(float)) + 1023) / 1024 * 1024);
    const size_t piece_rows = std::max(min_rows, ((n + 15) / 16 + 1023) / 1024 * 1024);
    const size_t pieces = (n + piece_rows - 1) / piece_rows;
    if (pieces < 4) return false;
    make_current();
    if (!arrival_fence_) VQB_CUDA_CHECK(cudaEventCreateWithFlags(&arrival_fence_, cudaEventDisableTiming));
    while (arrival_done_.size() < pieces) {
        cudaEvent_t e = nullptr;
        VQB_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        arrival_done_.push_back(e);
    }
    cudaStream_t up = aux_stream(0);
    // `dst` may be memory that earlier work of the working stream has just let go of
    VQB_CUDA_CHECK(cudaEventRecord(arrival_fence_, stream_));
    VQB_CUDA_CHECK(cudaStreamWaitEvent(up, arrival_fence_, 0));
    try {
        for (size_t i = 0; i < pieces; ++i) {
            const size_t r0 = i * piece_rows, rows = std::min(piece_rows, n - r0);
            VQB_CUDA_CHECK(cudaMemcpyAsync(dst + r0 * ld, host + r0 * ld, rows * ld * sizeof(float), cudaMemcpyHostToDevice, up));
            VQB_CUDA_CHECK(cudaEventRecord(arrival_done_[i], up));
        }
    } catch (...) {
        cudaStreamSynchronize(up); // the caller lets go of `dst`: no copy may still be writing to it
        throw;
    }
    arrival_.dev = dst;
    arrival_.host = host;
    arrival_.n = n;
    arrival_.ld = ld;
    arrival_.piece_rows = piece_rows;
    arrival_.pieces = pieces;
    arrival_.awaited = 0;
    return true;
}

void CudaDevice::end_arrival()
{
    // Nothing waited for the last pieces (an error, or a fit without iterations): the caller's buffer must not be read after
    // the call returns, and the working stream must not run ahead of the copies, so the host waits for them here.
    if (arrival_.dev && arrival_.awaited < arrival_.pieces) cudaStreamSynchronize(aux_[0]);
    arrival_ = Arrival();
}

size_t CudaDevice::arriving_pieces(const float *x)
{
    if (!arrival_.dev || x != arrival_.dev || arrival_.awaited == arrival_.pieces) return 0;
    if (arrival_.awaited == 0) return arrival_.pieces;
    // somebody stopped half way through the pieces: wait for the rest in one go
    VQB_CUDA_CHECK(cudaStreamWaitEvent(stream_, arrival_done_[arrival_.pieces - 1], 0));
    arrival_.awaited = arrival_.pieces;
    return 0;
}

size_t CudaDevice::await_piece(const float *x, size_t piece)
{
    if (!arrival_.dev || x != arrival_.dev || piece >= arrival_.pieces) throw Error(103, "no such piece of arriving rows");
    VQB_CUDA_CHECK(cudaStreamWaitEvent(stream_, arrival_done_[piece], 0));
    arrival_.awaited = std::max(arrival_.awaited, piece + 1);
    return std::min(arrival_.n, (piece + 1) * arrival_.piece_rows);
}

// Small downloads sit on the critical path of every k-means iteration (counts and "changed" flags): they go through a
// pinned staging buffer together with the tensor-core error word -- one copy, one event -- and the host polls the event
// instead of blocking in the driver, which keeps the latency at a few microseconds whatever the host scheduler does.
void CudaDevice::download(void *dst, const void *src, size_t bytes)
{
    if (!bytes) return;
    if (stage_ && bytes <= STAGE_BYTES - 16) {
        VQB_CUDA_CHECK(cudaMemcpyAsync(stage_ + 16, src, bytes, cudaMemcpyDeviceToHost, stream_));
        if (tc_error_) VQB_CUDA_CHECK(cudaMemcpyAsync(stage_, tc_error_, sizeof(int), cudaMemcpyDeviceToHost, stream_));
        VQB_CUDA_CHECK(cudaEventRecord(stage_event_, stream_));
        cudaError_t q;
        while ((q = cudaEventQuery(stage_event_)) == cudaErrorNotReady) {
        }
        VQB_CUDA_CHECK(q);
        std::memcpy(dst, stage_ + 16, bytes);
        if (tc_error_) {
            const int code = *reinterpret_cast<const int *>(stage_);
            if (code != 0) {
                cudaMemsetAsync(tc_error_, 0, sizeof(int), stream_);
                throw Error(100, "tensor-core kernel gave up waiting (stage " + std::to_string(code) + "); set VQB_NO_TENSOR=1 to use the CUDA-core path");
            }
        }
        return;
    }
    VQB_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream_));
    VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
    check_tc_error();
}

// ------------------------------------------------------------------------------------------------
// tensor-core path plumbing (kernels in dense_tc.cu / resolve.cu)
// ------------------------------------------------------------------------------------------------
void CudaDevice::ensure_tc_buffers(size_t n)
{
    if (!hn_scratch_) {
        device_allocs_ += 5;
        VQB_CUDA_CHECK(cudaMalloc(&rot_split_, opq_tc_split_floats(128) * sizeof(float)));
        VQB_CUDA_CHECK(cudaMalloc(&hn_scratch_, 260 * sizeof(float)));
        VQB_CUDA_CHECK(cudaMalloc(&pq_scratch_, pq_tc_scratch_floats() * sizeof(float)));
        VQB_CUDA_CHECK(cudaMemsetAsync(pq_scratch_, 0, pq_tc_scratch_floats() * sizeof(float), stream_));
        VQB_CUDA_CHECK(cudaMalloc(&tc_stats_, 3 * sizeof(unsigned long long)));
        VQB_CUDA_CHECK(cudaMalloc(&tc_error_, sizeof(int)));
        VQB_CUDA_CHECK(cudaMemsetAsync(tc_stats_, 0, 3 * sizeof(unsigned long long), stream_));
        VQB_CUDA_CHECK(cudaMemsetAsync(tc_error_, 0, sizeof(int), stream_));
    }
    if (n > rows_cap_) {
        VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
        cudaFree(rownorm_);
        cudaFree(cand_);
        cudaFree(list_);
        rownorm_ = nullptr;
        cand_ = nullptr;
        list_ = nullptr;
        list_count_ = nullptr;
        rows_cap_ = 0;
        device_allocs_ += 3;
        VQB_CUDA_CHECK(cudaMalloc(&rownorm_, n * sizeof(float)));
        VQB_CUDA_CHECK(cudaMalloc(&cand_, n * DENSE_MASK_WORDS * sizeof(uint32_t)));
        VQB_CUDA_CHECK(cudaMalloc(&list_, (n + 1) * sizeof(uint32_t))); // rows left for the exact kernel, then their count
        list_count_ = list_ + n;
        rows_cap_ = n;
    }
}

uint8_t *CudaDevice::pq_mark_buffer(size_t bytes)
{
    if (bytes > pq_marks_cap_) {
        VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
        cudaFree(pq_marks_);
        pq_marks_ = nullptr;
        pq_marks_cap_ = 0;
        const size_t cap = bytes + bytes / 4;
        ++device_allocs_;
        VQB_CUDA_CHECK(cudaMalloc(&pq_marks_, cap));
        pq_marks_cap_ = cap;
        VQB_CUDA_CHECK(cudaMemsetAsync(pq_marks_, 0, cap, stream_));
    }
    return pq_marks_;
}

// Called at host synchronisation points: a tensor-core kernel whose bounded wait expired leaves a code here.
void CudaDevice::check_tc_error()
{
    if (!tc_error_) return;
    int code = 0;
    VQB_CUDA_CHECK(cudaMemcpyAsync(&code, tc_error_, sizeof(int), cudaMemcpyDeviceToHost, stream_));
    VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
    if (code != 0) {
        cudaMemsetAsync(tc_error_, 0, sizeof(int), stream_);
        throw Error(100, "tensor-core kernel gave up waiting (stage " + std::to_string(code) + "); set VQB_NO_TENSOR=1 to use the CUDA-core path");
    }
}

void CudaDevice::prepare_rows(const Shape &sh, const float *x)
{
    prepared_x_ = nullptr;
    bop_fresh_ = nullptr;
    if (!tensor_enabled_ || sh.m != 1 || sh.ld != sh.sd || sh.n_local == 0) return;
    if (!dense_tc_applicable(sh.n_local, sh.sd, sh.k, M_SQ, x)) return;
    ensure_tc_buffers(sh.n_local);
    if (x == arrival_.dev) end_arrival(); // the norms need all rows: the host waits for the copies
    dense_row_norms(*this, x, sh.n_local, sh.sd, rownorm_);
    prepared_x_ = x;
    prepared_n_ = sh.n_local;
    prepared_dim_ = sh.sd;
}

void CudaDevice::dense_debug(const float *x, size_t n, size_t dim, const float *codebook, size_t k, float *dots,
                             unsigned long long *stats3)
{
    if (!dense_tc_applicable(n, dim, k, M_SQ, x)) throw Error(103, "shape not covered by the tensor-core path");
    ensure_tc_buffers(n);
    VQB_CUDA_CHECK(cudaMemsetAsync(tc_stats_, 0, 3 * sizeof(unsigned long long), stream_));
    dense_row_norms(*this, x, n, dim, rownorm_);
    dense_shortlist(*this, x, n, dim, codebook, k, rownorm_, hn_scratch_, cand_, tc_stats_, tc_error_, dots);
    download(stats3, tc_stats_, 3 * sizeof(unsigned long long));
    prepared_x_ = nullptr;
}

void CudaDevice::pq_tensor_debug(const float *x, size_t n, size_t m, const float *codebooks, size_t k, float *scores, uint32_t *codes,
                                 unsigned long long *marked)
{
    AssignParams p = {};
    p.x = x;
    p.n = n;
    p.ld = m * 8;
    p.m = (int)m;
    p.k = (int)k;
    p.sd = 8;
    p.centroids = codebooks;
    p.out_codes = codes;
    p.x_vec4 = 1;
    if (!pq_tc_applicable(p, M_SQ)) throw Error(103, "shape not covered by the product-quantizer tensor-core path");
    ensure_tc_buffers(0);
    bop_fresh_ = nullptr;
    unsigned long long before = 0, after = 0;
    download(&before, pq_scratch_ + pq_tc_stats_offset_floats(), sizeof before);
    PqTcBuffers tb;
    tb.scratch = pq_scratch_;
    tb.marks = pq_mark_buffer(pq_tc_mark_bytes(n, m));
    tb.error_word = tc_error_;
    tb.dbg_scores = scores;
    launch_pq_tc(*this, p, M_SQ, false, 4, tb);
    download(&after, pq_scratch_ + pq_tc_stats_offset_floats(), sizeof after);
    *marked = after - before;
}

void CudaDevice::copy(void *dst, const void *src, size_t bytes)
{
    if (!bytes) return;
    VQB_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream_));
}

void CudaDevice::zero(void *dst, size_t bytes)
{
    if (!bytes) return;
    VQB_CUDA_CHECK(cudaMemsetAsync(dst, 0, bytes, stream_));
}

static inline unsigned blocks_for(size_t items, int threads, size_t cap = 1u << 20)
{
    size_t b = (items + threads - 1) / threads;
    return (unsigned)std::max<size_t>(1, std::min(b, cap));
}

// ------------------------------------------------------------------------------------------------
// row patches: initial sample (src/utils.rs:54) and empty-cluster re-seed (src/utils.rs:100)
// ------------------------------------------------------------------------------------------------
__global__ void patch_fill_kernel(const float *x, unsigned long long n_local, unsigned long long ld, int sd,
                                  unsigned long long row_begin, const RowPatch *patches, unsigned long long n_patches,
                                  uint32_t *stage)
{
    const unsigned long long total = n_patches * sd;
    for (unsigned long long t = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; t < total;
         t += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long pi = t / sd;
        const int d = (int)(t % sd);
        const RowPatch pt = patches[pi];
        uint32_t bits = 0;
        if (pt.row >= row_begin && pt.row - row_begin < n_local)
            bits = __float_as_uint(x[(pt.row - row_begin) * ld + (size_t)pt.subspace * sd + d]);
        stage[t] = bits;
    }
}

__global__ void patch_scatter_kernel(const uint32_t *stage, const RowPatch *patches, unsigned long long n_patches, int k,
                                     int sd, float *centroids)
{
    const unsigned long long total = n_patches * sd;
    for (unsigned long long t = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; t < total;
         t += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long pi = t / sd;
        const int d = (int)(t % sd);
        const RowPatch pt = patches[pi];
        centroids[((size_t)pt.subspace * k + pt.cluster) * sd + d] = __uint_as_float(stage[t]);
    }
}

void CudaDevice::patch_centroids(const Shape &sh, const float *x, uint64_t row_begin, const RowPatch *patches,
                                 size_t n_patches, float *centroids, Comm *comm)
{
    if (n_patches == 0) return;
    bop_fresh_ = nullptr; // the centroids change behind the fused update's back
    RowPatch *pd = (RowPatch *)alloc(sizeof(RowPatch) * n_patches);
    uint32_t *stage = (uint32_t *)alloc(sizeof(uint32_t) * n_patches * sh.sd);
    upload(pd, patches, sizeof(RowPatch) * n_patches);
    const size_t total = n_patches * sh.sd;
    KernelScope ks(*this, "patch_centroids");
    if (arrival_.dev && x == arrival_.dev && arrival_.awaited < arrival_.pieces) {
        // the rows are still being copied in: take the wanted ones from the caller's host buffer
        std::vector<uint32_t> bits(total, 0u);
        for (size_t i = 0; i < n_patches; ++i) {
            const RowPatch &pt = patches[i];
            if (pt.row >= row_begin && pt.row - row_begin < sh.n_local)
                std::memcpy(&bits[i * sh.sd], arrival_.host + (pt.row - row_begin) * sh.ld + (size_t)pt.subspace * sh.sd, sizeof(float) * sh.sd);
        }
        upload(stage, bits.data(), sizeof(uint32_t) * total);
    } else {
        patch_fill_kernel<<<blocks_for(total, 256, 4096), 256, 0, stream_>>>(x, sh.n_local, sh.ld, (int)sh.sd, row_begin, pd,
                                                                           n_patches, stage);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
    if (comm && comm->world() > 1) comm->allreduce_max_u32(stage, total);
    patch_scatter_kernel<<<blocks_for(total, 256, 4096), 256, 0, stream_>>>(stage, pd, n_patches, (int)sh.k, (int)sh.sd,
                                                                          centroids);
    VQB_CUDA_CHECK(cudaGetLastError());
    count_launch();
    release(stage);
    release(pd);
}

// ------------------------------------------------------------------------------------------------
// assignment (training) and encode: thin wrappers over the kernel launchers
// ------------------------------------------------------------------------------------------------
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

void CudaDevice::assign_train(const Shape &sh, const float *x, const float *centroids, void *codes, const uint32_t *active,
                              const IterBuffers &buf)
{
    if (sh.n_local == 0) return;
    uint32_t *changed = buf.moved;
    if (prepared_x_ == x && prepared_n_ == sh.n_local && prepared_dim_ == sh.sd && sh.m == 1 &&
        dense_tc_applicable(sh.n_local, sh.sd, sh.k, M_SQ, x)) {
        // full-width k-means step: tensor-core shortlist, then the exact decision among the candidates
        static const bool stats_on = std::getenv("VQB_TC_STATS") != nullptr; // diagnostic: shortlist sizes per training pass on stderr
        if (stats_on) VQB_CUDA_CHECK(cudaMemsetAsync(tc_stats_, 0, 3 * sizeof(unsigned long long), stream_));
        // the shortlist kernel decides the rows with one candidate itself and lists the others for the exact kernel
        if (code_bytes(sh.k) != 1) throw Error(103, "full-width tensor path with assignments wider than one byte");
        VQB_CUDA_CHECK(cudaMemsetAsync(list_count_, 0, sizeof(uint32_t), stream_));
        ShortlistTrain tr = {static_cast<uint8_t *>(codes), changed, list_, list_count_};
        dense_shortlist(*this, x, sh.n_local, sh.sd, centroids, sh.k, rownorm_, hn_scratch_, cand_, stats_on ? tc_stats_ : nullptr, tc_error_, nullptr, &tr);
        if (stats_on) {
            unsigned long long st3[3] = {0, 0, 0};
            download(st3, tc_stats_, sizeof st3);
            uint32_t listed = 0;
            download(&listed, list_count_, sizeof listed);
            std::fprintf(stderr, "[vqb] shortlist: rows %llu candidates %llu (%.2f per row) full scans %llu, %u rows left for the exact kernel\n", st3[0],
                         st3[1], st3[0] ? (double)st3[1] / (double)st3[0] : 0.0, st3[2], listed);
        }
        ResolveParams r = {};
        r.x = x;
        r.n = sh.n_local;
        r.dim = (int)sh.sd;
        r.k = (int)sh.k;
        r.codebook = centroids;
        r.cand = cand_;
        r.euclid = 0;
        r.codes = codes;
        r.changed = changed;
        r.list = list_;
        r.list_count = list_count_;
        launch_resolve(*this, r, R_TRAIN, code_bytes(sh.k));
        return;
    }
    AssignParams p = {};
    p.x = x;
    p.n = sh.n_local;
    p.ld = sh.ld;
    p.m = (int)sh.m;
    p.k = (int)sh.k;
    p.sd = (int)sh.sd;
    p.centroids = centroids;
    p.codes = codes;
    p.active = active;
    p.changed = changed;
    p.x_vec4 = aligned16(x) && (sh.ld % 4 == 0) && (sh.sd % 4 == 0);
    if (pq_tensor_enabled_ && pq_tc_applicable(p, M_SQ)) {
        ensure_tc_buffers(0);
        PqTcBuffers tb;
        tb.scratch = pq_scratch_;
        tb.marks = pq_mark_buffer(pq_tc_mark_bytes(sh.n_local, sh.m));
        tb.error_word = tc_error_;
        tb.prepare_operand = (bop_fresh_ != centroids);
        launch_pq_tc(*this, p, M_SQ, true, code_bytes(sh.k), tb);
        bop_fresh_ = nullptr;
        return;
    }
    if (launch_assign_reg(*this, p, M_SQ, true, code_bytes(sh.k))) return;
    GenericParams g = {};
    g.x = x;
    g.n = sh.n_local;
    g.ld = sh.ld;
    g.m = (int)sh.m;
    g.k = (int)sh.k;
    g.sd = (int)sh.sd;
    g.centroids = centroids;
    g.codes = codes;
    g.active = active;
    g.changed = changed;
    launch_assign_generic(*this, g, M_SQ, G_TRAIN, code_bytes(sh.k));
    return;
}

void CudaDevice::pq_encode_impl(const Shape &sh, const float *x, const float *codebooks, int metric, double pm,
                                uint16_t *out_f16, uint32_t *out_codes, float *out_f32, bool cuda_cores_only)
{
    if (sh.n_local == 0) return;
    const size_t dim = sh.m * sh.sd;
    AssignParams p = {};
    p.x = x;
    p.n = sh.n_local;
    p.ld = sh.ld;
    p.m = (int)sh.m;
    p.k = (int)sh.k;
    p.sd = (int)sh.sd;
    p.centroids = codebooks;
    p.out_f16 = out_f16;
    p.out_codes = out_codes;
    p.out_f32 = out_f32;
    p.pv = (float)pm;
    p.x_vec4 = aligned16(x) && (sh.ld % 4 == 0) && (sh.sd % 4 == 0);
    p.out_vec = (!out_f16 || (aligned16(out_f16) && dim % 8 == 0)) && (!out_f32 || (aligned16(out_f32) && dim % 4 == 0));
    if (!cuda_cores_only && pq_tensor_enabled_ && pq_tc_applicable(p, metric)) {
        ensure_tc_buffers(0);
        bop_fresh_ = nullptr;
        PqTcBuffers tb;
        tb.scratch = pq_scratch_;
        tb.marks = pq_mark_buffer(pq_tc_mark_bytes(sh.n_local, sh.m));
        tb.error_word = tc_error_;
        launch_pq_tc(*this, p, metric, false, 4, tb);
        return;
    }
    if (launch_assign_reg(*this, p, metric, false, 4)) return;
    GenericParams g = {};
    g.x = x;
    g.n = sh.n_local;
    g.ld = sh.ld;
    g.m = (int)sh.m;
    g.k = (int)sh.k;
    g.sd = (int)sh.sd;
    g.centroids = codebooks;
    g.out_f16 = out_f16;
    g.out_codes = out_codes;
    g.out_f32 = out_f32;
    g.pv = (float)pm;
    launch_assign_generic(*this, g, metric, G_ENCODE, 4);
}

void CudaDevice::pq_encode(const Shape &sh, const float *x, const float *codebooks, int metric, double pm, uint16_t *out_f16,
                           uint32_t *out_codes, float *out_f32)
{
    pq_encode_impl(sh, x, codebooks, metric, pm, out_f16, out_codes, out_f32, false);
}

void CudaDevice::pq_encode_no_scratch(const Shape &sh, const float *x, const float *codebooks, int metric, double pm, uint16_t *out_f16,
                                      uint32_t *out_codes)
{
    pq_encode_impl(sh, x, codebooks, metric, pm, out_f16, out_codes, nullptr, true);
}

void CudaDevice::rvq_update(float *res, size_t n, size_t dim, const float *centroids, size_t k, int metric, double pm,
                            double *norm_sum)
{
    if (n == 0) return;
    if (tensor_enabled_ && prepared_x_ == res && prepared_n_ == n && prepared_dim_ == dim && dense_tc_applicable(n, dim, k, metric, res)) {
        // the rows have not changed since the stage's k-means announced them, so their norms are still valid
        dense_shortlist(*this, res, n, dim, centroids, k, rownorm_, hn_scratch_, cand_, nullptr, tc_error_, nullptr);
        ResolveParams r = {};
        r.x = res;
        r.res = res;
        r.n = n;
        r.dim = (int)dim;
        r.k = (int)k;
        r.codebook = centroids;
        r.cand = cand_;
        r.euclid = (metric == M_EUCLID);
        r.norm_sum = norm_sum;
        launch_resolve(*this, r, R_RVQ_UPDATE, 4);
        prepared_x_ = nullptr; // the residuals changed
        return;
    }
    prepared_x_ = nullptr;
    GenericParams g = {};
    g.x = res;
    g.res = res;
    g.n = n;
    g.ld = dim;
    g.m = 1;
    g.k = (int)k;
    g.sd = (int)dim;
    g.centroids = centroids;
    g.pv = (float)pm;
    g.norm_sum = norm_sum;
    launch_assign_generic(*this, g, metric, G_RVQ_UPDATE, 4);
}

__global__ void f32_to_f16_kernel(const float *in, unsigned long long n, uint16_t *out)
{
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < n; i += (unsigned long long)gridDim.x * blockDim.x)
        out[i] = f32_to_f16_bits(in[i]);
}

void CudaDevice::f32_to_f16_rows(const float *in, size_t n, uint16_t *out)
{
    if (n == 0) return;
    KernelScope ks(*this, "f32_to_f16");
    f32_to_f16_kernel<<<blocks_for(n, 256, (size_t)sm_count_ * 16), 256, 0, stream_>>>(in, n, out);
    VQB_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

void CudaDevice::rvq_quantize(const float *x, size_t n, size_t dim, const float *codebooks, size_t stages, size_t k,
                              float epsilon, int metric, double pm, uint16_t *out_f16, uint32_t *out_codes)
{
    if (n == 0) return;
    if (out_codes) VQB_CUDA_CHECK(cudaMemsetAsync(out_codes, 0xFF, sizeof(uint32_t) * n * stages, stream_));
    if (tensor_enabled_ && dense_tc_applicable(n, dim, k, metric, x)) {
        // stage by stage: norms of the current residuals, tensor-core shortlist, exact resolve that subtracts the chosen
        // centroid, adds it to the running sum and retires rows whose residual norm fell below epsilon
        ensure_tc_buffers(n);
        prepared_x_ = nullptr;
        float *res = (float *)alloc(sizeof(float) * n * dim), *qsum = (float *)alloc(sizeof(float) * n * dim);
        uint8_t *done = (uint8_t *)alloc(n);
        copy(res, x, sizeof(float) * n * dim);
        zero(qsum, sizeof(float) * n * dim);
        zero(done, n);
        for (size_t st = 0; st < stages; ++st) {
            const float *cb = codebooks + st * k * dim;
            dense_row_norms(*this, res, n, dim, rownorm_);
            dense_shortlist(*this, res, n, dim, cb, k, rownorm_, hn_scratch_, cand_, nullptr, tc_error_, nullptr);
            ResolveParams r = {};
            r.x = res;
            r.res = res;
            r.n = n;
            r.dim = (int)dim;
            r.k = (int)k;
            r.codebook = cb;
            r.cand = cand_;
            r.euclid = (metric == M_EUCLID);
            r.qsum = qsum;
            r.done = done;
            r.out_codes = out_codes;
            r.stage = (int)st;
            r.stages = (int)stages;
            r.epsilon = epsilon;
            launch_resolve(*this, r, R_RVQ_STAGE, 4);
        }
        if (out_f16) f32_to_f16_rows(qsum, n * dim, out_f16);
        release(done);
        release(qsum);
        release(res);
        return;
    }
    GenericParams g = {};
    g.x = x;
    g.n = n;
    g.ld = dim;
    g.m = 1;
    g.k = (int)k;
    g.sd = (int)dim;
    g.centroids = codebooks;
    g.pv = (float)pm;
    g.out_f16 = out_f16;
    g.out_codes = out_codes;
    g.stages = (int)stages;
    g.epsilon = epsilon;
    launch_assign_generic(*this, g, metric, G_RVQ_QUANT, 4);
}

// ------------------------------------------------------------------------------------------------
// cluster sums and counts (src/utils.rs:83-92 + src/vector.rs:297-314)
// ------------------------------------------------------------------------------------------------
// FAST, narrow subspaces: one thread per (row, subspace); shared-memory sums laid out [s][d][code] so
// that the 32 lanes of a warp (different rows, arbitrary codes) spread over the banks.
// counts hold u32 values, or f32 values when counts_f32 is set (IterBuffers)
__device__ __forceinline__ void add_count(uint32_t *counts, size_t at, uint32_t c, int counts_f32)
{
    if (counts_f32) atomicAdd(reinterpret_cast<float *>(counts) + at, (float)c);
    else atomicAdd(counts + at, c);
}

template <typename CodeT>
__global__ void accum_small_kernel(const float *x, unsigned long long n, unsigned long long ld, int m, int k, int sd,
                                   int group, const CodeT *codes, const uint32_t *active, float *sums, uint32_t *counts, int counts_f32)
{
    const bool vec4 = (sd % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
    extern __shared__ __align__(16) float smem[];
    const int g0 = blockIdx.y * group;
    const int gcount = min(group, m - g0);
    float *ssum = smem;                                               // [gcount][sd][k]
    uint32_t *scnt = reinterpret_cast<uint32_t *>(smem + (size_t)group * sd * k); // [gcount][k]
    for (int t = threadIdx.x; t < gcount * sd * k; t += blockDim.x) ssum[t] = 0.0f;
    for (int t = threadIdx.x; t < gcount * k; t += blockDim.x) scnt[t] = 0u;
    __syncthreads();
    const unsigned long long total = n * gcount;
    for (unsigned long long pidx = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; pidx < total;
         pidx += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long row = pidx / gcount;
        const int sl = (int)(pidx % gcount);
        const int s = g0 + sl;
        if (active && active[s] == 0) continue;
        const int code = (int)codes[row * m + s];
        const float *xp = x + row * ld + (size_t)s * sd;
        float *dst = ssum + (size_t)sl * sd * k + code;
        if (vec4) { // 128-bit loads of the row slice
            for (int d = 0; d < sd; d += 4) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(xp + d));
                atomicAdd(dst + (size_t)d * k, v.x);
                atomicAdd(dst + (size_t)(d + 1) * k, v.y);
                atomicAdd(dst + (size_t)(d + 2) * k, v.z);
                atomicAdd(dst + (size_t)(d + 3) * k, v.w);
            }
        } else {
            for (int d = 0; d < sd; ++d) atomicAdd(dst + (size_t)d * k, xp[d]);
        }
        atomicAdd(scnt + sl * k + code, 1u);
    }
    __syncthreads();
    for (int t = threadIdx.x; t < gcount * k * sd; t += blockDim.x) {
        const int sl = t / (k * sd), rem = t % (k * sd);
        const int j = rem / sd, d = rem % sd;
        if (scnt[sl * k + j] != 0u) atomicAdd(sums + ((size_t)(g0 + sl) * k + j) * sd + d, ssum[((size_t)sl * sd + d) * k + j]);
    }
    for (int t = threadIdx.x; t < gcount * k; t += blockDim.x)
        if (scnt[t] != 0u) add_count(counts, (size_t)g0 * k + t, scnt[t], counts_f32);
}

// FAST, wide rows: one warp per (row, subspace), lanes over dimensions; sums laid out [code][d].
// With shared == false the atomics go straight to global memory (codebook too large for shared memory).
template <typename CodeT, bool SHARED>
__global__ void accum_wide_kernel(const float *x, unsigned long long n, unsigned long long ld, int m, int k, int sd,
                                  const CodeT *codes, const uint32_t *active, float *sums, uint32_t *counts, int counts_f32)
{
    extern __shared__ __align__(16) float smem[];
    const int s = blockIdx.y;
    if (active && active[s] == 0) return;
    float *ssum = smem;                                                    // [k][sd]
    uint32_t *scnt = reinterpret_cast<uint32_t *>(smem + (size_t)k * sd); // [k]
    float *gsum = sums + (size_t)s * k * sd;
    uint32_t *gcnt = counts + (size_t)s * k;
    if (SHARED) {
        for (int t = threadIdx.x; t < k * sd; t += blockDim.x) ssum[t] = 0.0f;
        for (int t = threadIdx.x; t < k; t += blockDim.x) scnt[t] = 0u;
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const unsigned long long warps = (unsigned long long)gridDim.x * (blockDim.x >> 5);
    // four rows per step so that enough loads are in flight to cover the memory latency
    constexpr int RB = 4;
    for (unsigned long long row0 = (blockIdx.x * (unsigned long long)(blockDim.x >> 5) + (threadIdx.x >> 5)) * RB; row0 < n; row0 += warps * RB) {
        int code[RB];
#pragma unroll
        for (int r = 0; r < RB; ++r) code[r] = (row0 + r < n) ? (int)codes[(row0 + r) * m + s] : -1;
        for (int d0 = 0; d0 < sd; d0 += 128) {
            float v[RB][4];
#pragma unroll
            for (int r = 0; r < RB; ++r)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int d = d0 + e * 32 + lane;
                    v[r][e] = (code[r] >= 0 && d < sd) ? x[(row0 + r) * ld + (size_t)s * sd + d] : 0.0f;
                }
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                if (code[r] < 0) continue;
                float *dst = (SHARED ? ssum : gsum) + (size_t)code[r] * sd;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int d = d0 + e * 32 + lane;
                    if (d < sd) atomicAdd(dst + d, v[r][e]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r)
            if (lane == 0 && code[r] >= 0) {
                if (SHARED) atomicAdd(scnt + code[r], 1u);
                else add_count(gcnt, (size_t)code[r], 1u, counts_f32);
            }
    }
    if (SHARED) {
        __syncthreads();
        for (int t = threadIdx.x; t < k * sd; t += blockDim.x)
            if (scnt[t / sd] != 0u) atomicAdd(gsum + t, ssum[t]);
        for (int t = threadIdx.x; t < k; t += blockDim.x)
            if (scnt[t] != 0u) add_count(gcnt, (size_t)t, scnt[t], counts_f32);
    }
}

// FAST, narrow sub-spaces, from the second iteration on: only the (row, sub-space) pairs whose code changed are touched --
// their slice is added to the new cluster's sums and subtracted from the old one's, the counts move by one.  Same layout and
// per-CTA shared-memory sums as accum_small_kernel; the flush adds the CTA's net changes to the running totals.
template <typename CodeT>
__global__ void accum_moved_kernel(const float *x, unsigned long long n, unsigned long long ld, int m, int k, int sd, int group,
                                   CodeT *codes_prev, const CodeT *codes, const uint32_t *active, float *sums, uint32_t *counts, int counts_f32)
{
    const bool vec4 = (sd % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
    extern __shared__ __align__(16) float smem[];
    const int g0 = blockIdx.y * group;
    const int gcount = min(group, m - g0);
    float *ssum = smem;                                                        // [gcount][sd][k] net change of the sums
    int *scnt = reinterpret_cast<int *>(smem + (size_t)group * sd * k);        // [gcount][k] net change of the counts
    uint32_t *touched = reinterpret_cast<uint32_t *>(scnt + (size_t)group * k); // [gcount][k] a row joined or left
    for (int t = threadIdx.x; t < gcount * sd * k; t += blockDim.x) ssum[t] = 0.0f;
    for (int t = threadIdx.x; t < gcount * k; t += blockDim.x) scnt[t] = 0, touched[t] = 0u;
    __syncthreads();
    auto move_pair = [&](unsigned long long row, int sl, int was, int now) {
        const float *xp = x + row * ld + (size_t)(g0 + sl) * sd;
        float *add = ssum + (size_t)sl * sd * k + now, *sub = ssum + (size_t)sl * sd * k + was;
        if (vec4) {
            for (int d = 0; d < sd; d += 4) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(xp + d));
                atomicAdd(add + (size_t)d * k, v.x), atomicAdd(sub + (size_t)d * k, -v.x);
                atomicAdd(add + (size_t)(d + 1) * k, v.y), atomicAdd(sub + (size_t)(d + 1) * k, -v.y);
                atomicAdd(add + (size_t)(d + 2) * k, v.z), atomicAdd(sub + (size_t)(d + 2) * k, -v.z);
                atomicAdd(add + (size_t)(d + 3) * k, v.w), atomicAdd(sub + (size_t)(d + 3) * k, -v.w);
            }
        } else {
            for (int d = 0; d < sd; ++d) {
                const float v = xp[d];
                atomicAdd(add + (size_t)d * k, v), atomicAdd(sub + (size_t)d * k, -v);
            }
        }
        atomicAdd(scnt + sl * k + now, 1), atomicAdd(scnt + sl * k + was, -1);
        touched[sl * k + now] = 1u, touched[sl * k + was] = 1u;
    };
    if (sizeof(CodeT) == 1 && gcount == 8 && m % 8 == 0 && g0 % 8 == 0 && (reinterpret_cast<uintptr_t>(codes) & 7u) == 0 &&
        (reinterpret_cast<uintptr_t>(codes_prev) & 7u) == 0) {
        // one thread per row: the eight codes of the CTA's sub-spaces are one 64-bit word, and most rows have not moved at all
        uint32_t act_mask = 0;
        for (int sl = 0; sl < 8; ++sl) act_mask |= (!active || active[g0 + sl] != 0) ? (1u << sl) : 0u;
        for (unsigned long long row = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; row < n; row += (unsigned long long)gridDim.x * blockDim.x) {
            const unsigned long long was8 = *reinterpret_cast<const unsigned long long *>(codes_prev + row * m + g0);
            const unsigned long long now8 = *reinterpret_cast<const unsigned long long *>(codes + row * m + g0);
            unsigned long long diff = was8 ^ now8;
            if (diff) *reinterpret_cast<unsigned long long *>(codes_prev + row * m + g0) = now8; // up to date for the next iteration
            while (diff) {
                const int sl = (__ffsll((long long)diff) - 1) >> 3;
                diff &= ~(0xFFull << (8 * sl));
                if (act_mask >> sl & 1u) move_pair(row, sl, (int)((was8 >> (8 * sl)) & 0xFFu), (int)((now8 >> (8 * sl)) & 0xFFu));
            }
        }
    } else {
        const unsigned long long total = n * gcount;
        for (unsigned long long pidx = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; pidx < total;
             pidx += (unsigned long long)gridDim.x * blockDim.x) {
            const unsigned long long row = pidx / gcount;
            const int sl = (int)(pidx % gcount);
            const int s = g0 + sl;
            const int was = (int)codes_prev[row * m + s], now = (int)codes[row * m + s];
            if (was == now || (active && active[s] == 0)) continue;
            codes_prev[row * m + s] = (CodeT)now;
            move_pair(row, sl, was, now);
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < gcount * k * sd; t += blockDim.x) {
        const int sl = t / (k * sd), rem = t % (k * sd);
        const int j = rem / sd, d = rem % sd;
        if (touched[sl * k + j]) atomicAdd(sums + ((size_t)(g0 + sl) * k + j) * sd + d, ssum[((size_t)sl * sd + d) * k + j]);
    }
    for (int t = threadIdx.x; t < gcount * k; t += blockDim.x) {
        const int dc = scnt[t];
        if (dc == 0) continue;
        if (counts_f32) atomicAdd(reinterpret_cast<float *>(counts) + (size_t)g0 * k + t, (float)dc);
        else atomicAdd(counts + (size_t)g0 * k + t, (uint32_t)dc); // modulo 2^32: the total is the true count
    }
}

// FAST, wide rows in whole 16-byte pieces: the warps of a CTA share out the CLUSTERS (warp w owns the clusters j with
// j mod W == w), so the per-CTA sums need no atomics at all.  Every warp looks at the codes of a 256-row piece (one byte or
// word per row), lists the rows of its own clusters, fetches those rows eight at a time (128-bit loads, the lanes along the
// dimensions) and adds them into shared memory with ordinary 128-bit loads and stores: a lane always touches the same
// addresses of a cluster, so its own program order keeps repeated clusters right.  The shared-memory atomics of
// accum_wide_kernel ran at a third of the memory rate (0.22 ms per 1M x 128 rows); what is left here is the row traffic.
constexpr int AO_PIECE = 256, AO_BATCH = 8, AO_WARPS = 32;
template <typename CodeT>
__global__ void __launch_bounds__(32 * AO_WARPS) accum_owner_kernel(const float *__restrict__ x, unsigned long long n, unsigned long long ld, int m, int k,
                                                                    int sd, const CodeT *__restrict__ codes, const uint32_t *active, float *sums,
                                                                    uint32_t *counts, int counts_f32)
{
    extern __shared__ __align__(16) float smem[];
    const int s = blockIdx.y;
    if (active && active[s] == 0) return;
    float *ssum = smem;                                                    // [k][sd]
    uint32_t *scnt = reinterpret_cast<uint32_t *>(smem + (size_t)k * sd); // [k]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t *list = scnt + k + warp * AO_PIECE;                           // [AO_PIECE] per warp: row in piece | code << 8
    float *gsum = sums + (size_t)s * k * sd;
    uint32_t *gcnt = counts + (size_t)s * k;
    for (int t = threadIdx.x; t < k * sd; t += blockDim.x) ssum[t] = 0.0f;
    for (int t = threadIdx.x; t < k; t += blockDim.x) scnt[t] = 0u;
    __syncthreads();
    const unsigned long long pieces = (n + AO_PIECE - 1) / AO_PIECE;
    const float *xs = x + (size_t)s * sd;
    uint32_t cnext[AO_PIECE / 32];
    auto fetch_codes = [&](unsigned long long piece) {
#pragma unroll
        for (int i = 0; i < AO_PIECE / 32; ++i) {
            const unsigned long long row = piece * AO_PIECE + i * 32 + lane;
            cnext[i] = (piece < pieces && row < n) ? (uint32_t)codes[row * m + s] : 0xFFFFFFFFu;
        }
    };
    fetch_codes(blockIdx.x);
    for (unsigned long long piece = blockIdx.x; piece < pieces; piece += gridDim.x) {
        const unsigned long long row0 = piece * AO_PIECE;
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < AO_PIECE / 32; ++i) {
            const uint32_t c = cnext[i];
            const bool mine = c != 0xFFFFFFFFu && (int)(c % AO_WARPS) == warp;
            const unsigned bal = __ballot_sync(0xffffffffu, mine);
            if (mine) list[cnt + __popc(bal & ((1u << lane) - 1u))] = (uint32_t)(i * 32 + lane) | (c << 8);
            cnt += __popc(bal);
        }
        fetch_codes(piece + gridDim.x); // the next piece's codes travel while this piece's rows are added
        __syncwarp();
        for (int i0 = 0; i0 < cnt; i0 += AO_BATCH) {
            for (int d0 = 0; d0 < sd; d0 += 128) {
                const int d = d0 + 4 * lane;
                float4 v[AO_BATCH];
                uint32_t e[AO_BATCH];
#pragma unroll
                for (int u = 0; u < AO_BATCH; ++u) {
                    e[u] = i0 + u < cnt ? list[i0 + u] : 0xFFFFFFFFu;
                    v[u] = (e[u] != 0xFFFFFFFFu && d < sd) ? __ldg(reinterpret_cast<const float4 *>(xs + (row0 + (e[u] & 0xFFu)) * ld + d))
                                                            : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < AO_BATCH; ++u) {
                    if (e[u] == 0xFFFFFFFFu) continue;
                    const uint32_t code = e[u] >> 8;
                    if (d < sd) {
                        float4 *dst = reinterpret_cast<float4 *>(ssum + (size_t)code * sd + d);
                        float4 a = *dst;
                        a.x += v[u].x, a.y += v[u].y, a.z += v[u].z, a.w += v[u].w;
                        *dst = a;
                    }
                    if (d0 == 0 && lane == 0) scnt[code] += 1u;
                }
            }
        }
        __syncwarp();
    }
    __syncthreads();
    // every CTA starts its flush at another cluster, so that the CTAs that finish together do not queue on the same addresses
    const int total = k * sd, shift = (int)(((unsigned long long)blockIdx.x * 37u % (unsigned)k) * sd);
    for (int t0 = threadIdx.x; t0 < total; t0 += blockDim.x) {
        const int t = t0 + shift < total ? t0 + shift : t0 + shift - total;
        if (scnt[t / sd] != 0u) atomicAdd(gsum + t, ssum[t]);
    }
    for (int t = threadIdx.x; t < k; t += blockDim.x)
        if (scnt[t] != 0u) add_count(gcnt, (size_t)t, scnt[t], counts_f32);
}

// 8-wide sub-spaces with one-byte codes (the product quantizer's benchmark shape), iterations after the first: one thread per
// (row, eight sub-spaces) compares the eight old and new codes as one 64-bit word; a pair that moved adds its 32-byte slice to
// the new cluster's running sums and subtracts it from the old one's with two 128-bit atomics each, straight on global memory.
// No per-CTA sums to clear and flush, so the cost follows the number of moved pairs (and shrinks with the shard).
__global__ void __launch_bounds__(256) accum_pairs_moved_kernel(const float *__restrict__ x, unsigned long long n, unsigned long long ld, int m, int k,
                                                                uint8_t *codes_prev, const uint8_t *codes,
                                                                const uint32_t *active, float *sums, uint32_t *counts, int counts_f32)
{
    const int words = m >> 3; // 64-bit code words per row
    const unsigned long long total = n * words;
    for (unsigned long long t = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; t < total; t += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long row = t / words;
        const int g0 = (int)(t % words) * 8;
        const unsigned long long was8 = *reinterpret_cast<const unsigned long long *>(codes_prev + row * m + g0);
        const unsigned long long now8 = *reinterpret_cast<const unsigned long long *>(codes + row * m + g0);
        unsigned long long diff = was8 ^ now8;
        if (diff) *reinterpret_cast<unsigned long long *>(codes_prev + row * m + g0) = now8; // up to date for the next iteration
        while (diff) {
            const int sl = (__ffsll((long long)diff) - 1) >> 3;
            diff &= ~(0xFFull << (8 * sl));
            const int s = g0 + sl;
            if (active && active[s] == 0) continue;
            const uint32_t was = (uint32_t)((was8 >> (8 * sl)) & 0xFFu), now = (uint32_t)((now8 >> (8 * sl)) & 0xFFu);
            const float4 *xp = reinterpret_cast<const float4 *>(x + row * ld + (size_t)s * 8);
            const float4 a = __ldg(xp), b = __ldg(xp + 1);
            float4 *add = reinterpret_cast<float4 *>(sums + ((size_t)s * k + now) * 8), *sub = reinterpret_cast<float4 *>(sums + ((size_t)s * k + was) * 8);
            atomicAdd(add, a), atomicAdd(add + 1, b);
            atomicAdd(sub, make_float4(-a.x, -a.y, -a.z, -a.w)), atomicAdd(sub + 1, make_float4(-b.x, -b.y, -b.z, -b.w));
            if (counts_f32) {
                atomicAdd(reinterpret_cast<float *>(counts) + (size_t)s * k + now, 1.0f);
                atomicAdd(reinterpret_cast<float *>(counts) + (size_t)s * k + was, -1.0f);
            } else {
                atomicAdd(counts + (size_t)s * k + now, 1u);
                atomicAdd(counts + (size_t)s * k + was, 0xFFFFFFFFu); // minus one modulo 2^32
            }
        }
    }
}

// Wide rows, iterations after the first: a warp looks at 32 rows' old and new codes; for every row that moved, the lanes
// fetch the row in 16-byte pieces and add it to the new cluster's running sums and subtract it from the old one's with
// 128-bit atomics on global memory.  Few rows move, so neither per-CTA sums (whose clearing and flushing would dominate)
// nor an ownership split are worth their fixed cost here.
template <typename CodeT>
__global__ void __launch_bounds__(256) accum_rows_moved_kernel(const float *__restrict__ x, unsigned long long n, unsigned long long ld, int m, int k, int sd,
                                                               CodeT *codes_prev, const CodeT *codes,
                                                               const uint32_t *active, float *sums, uint32_t *counts, int counts_f32)
{
    const int s = blockIdx.y;
    if (active && active[s] == 0) return;
    const int lane = threadIdx.x & 31;
    const unsigned long long warps = (unsigned long long)gridDim.x * (blockDim.x >> 5);
    float *gsum = sums + (size_t)s * k * sd;
    uint32_t *gcnt = counts + (size_t)s * k;
    const float *xs = x + (size_t)s * sd;
    for (unsigned long long r0 = (blockIdx.x * (unsigned long long)(blockDim.x >> 5) + (threadIdx.x >> 5)) * 32; r0 < n; r0 += warps * 32) {
        const unsigned long long row = r0 + lane;
        uint32_t was = 0, now = 0;
        if (row < n) was = (uint32_t)codes_prev[row * m + s], now = (uint32_t)codes[row * m + s];
        if (was != now) codes_prev[row * m + s] = (CodeT)now; // up to date for the next iteration
        unsigned moved = __ballot_sync(0xffffffffu, was != now);
        while (moved) {
            const int src = __ffs(moved) - 1;
            moved &= moved - 1;
            const uint32_t cw = __shfl_sync(0xffffffffu, was, src), cn = __shfl_sync(0xffffffffu, now, src);
            const float *xr = xs + (r0 + src) * ld;
            for (int d = 4 * lane; d < sd; d += 128) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(xr + d));
                atomicAdd(reinterpret_cast<float4 *>(gsum + (size_t)cn * sd + d), v);
                atomicAdd(reinterpret_cast<float4 *>(gsum + (size_t)cw * sd + d), make_float4(-v.x, -v.y, -v.z, -v.w));
            }
            if (lane == 0) {
                if (counts_f32) {
                    atomicAdd(reinterpret_cast<float *>(gcnt) + cn, 1.0f);
                    atomicAdd(reinterpret_cast<float *>(gcnt) + cw, -1.0f);
                } else {
                    atomicAdd(gcnt + cn, 1u);
                    atomicAdd(gcnt + cw, 0xFFFFFFFFu); // minus one modulo 2^32
                }
            }
        }
    }
}

// ORDERED: one thread per (cluster, dimension) walks all rows in ascending order and adds the members
// of its cluster, which is exactly the serial branch of mean_vector (src/vector.rs:305-313).
template <typename CodeT>
__global__ void __launch_bounds__(256) accum_ordered_kernel(const float *x, unsigned long long n, unsigned long long ld, int m,
                                                            int k, int sd, const CodeT *codes, const uint32_t *active,
                                                            float *sums, uint32_t *counts, int counts_f32)
{
    __shared__ CodeT sc[2048];
    const int s = blockIdx.y;
    if (active && active[s] == 0) return;
    const int sdc = min(sd, 256);            // dimensions handled per pass
    const int cpb = max(1, 256 / sdc);       // clusters per block
    const int jl = threadIdx.x / sdc, dl = threadIdx.x % sdc;
    const int j = blockIdx.x * cpb + jl;
    for (int d0 = 0; d0 < sd; d0 += sdc) {
        const int d = d0 + dl;
        const bool mine = (jl < cpb) && (j < k) && (d < sd);
        float acc = 0.0f;
        uint32_t cnt = 0;
        for (unsigned long long r0 = 0; r0 < n; r0 += 2048) {
            const int cn = (int)min((unsigned long long)2048, n - r0);
            __syncthreads();
            for (int t = threadIdx.x; t < cn; t += blockDim.x) sc[t] = codes[(r0 + t) * m + s];
            __syncthreads();
            if (mine) {
                const float *xp = x + r0 * ld + (size_t)s * sd + d;
                for (int r = 0; r < cn; ++r)
                    if ((int)sc[r] == j) {
                        acc = __fadd_rn(acc, xp[(size_t)r * ld]);
                        ++cnt;
                    }
            }
        }
        if (mine) {
            sums[((size_t)s * k + j) * sd + d] = acc;
            if (d == 0) counts[(size_t)s * k + j] = counts_f32 ? __float_as_uint((float)cnt) : cnt;
        }
    }
}

template <typename CodeT>
static void accumulate_t(CudaDevice &dev, const Shape &sh, const float *x, const CodeT *codes, const uint32_t *active,
                         bool ordered, float *sums, uint32_t *counts, int counts_f32)
{
    const int m = (int)sh.m, k = (int)sh.k, sd = (int)sh.sd;
    cudaStream_t st = dev.stream();
    if (ordered) {
        const int sdc = std::min(sd, 256), cpb = std::max(1, 256 / sdc);
        dim3 grid((k + cpb - 1) / cpb, m);
        KernelScope ks(dev, "accumulate_ordered");
        accum_ordered_kernel<CodeT><<<grid, 256, 0, st>>>(x, sh.n_local, sh.ld, m, k, sd, codes, active, sums, counts, counts_f32);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
        return;
    }
    if (sh.n_local == 0) return;
    const size_t budget = dev.smem_limit() - 1024;
    const size_t per_sub = (size_t)k * (sd + 1) * sizeof(float);
    if (sd <= 32 && per_sub <= budget) {
        // two CTAs of 1024 threads per SM when the codebooks allow it: the shared-memory atomics are latency-bound
        const size_t half_budget = (budget - 2048) / 2;
        int group = (int)std::min<size_t>(m, std::max<size_t>(1, (per_sub <= half_budget ? half_budget : budget) / per_sub));
        group = (m + (m + group - 1) / group - 1) / ((m + group - 1) / group); // same number of CTAs, even share of subspaces
        const size_t smem = (size_t)group * per_sub;
        const int ctas_per_sm = (int)std::max<size_t>(1, std::min<size_t>(2, budget / (smem + 1024)));
        auto kernel = accum_small_kernel<CodeT>;
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const int threads = 1024;
        const unsigned long long pairs = (unsigned long long)sh.n_local * group;
        const unsigned ny = (unsigned)((m + group - 1) / group);
        unsigned gx = (unsigned)std::min<unsigned long long>((pairs + threads - 1) / threads,
                                                             std::max<unsigned long long>(1, (unsigned long long)dev.sm_count() * ctas_per_sm / ny));
        dim3 grid(std::max(1u, gx), (m + group - 1) / group);
        KernelScope ks(dev, "accumulate_fast");
        kernel<<<grid, threads, smem, st>>>(x, sh.n_local, sh.ld, m, k, sd, group, codes, active, sums, counts, counts_f32);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
        return;
    }
    const int threads = 512;
    KernelScope ks(dev, "accumulate_fast");
    const size_t owner_smem = per_sub + (size_t)AO_WARPS * AO_PIECE * sizeof(uint32_t);
    if (owner_smem <= budget && sd % 4 == 0 && sh.ld % 4 == 0 && sd >= 64 && k >= 2 * AO_WARPS && k <= (1 << 24) &&
        (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && getenv("VQB_ACCUM_ATOMICS") == nullptr) {
        auto kernel = accum_owner_kernel<CodeT>;
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)owner_smem));
        const unsigned long long pieces = (sh.n_local + AO_PIECE - 1) / AO_PIECE;
        unsigned gx = (unsigned)std::min<unsigned long long>(pieces, (unsigned long long)std::max(1, dev.sm_count() / m));
        dim3 grid(std::max(1u, gx), m);
        kernel<<<grid, 32 * AO_WARPS, owner_smem, st>>>(x, sh.n_local, sh.ld, m, k, sd, codes, active, sums, counts, counts_f32);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
        return;
    }
    if (per_sub <= budget) {
        auto kernel = accum_wide_kernel<CodeT, true>;
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)per_sub));
        unsigned gx = (unsigned)std::min<unsigned long long>((sh.n_local + 15) / 16, (unsigned long long)std::max(1, dev.sm_count() / m));
        dim3 grid(std::max(1u, gx), m);
        kernel<<<grid, threads, per_sub, st>>>(x, sh.n_local, sh.ld, m, k, sd, codes, active, sums, counts, counts_f32);
    } else {
        unsigned gx = (unsigned)std::min<unsigned long long>((sh.n_local + 15) / 16, (unsigned long long)dev.sm_count() * 4);
        dim3 grid(std::max(1u, gx), m);
        accum_wide_kernel<CodeT, false><<<grid, threads, 0, st>>>(x, sh.n_local, sh.ld, m, k, sd, codes, active, sums, counts, counts_f32);
    }
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

template <typename CodeT>
static bool accumulate_moved_t(CudaDevice &dev, const Shape &sh, const float *x, CodeT *codes_prev, const CodeT *codes, const uint32_t *active,
                               float *sums, uint32_t *counts, int counts_f32)
{
    const int m = (int)sh.m, k = (int)sh.k, sd = (int)sh.sd;
    const size_t budget = dev.smem_limit() - 1024;
    const size_t per_sub = (size_t)k * (sd + 2) * sizeof(float); // sums, count changes, touched flags
    if (sd >= 64 && sd % 4 == 0 && sh.ld % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(sums) & 15u) == 0) {
        const unsigned long long groups = (sh.n_local + 31) / 32;
        const unsigned gx = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((groups + 7) / 8, (unsigned long long)dev.sm_count() * 8 / m + 1));
        KernelScope ks(dev, "accumulate_moved");
        accum_rows_moved_kernel<CodeT><<<dim3(gx, m), 256, 0, dev.stream()>>>(x, sh.n_local, sh.ld, m, k, sd, codes_prev, codes, active, sums, counts,
                                                                              counts_f32);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
        return true;
    }
    // measured on a B200: 0.006 ms + 0.148 ms per million rows for the direct kernel, 0.03 ms + 0.097 ms per million rows for the
    // one with per-CTA sums below, so shards below about 450,000 rows take the direct one
    if (sh.n_local <= 450000 && sd == 8 && sizeof(CodeT) == 1 && m % 8 == 0 && sh.ld % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(sums) & 15u) == 0 && (reinterpret_cast<uintptr_t>(codes) & 7u) == 0 && (reinterpret_cast<uintptr_t>(codes_prev) & 7u) == 0 &&
        getenv("VQB_ACCUM_ATOMICS") == nullptr) {
        const unsigned long long total = (unsigned long long)sh.n_local * (m / 8);
        const unsigned gx = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((total + 255) / 256, (unsigned long long)dev.sm_count() * 32));
        KernelScope ks(dev, "accumulate_moved");
        accum_pairs_moved_kernel<<<gx, 256, 0, dev.stream()>>>(x, sh.n_local, sh.ld, m, k, reinterpret_cast<uint8_t *>(codes_prev),
                                                               reinterpret_cast<const uint8_t *>(codes), active, sums, counts, counts_f32);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
        return true;
    }
    if (sd > 32 || per_sub > budget) return false;
    const size_t half_budget = (budget - 2048) / 2;
    int group = (int)std::min<size_t>(m, std::max<size_t>(1, (per_sub <= half_budget ? half_budget : budget) / per_sub));
    group = (m + (m + group - 1) / group - 1) / ((m + group - 1) / group);
    const size_t smem = (size_t)group * per_sub;
    const int ctas_per_sm = (int)std::max<size_t>(1, std::min<size_t>(2, budget / (smem + 1024)));
    auto kernel = accum_moved_kernel<CodeT>;
    VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int threads = 1024;
    const unsigned long long pairs = (unsigned long long)sh.n_local * group;
    const unsigned ny = (unsigned)((m + group - 1) / group);
    const unsigned gx = (unsigned)std::min<unsigned long long>((pairs + threads - 1) / threads,
                                                               std::max<unsigned long long>(1, (unsigned long long)dev.sm_count() * ctas_per_sm / ny));
    KernelScope ks(dev, "accumulate_moved");
    kernel<<<dim3(std::max(1u, gx), ny), threads, smem, dev.stream()>>>(x, sh.n_local, sh.ld, m, k, sd, group, codes_prev, codes, active, sums, counts,
                                                                        counts_f32);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
    return true;
}

bool CudaDevice::accumulate_moved(const Shape &sh, const float *x, void *codes_prev, const void *codes, const uint32_t *active,
                                  const IterBuffers &local)
{
    static const bool off = std::getenv("VQB_ACCUM_FULL") != nullptr; // A/B switch: add up all rows in every iteration
    if (off || sh.n_local == 0) return !off;
    const size_t cb = code_bytes(sh.k);
    const int cf = local.counts_f32 ? 1 : 0;
    if (cb == 1) return accumulate_moved_t<uint8_t>(*this, sh, x, (uint8_t *)codes_prev, (const uint8_t *)codes, active, local.sums, local.counts, cf);
    if (cb == 2) return accumulate_moved_t<uint16_t>(*this, sh, x, (uint16_t *)codes_prev, (const uint16_t *)codes, active, local.sums, local.counts, cf);
    return accumulate_moved_t<uint32_t>(*this, sh, x, (uint32_t *)codes_prev, (const uint32_t *)codes, active, local.sums, local.counts, cf);
}

void CudaDevice::accumulate(const Shape &sh, const float *x, const void *codes, const uint32_t *active, bool ordered,
                            const IterBuffers &buf)
{
    // the buffer arrives zero-filled (update_centroids clears what it has read); the ordered kernel overwrites every entry
    const size_t cb = code_bytes(sh.k);
    const int cf = buf.counts_f32 ? 1 : 0;
    if (cb == 1) accumulate_t<uint8_t>(*this, sh, x, (const uint8_t *)codes, active, ordered, buf.sums, buf.counts, cf);
    else if (cb == 2) accumulate_t<uint16_t>(*this, sh, x, (const uint16_t *)codes, active, ordered, buf.sums, buf.counts, cf);
    else accumulate_t<uint32_t>(*this, sh, x, (const uint32_t *)codes, active, ordered, buf.sums, buf.counts, cf);
}

// ------------------------------------------------------------------------------------------------
// centroid update (src/utils.rs:95-106): centroid = sum / (count as f32), IEEE division (src/vector.rs:315-316); empty
// clusters keep their old value until the host patches them (src/utils.rs:99-101).  The same launch reports the iteration's
// flags to the host through the status page and clears sums, counts and flags for the next iteration.
// One CTA of 8 warps per (sub-space, 32 clusters): a warp takes four clusters, its lanes the dimensions.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) update_centroids_kernel(float *sums, uint32_t *counts, uint32_t *moved, int counts_f32, const uint32_t *active,
                                                               int k, int sd, float *centroids, StatusPage sp, const PeerView pv)
{
    __shared__ uint32_t s_bits;
    const int s = blockIdx.x, word = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool act = !active || active[s] != 0;
    const bool direct = pv.world > 1; // the parts of all ranks are added here, in rank order (peer_exchange.cuh)
    if (threadIdx.x == 0) s_bits = 0u;
    peer_arrive_and_wait(pv);
    __syncthreads();
    if (act) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int j = word * 32 + warp * 4 + q;
            if (j >= k) break;
            const size_t cj = (size_t)s * k + j;
            float cf;
            if (direct) {
                // all peer loads are issued before the first is used (a warp stops at the first use of a pending load, so a
                // load-then-add loop would pay one NVLink round trip per rank)
                uint32_t pc[VQB_MAX_PEERS];
#pragma unroll
                for (int r = 0; r < VQB_MAX_PEERS; ++r) pc[r] = r < pv.world ? peer_ld(pv.words[r] + pv.off_counts + cj) : 0u;
                uint32_t cnt = 0;
#pragma unroll
                for (int r = 0; r < VQB_MAX_PEERS; ++r) cnt += pc[r];
                cf = __uint2float_rn(cnt);
            } else {
                const uint32_t cw = counts[cj];
                cf = counts_f32 ? __uint_as_float(cw) : __uint2float_rn(cw);
            }
            if (direct) {
                for (int d = lane; d < sd; d += 32) {
                    float part[VQB_MAX_PEERS];
#pragma unroll
                    for (int r = 0; r < VQB_MAX_PEERS; ++r) part[r] = r < pv.world ? __uint_as_float(peer_ld(pv.words[r] + cj * sd + d)) : 0.0f;
                    float v = part[0];
#pragma unroll
                    for (int r = 1; r < VQB_MAX_PEERS; ++r)
                        if (r < pv.world) v = __fadd_rn(v, part[r]);
                    if (cf != 0.0f) centroids[cj * sd + d] = __fdiv_rn(v, cf);
                    pv.stale[cj * sd + d] = 0u;
                }
                if (cf == 0.0f && lane == 0) atomicOr(&s_bits, 1u << (warp * 4 + q));
                if (lane == 0) pv.stale[pv.off_counts + cj] = 0u;
            } else {
                if (cf != 0.0f) {
                    for (int d = lane; d < sd; d += 32) {
                        centroids[cj * sd + d] = __fdiv_rn(sums[cj * sd + d], cf);
                        sums[cj * sd + d] = 0.0f;
                    }
                } else if (lane == 0) {
                    atomicOr(&s_bits, 1u << (warp * 4 + q));
                }
                __syncwarp();
                if (lane == 0) counts[cj] = 0u;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        sp.put(sp.idx_bitmap(s, word), s_bits);
        if (word == 0) {
            uint32_t mv = 0u;
            if (direct) {
                uint32_t part[VQB_MAX_PEERS];
#pragma unroll
                for (int r = 0; r < VQB_MAX_PEERS; ++r) part[r] = r < pv.world ? peer_ld(pv.words[r] + pv.off_moved + s) : 0u;
#pragma unroll
                for (int r = 0; r < VQB_MAX_PEERS; ++r) mv |= part[r];
                pv.stale[pv.off_moved + s] = 0u;
            } else {
                mv = moved[s];
                moved[s] = 0u;
            }
            sp.put(sp.idx_moved(s), act ? mv : 0u);
            if (s == 0) sp.put_error();
        }
    }
}

// what the update kernels need to know of a direct exchange
static PeerView peer_view(const PeerExchange *px, const Shape &sh, int *error)
{
    PeerView pv;
    if (!px || px->world <= 1) return pv;
    if (px->world > VQB_MAX_PEERS) throw Error(103, "direct exchange between more than 8 ranks is not supported");
    pv.world = px->world;
    pv.rank = px->rank;
    pv.epoch = px->epoch;
    for (int r = 0; r < px->world; ++r) pv.words[r] = px->words[r], pv.flags[r] = px->flags[r];
    pv.stale = px->stale;
    pv.off_counts = (unsigned long long)sh.m * sh.k * sh.sd;
    pv.off_moved = pv.off_counts + (unsigned long long)sh.m * sh.k;
    pv.error = error;
    return pv;
}

StatusPage CudaDevice::status_page(size_t m, size_t k)
{
    const size_t need = StatusPage::words(m, k);
    if (need > status_cap_words_) {
        VQB_CUDA_CHECK(cudaStreamSynchronize(stream_));
        if (status_host_) cudaFreeHost(status_host_);
        status_host_ = nullptr;
        status_cap_words_ = 0;
        const size_t cap = std::max<size_t>(need + need / 2, 2048);
        ++device_allocs_;
        VQB_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void **>(&status_host_), cap * sizeof(unsigned long long), cudaHostAllocMapped));
        VQB_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void **>(&status_dev_), status_host_, 0));
        std::memset(status_host_, 0, cap * sizeof(unsigned long long));
        status_cap_words_ = cap;
        status_seq_ = 0;
    }
    StatusPage sp;
    sp.host_words = status_dev_;
    sp.tc_error = tc_error_;
    sp.seq = ++status_seq_;
    if (sp.seq == 0) sp.seq = ++status_seq_; // zero is the page's initial value
    sp.m = (uint32_t)m;
    sp.words_per_subspace = (uint32_t)((k + 31) / 32);
    return sp;
}

// The host polls the page (reads of its own memory) instead of queueing a copy and waiting on an event: every entry is
// valid once it carries this update's number.
void CudaDevice::wait_status(const StatusPage &sp, size_t m, size_t k, IterStatus &out)
{
    volatile unsigned long long *page = status_host_;
    const size_t need = StatusPage::words(m, k);
    const auto t0 = std::chrono::steady_clock::now();
    size_t next = 0; // entries below `next` have arrived
    for (uint64_t spin = 1; next < need; ++spin) {
        while (next < need && (uint32_t)(page[next] >> 32) == sp.seq) ++next;
        if (next == need) break;
        if ((spin & 0xFFFFu) == 0) {
            const cudaError_t q = cudaStreamQuery(stream_);
            if (q != cudaSuccess && q != cudaErrorNotReady) VQB_CUDA_CHECK(q);
            if (q == cudaSuccess) {
                // the stream has drained: the writes to the page must have landed by now
                while (next < need && (uint32_t)(page[next] >> 32) == sp.seq) ++next;
                if (next == need) break;
                throw Error(100, "centroid update finished without reporting its status");
            }
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(120))
                throw Error(100, "timed out waiting for the centroid update's status");
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    const size_t wps = (k + 31) / 32;
    out.moved.assign(m, 0);
    out.has_empty.assign(m, 0);
    out.empty_bits.assign(m * wps, 0u);
    for (size_t s = 0; s < m; ++s) {
        out.moved[s] = (uint32_t)page[sp.idx_moved(s)] != 0u;
        for (size_t w = 0; w < wps; ++w) {
            const uint32_t bits = (uint32_t)page[sp.idx_bitmap(s, w)];
            out.empty_bits[s * wps + w] = bits;
            if (bits) out.has_empty[s] = 1;
        }
    }
    const int code = (int)(uint32_t)page[sp.idx_error()];
    if (code != 0) {
        cudaMemsetAsync(tc_error_, 0, sizeof(int), stream_);
        if (code == PEER_ERR_WAIT) throw Error(101, "a rank did not arrive at the exchange of an iteration within four seconds");
        throw Error(100, "tensor-core kernel gave up waiting (stage " + std::to_string(code) + "); set VQB_NO_TENSOR=1 to use the CUDA-core path");
    }
}

void CudaDevice::update_centroids(const Shape &sh, const IterBuffers &buf, const uint32_t *active, float *centroids, IterStatus &status,
                                  const PeerExchange *px)
{
    const size_t m = sh.m, k = sh.k;
    if (m * k * sh.sd == 0) {
        status.moved.assign(m, 0);
        status.has_empty.assign(m, 0);
        status.empty_bits.clear();
        return;
    }
    // shapes of the product-quantizer tensor kernel: the same launch writes the operand of the next assignment pass
    const bool pq8 = pq_tensor_enabled_ && sh.sd == 8 && sh.m >= 4 && sh.m <= 64 && sh.m % 4 == 0 && k >= 2 && k <= 256 && pq_scratch_ != nullptr &&
                     (reinterpret_cast<uintptr_t>(centroids) & 15u) == 0 && (reinterpret_cast<uintptr_t>(buf.sums) & 15u) == 0;
    const PeerView pv = peer_view(px, sh, tc_error_);
    if (pq8) {
        const StatusPage sp = status_page(m, k);
        launch_pq_update_centroids(*this, (int)m, (int)k, buf.sums, buf.counts, buf.moved, buf.counts_f32, active, centroids, pq_scratch_, sp, pv);
        bop_fresh_ = centroids;
        wait_status(sp, m, k, status);
        return;
    }
    const unsigned wps = (unsigned)((k + 31) / 32);
    if (wps > 65535u) throw Error(103, "more than 2,097,120 clusters per sub-space are not supported");
    const StatusPage sp = status_page(m, k);
    {
        KernelScope ks(*this, "update_centroids");
        update_centroids_kernel<<<dim3((unsigned)m, wps), 256, 0, stream_>>>(buf.sums, buf.counts, buf.moved, buf.counts_f32 ? 1 : 0, active, (int)k,
                                                                            (int)sh.sd, centroids, sp, pv);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
    wait_status(sp, m, k, status);
}

// ------------------------------------------------------------------------------------------------
// OPQ: y = R x per row (src/opq.rs:186-194, 232-234) and A = Y X^T (src/opq.rs:172-179)
// ------------------------------------------------------------------------------------------------
// 64x64 output tile per CTA, 4x4 per thread, 16-wide steps over the contraction index.
__global__ void __launch_bounds__(256) rotate_rows_kernel(const float *rot, int dim, const float *x, unsigned long long n, float *y)
{
    __shared__ float xs[16][64 + 1]; // [jj][row]
    __shared__ float rs[16][64 + 1]; // [jj][out]
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const unsigned long long row0 = (unsigned long long)blockIdx.y * 64;
    const int out0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int j0 = 0; j0 < dim; j0 += 16) {
        for (int t = threadIdx.x; t < 64 * 16; t += 256) {
            const int r = t >> 4, jj = t & 15;
            const unsigned long long row = row0 + r;
            const int j = j0 + jj;
            xs[jj][r] = (row < n && j < dim) ? x[row * dim + j] : 0.0f;
            const int o = out0 + r;
            rs[jj][r] = (o < dim && j < dim) ? rot[(size_t)o * dim + j] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = xs[jj][ty * 4 + i];
                b[i] = rs[jj][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int l = 0; l < 4; ++l) acc[i][l] = fmaf(a[i], b[l], acc[i][l]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned long long row = row0 + ty * 4 + i;
        if (row >= n) continue;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const int o = out0 + tx * 4 + l;
            if (o < dim) y[row * dim + o] = acc[i][l];
        }
    }
}

void CudaDevice::rotate_rows(const float *rot, size_t dim, const float *x, size_t n, float *y)
{
    if (n == 0 || dim == 0) return;
    if (opq_tensor_enabled_ && opq_tc_applicable(dim, x, y) && (reinterpret_cast<uintptr_t>(rot) & 15u) == 0) {
        launch_opq_rotate(*this, rot, dim, x, n, y, rot_split_, tc_error_);
        return;
    }
    const unsigned long long row_tiles = (n + 63) / 64;
    // gridDim.y is limited to 65535: walk the rows in slabs
    const unsigned long long slab = 65535ull;
    for (unsigned long long t0 = 0; t0 < row_tiles; t0 += slab) {
        const unsigned long long tiles = std::min(slab, row_tiles - t0);
        const unsigned long long r0 = t0 * 64;
        const unsigned long long rows = std::min<unsigned long long>(n - r0, tiles * 64);
        dim3 grid((unsigned)((dim + 63) / 64), (unsigned)tiles);
        KernelScope ks(*this, "rotate_rows");
        rotate_rows_kernel<<<grid, 256, 0, stream_>>>(rot, (int)dim, x + r0 * dim, rows, y + r0 * dim);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
}

// Each CTA reduces `rows_per_cta` rows into a 64x64 tile of A in f32 and adds it to the f64 result.
__global__ void __launch_bounds__(256) cross_cov_kernel(const float *y, const float *x, unsigned long long n, int dim,
                                                        unsigned long long rows_per_cta, double *a)
{
    __shared__ float ys[16][64 + 4];
    __shared__ float xs[16][64 + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
    const unsigned long long r_begin = (unsigned long long)blockIdx.z * rows_per_cta;
    const unsigned long long r_end = min(n, r_begin + rows_per_cta);
    float acc[4][4] = {};
    for (unsigned long long r0 = r_begin; r0 < r_end; r0 += 16) {
        for (int t = threadIdx.x; t < 16 * 64; t += 256) {
            const int rr = t >> 6, c = t & 63;
            const unsigned long long row = r0 + rr;
            const bool ok = row < r_end;
            ys[rr][c] = (ok && i0 + c < dim) ? y[row * dim + i0 + c] : 0.0f;
            xs[rr][c] = (ok && j0 + c < dim) ? x[row * dim + j0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) {
            float p[4], q[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                p[i] = ys[rr][ty * 4 + i];
                q[i] = xs[rr][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int l = 0; l < 4; ++l) acc[i][l] = fmaf(p[i], q[l], acc[i][l]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const int ii = i0 + ty * 4 + i, jj = j0 + tx * 4 + l;
            if (ii < dim && jj < dim) atomicAdd(a + (size_t)ii * dim + jj, (double)acc[i][l]);
        }
}

void CudaDevice::cross_cov(const float *y, const float *x, size_t n, size_t dim, double *a)
{
    zero(a, sizeof(double) * dim * dim);
    if (n == 0 || dim == 0) return;
    if (opq_tensor_enabled_ && opq_tc_applicable(dim, x, y)) {
        launch_opq_cross_cov(*this, y, x, n, dim, a, tc_error_);
        return;
    }
    const unsigned long long rows_per_cta = 2048;
    const unsigned long long splits = (n + rows_per_cta - 1) / rows_per_cta;
    const unsigned long long slab = 65535ull;
    const unsigned tiles = (unsigned)((dim + 63) / 64);
    for (unsigned long long z0 = 0; z0 < splits; z0 += slab) {
        const unsigned long long zs = std::min(slab, splits - z0);
        const unsigned long long r0 = z0 * rows_per_cta;
        const unsigned long long rows = std::min<unsigned long long>(n - r0, zs * rows_per_cta);
        dim3 grid(tiles, tiles, (unsigned)zs);
        KernelScope ks(*this, "cross_cov");
        cross_cov_kernel<<<grid, 256, 0, stream_>>>(y + r0 * dim, x + r0 * dim, rows, (int)dim, rows_per_cta, a);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
}

// ------------------------------------------------------------------------------------------------
// Distance::compute per row pair (src/distances.rs:115-172)
// ------------------------------------------------------------------------------------------------
template <int METRIC>
__global__ void distance_rows_kernel(const float *a, const float *b, int d, unsigned long long n, float pv, float *out)
{
    for (unsigned long long r = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; r < n;
         r += (unsigned long long)gridDim.x * blockDim.x) {
        const float *pa = a + r * d, *pb = b + r * d;
        float na = 0.0f;
        if (METRIC == M_COSINE) na = norm_chain(pa, d, 1);
        DistAcc<METRIC> acc;
        acc.init();
        for (int i = 0; i < d; ++i) acc.step(pa[i], pb[i], pv);
        out[r] = acc.finish(pv, na);
    }
}

void CudaDevice::distance_rows(int metric, double p, const float *a, const float *b, size_t d, size_t n, float *out)
{
    if (n == 0) return;
    const unsigned grid = blocks_for(n, 128, 4096);
    const float pv = (float)p;
#define VQB_DR(M) distance_rows_kernel<M><<<grid, 128, 0, stream_>>>(a, b, (int)d, n, pv, out)
    switch (metric) {
    case M_SQ: VQB_DR(M_SQ); break;
    case M_EUCLID: VQB_DR(M_EUCLID); break;
    case M_COSINE: VQB_DR(M_COSINE); break;
    case M_MANHATTAN: VQB_DR(M_MANHATTAN); break;
    case M_CHEBYSHEV: VQB_DR(M_CHEBYSHEV); break;
    case M_MINKOWSKI: VQB_DR(M_MINKOWSKI); break;
    case M_HAMMING: VQB_DR(M_HAMMING); break;
    default: throw Error(90, "unknown metric");
    }
#undef VQB_DR
    VQB_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

// ------------------------------------------------------------------------------------------------
// ScalarQuantizer / BinaryQuantizer (src/sq.rs:117-127, src/bq.rs:94-100): pure streaming kernels,
// 16 values per thread step (4 x 128-bit loads, one 128-bit store), 5 bytes of traffic per value.
// ------------------------------------------------------------------------------------------------
struct SqOp {
    static constexpr bool TWO_PIECES = false;
    float mn, mx, step, inv; // inv = fl(1 / step)
    unsigned last;
    // The reference's arithmetic, operation by operation (src/sq.rs:117-127).
    __device__ __forceinline__ unsigned exact(float v) const
    {
        const float c = (v < mn) ? mn : ((v > mx) ? mx : v); // NaN passes through both tests
        const float q = __fdiv_rn(__fsub_rn(c, mn), step);
        const unsigned idx = __float2uint_rz(roundf(q)); // round half away from zero; saturating, NaN -> 0 (`as usize`)
        return min(idx, last);
    }
    // Same result with a multiply instead of the IEEE division: q' = (c - min) * inv differs from the reference's
    // quotient q by at most 3.1 * 2^-24 * q (< 2e-4 for q < 1024), so whenever q' is farther than 2e-4 from a
    // half-integer, round(q) is the integer nearest to q'; that integer is read from the mantissa after adding
    // 1.5 * 2^23.  Values close to a half-integer (or out of range) take the exact path.  NaN clamps to min here and
    // yields level 0, which is also what the reference's saturating cast gives.
    __device__ __forceinline__ unsigned operator()(float v) const
    {
        const float c = fminf(fmaxf(v, mn), mx);
        const float qp = __fmul_rn(__fsub_rn(c, mn), inv);
        const float t = __fadd_rn(qp, 12582912.0f);
        const float diff = __fsub_rn(qp, __fsub_rn(t, 12582912.0f));
        if (!(fabsf(diff) < 0.4998f && qp < 1024.0f)) return exact(v);
        const unsigned idx = (unsigned)(__float_as_int(t) - 0x4B400000);
        return min(idx, last);
    }
};

struct BqOp {
    static constexpr bool TWO_PIECES = true;
    float thr;
    unsigned low, high;
    __device__ __forceinline__ unsigned operator()(float v) const { return (v >= thr) ? high : low; }
};

__device__ __forceinline__ float4 ld_stream(const float4 *p)
{
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

template <typename Op>
__global__ void __launch_bounds__(256) elementwise_u8_kernel(const float *__restrict__ x, unsigned long long n, Op op,
                                                             uint8_t *__restrict__ out, int vec)
{
    const unsigned long long tid = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x;
    const unsigned long long nthreads = (unsigned long long)gridDim.x * blockDim.x;
    if (vec) {
        const unsigned long long n16 = n / 16;
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        uint4 *o4 = reinterpret_cast<uint4 *>(out);
        // Op::TWO_PIECES: two 64-byte pieces per trip, eight 128-bit loads in flight per thread.  Measured at 10M x 128: the
        // threshold test gains (1.20 -> 1.07 ms), the scalar quantizer with its longer arithmetic loses (1.10 -> 1.19 ms).
        unsigned long long i = tid;
        for (; Op::TWO_PIECES && i + nthreads < n16; i += 2 * nthreads) {
            float4 v[8];
#pragma unroll
            for (int t = 0; t < 4; ++t) v[t] = ld_stream(x4 + 4 * i + t);
#pragma unroll
            for (int t = 0; t < 4; ++t) v[4 + t] = ld_stream(x4 + 4 * (i + nthreads) + t);
            unsigned w[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) w[t] = op(v[t].x) | (op(v[t].y) << 8) | (op(v[t].z) << 16) | (op(v[t].w) << 24);
            __stcs(o4 + i, make_uint4(w[0], w[1], w[2], w[3]));
            __stcs(o4 + i + nthreads, make_uint4(w[4], w[5], w[6], w[7]));
        }
        for (; i < n16; i += nthreads) {
            float4 v[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) v[t] = ld_stream(x4 + 4 * i + t);
            unsigned w[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) w[t] = op(v[t].x) | (op(v[t].y) << 8) | (op(v[t].z) << 16) | (op(v[t].w) << 24);
            __stcs(o4 + i, make_uint4(w[0], w[1], w[2], w[3]));
        }
        for (unsigned long long i = n16 * 16 + tid; i < n; i += nthreads) out[i] = (uint8_t)op(x[i]);
    } else {
        for (unsigned long long i = tid; i < n; i += nthreads) out[i] = (uint8_t)op(x[i]);
    }
}

template <typename Op> static void launch_elementwise(CudaDevice &dev, const char *name, const float *x, size_t n, Op op, uint8_t *out)
{
    if (n == 0) return;
    const int vec = aligned16(x) && aligned16(out);
    const size_t items = vec ? (n + 15) / 16 : n;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>((items + 255) / 256, (size_t)dev.sm_count() * 32));
    KernelScope ks(dev, name);
    elementwise_u8_kernel<Op><<<grid, 256, 0, dev.stream()>>>(x, n, op, out, vec);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

void CudaDevice::sq_quantize(float mn, float mx, size_t levels, float step, const float *x, size_t n, uint8_t *out)
{
    SqOp op{mn, mx, step, 1.0f / step, (unsigned)(levels - 1)};
    launch_elementwise(*this, "sq_quantize", x, n, op, out);
}

void CudaDevice::bq_quantize(float threshold, uint8_t low, uint8_t high, const float *x, size_t n, uint8_t *out)
{
    BqOp op{threshold, low, high};
    launch_elementwise(*this, "bq_quantize", x, n, op, out);
}

} // namespace vqb
