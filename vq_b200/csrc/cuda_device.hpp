// cuda_device.hpp -- the sm_100a implementation of vqb::Device plus the element-wise quantizers.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <string>
#include <vector>

#include "backend.hpp"
#include "iter_status.cuh"

namespace vqb {

#define VQB_CUDA_CHECK(expr)                                                                                       \
    do {                                                                                                           \
        cudaError_t _e = (expr);                                                                                   \
        if (_e != cudaSuccess)                                                                                     \
            throw ::vqb::Error(100, std::string("CUDA error: ") + cudaGetErrorString(_e) + " at " + __FILE__ + ":" + \
                                        std::to_string(__LINE__));                                                 \
    } while (0)

class CudaDevice : public Device {
  public:
    explicit CudaDevice(int device);
    ~CudaDevice() override;

    void *alloc(size_t bytes) override;
    void release(void *p) override;
    void upload(void *dst, const void *src, size_t bytes) override;
    void download(void *dst, const void *src, size_t bytes) override;
    void copy(void *dst, const void *src, size_t bytes) override;
    void zero(void *dst, size_t bytes) override;
    size_t code_bytes(size_t k) const override { return k <= 256 ? 1 : (k <= 65536 ? 2 : 4); }

    void prepare_rows(const Shape &sh, const float *x) override;
    size_t arriving_pieces(const float *x) override;
    size_t await_piece(const float *x, size_t piece) override;
    // Starts copying n rows of ld floats from the caller's host buffer to `dst` in pieces on a helper stream and remembers
    // them as arriving (Device::arriving_pieces).  Returns false, having copied nothing, when the rows are too few for pieces
    // to pay.  end_arrival waits (on the host) for whatever nobody has awaited yet; the owner of `dst` calls it before it
    // lets go of the memory or returns to the caller.
    bool begin_arrival(float *dst, const float *host, size_t n, size_t ld);
    void end_arrival();
    bool svd_sweeps(double *gt, double *vt, size_t n) override;
    bool polar_rotation(const double *a_dev, size_t n, float *rot_dev) override;
    // Zero-filled map of at least `bytes` bytes for the product-quantizer tensor kernel; its users leave it zero-filled.
    uint8_t *pq_mark_buffer(size_t bytes);
    void patch_centroids(const Shape &sh, const float *x, uint64_t row_begin, const RowPatch *patches, size_t n_patches,
                         float *centroids, Comm *comm) override;
    void assign_train(const Shape &sh, const float *x, const float *centroids, void *codes, const uint32_t *active,
                      const IterBuffers &buf) override;
    void accumulate(const Shape &sh, const float *x, const void *codes, const uint32_t *active, bool ordered,
                    const IterBuffers &buf) override;
    bool accumulate_moved(const Shape &sh, const float *x, void *codes_prev, const void *codes, const uint32_t *active,
                          const IterBuffers &local) override;
    void update_centroids(const Shape &sh, const IterBuffers &buf, const uint32_t *active, float *centroids,
                          IterStatus &status, const PeerExchange *px = nullptr) override;
    void rvq_update(float *res, size_t n, size_t dim, const float *centroids, size_t k, int metric, double p,
                    double *norm_sum) override;
    void pq_encode(const Shape &sh, const float *x, const float *codebooks, int metric, double p, uint16_t *out_f16,
                   uint32_t *out_codes, float *out_f32) override;
    // The same encode on the CUDA-core kernels only: they work out of shared memory and registers and need no device
    // memory besides inputs and outputs.  Results are identical to pq_encode.
    void pq_encode_no_scratch(const Shape &sh, const float *x, const float *codebooks, int metric, double p, uint16_t *out_f16,
                              uint32_t *out_codes);
    void rotate_rows(const float *rot, size_t dim, const float *x, size_t n, float *y) override;
    void cross_cov(const float *y, const float *x, size_t n, size_t dim, double *a) override;

    // Not part of the training loops:
    void rvq_quantize(const float *x, size_t n, size_t dim, const float *codebooks, size_t stages, size_t k,
                      float epsilon, int metric, double p, uint16_t *out_f16, uint32_t *out_codes);
    void f32_to_f16_rows(const float *in, size_t n, uint16_t *out);
    // Raw scores, codes and the number of pairs left to the exact scan of the product-quantizer tensor-core kernel.
    void pq_tensor_debug(const float *x, size_t n, size_t m, const float *codebooks, size_t k, float *scores, uint32_t *codes,
                         unsigned long long *marked);
    // Reconstruction error and windowed recall@k of an f16 reconstruction (the reference's evaluation metrics).
    void evaluate_f16(const float *x, const uint16_t *q, size_t n, size_t dim, size_t k, float *mse_out, float *recall_out);
    void distance_rows(int metric, double p, const float *a, const float *b, size_t d, size_t n, float *out);
    void sq_quantize(float mn, float mx, size_t levels, float step, const float *x, size_t n, uint8_t *out);
    void bq_quantize(float threshold, uint8_t low, uint8_t high, const float *x, size_t n, uint8_t *out);

    // Two helper streams for overlapping host<->device copies with kernels (created on first use).
    cudaStream_t aux_stream(int i);
    void set_stream(cudaStream_t s) { stream_ = s; } // nullptr = the CUDA default stream
    void reset_stream() { stream_ = own_stream_; }
    cudaStream_t stream() const { return stream_; }
    void synchronize();
    int device() const { return device_; }
    int sm_count() const { return sm_count_; }
    size_t smem_limit() const { return smem_limit_; }
    uint64_t launches() const { return launches_.load(); }
    void count_launch(uint64_t n = 1) { launches_ += n; }
    // How often this context has asked CUDA for device or pinned memory (cudaMalloc, cudaMallocAsync, cudaHostAlloc).
    uint64_t device_allocs() const { return device_allocs_.load(); }
    void make_current() const;
    // Optional per-kernel timing with CUDA events on the launching stream (off by default).
    void set_timing(bool on);
    bool timing() const { return timing_; }
    void timing_begin(const char *name);
    void timing_end();
    // {"name": {"launches": L, "ms": T}, ...}; clears the record.
    std::string timing_report();
    // Diagnostic: raw tensor-core dot products (n x 256) and shortlist statistics {rows, candidates, full scans}.
    void dense_debug(const float *x, size_t n, size_t dim, const float *codebook, size_t k, float *dots, unsigned long long *stats3);
    // True when p points to device memory usable by kernels on this GPU.
    bool is_device_pointer(const void *p) const;

  private:
    int device_;
    int sm_count_ = 148;
    size_t smem_limit_ = 0;
    cudaStream_t own_stream_ = nullptr, stream_ = nullptr, aux_[2] = {nullptr, nullptr};
    static constexpr size_t STAGE_BYTES = 1u << 20; // pinned staging for small downloads
    unsigned char *stage_ = nullptr, *stage_dev_ = nullptr; // stage_dev_: the same bytes as kernels on this GPU address them
    cudaEvent_t stage_event_ = nullptr;
    std::atomic<uint64_t> launches_{0}, device_allocs_{0};
    // page of mapped pinned memory the centroid-update kernels report to (iter_status.cuh)
    unsigned long long *status_host_ = nullptr, *status_dev_ = nullptr;
    size_t status_cap_words_ = 0;
    uint32_t status_seq_ = 0;
    StatusPage status_page(size_t m, size_t k);
    void wait_status(const StatusPage &sp, size_t m, size_t k, IterStatus &out);
    // centroids whose operand B (pq_tc.cu) the scratch currently holds, written by the fused centroid update
    const float *bop_fresh_ = nullptr;
    // tensor-core path state (dense_tc.cu): row norms of the rows announced by prepare_rows, shortlist scratch
    bool tensor_enabled_ = true;
    const float *prepared_x_ = nullptr;
    size_t prepared_n_ = 0, prepared_dim_ = 0;
    float *rownorm_ = nullptr, *hn_scratch_ = nullptr, *pq_scratch_ = nullptr;
    float *rot_split_ = nullptr; // TF32 high and low parts of the rotation matrix of the current rotate_rows call (dim <= 128)
    bool opq_tensor_enabled_ = true;
    uint8_t *pq_marks_ = nullptr;
    size_t pq_marks_cap_ = 0;
    bool pq_tensor_enabled_ = false;
    uint32_t *cand_ = nullptr;
    uint32_t *list_ = nullptr, *list_count_ = nullptr; // rows the shortlist kernel leaves to the exact kernel (training passes)
    size_t rows_cap_ = 0;
    unsigned long long *tc_stats_ = nullptr;
    int *tc_error_ = nullptr;
    void ensure_tc_buffers(size_t n);
    void pq_encode_impl(const Shape &sh, const float *x, const float *codebooks, int metric, double p, uint16_t *out_f16,
                        uint32_t *out_codes, float *out_f32, bool cuda_cores_only);

    void check_tc_error();
    // rows on their way from a host buffer (begin_arrival): piece i is complete when arrival_done_[i] has fired
    struct Arrival {
        const float *dev = nullptr, *host = nullptr;
        size_t n = 0, ld = 0, piece_rows = 0, pieces = 0, awaited = 0;
    } arrival_;
    std::vector<cudaEvent_t> arrival_done_; // created once, re-used
    cudaEvent_t arrival_fence_ = nullptr;
    bool timing_ = false;
    struct Span {
        const char *name;
        cudaEvent_t a, b;
    };
    std::vector<Span> spans_;
    std::vector<cudaEvent_t> event_pool_; // timing events are created once and re-used
    cudaEvent_t take_event();
};

// Brackets one kernel launch for the optional timing record.
struct KernelScope {
    CudaDevice &dev;
    KernelScope(CudaDevice &d, const char *name) : dev(d)
    {
        if (dev.timing()) dev.timing_begin(name);
    }
    ~KernelScope()
    {
        if (dev.timing()) dev.timing_end();
    }
};

// assign_launch.cu
struct AssignParams;
struct GenericParams;
// Returns false when the register kernel does not cover this shape/metric.
bool launch_assign_reg(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t code_bytes);
void launch_assign_generic(CudaDevice &dev, GenericParams &p, int metric, int mode, size_t code_bytes);

} // namespace vqb
