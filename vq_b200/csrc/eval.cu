// eval.cu -- the reference's quality metrics on the device (src/bin/utils.rs:50-67 reconstruction error,
// src/bin/utils.rs:70-127 windowed recall@k), so that a 1M-row evaluation needs no host copy of the f16 output.
#include <algorithm>
#include <vector>

#include "cuda_device.hpp"
#include "kernels_common.cuh"

namespace vqb {

namespace {

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// sum over all elements of (x - q)^2 in f64 (the reference sums f32 partial results in an unspecified order)
__global__ void sq_error_kernel(const float *x, const uint16_t *q, unsigned long long total, double *out)
{
    double acc = 0.0;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < total;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const float d = x[i] - f16_bits_to_f32(q[i]);
        acc += (double)d * (double)d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __shared__ double part[32];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += part[w];
        atomicAdd(out, s);
    }
}

// One CTA per query: Euclidean distances (the reference's chain: sub, mul, serial add, then sqrt) from the query to
// every other row of its window, in the original and in the reconstructed space; the k nearest of each by (distance,
// index) -- what a stable sort by distance keeps -- and the size of their intersection.
template <int MAXK>
__global__ void __launch_bounds__(256) recall_kernel(const float *x, const uint16_t *q, unsigned long long n, int dim, int k,
                                                     unsigned long long step, unsigned long long window, uint32_t *hits)
{
    extern __shared__ float sm[];
    float *qx = sm;            // [dim] query, original space
    float *qa = sm + dim;      // [dim] query, reconstructed space
    float *dx = qa + dim;      // [window] distances, original
    float *da = dx + window;   // [window] distances, reconstructed
    __shared__ float red_d[256];
    __shared__ int red_i[256];
    __shared__ int top[2][MAXK];
    const unsigned long long i = (unsigned long long)blockIdx.x * step;
    const unsigned long long half = window / 2;
    const unsigned long long start = (i > half) ? i - half : 0ull;
    const unsigned long long end = min(i + half, n);
    const int cnt = (int)(end - start);
    for (int t = threadIdx.x; t < dim; t += blockDim.x) {
        qx[t] = x[i * dim + t];
        qa[t] = f16_bits_to_f32(q[i * dim + t]);
    }
    __syncthreads();
    for (int j = threadIdx.x; j < cnt; j += blockDim.x) {
        const unsigned long long row = start + j;
        float ax = 0.0f, aa = 0.0f;
        for (int t = 0; t < dim; ++t) {
            const float d0 = __fsub_rn(qx[t], x[row * dim + t]);
            ax = __fadd_rn(ax, __fmul_rn(d0, d0));
            const float d1 = __fsub_rn(qa[t], f16_bits_to_f32(q[row * dim + t]));
            aa = __fadd_rn(aa, __fmul_rn(d1, d1));
        }
        const bool self = (row == i);
        ax = __fsqrt_rn(ax);
        aa = __fsqrt_rn(aa);
        dx[j] = (self || !(ax == ax)) ? VQB_INF : ax; // the query itself is excluded (src/bin/utils.rs:97,105)
        da[j] = (self || !(aa == aa)) ? VQB_INF : aa;
    }
    __syncthreads();
    for (int space = 0; space < 2; ++space) {
        float *d = space ? da : dx;
        for (int r = 0; r < k; ++r) {
            float bd = VQB_INF;
            int bi = 0x7fffffff;
            for (int j = threadIdx.x; j < cnt; j += blockDim.x)
                if (d[j] < bd) { // ascending j within a thread: the first of equal distances stays
                    bd = d[j];
                    bi = j;
                }
            red_d[threadIdx.x] = bd;
            red_i[threadIdx.x] = bi;
            __syncthreads();
            for (int o = 128; o > 0; o >>= 1) {
                if ((int)threadIdx.x < o) {
                    const float od = red_d[threadIdx.x + o];
                    const int oi = red_i[threadIdx.x + o];
                    if (od < red_d[threadIdx.x] || (od == red_d[threadIdx.x] && oi < red_i[threadIdx.x])) {
                        red_d[threadIdx.x] = od;
                        red_i[threadIdx.x] = oi;
                    }
                }
                __syncthreads();
            }
            if (threadIdx.x == 0) {
                top[space][r] = red_i[0];
                if (red_i[0] != 0x7fffffff) d[red_i[0]] = VQB_INF; // taken
            }
            __syncthreads();
        }
    }
    if (threadIdx.x == 0) {
        uint32_t h = 0;
        for (int a = 0; a < k; ++a) {
            if (top[0][a] == 0x7fffffff) continue;
            for (int b = 0; b < k; ++b)
                if (top[0][a] == top[1][b]) {
                    ++h;
                    break;
                }
        }
        hits[blockIdx.x] = h;
    }
}

} // namespace

void CudaDevice::evaluate_f16(const float *x, const uint16_t *q, size_t n, size_t dim, size_t k, float *mse_out, float *recall_out)
{
    if (n == 0 || dim == 0) throw Error(1, "Empty input: at least one vector is required.");
    if (k == 0 || k > 32) throw Error(2, "Invalid parameter: k must be between 1 and 32");
    // reconstruction error: sum of squared differences / (rows * dim)    (src/bin/utils.rs:50-67)
    double *acc = (double *)alloc(sizeof(double));
    zero(acc, sizeof(double));
    {
        KernelScope ks(*this, "sq_error");
        const unsigned long long total = (unsigned long long)n * dim;
        const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((total + 255) / 256, (unsigned long long)sm_count_ * 16));
        sq_error_kernel<<<grid, 256, 0, stream_>>>(x, q, total, acc);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
    double total_err = 0.0;
    download(&total_err, acc, sizeof(double));
    release(acc);
    *mse_out = (float)(total_err / (double)((float)(n * dim))); // total_elements is an f32 in the reference
    // recall@k over at most 1000 evenly spaced queries, each against a window of 5000 rows when n > 10000  (70-127)
    const unsigned long long eval = std::min<unsigned long long>(n, 1000);
    const unsigned long long step = std::max<unsigned long long>(1, n / eval);
    const unsigned long long window = n > 10000 ? 5000 : n;
    const unsigned long long queries = (n + step - 1) / step;
    const size_t smem = (2 * dim + 2 * std::min<unsigned long long>(window, n)) * sizeof(float);
    if (smem > smem_limit_ - 4096) throw Error(103, "evaluation window does not fit in shared memory");
    uint32_t *hits = (uint32_t *)alloc(sizeof(uint32_t) * queries);
    {
        KernelScope ks(*this, "recall");
        auto kernel = recall_kernel<32>;
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<(unsigned)queries, 256, smem, stream_>>>(x, q, n, (int)dim, (int)k, step, window, hits);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
    std::vector<uint32_t> h(queries);
    download(h.data(), hits, sizeof(uint32_t) * queries);
    release(hits);
    float total_recall = 0.0f; // f32, in query order, as the reference accumulates it
    for (unsigned long long t = 0; t < queries; ++t) total_recall += (float)h[t] / (float)k;
    *recall_out = total_recall / (float)(n / step);
}

} // namespace vqb
