// assign_generic.cuh -- nearest-centroid search for any sub-space width and any metric.
//
// Used where the register kernel (assign_reg.cuh) does not apply: full-width k-means of the residual
// quantizer (src/rvq.rs:107,111-128,186-202), odd sub-space widths, and the rarely used metrics.
// One lane owns one row; the warp's 32 rows sit in shared memory dimension-major (stride 33 floats,
// conflict-free both for the coalesced fill and for the per-lane reads); centroids stream through a
// shared-memory chunk that every lane reads as a broadcast.  J centroids are evaluated side by side
// per lane, each keeping the reference's serial order over dimensions.
#pragma once
#include "kernels_common.cuh"

namespace vqb {

enum : int { G_TRAIN = 0, G_ENCODE = 1, G_RVQ_UPDATE = 2, G_RVQ_QUANT = 3 };

struct GenericParams {
    const float *x; // n rows, ld floats apart
    unsigned long long n, ld;
    int m, k, sd;
    const float *centroids; // [m][k][sd]; for G_RVQ_QUANT [stages][k][sd]
    void *codes;
    const uint32_t *active;
    uint32_t *changed;
    uint16_t *out_f16;
    uint32_t *out_codes;
    float *out_f32;
    float pv;
    int jc;        // centroids per shared-memory chunk
    int resident;  // whole codebook of the CTA's subspace fits in one chunk: load once
    float *res;    // G_RVQ_UPDATE: residual rows, updated in place (same buffer as x)
    double *norm_sum;
    int stages;
    float epsilon;
};

#define VQB_XS_STRIDE 33

template <int METRIC, int J, bool VEC4>
__device__ __forceinline__ void dist_block(const float *xcol, const float *cs, int sd, float pv, float na, float (&out)[J])
{
    DistAcc<METRIC> acc[J];
#pragma unroll
    for (int jj = 0; jj < J; ++jj) acc[jj].init();
    if (VEC4) {
        for (int i4 = 0; i4 < sd / 4; ++i4) {
            const float x0 = xcol[(4 * i4 + 0) * VQB_XS_STRIDE], x1 = xcol[(4 * i4 + 1) * VQB_XS_STRIDE];
            const float x2 = xcol[(4 * i4 + 2) * VQB_XS_STRIDE], x3 = xcol[(4 * i4 + 3) * VQB_XS_STRIDE];
#pragma unroll
            for (int jj = 0; jj < J; ++jj) {
                const float4 c = reinterpret_cast<const float4 *>(cs + (size_t)jj * sd)[i4];
                acc[jj].step(x0, c.x, pv);
                acc[jj].step(x1, c.y, pv);
                acc[jj].step(x2, c.z, pv);
                acc[jj].step(x3, c.w, pv);
            }
        }
    } else {
        for (int i = 0; i < sd; ++i) {
            const float xi = xcol[i * VQB_XS_STRIDE];
#pragma unroll
            for (int jj = 0; jj < J; ++jj) acc[jj].step(xi, cs[(size_t)jj * sd + i], pv);
        }
    }
#pragma unroll
    for (int jj = 0; jj < J; ++jj) out[jj] = acc[jj].finish(pv, na);
}

template <int METRIC, int MODE, typename CodeT, bool VEC4>
__global__ void __launch_bounds__(256) assign_generic_kernel(const GenericParams P)
{
    extern __shared__ __align__(16) float smem[];
    constexpr int J = 4;
    const int sd = P.sd, k = P.k;
    const int W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.y;
    if (MODE == G_TRAIN && P.active && P.active[s] == 0) return; // uniform over the CTA
    const size_t tile_floats = (size_t)sd * VQB_XS_STRIDE;
    float *xs = smem + (size_t)warp * tile_floats;
    float *qs = (MODE == G_RVQ_QUANT) ? smem + (size_t)(W + warp) * tile_floats : nullptr;
    size_t cs_off = (size_t)W * tile_floats * ((MODE == G_RVQ_QUANT) ? 2 : 1);
    cs_off = (cs_off + 3) & ~(size_t)3;
    float *cs = smem + cs_off; // [jc][sd]
    const int dim = P.m * sd;
    const unsigned long long rows_per_tile = 32ull * W;
    const unsigned long long n_tiles = (P.n + rows_per_tile - 1) / rows_per_tile;
    const int nstages = (MODE == G_RVQ_QUANT) ? P.stages : 1;
    bool moved = false;
    bool chunk_loaded = false;
    double warp_norm = 0.0;

    for (unsigned long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const unsigned long long wrow0 = tile * rows_per_tile + 32ull * warp;
        const unsigned long long row = wrow0 + lane;
        const bool valid = row < P.n;
        // fill the warp's row tile: consecutive lanes read consecutive columns of a row
        for (int r = 0; r < 32; ++r) {
            const unsigned long long rr = wrow0 + r;
            const float *src = P.x + rr * P.ld + (size_t)s * sd;
            for (int i = lane; i < sd; i += 32) {
                xs[i * VQB_XS_STRIDE + r] = (rr < P.n) ? src[i] : 0.0f;
                if (MODE == G_RVQ_QUANT) qs[i * VQB_XS_STRIDE + r] = 0.0f;
            }
        }
        __syncwarp();
        const float *xcol = xs + lane;
        bool done = false;

        for (int st = 0; st < nstages; ++st) {
            const float *cb = P.centroids + (size_t)((MODE == G_RVQ_QUANT) ? st : s) * k * sd;
            float na = 0.0f;
            if (METRIC == M_COSINE) na = norm_chain(xcol, sd, VQB_XS_STRIDE);
            float best = 0.0f;
            int idx = 0;
            for (int j0 = 0; j0 < k; j0 += P.jc) {
                const int jcnt = min(P.jc, k - j0);
                if (!(P.resident && chunk_loaded)) {
                    __syncthreads();
                    const float *src = cb + (size_t)j0 * sd;
                    for (int t = threadIdx.x; t < jcnt * sd; t += blockDim.x) cs[t] = src[t];
                    __syncthreads();
                    chunk_loaded = true;
                }
                if (valid && !done) {
                    int jj = 0;
                    for (; jj + J <= jcnt; jj += J) {
                        float d[J];
                        dist_block<METRIC, J, VEC4>(xcol, cs + (size_t)jj * sd, sd, P.pv, na, d);
#pragma unroll
                        for (int t = 0; t < J; ++t) {
                            const int j = j0 + jj + t;
                            if (j == 0) {
                                best = d[t];
                                idx = 0;
                            } else {
                                argmin_update(d[t], j, best, idx);
                            }
                        }
                    }
                    for (; jj < jcnt; ++jj) {
                        float d[1];
                        dist_block<METRIC, 1, VEC4>(xcol, cs + (size_t)jj * sd, sd, P.pv, na, d);
                        const int j = j0 + jj;
                        if (j == 0) {
                            best = d[0];
                            idx = 0;
                        } else {
                            argmin_update(d[0], j, best, idx);
                        }
                    }
                }
            }

            if (!valid || done) continue;
            if (MODE == G_TRAIN) {
                CodeT *cp = reinterpret_cast<CodeT *>(P.codes) + row * P.m + s;
                const CodeT nc = (CodeT)idx;
                if (*cp != nc) moved = true;
                *cp = nc;
            } else if (MODE == G_ENCODE) {
                const float *cw = cb + (size_t)idx * sd;
                if (P.out_codes) P.out_codes[row * P.m + s] = (uint32_t)idx;
                if (P.out_f16) {
                    uint16_t *o = P.out_f16 + row * dim + (size_t)s * sd;
                    for (int i = 0; i < sd; ++i) o[i] = f32_to_f16_bits(cw[i]);
                }
                if (P.out_f32) {
                    float *o = P.out_f32 + row * dim + (size_t)s * sd;
                    for (int i = 0; i < sd; ++i) o[i] = cw[i];
                }
            } else { // residual update: res -= chosen, then its L2 norm (src/rvq.rs:127,133-135 / 200-207)
                const float *cw = cb + (size_t)idx * sd;
                float nsq = 0.0f;
                for (int i = 0; i < sd; ++i) {
                    const float c = cw[i];
                    const float r = __fsub_rn(xs[i * VQB_XS_STRIDE + lane], c);
                    xs[i * VQB_XS_STRIDE + lane] = r;
                    nsq = __fadd_rn(nsq, __fmul_rn(r, r));
                    if (MODE == G_RVQ_QUANT) qs[i * VQB_XS_STRIDE + lane] = __fadd_rn(qs[i * VQB_XS_STRIDE + lane], c);
                }
                const float nrm = __fsqrt_rn(nsq);
                if (MODE == G_RVQ_UPDATE) warp_norm += (double)nrm;
                if (MODE == G_RVQ_QUANT) {
                    if (P.out_codes) P.out_codes[row * (unsigned long long)P.stages + st] = (uint32_t)idx;
                    if (nrm < P.epsilon) done = true;
                }
            }
        }

        if (MODE == G_RVQ_UPDATE || MODE == G_RVQ_QUANT) {
            __syncwarp();
            for (int r = 0; r < 32; ++r) {
                const unsigned long long rr = wrow0 + r;
                if (rr >= P.n) break;
                for (int i = lane; i < sd; i += 32) {
                    if (MODE == G_RVQ_UPDATE) {
                        P.res[rr * P.ld + i] = xs[i * VQB_XS_STRIDE + r];
                    } else {
                        const float q = qs[i * VQB_XS_STRIDE + r];
                        if (P.out_f16) P.out_f16[rr * sd + i] = f32_to_f16_bits(q);
                        if (P.out_f32) P.out_f32[rr * sd + i] = q;
                    }
                }
            }
            __syncwarp();
        }
    }
    if (MODE == G_TRAIN) {
        if (__any_sync(0xffffffffu, moved) && lane == 0) atomicOr(P.changed + s, VQB_MOVED_BITS);
    }
    if (MODE == G_RVQ_UPDATE) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) warp_norm += __shfl_xor_sync(0xffffffffu, warp_norm, o);
        if (lane == 0 && warp_norm != 0.0) atomicAdd(P.norm_sum, warp_norm);
    }
}

} // namespace vqb
