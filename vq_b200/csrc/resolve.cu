// resolve.cu -- exact decision among shortlisted centroids (the second half of the tensor-core path, dense_tc.cu).
//
// For every row the shortlist holds, in ascending order, every centroid that can be the reference's choice.  Here each
// candidate's distance is evaluated with the reference's own f32 arithmetic (src/vector.rs:198-220, src/distances.rs:
// 130-140) and compared with strict '<', so the outcome equals the reference's full scan; rows marked "scan all" get that
// full scan.  The epilogue is the caller's: new assignment (training), residual update (src/rvq.rs:127,133-138), or one
// stage of the residual encoder (src/rvq.rs:186-207).
#include <algorithm>

#include "cuda_device.hpp"
#include "dense_tc.hpp"
#include "kernels_common.cuh"

namespace vqb {

namespace {

// Index of the lowest set bit at or above `from` in a 256-bit mask, or 256.
__device__ __forceinline__ int next_bit(const uint32_t (&w)[8], int from)
{
    for (int wd = from >> 5; wd < 8; ++wd) {
        uint32_t m = w[wd];
        if (wd == (from >> 5)) m &= 0xFFFFFFFFu << (from & 31);
        if (m) return wd * 32 + __ffs(m) - 1;
    }
    return 256;
}

// Reference distance of one row (xcol, stride XT_STRIDE) to two centroids at once: two independent serial chains.
#define XT_STRIDE 17
__device__ __forceinline__ void exact_dist2(const float *xcol, const float *c0, const float *c1, int dim, bool euclid, float (&out)[2])
{
    float a0 = 0.0f, a1 = 0.0f;
    for (int i0 = 0; i0 < dim; i0 += 8) {
        float xv[8], v0[8], v1[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            xv[u] = xcol[(i0 + u) * XT_STRIDE];
            v0[u] = c0[i0 + u], v1[u] = c1[i0 + u];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float d0 = __fsub_rn(xv[u], v0[u]), d1 = __fsub_rn(xv[u], v1[u]);
            a0 = __fadd_rn(a0, __fmul_rn(d0, d0));
            a1 = __fadd_rn(a1, __fmul_rn(d1, d1));
        }
    }
    out[0] = euclid ? __fsqrt_rn(a0) : a0;
    out[1] = euclid ? __fsqrt_rn(a1) : a1;
}

// Tiles of 16 rows, two lanes per row (see resolve_train_kernel below for why): both lanes of a row evaluate two of its next
// four candidates each and walk through the four distances in ascending centroid order; the row's epilogue (residual, norm,
// flags) is the first lane's.
constexpr int RT_MAX_WARPS = 12;
template <int MODE, typename CodeT> __global__ void __launch_bounds__(32 * RT_MAX_WARPS, 1) resolve_kernel(const ResolveParams P)
{
    extern __shared__ __align__(16) float smem[];
    const int dim = P.dim, k = P.k, cstride = dim + 1; // odd stride: lanes reading different centroids hit different banks
    const int W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *cpad = smem;                                   // [k][dim + 1]
    float *xs = smem + (size_t)k * cstride + (size_t)warp * dim * XT_STRIDE; // [dim][17] per warp
    {
        // codebook -> shared memory, eight 128-bit loads in flight per thread (dim is a multiple of 4 on this path)
        const int total4 = k * dim / 4, dim4 = dim / 4;
        const float4 *src = reinterpret_cast<const float4 *>(P.codebook);
        for (int base = 0; base < total4; base += 8 * (int)blockDim.x) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = base + u * (int)blockDim.x + (int)threadIdx.x;
                v[u] = (t < total4) ? __ldg(src + t) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = base + u * (int)blockDim.x + (int)threadIdx.x;
                if (t < total4) {
                    float *d = cpad + (size_t)(t / dim4) * cstride + (size_t)(t % dim4) * 4;
                    d[0] = v[u].x, d[1] = v[u].y, d[2] = v[u].z, d[3] = v[u].w;
                }
            }
        }
    }
    __syncthreads();
    const bool euclid = P.euclid != 0;
    const unsigned long long tiles = (P.n + 15) / 16;
    bool moved = false;
    double warp_norm = 0.0;
    const int r = lane & 15, half = lane >> 4;

    // A warp's next tile (16 rows, up to 8 KiB) is requested into registers while the current one is worked on.
    const int dim4 = dim / 4, total4 = 16 * dim4;
    float4 pre[16];
    auto request = [&](unsigned long long tile) {
        const unsigned long long r0 = tile * 16;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int idx = u * 32 + lane;
            const unsigned long long rr = r0 + idx / dim4;
            pre[u] = (tile < tiles && idx < total4 && rr < P.n) ? __ldg(reinterpret_cast<const float4 *>(P.x + rr * dim) + idx % dim4)
                                                              : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    request((unsigned long long)blockIdx.x * W + warp);
    for (unsigned long long tile = (unsigned long long)blockIdx.x * W + warp; tile < tiles; tile += (unsigned long long)gridDim.x * W) {
        const unsigned long long row0 = tile * 16, row = row0 + r;
        const bool valid = row < P.n;
        bool skip = false;
        if (MODE == R_RVQ_STAGE && valid) skip = P.done[row] != 0;
        // stage the 16 rows dimension-major (lanes walked along a row when they were loaded: coalesced), then ask for the next tile
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int idx = u * 32 + lane;
            if (idx < total4) {
                float *d = xs + (size_t)(idx % dim4) * 4 * XT_STRIDE + idx / dim4;
                d[0] = pre[u].x, d[XT_STRIDE] = pre[u].y, d[2 * XT_STRIDE] = pre[u].z, d[3 * XT_STRIDE] = pre[u].w;
            }
        }
        request(tile + (unsigned long long)gridDim.x * W);
        __syncwarp();
        const float *xcol = xs + r;
        int best = 0;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int ncand = 0;
        if (valid && !skip) {
            const uint4 lo = reinterpret_cast<const uint4 *>(P.cand + row * 8)[0], hi = reinterpret_cast<const uint4 *>(P.cand + row * 8)[1];
            w[0] = lo.x, w[1] = lo.y, w[2] = lo.z, w[3] = lo.w, w[4] = hi.x, w[5] = hi.y, w[6] = hi.z, w[7] = hi.w;
#pragma unroll
            for (int t = 0; t < 8; ++t) ncand += __popc(w[t]);
        }
        // Rows with many candidates (or marked "examine all") are scanned by the whole warp: lane L takes centroids
        // L, L+32, ... in ascending order, then the warp keeps the smallest distance, lowest index on ties.  A NaN never
        // wins in the reference unless it sits at centroid 0, where the scan starts.
        const bool wide = ncand > 12;
        unsigned wide_rows = __ballot_sync(0xffffffffu, wide) & 0xFFFFu;
        while (wide_rows) {
            const int wr = __ffs(wide_rows) - 1;
            wide_rows &= wide_rows - 1;
            const float *xr = xs + wr;
            float bd = VQB_DENSE_INF;
            int bi = 0x7fffffff;
            float d0 = 0.0f;
            for (int j = lane; j < k; j += 32) {
                const float *c = cpad + (size_t)j * cstride;
                float acc = 0.0f;
#pragma unroll 8
                for (int i = 0; i < dim; ++i) {
                    const float d = __fsub_rn(xr[i * XT_STRIDE], c[i]);
                    acc = __fadd_rn(acc, __fmul_rn(d, d));
                }
                const float d = euclid ? __fsqrt_rn(acc) : acc;
                if (j == 0) d0 = d;
                if (d < bd) {
                    bd = d;
                    bi = j;
                }
            }
            d0 = __shfl_sync(0xffffffffu, d0, 0);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float od = __shfl_xor_sync(0xffffffffu, bd, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (od < bd || (od == bd && oi < bi)) {
                    bd = od;
                    bi = oi;
                }
            }
            int res = (bi == 0x7fffffff) ? 0 : bi; // nothing finite below +inf: the reference keeps centroid 0
            if (!(d0 == d0)) res = 0;               // NaN at centroid 0: nothing ever replaces it (src/utils.rs:62-66)
            if (bd == VQB_DENSE_INF) res = 0;       // all distances +inf (or NaN): strict '<' never fires
            if (r == wr) best = res;
        }
        // the other rows: rounds of four candidates, two per lane of the pair; every lane of the warp takes part in a round
        {
            float bd = VQB_DENSE_INF;
            int bi = -1;
            int j = (valid && !skip && !wide) ? next_bit(w, 0) : 256;
            while (__any_sync(0xffffffffu, j < k)) {
                int js[4];
                js[0] = j;
#pragma unroll
                for (int t = 1; t < 4; ++t) js[t] = (js[t - 1] < 256) ? next_bit(w, js[t - 1] + 1) : 256;
                const int ja = half ? js[2] : js[0], jb = half ? js[3] : js[1];
                float mine[2];
                exact_dist2(xcol, cpad + (size_t)min(ja, k - 1) * cstride, cpad + (size_t)min(jb, k - 1) * cstride, dim, euclid, mine);
                const float o0 = __shfl_xor_sync(0xffffffffu, mine[0], 16), o1 = __shfl_xor_sync(0xffffffffu, mine[1], 16);
                const float d[4] = {half ? o0 : mine[0], half ? o1 : mine[1], half ? mine[0] : o0, half ? mine[1] : o1};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    if (js[t] >= k) break;
                    if (js[t] == 0) { // the reference's scan starts at centroid 0 whatever its value
                        bd = d[t];
                        bi = 0;
                    } else {
                        argmin_update(d[t], js[t], bd, bi); // a skipped centroid 0 is provably farther than the winner
                    }
                }
                j = (js[3] < 256) ? next_bit(w, js[3] + 1) : 256;
            }
            if (valid && !skip && !wide) best = bi < 0 ? 0 : bi;
        }
        if (valid && !skip && half == 0) {
            if (MODE == R_TRAIN) {
                CodeT *cp = reinterpret_cast<CodeT *>(P.codes) + row;
                const CodeT nc = (CodeT)best;
                if (*cp != nc) moved = true;
                *cp = nc;
            } else {
                const float *cw = cpad + (size_t)best * cstride;
                float nsq = 0.0f;
#pragma unroll 8
                for (int i = 0; i < dim; ++i) {
                    const float rv = __fsub_rn(xs[i * XT_STRIDE + r], cw[i]);
                    xs[i * XT_STRIDE + r] = rv;
                    nsq = __fadd_rn(nsq, __fmul_rn(rv, rv));
                }
                const float nrm = __fsqrt_rn(nsq);
                if (MODE == R_RVQ_UPDATE) warp_norm += (double)nrm;
                if (MODE == R_RVQ_STAGE) {
                    if (P.out_codes) P.out_codes[row * (unsigned long long)P.stages + P.stage] = (uint32_t)best;
                    if (nrm < P.epsilon) P.done[row] = 1;
                }
            }
        }
        if (MODE != R_TRAIN) {
            // write the residual tile back; R_RVQ_STAGE also adds the chosen centroid to the running sum
            const int mybest = (valid && !skip) ? best : -1;
            __syncwarp();
            // four rows per step; the running-sum reads of a step are all issued before any is used
            for (int r0 = 0; r0 < 16; r0 += 4) {
                int b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    b[u] = __shfl_sync(0xffffffffu, mybest, r0 + u);
                    if (row0 + r0 + u >= P.n) b[u] = -1;
                }
                for (int i0 = 0; i0 < dim; i0 += 128) {
                    float q[4][4];
                    if (MODE == R_RVQ_STAGE) {
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int i = i0 + e * 32 + lane;
                                q[u][e] = (b[u] >= 0 && i < dim) ? P.qsum[(row0 + r0 + u) * dim + i] : 0.0f;
                            }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (b[u] < 0) continue;
                        const unsigned long long rr = row0 + r0 + u;
                        const float *cw = cpad + (size_t)b[u] * cstride;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = i0 + e * 32 + lane;
                            if (i >= dim) continue;
                            P.res[rr * dim + i] = xs[i * XT_STRIDE + r0 + u];
                            if (MODE == R_RVQ_STAGE) P.qsum[rr * dim + i] = __fadd_rn(q[u][e], cw[i]);
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
    if (MODE == R_TRAIN) {
        if (__any_sync(0xffffffffu, moved) && lane == 0) atomicOr(P.changed, VQB_MOVED_BITS);
    }
    if (MODE == R_RVQ_UPDATE) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) warp_norm += __shfl_xor_sync(0xffffffffu, warp_norm, o);
        if (lane == 0 && warp_norm != 0.0) atomicAdd(P.norm_sum, warp_norm);
    }
}

// Training assignment of the rows the shortlist kernel could not decide (more than one candidate, or "examine all"); the
// rows with a single candidate got their assignment there and are never read here.  A warp takes 16 listed rows at a time and
// gives every row TWO lanes, each of which evaluates two of the row's next four candidates with the exact arithmetic; the pair
// then goes through the four distances in ascending centroid order like the reference.  Sixteen-row groups halve a warp's
// staging buffer, which is what lets ten warps instead of four sit beside the 132 KB codebook: with one warp per scheduler
// the serial chains ran at a quarter of the issue rate.
template <typename CodeT> __global__ void __launch_bounds__(32 * RT_MAX_WARPS, 1) resolve_train_kernel(const ResolveParams P)
{
    extern __shared__ __align__(16) float smem[];
    const int dim = P.dim, k = P.k, cstride = dim + 1;
    const int W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long cnt = *reinterpret_cast<const volatile uint32_t *>(P.list_count);
    const unsigned long long groups = (cnt + 15) / 16;
    if ((unsigned long long)blockIdx.x * W >= groups) return; // nothing for this CTA: skip the codebook copy as well
    float *cpad = smem;                                                                   // [k][dim + 1]
    float *xs = smem + (size_t)k * cstride + (size_t)warp * dim * XT_STRIDE;              // [dim][17] per warp
    {
        const int total4 = k * dim / 4, dim4 = dim / 4;
        const float4 *src = reinterpret_cast<const float4 *>(P.codebook);
        for (int base = 0; base < total4; base += 8 * (int)blockDim.x) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = base + u * (int)blockDim.x + (int)threadIdx.x;
                v[u] = (t < total4) ? __ldg(src + t) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = base + u * (int)blockDim.x + (int)threadIdx.x;
                if (t < total4) {
                    float *d = cpad + (size_t)(t / dim4) * cstride + (size_t)(t % dim4) * 4;
                    d[0] = v[u].x, d[1] = v[u].y, d[2] = v[u].z, d[3] = v[u].w;
                }
            }
        }
    }
    __syncthreads();
    const bool euclid = P.euclid != 0;
    bool moved = false;
    CodeT *codes = reinterpret_cast<CodeT *>(P.codes);
    const int r = lane & 15, half = lane >> 4;
    const int dim4 = dim / 4;
    // the next group's rows are requested into registers while this one is evaluated
    float4 pre[16];
    auto request = [&](unsigned long long g) {
        const int nb = g < groups ? (int)min(16ull, cnt - g * 16) : 0, total4 = nb * dim4;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int idx = u * 32 + lane;
            pre[u] = idx < total4 ? __ldg(reinterpret_cast<const float4 *>(P.x + (unsigned long long)P.list[g * 16 + idx / dim4] * dim) + idx % dim4)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    const unsigned long long g0 = (unsigned long long)blockIdx.x * W + warp, gstep = (unsigned long long)gridDim.x * W;
    request(g0);
    for (unsigned long long g = g0; g < groups; g += gstep) {
        const int nb = (int)min(16ull, cnt - g * 16);
        {
            const int total4 = nb * dim4;
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int idx = u * 32 + lane;
                if (idx < total4) {
                    float *d = xs + (size_t)(idx % dim4) * 4 * XT_STRIDE + idx / dim4;
                    d[0] = pre[u].x, d[XT_STRIDE] = pre[u].y, d[2 * XT_STRIDE] = pre[u].z, d[3 * XT_STRIDE] = pre[u].w;
                }
            }
        }
        request(g + gstep);
        __syncwarp();
        const bool valid = r < nb; // both lanes of a row agree on everything below
        const unsigned long long row = valid ? P.list[g * 16 + r] : 0ull;
        const float *xcol = xs + r;
        int best = 0, ncand = 0;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (valid) {
            const uint4 lo = __ldg(reinterpret_cast<const uint4 *>(P.cand + row * 8)), hi = __ldg(reinterpret_cast<const uint4 *>(P.cand + row * 8) + 1);
            w[0] = lo.x, w[1] = lo.y, w[2] = lo.z, w[3] = lo.w, w[4] = hi.x, w[5] = hi.y, w[6] = hi.z, w[7] = hi.w;
#pragma unroll
            for (int e = 0; e < 8; ++e) ncand += __popc(w[e]);
        }
        // rows with many candidates (or marked "examine all"): the whole warp scans all centroids, as in resolve_kernel
        const bool wide = valid && (ncand > 12 || ncand == 0);
        unsigned wide_rows = __ballot_sync(0xffffffffu, wide) & 0xFFFFu;
        while (wide_rows) {
            const int wr = __ffs(wide_rows) - 1;
            wide_rows &= wide_rows - 1;
            const float *xr = xs + wr;
            float bd = VQB_DENSE_INF, d0 = 0.0f;
            int bi = 0x7fffffff;
            for (int j = lane; j < k; j += 32) {
                const float *c = cpad + (size_t)j * cstride;
                float acc = 0.0f;
#pragma unroll 8
                for (int i = 0; i < dim; ++i) {
                    const float d = __fsub_rn(xr[i * XT_STRIDE], c[i]);
                    acc = __fadd_rn(acc, __fmul_rn(d, d));
                }
                const float d = euclid ? __fsqrt_rn(acc) : acc;
                if (j == 0) d0 = d;
                if (d < bd) {
                    bd = d;
                    bi = j;
                }
            }
            d0 = __shfl_sync(0xffffffffu, d0, 0);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float od = __shfl_xor_sync(0xffffffffu, bd, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (od < bd || (od == bd && oi < bi)) {
                    bd = od;
                    bi = oi;
                }
            }
            int res = (bi == 0x7fffffff) ? 0 : bi;
            if (!(d0 == d0)) res = 0;
            if (bd == VQB_DENSE_INF) res = 0;
            if (r == wr) best = res;
        }
        // the other rows: rounds of four candidates, two per lane of the pair
        float bd = VQB_DENSE_INF;
        int bi = -1;
        int j = (valid && !wide) ? next_bit(w, 0) : 256;
        while (__any_sync(0xffffffffu, j < k)) {
            int js[4];
            js[0] = j;
#pragma unroll
            for (int t = 1; t < 4; ++t) js[t] = (js[t - 1] < 256) ? next_bit(w, js[t - 1] + 1) : 256;
            const int ja = half ? js[2] : js[0], jb = half ? js[3] : js[1];
            float mine[2];
            exact_dist2(xcol, cpad + (size_t)min(ja, k - 1) * cstride, cpad + (size_t)min(jb, k - 1) * cstride, dim, euclid, mine);
            const float o0 = __shfl_xor_sync(0xffffffffu, mine[0], 16), o1 = __shfl_xor_sync(0xffffffffu, mine[1], 16);
            const float d[4] = {half ? o0 : mine[0], half ? o1 : mine[1], half ? mine[0] : o0, half ? mine[1] : o1};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                if (js[t] >= k) break;
                if (js[t] == 0) {
                    bd = d[t];
                    bi = 0;
                } else {
                    argmin_update(d[t], js[t], bd, bi);
                }
            }
            j = (js[3] < 256) ? next_bit(w, js[3] + 1) : 256;
        }
        if (valid && half == 0) {
            if (!wide) best = bi < 0 ? 0 : bi;
            const CodeT nc = (CodeT)best;
            if (codes[row] != nc) moved = true;
            codes[row] = nc;
        }
        __syncwarp();
    }
    if (__any_sync(0xffffffffu, moved) && lane == 0) atomicOr(P.changed, VQB_MOVED_BITS);
}

// as many warps as fit beside the padded codebook (ten at k = 256, dim = 128)
static int resolve_warps(const ResolveParams &p, size_t extra_per_warp, size_t *smem)
{
    const size_t book = (size_t)p.k * (p.dim + 1) * sizeof(float), per_warp = (size_t)p.dim * XT_STRIDE * sizeof(float) + extra_per_warp;
    const size_t budget = 226 * 1024;
    const int warps = (int)std::max<size_t>(1, std::min<size_t>(RT_MAX_WARPS, book < budget ? (budget - book) / per_warp : 1));
    *smem = book + (size_t)warps * per_warp;
    return warps;
}

template <int MODE, typename CodeT> void launch_t(CudaDevice &dev, const ResolveParams &p, const char *name)
{
    size_t smem = 0;
    const int warps = resolve_warps(p, 0, &smem);
    auto kernel = resolve_kernel<MODE, CodeT>;
    VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned long long tiles = (p.n + 15) / 16;
    const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((tiles + warps - 1) / warps, (unsigned long long)dev.sm_count()));
    KernelScope ks(dev, name);
    kernel<<<grid, 32 * warps, smem, dev.stream()>>>(p);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

template <typename CodeT> void launch_train(CudaDevice &dev, const ResolveParams &p)
{
    size_t smem = 0;
    const int warps = resolve_warps(p, 0, &smem);
    auto kernel = resolve_train_kernel<CodeT>;
    VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // the number of listed rows is only known on the device: CTAs without a group leave at once
    const unsigned long long groups = (p.n + 15) / 16;
    const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((groups + warps - 1) / warps, (unsigned long long)dev.sm_count()));
    KernelScope ks(dev, "resolve_train");
    kernel<<<grid, 32 * warps, smem, dev.stream()>>>(p);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

} // namespace

void launch_resolve(CudaDevice &dev, const ResolveParams &p, int mode, size_t cb)
{
    if (p.n == 0) return;
    if (mode == R_TRAIN) {
        if (cb == 1) launch_train<uint8_t>(dev, p);
        else if (cb == 2) launch_train<uint16_t>(dev, p);
        else launch_train<uint32_t>(dev, p);
    } else if (mode == R_RVQ_UPDATE) {
        launch_t<R_RVQ_UPDATE, uint32_t>(dev, p, "resolve_rvq_update");
    } else {
        launch_t<R_RVQ_STAGE, uint32_t>(dev, p, "resolve_rvq_stage");
    }
}

} // namespace vqb
