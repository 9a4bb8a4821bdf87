// assign_filter.cuh -- the fast form of the narrow-subspace nearest-centroid search (squared Euclidean and
// Euclidean; training src/utils.rs:59-73 and encode src/pq.rs:159-182).
//
// The reference's distance needs 3 un-fused f32 operations per dimension.  This kernel ranks centroids with the
// FMA form  S_j = |c_j|^2/2 - x.c_j  (one FFMA per dimension;  |x - c_j|^2 = |x|^2 + 2 S_j), keeps the best and the
// runner-up, and accepts the best ONLY when the gap to the runner-up exceeds a proven bound on everything that can
// separate the two rankings: the rounding of the FMA chain, the rounding of the reference's own chain, and (for the
// Euclidean metric) the merging of neighbouring sums by sqrt.  Otherwise the row slice is re-examined: every centroid
// whose S lies within the bound of the best is evaluated with the reference's exact arithmetic, in ascending index
// with strict '<', which reproduces the reference's choice.  The result is therefore identical to the exact kernel.
//
// Bound.  u = 2^-24.  Let d_j be the true squared distance, D_j the reference's f32 value, xh = |x|^2/2,
// HN_j the stored f32 value of |c_j|^2/2.
//   reference chain:   |D_j - d_j| <= 10u d_j                 (sub, mul, <= 7 adds of non-negative terms)
//   FMA chain:         |S_j - (HN_j - x.c_j)| <= 8.1u (HN_j + sum|x_i c_ji|) <= 8.1u (xh + 2.001 hn_j)
//   stored half norm:  |HN_j - hn_j| <= 9u hn_j
//   =>  |d_j/2 - (xh + S_j)| <= E := 9u xh + 26u HNmax.
// If the reference picks w != a (a = argmin S) then D_w <= D_a (or, Euclidean, sqrt(D_w) <= sqrt(D_a), which allows
// D_w <= D_a (1 + 4u)), hence  S_w <= S_a + 2E + 13u d_a  with  d_a <= 2 (xh + S_a + E).  With the comparison's own
// rounding this is covered by   margin = 64u (xh + HNmax + |S_a| + |S_b|) + 1e-36   (coefficients: xh 18+26 <= 64,
// HNmax 52 <= 64, |S_a| 26+4 <= 64).  Any non-finite value makes the comparison fail and sends the row to the re-check.
#pragma once
#include "assign_reg.cuh"

namespace vqb {

#define VQB_FILTER_COEF 3.814697265625e-06f /* 64 * 2^-24 */

// Packed pair of f32 in one 64-bit register (sm_100 issues one FFMA2 for two FMAs).
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float lo, float hi)
{
    f32x2 r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ float hsum2(f32x2 v)
{
    float lo, hi;
    asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo + hi;
}

// S = hn - x.c with the dimensions split into (even, odd) lanes of packed FMAs; nx holds (-x[2t], -x[2t+1]),
// c the centroid's packed pairs, h0 = (hn, 0).  The same instruction sequence is used by the scan and by the
// re-check, so a given (row, centroid) always yields the same bits.
template <int SD> __device__ __forceinline__ float fma_score(const f32x2 (&nx)[SD / 2], const f32x2 (&c)[SD / 2], f32x2 h0)
{
    f32x2 acc = h0;
#pragma unroll
    for (int t = 0; t < SD / 2; ++t) acc = fma2(nx[t], c[t], acc);
    return hsum2(acc);
}

template <int SD> __device__ __forceinline__ void load_centroid2(f32x2 (&c)[SD / 2], const float *p)
{
    if (SD % 4 == 0) {
#pragma unroll
        for (int i = 0; i < SD / 4; ++i) {
            const ulonglong2 q = reinterpret_cast<const ulonglong2 *>(p)[i];
            c[2 * i] = q.x;
            c[2 * i + 1] = q.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < SD / 2; ++i) c[i] = reinterpret_cast<const unsigned long long *>(p)[i];
    }
}

template <int SD> __device__ __forceinline__ void unpack_centroid(float (&c)[SD], const f32x2 (&c2)[SD / 2])
{
#pragma unroll
    for (int t = 0; t < SD / 2; ++t) asm("mov.b64 {%0,%1}, %2;" : "=f"(c[2 * t]), "=f"(c[2 * t + 1]) : "l"(c2[t]));
}

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN>
__global__ void __launch_bounds__((SD == 8 && V == 2) ? 1024 : 512, 1) assign_filter_kernel(const AssignParams P)
{
    static_assert(METRIC == M_SQ || METRIC == M_EUCLID, "the FMA filter is defined for the Euclidean metrics");
    static_assert(SD % 2 == 0, "even sub-space width");
    extern __shared__ __align__(16) float smem[];
    const int k = P.k, G = P.group;
    const int g0 = blockIdx.y * G;
    const int gcount = min(G, P.m - g0);
    float *cb = smem;                         // [G][k][SD]
    float *hn = smem + (size_t)G * k * SD;    // [G][k]   |c|^2 / 2
    float *hmax = hn + (size_t)G * k;         // [G]      max_j hn

    {
        const float *src = P.centroids + (size_t)g0 * k * SD;
        const int total = gcount * k * SD;
        for (int t = threadIdx.x; t < total; t += blockDim.x) cb[t] = src[t];
    }
    __syncthreads();
    for (int t = threadIdx.x; t < gcount * k; t += blockDim.x) {
        const float *c = cb + (size_t)t * SD;
        float a = 0.0f;
#pragma unroll
        for (int i = 0; i < SD; ++i) a = fmaf(c[i], c[i], a);
        hn[t] = 0.5f * a;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp < gcount) { // one warp per subspace reduces the largest half norm
        float mx = 0.0f;
        for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(hn[(size_t)warp * k + j]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) hmax[warp] = mx;
    }
    __syncthreads();

    const int W = blockDim.x >> 5;
    const int rbw = W / G;
    const int s_local = warp % G;
    const int s = g0 + s_local;
    if (s >= P.m) return;
    if (TRAIN && P.active && P.active[s] == 0) return;
    const float *cbs = cb + (size_t)s_local * k * SD;
    const float *hns = hn + (size_t)s_local * k;
    const float hnmax = hmax[s_local];
    const unsigned long long rows_per_block = 32ull * V;
    const unsigned long long n_blocks = (P.n + rows_per_block - 1) / rows_per_block;
    bool moved = false;

    for (unsigned long long blk = (unsigned long long)blockIdx.x * rbw + (warp / G); blk < n_blocks;
         blk += (unsigned long long)gridDim.x * rbw) {
        const unsigned long long row0 = blk * rows_per_block + lane;
        float x[V][SD];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            unsigned long long row = row0 + 32ull * v;
            if (row < P.n) {
                load_slice<SD>(x[v], P.x + row * P.ld + (size_t)s * SD, P.x_vec4 != 0);
            } else {
#pragma unroll
                for (int i = 0; i < SD; ++i) x[v][i] = 0.0f;
            }
        }

        f32x2 nx[V][SD / 2];
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int t = 0; t < SD / 2; ++t) nx[v][t] = pack2(-x[v][2 * t], -x[v][2 * t + 1]);

        float best[V], second[V];
        int idx[V];
        bool force[V]; // centroid 0 not comparable (NaN score): the reference's scan depends on it, so re-examine
        {
            f32x2 c[SD / 2];
            load_centroid2<SD>(c, cbs);
            const f32x2 h0 = pack2(hns[0], 0.0f);
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float s0 = fma_score<SD>(nx[v], c, h0);
                force[v] = !(s0 == s0);
                best[v] = VQB_INF;
                second[v] = VQB_INF;
                idx[v] = 0;
            }
        }
        // two centroids per step: lo/hi of the pair, then one update of (best, second, idx)
        int j = 0;
        for (; j + 2 <= k; j += 2) {
            f32x2 ca[SD / 2], cb2[SD / 2];
            load_centroid2<SD>(ca, cbs + (size_t)j * SD);
            load_centroid2<SD>(cb2, cbs + (size_t)(j + 1) * SD);
            const f32x2 ha = pack2(hns[j], 0.0f), hb = pack2(hns[j + 1], 0.0f);
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float sa = fma_score<SD>(nx[v], ca, ha);
                const float sb = fma_score<SD>(nx[v], cb2, hb);
                const float lo = fminf(sa, sb), hi = fmaxf(sa, sb);
                const int jlo = (sb < sa) ? j + 1 : j; // equal scores keep the lower index
                const bool lt = lo < best[v];
                second[v] = min3f(second[v], fmaxf(best[v], lo), hi); // second smallest of {best, second, lo, hi}
                best[v] = fminf(best[v], lo);
                idx[v] = lt ? jlo : idx[v];
            }
        }
        for (; j < k; ++j) {
            f32x2 c[SD / 2];
            load_centroid2<SD>(c, cbs + (size_t)j * SD);
            const f32x2 h0 = pack2(hns[j], 0.0f);
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float sc = fma_score<SD>(nx[v], c, h0);
                const bool lt = sc < best[v];
                second[v] = fmaxf(best[v], fminf(second[v], sc));
                best[v] = fminf(best[v], sc);
                idx[v] = lt ? j : idx[v];
            }
        }

        // accept, or re-examine the near candidates with the reference's arithmetic
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float xh = 0.0f;
#pragma unroll
            for (int i = 0; i < SD; ++i) xh = fmaf(x[v][i], x[v][i], xh);
            xh *= 0.5f;
            const float margin = VQB_FILTER_COEF * (xh + hnmax + fabsf(best[v]) + fabsf(second[v])) + 1e-36f;
            const float limit = best[v] + margin;
            if (force[v] || !(second[v] > limit)) { // also taken when anything is NaN or infinite
                float bd = VQB_INF;
                int bi = -1;
                for (int jj = 0; jj < k; ++jj) {
                    f32x2 c2[SD / 2];
                    load_centroid2<SD>(c2, cbs + (size_t)jj * SD);
                    const float sc = fma_score<SD>(nx[v], c2, pack2(hns[jj], 0.0f));
                    if (!(sc > limit)) { // candidate (or not comparable): exact distance, reference order
                        float c[SD];
                        unpack_centroid<SD>(c, c2);
                        float d = reg_dist<SD, M_SQ>(x[v], c, 0.0f, 0.0f, 0.0f);
                        if (METRIC == M_EUCLID) d = __fsqrt_rn(d);
                        if (jj == 0) { // the reference's scan starts here, whatever the value (even NaN)
                            bd = d;
                            bi = 0;
                        } else {
                            // if centroid 0 was skipped it is provably farther than the winner, so starting the
                            // strict-'<' scan from +inf at the first candidate gives the same answer
                            argmin_update(d, jj, bd, bi);
                        }
                    }
                }
                idx[v] = bi < 0 ? 0 : bi;
            }
        }

#pragma unroll
        for (int v = 0; v < V; ++v) {
            unsigned long long row = row0 + 32ull * v;
            if (row < P.n) store_result<SD, CodeT, TRAIN>(P, row, s, idx[v], cbs, moved);
        }
    }
    if (TRAIN) {
        if (__any_sync(0xffffffffu, moved) && lane == 0) atomicOr(P.changed + s, VQB_MOVED_BITS);
    }
}

} // namespace vqb
