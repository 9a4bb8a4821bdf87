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

template <int SD> __device__ __forceinline__ float fma_score(const float (&x)[SD], const float (&c)[SD], float hn)
{
    // two interleaved chains (even / odd dimensions) so that consecutive FFMAs are independent
    float a0 = hn, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < SD; i += 2) {
        a0 = fmaf(-x[i], c[i], a0);
        a1 = fmaf(-x[i + 1], c[i + 1], a1);
    }
    return a0 + a1;
}

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN>
__global__ void __launch_bounds__(512, 1) assign_filter_kernel(const AssignParams P)
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

        float best[V], second[V];
        int idx[V];
        bool force[V]; // centroid 0 not comparable (NaN score): the reference's scan depends on it, so re-examine
        {
            float c[SD];
            load_centroid<SD>(c, cbs);
            const float h = hns[0];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float s0 = fma_score<SD>(x[v], c, h);
                force[v] = !(s0 == s0);
                best[v] = VQB_INF;
                second[v] = VQB_INF;
                idx[v] = 0;
            }
        }
#pragma unroll 2
        for (int j = 0; j < k; ++j) {
            float c[SD];
            load_centroid<SD>(c, cbs + (size_t)j * SD);
            const float h = hns[j];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float sc = fma_score<SD>(x[v], c, h);
                const bool lt = sc < best[v];
                second[v] = fmaxf(best[v], fminf(second[v], sc)); // second smallest of {best, second, sc}
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
                for (int j = 0; j < k; ++j) {
                    float c[SD];
                    load_centroid<SD>(c, cbs + (size_t)j * SD);
                    const float sc = fma_score<SD>(x[v], c, hns[j]);
                    if (!(sc > limit)) { // candidate (or not comparable): exact distance, reference order
                        float d = reg_dist<SD, M_SQ>(x[v], c, 0.0f, 0.0f, 0.0f);
                        if (METRIC == M_EUCLID) d = __fsqrt_rn(d);
                        if (j == 0) { // the reference's scan starts here, whatever the value (even NaN)
                            bd = d;
                            bi = 0;
                        } else {
                            // if centroid 0 was skipped it is provably farther than the winner, so starting the
                            // strict-'<' scan from +inf at the first candidate gives the same answer
                            argmin_update(d, j, bd, bi);
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
        if (__any_sync(0xffffffffu, moved) && lane == 0) atomicOr(P.changed + s, 1u);
    }
}

} // namespace vqb
