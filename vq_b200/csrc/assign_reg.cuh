// assign_reg.cuh -- nearest-centroid search for narrow subspaces (sub_dim 4, 8 or 16), the PQ hot loop.
//
// Replaces the per-point scan of src/utils.rs:59-73 (training, always squared Euclidean) and of
// src/pq.rs:159-182 / src/opq.rs:146-168,246-261 (encode, stored metric).
//
// Layout: a CTA keeps the codebooks of `group` consecutive subspaces in shared memory; each warp
// owns one subspace of the group and V*32 rows at a time, one row slice per lane and register set,
// so every centroid read is a shared-memory broadcast and every row slice is read from HBM once.
// Arithmetic is the reference's (see kernels_common.cuh); ties keep the lowest index.
#pragma once
#include "kernels_common.cuh"

namespace vqb {

struct AssignParams {
    const float *x;         // n rows, ld floats apart
    unsigned long long n;
    unsigned long long ld;
    int m, k, sd;
    int group;              // subspaces per CTA (gridDim.y = ceil(m / group)); divides the warp count
    const float *centroids; // [m][k][sd]
    void *codes;            // training: [n][m] previous assignment in, new assignment out
    const uint32_t *active; // training: per-subspace mask (may be null = all)
    uint32_t *changed;      // training: per-subspace "some row moved" flag
    uint16_t *out_f16;      // encode: [n][m*sd] binary16 bits (may be null)
    uint32_t *out_codes;    // encode: [n][m] (may be null)
    float *out_f32;         // encode: [n][m*sd] chosen centroid values in f32 (may be null)
    float pv;               // Minkowski p
    int x_vec4;             // row slices may be read with 128-bit loads
    int out_vec;            // f16 / f32 outputs may be written with 128-bit stores
};

template <int SD> __device__ __forceinline__ void load_slice(float (&v)[SD], const float *p, bool vec4)
{
    if (vec4 && (SD % 4 == 0)) {
#pragma unroll
        for (int i = 0; i < SD / 4; ++i) {
            float4 t = __ldg(reinterpret_cast<const float4 *>(p) + i);
            v[4 * i + 0] = t.x;
            v[4 * i + 1] = t.y;
            v[4 * i + 2] = t.z;
            v[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < SD; ++i) v[i] = __ldg(p + i);
    }
}

template <int SD> __device__ __forceinline__ void load_centroid(float (&c)[SD], const float *p)
{
    if (SD % 4 == 0) {
#pragma unroll
        for (int i = 0; i < SD / 4; ++i) {
            float4 t = reinterpret_cast<const float4 *>(p)[i];
            c[4 * i + 0] = t.x;
            c[4 * i + 1] = t.y;
            c[4 * i + 2] = t.z;
            c[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < SD; ++i) c[i] = p[i];
    }
}

// Distance of one register-resident row slice to one centroid, comparison form.
// For the Euclidean metric the fast scan compares squared sums; the caller resolves sqrt-merged ties.
template <int SD, int METRIC>
__device__ __forceinline__ float reg_dist(const float (&x)[SD], const float (&c)[SD], float pv, float norm_a, float norm_b)
{
    if (METRIC == M_SQ || METRIC == M_EUCLID) {
        float d0 = __fsub_rn(x[0], c[0]);
        float acc = __fmul_rn(d0, d0); // 0.0 + d0*d0 == d0*d0 exactly (a square is never -0.0)
#pragma unroll
        for (int i = 1; i < SD; ++i) {
            float d = __fsub_rn(x[i], c[i]);
            acc = __fadd_rn(acc, __fmul_rn(d, d));
        }
        return acc;
    } else if (METRIC == M_MANHATTAN) {
        float acc = fabsf(__fsub_rn(x[0], c[0]));
#pragma unroll
        for (int i = 1; i < SD; ++i) acc = __fadd_rn(acc, fabsf(__fsub_rn(x[i], c[i])));
        return acc;
    } else { // cosine; norm_b precomputed with the same serial chain
        float dot = __fadd_rn(0.0f, __fmul_rn(x[0], c[0]));
#pragma unroll
        for (int i = 1; i < SD; ++i) dot = __fadd_rn(dot, __fmul_rn(x[i], c[i]));
        if (norm_a == 0.0f || norm_b == 0.0f) return 1.0f;
        return __fsub_rn(1.0f, __fdiv_rn(dot, __fmul_rn(norm_a, norm_b)));
    }
}

// Writes the outcome for one (row, subspace): the new assignment while training (noting whether it moved), or
// the code / f16 / f32 image of the chosen centroid while encoding (src/pq.rs:176-180).
template <int SD, typename CodeT, bool TRAIN>
__device__ __forceinline__ void store_result(const AssignParams &P, unsigned long long row, int s, int idx, const float *cbs, bool &moved)
{
    const int dim = P.m * SD;
    if (TRAIN) {
        CodeT *cp = reinterpret_cast<CodeT *>(P.codes) + row * P.m + s;
        const CodeT nc = (CodeT)idx;
        if (*cp != nc) moved = true;
        *cp = nc;
    } else {
        if (P.out_codes) P.out_codes[row * P.m + s] = (uint32_t)idx;
        const float *cw = cbs + (size_t)idx * SD;
        if (P.out_f16) {
            uint16_t *o = P.out_f16 + row * dim + (size_t)s * SD;
            if (P.out_vec && SD % 8 == 0) {
#pragma unroll
                for (int i = 0; i < SD / 8; ++i) {
                    float4 a = reinterpret_cast<const float4 *>(cw)[2 * i], b = reinterpret_cast<const float4 *>(cw)[2 * i + 1];
                    uint4 pk;
                    pk.x = f32_to_f16_bits(a.x) | ((uint32_t)f32_to_f16_bits(a.y) << 16);
                    pk.y = f32_to_f16_bits(a.z) | ((uint32_t)f32_to_f16_bits(a.w) << 16);
                    pk.z = f32_to_f16_bits(b.x) | ((uint32_t)f32_to_f16_bits(b.y) << 16);
                    pk.w = f32_to_f16_bits(b.z) | ((uint32_t)f32_to_f16_bits(b.w) << 16);
                    reinterpret_cast<uint4 *>(o)[i] = pk;
                }
            } else {
#pragma unroll
                for (int i = 0; i < SD; ++i) o[i] = f32_to_f16_bits(cw[i]);
            }
        }
        if (P.out_f32) {
            float *o = P.out_f32 + row * dim + (size_t)s * SD;
            if (P.out_vec && SD % 4 == 0) {
#pragma unroll
                for (int i = 0; i < SD / 4; ++i) reinterpret_cast<float4 *>(o)[i] = reinterpret_cast<const float4 *>(cw)[i];
            } else {
#pragma unroll
                for (int i = 0; i < SD; ++i) o[i] = cw[i];
            }
        }
    }
}

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN>
__global__ void __launch_bounds__(512, 1) assign_reg_kernel(const AssignParams P)
{
    extern __shared__ __align__(16) float smem[];
    const int k = P.k, G = P.group;
    const int g0 = blockIdx.y * G;
    const int gcount = min(G, P.m - g0);
    float *cb = smem;                           // [G][k][SD]
    float *cnorm = smem + (size_t)G * k * SD;   // [G][k], cosine only

    {
        const float *src = P.centroids + (size_t)g0 * k * SD;
        const int total = gcount * k * SD;
        for (int t = threadIdx.x; t < total; t += blockDim.x) cb[t] = src[t];
    }
    __syncthreads();
    if (METRIC == M_COSINE) {
        for (int t = threadIdx.x; t < gcount * k; t += blockDim.x) cnorm[t] = norm_chain(cb + (size_t)t * SD, SD, 1);
        __syncthreads();
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = blockDim.x >> 5;
    const int rbw = W / G; // row blocks handled side by side
    const int s_local = warp % G;
    const int s = g0 + s_local;
    if (s >= P.m) return;
    if (TRAIN && P.active && P.active[s] == 0) return;
    const float *cbs = cb + (size_t)s_local * k * SD;
    const float *cns = cnorm + (size_t)s_local * k;
    const unsigned long long rows_per_block = 32ull * V;
    const unsigned long long n_blocks = (P.n + rows_per_block - 1) / rows_per_block;
    bool moved = false;

    for (unsigned long long blk = (unsigned long long)blockIdx.x * rbw + (warp / G); blk < n_blocks;
         blk += (unsigned long long)gridDim.x * rbw) {
        const unsigned long long row0 = blk * rows_per_block + lane;
        float x[V][SD];
        float na[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            unsigned long long row = row0 + 32ull * v;
            if (row < P.n) {
                load_slice<SD>(x[v], P.x + row * P.ld + (size_t)s * SD, P.x_vec4 != 0);
            } else {
#pragma unroll
                for (int i = 0; i < SD; ++i) x[v][i] = 0.0f;
            }
            na[v] = 0.0f;
            if (METRIC == M_COSINE) {
                float a2 = 0.0f;
#pragma unroll
                for (int i = 0; i < SD; ++i) a2 = __fadd_rn(a2, __fmul_rn(x[v][i], x[v][i]));
                na[v] = __fsqrt_rn(a2);
            }
        }

        float best[V], second[V];
        int idx[V];
        {
            float c[SD];
            load_centroid<SD>(c, cbs);
            const float nb = (METRIC == M_COSINE) ? cns[0] : 0.0f;
#pragma unroll
            for (int v = 0; v < V; ++v) {
                best[v] = reg_dist<SD, METRIC>(x[v], c, P.pv, na[v], nb);
                idx[v] = 0;
                second[v] = VQB_INF;
            }
        }
#pragma unroll 2
        for (int j = 1; j < k; ++j) {
            float c[SD];
            load_centroid<SD>(c, cbs + (size_t)j * SD);
            const float nb = (METRIC == M_COSINE) ? cns[j] : 0.0f;
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float d = reg_dist<SD, METRIC>(x[v], c, P.pv, na[v], nb);
                const bool lt = d < best[v];
                if (METRIC == M_EUCLID) second[v] = fminf(second[v], lt ? best[v] : d); // smallest non-winning sum
                best[v] = lt ? d : best[v];
                idx[v] = lt ? j : idx[v];
            }
        }

        if (METRIC == M_EUCLID) {
            // The reference compares sqrt() values (src/distances.rs:134-140): two different sums can round to
            // the same root, and then the LOWER index keeps the win.  Only possible when the runner-up's root
            // equals the winner's; redo such rows with the root in the comparison.
#pragma unroll
            for (int v = 0; v < V; ++v) {
                if (__fsqrt_rn(second[v]) == __fsqrt_rn(best[v])) {
                    float c[SD];
                    load_centroid<SD>(c, cbs);
                    float bd = __fsqrt_rn(reg_dist<SD, M_SQ>(x[v], c, 0.0f, 0.0f, 0.0f));
                    int bi = 0;
                    for (int j = 1; j < k; ++j) {
                        load_centroid<SD>(c, cbs + (size_t)j * SD);
                        float d = __fsqrt_rn(reg_dist<SD, M_SQ>(x[v], c, 0.0f, 0.0f, 0.0f));
                        argmin_update(d, j, bd, bi);
                    }
                    idx[v] = bi;
                }
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
