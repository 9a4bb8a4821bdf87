// kernels_common.cuh -- device-side arithmetic shared by every kernel.
//
// The exact distance forms reproduce the reference's f32 operation order: element-wise subtract
// (rounded), multiply (rounded), then a serial left fold (src/vector.rs:198-201,214-220,259-264;
// src/distances.rs:27-30,130-170).  The _rn intrinsics are never contracted into FMAs by nvcc.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vqb {

enum : int { M_SQ = 0, M_EUCLID = 1, M_COSINE = 2, M_MANHATTAN = 3, M_CHEBYSHEV = 4, M_MINKOWSKI = 5, M_HAMMING = 6 };

#define VQB_INF __int_as_float(0x7f800000)
// What the assignment kernels OR into a sub-space's "some row moved" word: the bits of 1.0f, so that the word is non-zero
// as an integer and, when the words of several ranks are added up as f32 in one all-reduce with the cluster sums, as a float.
#define VQB_MOVED_BITS 0x3F800000u

// ---- running state of one distance evaluation, advanced one dimension at a time ----------------
// `b` carries the centroid's sum of squares for the cosine metric (src/distances.rs:141-144).
template <int METRIC> struct DistAcc {
    float a, b;
    __device__ __forceinline__ void init()
    {
        a = 0.0f;
        b = 0.0f;
    }
    __device__ __forceinline__ void step(float x, float c, float pv)
    {
        if (METRIC == M_SQ || METRIC == M_EUCLID) {
            float d = __fsub_rn(x, c);
            a = __fadd_rn(a, __fmul_rn(d, d));
        } else if (METRIC == M_COSINE) {
            a = __fadd_rn(a, __fmul_rn(x, c));
            b = __fadd_rn(b, __fmul_rn(c, c));
        } else if (METRIC == M_MANHATTAN) {
            a = __fadd_rn(a, fabsf(__fsub_rn(x, c)));
        } else if (METRIC == M_CHEBYSHEV) {
            float v = fabsf(__fsub_rn(x, c));
            if (v > a) a = v; // src/distances.rs:47-50
        } else if (METRIC == M_MINKOWSKI) {
            a = __fadd_rn(a, powf(fabsf(__fsub_rn(x, c)), pv));
        } else { // Hamming
            a = __fadd_rn(a, (x == c) ? 0.0f : 1.0f);
        }
    }
    // norm_a = sqrt(sum x^2) of the query, cosine only.
    __device__ __forceinline__ float finish(float pv, float norm_a) const
    {
        if (METRIC == M_EUCLID) return __fsqrt_rn(a);
        if (METRIC == M_COSINE) {
            float norm_b = __fsqrt_rn(b);
            if (norm_a == 0.0f || norm_b == 0.0f) return 1.0f; // src/distances.rs:146-147
            return __fsub_rn(1.0f, __fdiv_rn(a, __fmul_rn(norm_a, norm_b)));
        }
        if (METRIC == M_MINKOWSKI) return powf(a, __fdiv_rn(1.0f, pv));
        return a;
    }
};

// sqrt(sum x^2), serial fold (map_sum, src/distances.rs:66-69).
__device__ __forceinline__ float norm_chain(const float *x, int d, int stride)
{
    float s = 0.0f;
    for (int i = 0; i < d; ++i) {
        float v = x[(size_t)i * stride];
        s = __fadd_rn(s, __fmul_rn(v, v));
    }
    return __fsqrt_rn(s);
}

// Strict '<' update (src/utils.rs:66, src/pq.rs:170): NaN never wins, lowest index wins ties.
__device__ __forceinline__ void argmin_update(float d, int j, float &best, int &idx)
{
    if (d < best) {
        best = d;
        idx = j;
    }
}

__device__ __forceinline__ unsigned short f32_to_f16_bits(float v)
{
    return __half_as_ushort(__float2half_rn(v)); // IEEE round-to-nearest-even == half::f16::from_f32
}

// Three-input minimum (one instruction on sm_100); NaN operands are ignored like fminf.
__device__ __forceinline__ float min3f(float a, float b, float c)
{
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ float max3f(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// nearest TF32 number (10-bit mantissa), ties away from zero
__device__ __forceinline__ float tf32_round(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

template <typename CodeT> __device__ __forceinline__ CodeT to_code(int j) { return (CodeT)j; }

} // namespace vqb
