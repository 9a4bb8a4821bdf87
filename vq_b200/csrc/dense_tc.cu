// dense_tc.cu -- full-width nearest-centroid search on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// The residual quantizer's k-means and encode (src/rvq.rs:107,111-128,186-202) compare every row with every centroid
// over the full dimension: a dense n x k x dim contraction.  This file ranks centroids with
//        S_j = |c_j|^2/2 - x.c_j          (|x - c_j|^2 = |x|^2 + 2 S_j)
// where the dot products come from tcgen05.mma (TF32 inputs, f32 accumulation in tensor memory), keeps for every row
// the SHORTLIST of centroids whose S lies within a proven error bound of the smallest one, and hands the shortlist
// to resolve kernels (resolve.cuh) that evaluate only those candidates with the reference's exact f32 arithmetic in
// ascending index order.  The final choice is therefore the reference's; the tensor cores only prune.
//
// Bound.  TF32 keeps 10 mantissa bits of each operand (the low 13 bits of the f32 container are ignored), so
//   |dot_tc - x.c| <= (2^-10 + 2^-10 + 2^-20 + 2 K 2^-24) sum|x_i c_ji| <= 2.1e-3 |x| |c_j|        (K <= 128)
// and with the reference's own chain error (<= (dim + 2) 2^-24 relative on the distance) the winner w satisfies
//   S_w <= S_min + 2 E + 1.05 (dim + 6) 2^-24 (|x|^2 + 2 S_min + 2 E),   E = 2.1e-3 |x| max_j |c_j|.
// Everything not finite falls out of the comparisons and marks the row for a full exact scan.
//
// Kernel layout (one CTA per SM, persistent over 128-row tiles):
//   warp 0      TMA producer: the codebook once (k x dim, resident in shared memory), then row tiles in 128-byte
//               column chunks through a 5-stage ring (cp.async.bulk.tensor, 128B swizzle, no multicast)
//   warp 1      allocates tensor memory and issues tcgen05.mma M128 x N256 x K8 (kind::tf32); two 256-column
//               accumulators so the next tile's MMAs overlap this tile's epilogue.  One more K = 8 step per tile multiplies
//               a constant (1, 1, 0, ...) row operand with (-hn_h, -hn_l, 0, ...) per centroid, so the accumulator holds
//               D = x.c - |c|^2/2 = -S and the epilogue never touches the half norms
//   warps 2..5  epilogue: tcgen05.ld the 128 x 256 values, one row per lane; pass 1 finds the largest D (3-input max), pass 2
//               shifts the sign of (D - limit) into a 256-bit candidate mask
// Every wait is bounded; on expiry the kernel records an error code, stops issuing work and frees its tensor memory.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "cuda_device.hpp"
#include "dense_tc.hpp"
#include "kernels_common.cuh"
#include "tma_host.hpp"
#include "umma.cuh"

namespace vqb {

namespace {

constexpr int BM = 128;          // rows per tile (= TMEM lanes)
constexpr int BN = 256;          // centroids per tile (= accumulator columns)
constexpr int CHUNK = 32;        // f32 per 128-byte swizzle row
constexpr int NSTAGE = 5;        // row-tile ring depth (stages of 128 rows x 128 bytes)
constexpr int MAX_KCHUNKS = 4;   // dim <= 128
constexpr uint32_t X_STAGE_BYTES = BM * 128;
constexpr uint32_t C_CHUNK_BYTES = BN * 128;

struct alignas(8) Barriers {
    unsigned long long full[NSTAGE], empty[NSTAGE], cfull, tfull[2], tempty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct ShortlistParams {
    unsigned long long n;
    int dim, k, kchunks;
    const float *hn;      // [256] |c_j|^2 / 2, +inf beyond k
    const float *cmax;    // [1]   max_j |c_j|
    const float *xnorm2;  // [n]   |x|^2 per row
    uint32_t *cand;       // [n][8] bit j set = centroid j may be the reference's choice (all k bits set: examine all)
    unsigned long long *stats; // [0] rows, [1] candidates, [2] rows needing a full scan   (may be null)
    float *debug_dots;    // [n][256] raw tensor-core dot products (may be null)
    int *error;           // device error word, 0 = ok
    // training passes (codes != null): a row with a single candidate gets its assignment here; the others are appended to
    // `list` (and only they get their mask written)
    uint8_t *codes;        // [n] previous assignment in, new assignment out
    uint32_t *changed;     // VQB_MOVED_BITS is OR-ed in when a row moved
    uint32_t *list;        // [n] rows left for the exact decision
    uint32_t *list_count;  // [1] zero on entry
};

__global__ void __launch_bounds__(192, 1) dense_shortlist_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c,
                                                                const ShortlistParams P)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *c_smem = base;                                            // kchunks x 32 KiB
    unsigned char *x_smem = base + (size_t)MAX_KCHUNKS * C_CHUNK_BYTES;       // NSTAGE x 16 KiB
    float *hn_s = reinterpret_cast<float *>(x_smem + (size_t)NSTAGE * X_STAGE_BYTES); // 256 floats (diagnostics only)
    // one more K = 8 step folds the half norms into the accumulator: operand A = (1, 1, 0, ...) for every row, operand B =
    // (-hn_h, -hn_l, 0, ...) per centroid, hn split into two TF32 numbers; both tiles K-major with 32-byte rows, 32B swizzle
    unsigned char *a1_smem = reinterpret_cast<unsigned char *>(hn_s + BN);            // 128 rows x 32 bytes
    unsigned char *bh_smem = a1_smem + BM * 32;                                       // 256 rows x 32 bytes
    Barriers *bars = reinterpret_cast<Barriers *>(bh_smem + BN * 32);
    volatile int *abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long n_tiles = (P.n + BM - 1) / BM;
    const int kchunks = P.kchunks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        mbar_init(&bars->cfull, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->tfull[b], 1);
            mbar_init(&bars->tempty[b], 4);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int t = threadIdx.x; t < BN; t += blockDim.x) {
        const float hn = P.hn[t]; // +inf beyond k
        hn_s[t] = hn;
        const bool pad = !(hn < VQB_DENSE_INF);
        const float hh = pad ? 1e30f : tf32_round(hn), hl = pad ? 0.0f : tf32_round(hn - hh);
        unsigned char *rowp = bh_smem + (size_t)(t >> 3) * 256 + (size_t)(t & 7) * 32;
        const int sw = ((t >> 2) & 1) * 16; // 32B swizzle: the two 16-byte halves of a row swap when bit 2 of the row is set
        *reinterpret_cast<float4 *>(rowp + sw) = make_float4(-hh, -hl, 0.0f, 0.0f);
        *reinterpret_cast<float4 *>(rowp + (16 - sw)) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (t < BM) {
            unsigned char *ap = a1_smem + (size_t)(t >> 3) * 256 + (size_t)(t & 7) * 32;
            *reinterpret_cast<float4 *>(ap + sw) = make_float4(1.0f, 1.0f, 0.0f, 0.0f);
            *reinterpret_cast<float4 *>(ap + (16 - sw)) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic writes -> visible to the MMA's reads
    if (warp == 1) { // tensor memory: 512 columns = two 128 x 256 f32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(&bars->cfull, (uint32_t)kchunks * C_CHUNK_BYTES);
            for (int kc = 0; kc < kchunks; ++kc) tma_load_2d(c_smem + (size_t)kc * C_CHUNK_BYTES, &map_c, kc * CHUNK, 0, &bars->cfull);
            uint32_t it = 0;
            for (unsigned long long tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x) {
                for (int kc = 0; kc < kchunks; ++kc, ++it) {
                    const int s = it % NSTAGE;
                    const uint32_t use = it / NSTAGE;
                    if (!mbar_wait(&bars->empty[s], (use & 1u) ^ 1u, abort_flag, P.error, 1)) break;
                    mbar_expect_tx(&bars->full[s], X_STAGE_BYTES);
                    tma_load_2d(x_smem + (size_t)s * X_STAGE_BYTES, &map_x, kc * CHUNK, (int)(tile * BM), &bars->full[s]);
                }
            }
            if (*abort_flag) {
                // gave up: let the copies already in flight land before the CTA retires (bounded; a phase the MMA warp
                // already consumed simply runs this short wait out)
                for (uint32_t back = 0; back < NSTAGE && back < it; ++back) {
                    const uint32_t j = it - 1 - back;
                    const uint32_t addr = smem_u32(&bars->full[j % NSTAGE]);
                    for (uint32_t spin = 0; spin < 20000u; ++spin) {
                        uint32_t done;
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done)
                                     : "r"(addr), "r"((j / NSTAGE) & 1u)
                                     : "memory");
                        if (done) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = mbar_wait(&bars->cfull, 0, abort_flag, P.error, 2);
            uint32_t it = 0, local = 0;
            for (unsigned long long tile = blockIdx.x; ok && tile < n_tiles && !*abort_flag; tile += gridDim.x, ++local) {
                const uint32_t b = local & 1u, buse = local >> 1;
                if (!mbar_wait(&bars->tempty[b], (buse & 1u) ^ 1u, abort_flag, P.error, 3)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + b * BN;
                for (int kc = 0; kc < kchunks; ++kc, ++it) {
                    const int s = it % NSTAGE;
                    const uint32_t use = it / NSTAGE;
                    if (!mbar_wait(&bars->full[s], use & 1u, abort_flag, P.error, 4)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = smem_desc_sw128(smem_u32(x_smem + (size_t)s * X_STAGE_BYTES));
                    const uint64_t bdesc = smem_desc_sw128(smem_u32(c_smem + (size_t)kc * C_CHUNK_BYTES));
#pragma unroll
                    for (int k8 = 0; k8 < CHUNK / 8; ++k8) // 8 f32 = 32 bytes = 2 descriptor units per MMA step
                        umma_tf32(d_tmem, adesc + (uint64_t)(2 * k8), bdesc + (uint64_t)(2 * k8), (kc | k8) ? 1u : 0u);
                    umma_commit(&bars->empty[s]); // the stage is free once these MMAs have read it
                }
                if (ok) {
                    umma_tf32(d_tmem, smem_desc_sw32(smem_u32(a1_smem)), smem_desc_sw32(smem_u32(bh_smem)), 1u); // D = x.c - hn
                    umma_commit(&bars->tfull[b]);
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue: one row per lane
        const int q = warp & 3; // TMEM lane quadrant this warp may read
        const float cmax = *P.cmax;
        unsigned long long cand_total = 0, full_scans = 0, rows_done = 0;
        bool moved = false;
        uint32_t local = 0;
        for (unsigned long long tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x, ++local) {
            const uint32_t b = local & 1u, buse = local >> 1;
            if (!mbar_wait(&bars->tfull[b], buse & 1u, abort_flag, P.error, 5)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned long long row = tile * BM + 32ull * q + lane;
            const bool valid = row < P.n;
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + b * BN;
            const float xn2 = valid ? P.xnorm2[row] : 0.0f;
            const int old_code = (P.codes && valid) ? (int)P.codes[row] : 0; // asked for now, needed after the two passes

            // pass 1: the largest D = x.c - hn, i.e. the smallest score S = -D (four chains of 3-input max); the next 32 columns
            // are in flight while these are processed
            float m0 = -VQB_DENSE_INF, m1 = -VQB_DENSE_INF, m2 = -VQB_DENSE_INF, m3 = -VQB_DENSE_INF;
            bool col0_nan = false;
            uint32_t ra[32], rb[32];
            tmem_ld32_issue(taddr, ra);
            tmem_wait();
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; cb += 2) {
                tmem_ld32_issue(taddr + (cb + 1) * 32, rb);
                if (P.debug_dots && valid) {
#pragma unroll
                    for (int t = 0; t < 32; ++t) P.debug_dots[row * BN + cb * 32 + t] = (cb * 32 + t < P.k) ? __uint_as_float(ra[t]) + hn_s[cb * 32 + t] : 0.0f;
                }
                if (cb == 0) {
                    const float s0 = __uint_as_float(ra[0]);
                    col0_nan = !(s0 == s0);
                }
#pragma unroll
                for (int t = 0; t < 32; t += 8) {
                    m0 = max3f(m0, __uint_as_float(ra[t]), __uint_as_float(ra[t + 1]));
                    m1 = max3f(m1, __uint_as_float(ra[t + 2]), __uint_as_float(ra[t + 3]));
                    m2 = max3f(m2, __uint_as_float(ra[t + 4]), __uint_as_float(ra[t + 5]));
                    m3 = max3f(m3, __uint_as_float(ra[t + 6]), __uint_as_float(ra[t + 7]));
                }
                tmem_wait();
                if (cb + 2 < BN / 32) tmem_ld32_issue(taddr + (cb + 2) * 32, ra);
                if (P.debug_dots && valid) {
#pragma unroll
                    for (int t = 0; t < 32; ++t)
                        P.debug_dots[row * BN + (cb + 1) * 32 + t] = ((cb + 1) * 32 + t < P.k) ? __uint_as_float(rb[t]) + hn_s[(cb + 1) * 32 + t] : 0.0f;
                }
#pragma unroll
                for (int t = 0; t < 32; t += 8) {
                    m0 = max3f(m0, __uint_as_float(rb[t]), __uint_as_float(rb[t + 1]));
                    m1 = max3f(m1, __uint_as_float(rb[t + 2]), __uint_as_float(rb[t + 3]));
                    m2 = max3f(m2, __uint_as_float(rb[t + 4]), __uint_as_float(rb[t + 5]));
                    m3 = max3f(m3, __uint_as_float(rb[t + 6]), __uint_as_float(rb[t + 7]));
                }
                tmem_wait();
            }
            const float best = -fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)); // smallest score
            // E = 2.1e-3 |x| cmax (+ the rounding of the half norms);
            // limit = best + 2E + 1.05 (dim + 6) u (|x|^2 + 2 best + 2E) + rounding slack of the comparison itself
            const float e2 = 2.0f * 2.1e-3f * sqrtf(xn2) * cmax + 8e-6f * cmax * cmax;
            const float d_a = fmaxf(xn2 + 2.0f * best + e2, 0.0f);
            const float limit = best + e2 + 1.05f * (float)(P.dim + 6) * 5.9604645e-8f * d_a + 2.4e-7f * (fabsf(best) + e2) + 1e-36f;
            const float lim_d = -limit; // centroid j is a candidate when D_j >= lim_d
            // a row the comparisons cannot rank (NaN / infinity somewhere, or centroid 0 not comparable, on which the
            // reference's scan depends) is handed over with every centroid marked
            // (also when a true distance could overflow f32: then the reference's own comparisons see infinities)
            const bool scan_all = col0_nan || !(best == best) || !(limit == limit) || !(fabsf(limit) < VQB_DENSE_INF) || !(xn2 + cmax * cmax < 1e37f);

            // pass 2: one bit per centroid, set when D_j >= lim_d.  The sign of (D_j - lim_d) is shifted into the word,
            // so the bits arrive in reverse order and inverted.
            uint32_t words[BN / 32];
            tmem_ld32_issue(taddr, ra);
            tmem_wait();
#pragma unroll
            for (int cb = 0; cb < BN / 32; cb += 2) {
                tmem_ld32_issue(taddr + (cb + 1) * 32, rb);
                uint32_t m = 0;
#pragma unroll
                for (int t = 0; t < 32; ++t) m = __funnelshift_l(__float_as_uint(__uint_as_float(ra[t]) - lim_d), m, 1);
                words[cb] = ~__brev(m);
                tmem_wait();
                if (cb + 2 < BN / 32) tmem_ld32_issue(taddr + (cb + 2) * 32, ra);
                m = 0;
#pragma unroll
                for (int t = 0; t < 32; ++t) m = __funnelshift_l(__float_as_uint(__uint_as_float(rb[t]) - lim_d), m, 1);
                words[cb + 1] = ~__brev(m);
                tmem_wait();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tempty[b]); // this accumulator may be overwritten
            bool listed = false;
            if (valid) {
                int cnt = 0;
#pragma unroll
                for (int wd = 0; wd < BN / 32; ++wd) {
                    const int lo = wd * 32;
                    const uint32_t in_range = (P.k >= lo + 32) ? 0xFFFFFFFFu : ((P.k > lo) ? ((1u << (P.k - lo)) - 1u) : 0u);
                    words[wd] = scan_all ? in_range : (words[wd] & in_range);
                    cnt += __popc(words[wd]);
                }
                if (scan_all) ++full_scans;
                else cand_total += cnt;
                ++rows_done;
                if (P.codes && cnt == 1) {
                    // the only candidate is the reference's choice (an unrankable row comes with all k >= 2 bits set)
                    int best_j = 0;
#pragma unroll
                    for (int wd = 0; wd < BN / 32; ++wd)
                        if (words[wd]) best_j = wd * 32 + __ffs(words[wd]) - 1;
                    if (best_j != old_code) {
                        moved = true;
                        P.codes[row] = (uint8_t)best_j;
                    }
                } else {
                    uint4 *o = reinterpret_cast<uint4 *>(P.cand + row * 8);
                    o[0] = make_uint4(words[0], words[1], words[2], words[3]);
                    o[1] = make_uint4(words[4], words[5], words[6], words[7]);
                    listed = P.codes != nullptr;
                }
            }
            if (P.codes) { // the rows that need the exact decision, appended in one step per warp
                const unsigned bal = __ballot_sync(0xffffffffu, listed);
                if (bal) {
                    uint32_t base = 0;
                    if (lane == 0) base = atomicAdd(P.list_count, (uint32_t)__popc(bal));
                    base = __shfl_sync(0xffffffffu, base, 0);
                    if (listed) P.list[base + __popc(bal & ((1u << lane) - 1u))] = (uint32_t)row;
                }
            }
        }
        if (P.codes && __any_sync(0xffffffffu, moved) && lane == 0) atomicOr(P.changed, VQB_MOVED_BITS);
        if (P.stats) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                cand_total += __shfl_xor_sync(0xffffffffu, cand_total, o);
                full_scans += __shfl_xor_sync(0xffffffffu, full_scans, o);
                rows_done += __shfl_xor_sync(0xffffffffu, rows_done, o);
            }
            if (lane == 0) {
                atomicAdd(P.stats + 0, rows_done);
                atomicAdd(P.stats + 1, cand_total);
                atomicAdd(P.stats + 2, full_scans);
            }
        }
    }

    // ---------------------------------------------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// |c_j|^2 / 2 for j < k (+inf beyond) and max_j |c_j|
// One CTA of eight warps; a warp takes every eighth centroid, its lanes the row's 16-byte pieces (dim <= 128 on this path), so
// all of a warp's rows are in flight together.  The order in which a row's squares are added is free: the shortlist's bound
// carries (dim + 1) roundings of slack for the half norms.  (One thread per centroid walking its row took 23 us per launch,
// 2 ms over a residual-quantizer fit.)
__global__ void __launch_bounds__(256) codebook_norms_kernel(const float *c, int k, int dim, float *hn, float *cmax)
{
    __shared__ float smax[256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dim4 = dim >> 2;
    smax[threadIdx.x] = 0.0f;
    hn[threadIdx.x] = VQB_DENSE_INF; // entries at and beyond k stay at +inf
    __syncthreads();
    float part[32];
#pragma unroll
    for (int t = 0; t < 32; ++t) {
        const int j = warp + 8 * t;
        float a = 0.0f;
        if (j < k && lane < dim4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(c + (size_t)j * dim) + lane);
            a = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
        }
        part[t] = a;
    }
#pragma unroll
    for (int t = 0; t < 32; ++t) {
        float a = part[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        const int j = warp + 8 * t;
        if (lane == 0 && j < k) {
            hn[j] = 0.5f * a;
            smax[j] = sqrtf(a);
        }
    }
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) smax[threadIdx.x] = fmaxf(smax[threadIdx.x], smax[threadIdx.x + o]);
        __syncthreads();
    }
    if (threadIdx.x == 0) *cmax = smax[0] * 1.000001f;
}

__global__ void row_norms_kernel(const float *x, unsigned long long n, int dim, float *out)
{
    const int lane = threadIdx.x & 31;
    const unsigned long long warps = (unsigned long long)gridDim.x * (blockDim.x >> 5);
    for (unsigned long long row = blockIdx.x * (unsigned long long)(blockDim.x >> 5) + (threadIdx.x >> 5); row < n; row += warps) {
        float a = 0.0f;
        for (int i = lane; i < dim; i += 32) {
            const float v = x[row * dim + i];
            a = fmaf(v, v, a);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) out[row] = a * 1.00001f; // an upper bound is what the filter needs
    }
}

CUtensorMap make_map(const float *ptr, unsigned long long rows, int dim, int box_rows)
{
    return make_tensor_map_2d(ptr, (unsigned long long)dim, rows, CHUNK, (unsigned)box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

} // namespace

bool dense_tc_applicable(size_t n, size_t dim, size_t k, int metric, const float *x)
{
    (void)n;
    return (metric == 0 || metric == 1) && dim >= 32 && dim <= 128 && dim % 32 == 0 && k >= 2 && k <= 256 &&
           (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
}

size_t dense_tc_smem_bytes()
{
    return 1024 + (size_t)MAX_KCHUNKS * C_CHUNK_BYTES + (size_t)NSTAGE * X_STAGE_BYTES + BN * sizeof(float) + (size_t)(BM + BN) * 32 + sizeof(Barriers) + 64;
}

void dense_row_norms(CudaDevice &dev, const float *x, size_t n, size_t dim, float *out)
{
    if (n == 0) return;
    KernelScope ks(dev, "row_norms");
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>((n + 7) / 8, (size_t)dev.sm_count() * 8));
    row_norms_kernel<<<grid, 256, 0, dev.stream()>>>(x, n, (int)dim, out);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

void dense_shortlist(CudaDevice &dev, const float *x, size_t n, size_t dim, const float *codebook, size_t k, const float *xnorm2,
                     float *hn_scratch /* 257 floats */, uint32_t *cand, unsigned long long *stats, int *error_word, float *debug_dots,
                     const ShortlistTrain *train)
{
    if (n == 0) return;
    {
        KernelScope ks(dev, "codebook_norms");
        codebook_norms_kernel<<<1, 256, 0, dev.stream()>>>(codebook, (int)k, (int)dim, hn_scratch, hn_scratch + 256);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
    }
    const CUtensorMap mx = make_map(x, n, (int)dim, BM);
    const CUtensorMap mc = make_map(codebook, k, (int)dim, BN);
    ShortlistParams p;
    p.n = n;
    p.dim = (int)dim;
    p.k = (int)k;
    p.kchunks = (int)(dim / CHUNK);
    p.hn = hn_scratch;
    p.cmax = hn_scratch + 256;
    p.xnorm2 = xnorm2;
    p.cand = cand;
    p.stats = stats;
    p.debug_dots = debug_dots;
    p.error = error_word;
    p.codes = train ? train->codes : nullptr;
    p.changed = train ? train->changed : nullptr;
    p.list = train ? train->list : nullptr;
    p.list_count = train ? train->list_count : nullptr;
    const size_t smem = dense_tc_smem_bytes();
    VQB_CUDA_CHECK(cudaFuncSetAttribute(dense_shortlist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned long long tiles = (n + BM - 1) / BM;
    const unsigned grid = (unsigned)std::min<unsigned long long>(tiles, (unsigned long long)dev.sm_count());
    KernelScope ks(dev, "dense_shortlist");
    dense_shortlist_kernel<<<grid, 192, smem, dev.stream()>>>(mx, mc, p);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

} // namespace vqb
