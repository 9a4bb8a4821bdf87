// pq_tc.cu -- product-quantizer nearest-centroid search (sub-space width 8) with the scores on the tensor cores.
//
// Replaces the per-point scan of src/utils.rs:59-73 (training) and src/pq.rs:159-182 (encode) for the Euclidean metrics.
//
// Scores.  S_j = |c_j|^2/2 - x.c_j ranks the centroids like the squared distance (|x - c_j|^2 = |x|^2 + 2 S_j).  Both
// operands are split into two TF32 numbers (x = xh + xl, c = ch + cl, each part exactly representable, so the hardware's
// treatment of the low mantissa bits does not matter) and one K = 32 tcgen05.mma chain per (128-row tile, sub-space)
// accumulates, in f32,
//     xh.(-ch) + xh.(-cl) + xl.(-ch) + 1*hn_h + 1*hn_l            (hn = |c|^2/2 split the same way)
// into tensor memory: 128 x 256 scores with about 2^-21 relative accuracy instead of TF32's 2^-11.
//
// Decision.  Per row the epilogue finds the smallest score, then counts the scores below
//     limit = best + 7e-6 (|x|^2/2 + 2 max_j hn_j + |best|)
// If exactly one score lies below the limit its centroid is the reference's answer; otherwise (two or more within the
// limit, NaN / infinity, values too small to rank) the (row, sub-space) pair is marked and a second kernel decides it with
// the reference's own f32 arithmetic over all centroids (ascending index, strict '<', sqrt inside the comparison for the
// Euclidean metric, scan started at centroid 0).  The result equals the exact scan's bit for bit.
//
// Bound behind 7e-6.  u = 2^-24, xh2 = |x|^2/2, HN = max_j hn_j.
//   operand split:   dropped xl.cl and the rounding of xl, cl to TF32: <= 3 * 2^-22 sum|x_i c_ji| <= 3 * 2^-22 (xh2 + hn_j)
//   half norm:       f32 chain 9u hn_j, split 2^-22 hn_j
//   accumulation:    26 exact products summed by the tensor core in f32; assumed error <= 2^-20 (hn_j + sum|x_i c_ji|),
//                    sixteen times what is measured (tests/test_gpu_pq_tensor.py measures it against f64)
//   => |S_j - true| <= E = 1.25 * 2^-19 (xh2 + 2 HN) = 2.4e-6 (xh2 + 2 HN)
//   the reference prefers w over a = argmin S only if D_w <= D_a (1 + 4u) in its own arithmetic (10u relative each), i.e.
//   S_w <= S_a + 2E + 25u (xh2 + |S_a| + E)  <=  S_a + 4.8e-6 (xh2 + 2HN) + 1.5e-6 (xh2 + |S_a|) + ...  <  limit.
// The count uses t = sat((limit - S) * 2^p) with p chosen per row so that limit * 2^p ~ 2^60: a score differs from the
// limit by nothing or by at least one unit in its last place (>= 2^-24 |limit|), so t is exactly 0 or 1, and the two sums
// total = sum t * (1 + (j mod 32) / 512) and offs = sum (j / 32) * t * (1 + (j mod 32) / 512) yield count and index at once on
// the FMA pipe.  Rows whose true distances could overflow f32 (|x|^2/2 + 2 HN >= 1e37) are marked as well: there the
// reference's own comparisons see infinities.
//
// CTA (1 per SM, persistent, 448 threads), owning 4 consecutive sub-spaces (m / 4 groups share the row tiles):
//   warp 0       loads the group's four operand-B tiles once (TMA, 128B swizzle, no multicast; 32 KiB each) and, for an
//                encode, the binary16 images of the group's centroids (16 KiB, bulk copy)
//   warp 1       owns tensor memory (two 128 x 256 f32 accumulators) and issues the MMAs
//   warps 2-5    read row slices from global memory, split them and write operand-A tiles (128 rows x 128 bytes, 128B
//                swizzle) into a 4-stage ring, plus |x|^2/2 per row
//   warps 6-13   epilogue: two teams of four warps (one row per lane, one TMEM lane quadrant per warp); team t serves
//                sub-spaces 2t, 2t+1 of the group through accumulator t
// Every wait is bounded; on expiry the CTA records a code, stops issuing, frees tensor memory and the host raises an error.
#include <algorithm>
#include <atomic>

#include "assign_reg.cuh"
#include "cuda_device.hpp"
#include "pq_tc.hpp"
#include "tma_host.hpp"
#include "umma.cuh"

namespace vqb {

namespace {

constexpr int BM = 128, BN = 256, SDW = 8, KOP = 32, NSTAGE = 4, MAXM = 64, XH_RING = 8, NTHREADS = 448;
constexpr uint32_t A_STAGE_BYTES = BM * 128; // 16 KiB
constexpr uint32_t B_BYTES = BN * 128;       // 32 KiB per sub-space
constexpr float PAD_SCORE = 1e30f;           // score of the columns beyond k
constexpr float MARGIN_COEF = 7e-6f;

// scratch layout (floats)
constexpr size_t OFF_BOP = 0;                                   // [MAXM][256][32] operand B
constexpr size_t OFF_C16 = OFF_BOP + (size_t)MAXM * BN * KOP;   // [MAXM][256] 8 halves (uint4)
constexpr size_t OFF_HMAX = OFF_C16 + (size_t)MAXM * BN * 4;    // [MAXM]
constexpr size_t OFF_STATS = OFF_HMAX + MAXM;                   // 2 x u64: marked pairs, launches
constexpr size_t SCRATCH_FLOATS = OFF_STATS + 4;

struct alignas(8) PqBarriers {
    unsigned long long afull[NSTAGE], aempty[NSTAGE], bfull, tfull[2], tempty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct PqTcParams {
    AssignParams a;
    const uint4 *c16;   // [m][256] centroid values as 8 binary16
    const float *hnmax; // [m]
    uint8_t *marks;     // [n][m/2]: bit h of byte (g, team) = pair (row, 4g + 2 team + h) needs the exact scan
    unsigned long long *stats;
    int *error;
    float *dbg_scores; // optional [n][m][256]
};

__device__ __forceinline__ float to_tf32(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

__device__ __forceinline__ float fma_sat(float a, float b, float c)
{
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// order in which the four sub-spaces of a group are issued: accumulator / team = ss >> 1 alternates
__device__ __forceinline__ int issue_order(int p) { return ((p & 1) << 1) | (p >> 1); } // 0, 2, 1, 3

constexpr size_t PQ_TC_SMEM = 1024 + 4 * (size_t)B_BYTES + (size_t)NSTAGE * A_STAGE_BYTES + ((size_t)XH_RING * BM + 4 * BN * 4) * sizeof(float) + sizeof(PqBarriers) + 64;

template <bool TRAIN, bool EUCLID>
__global__ void __launch_bounds__(NTHREADS, 1) pq_tc_kernel(const __grid_constant__ CUtensorMap map_b, const PqTcParams Q)
{
    extern __shared__ unsigned char smem_raw[];
    const AssignParams &P = Q.a;
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *b_smem = base;                                           // 4 x 32 KiB
    unsigned char *a_smem = base + 4 * (size_t)B_BYTES;                     // NSTAGE x 16 KiB
    float *xh_ring = reinterpret_cast<float *>(a_smem + (size_t)NSTAGE * A_STAGE_BYTES); // [XH_RING][128]
    const uint4 *c16_s = reinterpret_cast<const uint4 *>(xh_ring + XH_RING * BM);         // [4][256] binary16 images
    PqBarriers *bars = reinterpret_cast<PqBarriers *>(xh_ring + XH_RING * BM + 4 * BN * 4);
    volatile int *abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = P.m, k = P.k;
    const int ngroups = m >> 2;
    const int g = blockIdx.x % ngroups;
    const unsigned long long tile0 = blockIdx.x / ngroups, tstep = gridDim.x / ngroups;
    const unsigned long long n_tiles = (P.n + BM - 1) / BM;

    // the active sub-spaces of this group in issue order (identical in every thread), packed four bits apiece so that the
    // lookups below are shifts on a register: indexed local arrays would go through the L1 cache, which the row stream of
    // the producer warps keeps flushing (each lookup then costs a trip to L2 on the critical path of a unit)
    uint32_t list_p = 0, pos_p = 0xFFFFu; // list_p: nibble p = sub-space issued p-th; pos_p: nibble ss = its position, 0xF = inactive
    int nact = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int ss = issue_order(p);
        const bool act = !(TRAIN && P.active && P.active[g * 4 + ss] == 0);
        if (act) {
            pos_p = (pos_p & ~(0xFu << (4 * ss))) | ((uint32_t)nact << (4 * ss));
            list_p |= (uint32_t)ss << (4 * nact);
            ++nact;
        }
    }
    auto list_at = [&](int p) { return (int)((list_p >> (4 * p)) & 0xFu); };
    auto pos_of = [&](int ss) { return (int)((pos_p >> (4 * ss)) & 0xFu); }; // 15 = inactive

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&bars->afull[s], 4);
            mbar_init(&bars->aempty[s], 1);
        }
        mbar_init(&bars->bfull, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->tfull[b], 1);
            mbar_init(&bars->tempty[b], 4);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------ operand B: the group's four sub-spaces, once
        if (lane == 0 && nact > 0) {
            mbar_expect_tx(&bars->bfull, 4 * B_BYTES + (TRAIN ? 0u : 4u * BN * 16u));
            for (int ss = 0; ss < 4; ++ss) tma_load_2d(b_smem + (size_t)ss * B_BYTES, &map_b, 0, (g * 4 + ss) * BN, &bars->bfull);
            if (!TRAIN) bulk_load_1d(const_cast<uint4 *>(c16_s), Q.c16 + (size_t)g * 4 * BN, 4u * BN * 16u, &bars->bfull);
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0 && nact > 0) {
            bool ok = mbar_wait(&bars->bfull, 0, abort_flag, Q.error, 12);
            uint32_t it = 0, uses0 = 0, uses1 = 0;
            for (unsigned long long tile = tile0; ok && tile < n_tiles && !*abort_flag; tile += tstep) {
                for (int p = 0; ok && p < nact; ++p, ++it) {
                    const int ss = list_at(p);
                    const uint32_t b = (uint32_t)ss >> 1;
                    const int st = it % NSTAGE;
                    if (!mbar_wait(&bars->afull[st], (it / NSTAGE) & 1u, abort_flag, Q.error, 14)) {
                        ok = false;
                        break;
                    }
                    const uint32_t ub = b ? uses1 : uses0;
                    if (!mbar_wait(&bars->tempty[b], (ub & 1u) ^ 1u, abort_flag, Q.error, 13)) {
                        ok = false;
                        break;
                    }
                    if (b) ++uses1;
                    else ++uses0;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = smem_desc_sw128(smem_u32(a_smem + (size_t)st * A_STAGE_BYTES));
                    const uint64_t bdesc = smem_desc_sw128(smem_u32(b_smem + (size_t)ss * B_BYTES));
#pragma unroll
                    for (int k8 = 0; k8 < KOP / 8; ++k8) // 8 f32 = 32 bytes = 2 descriptor units per step
                        umma_tf32(tmem_base + b * BN, adesc + (uint64_t)(2 * k8), bdesc + (uint64_t)(2 * k8), k8 ? 1u : 0u);
                    umma_commit(&bars->aempty[st]);
                    umma_commit(&bars->tfull[b]);
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------ operand A: split row slices into the ring
        const int r = (warp - 2) * 32 + lane; // row of the tile
        uint32_t it = 0;
        float4 cur[8], nxt[8];
        auto fetch = [&](float4(&dst)[8], unsigned long long tile) {
            const unsigned long long row = tile * BM + r;
            if (tile < n_tiles && row < P.n) {
                const float4 *src = reinterpret_cast<const float4 *>(P.x + row * P.ld + (size_t)g * 32);
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i] = __ldg(src + i);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        if (nact > 0) fetch(nxt, tile0);
        for (unsigned long long tile = tile0; nact > 0 && tile < n_tiles && !*abort_flag; tile += tstep) {
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
            fetch(nxt, tile + tstep);
            bool ok = true;
#pragma unroll
            for (int ss4 = 0; ss4 < 4; ++ss4) { // static indexing of cur[]; issue order 0, 2, 1, 3
                const int ss = issue_order(ss4);
                if (pos_of(ss) == 15 || !ok) continue;
                const int st = it % NSTAGE;
                if (!mbar_wait(&bars->aempty[st], ((it / NSTAGE) & 1u) ^ 1u, abort_flag, Q.error, 11)) {
                    ok = false;
                    continue;
                }
                const float4 v0 = cur[2 * ss], v1 = cur[2 * ss + 1];
                const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                float hi[8], lo[8], sq = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    hi[i] = to_tf32(v[i]);
                    lo[i] = to_tf32(v[i] - hi[i]);
                    sq = fmaf(v[i], v[i], sq);
                }
                unsigned char *rowp = a_smem + (size_t)st * A_STAGE_BYTES + (size_t)r * 128;
                const int sw = r & 7;
                const float4 h0 = make_float4(hi[0], hi[1], hi[2], hi[3]), h1 = make_float4(hi[4], hi[5], hi[6], hi[7]);
                *reinterpret_cast<float4 *>(rowp + ((0 ^ sw) << 4)) = h0;
                *reinterpret_cast<float4 *>(rowp + ((1 ^ sw) << 4)) = h1;
                *reinterpret_cast<float4 *>(rowp + ((2 ^ sw) << 4)) = h0;
                *reinterpret_cast<float4 *>(rowp + ((3 ^ sw) << 4)) = h1;
                *reinterpret_cast<float4 *>(rowp + ((4 ^ sw) << 4)) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<float4 *>(rowp + ((5 ^ sw) << 4)) = make_float4(lo[4], lo[5], lo[6], lo[7]);
                *reinterpret_cast<float4 *>(rowp + ((6 ^ sw) << 4)) = make_float4(1.0f, 1.0f, 0.0f, 0.0f);
                *reinterpret_cast<float4 *>(rowp + ((7 ^ sw) << 4)) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                xh_ring[(it & (XH_RING - 1)) * BM + r] = 0.5f * sq;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic writes -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->afull[st]);
                ++it;
            }
            if (!ok) break;
        }
    } else {
        // ------------------------------------------------ epilogue
        const int q = warp & 3;           // TMEM lane quadrant
        const int team = (warp - 6) >> 2; // accumulator and sub-space pair
        const int nch = (k + 31) >> 5;    // 32-column chunks that hold centroids
        uint32_t uu = 0, moved_mask = 0, tile_iter = 0;
        const float hmax2_0 = 2.0f * Q.hnmax[g * 4 + team * 2], hmax2_1 = 2.0f * Q.hnmax[g * 4 + team * 2 + 1];
        if (!TRAIN && nact > 0) mbar_wait(&bars->bfull, 0, abort_flag, Q.error, 16); // the f16 images arrive with operand B
        for (unsigned long long tile = tile0; nact > 0 && tile < n_tiles && !*abort_flag; tile += tstep, ++tile_iter) {
            const unsigned long long row = tile * BM + 32ull * q + lane;
            const bool valid = row < P.n;
            uint32_t old2 = 0;
            if (TRAIN && valid) old2 = *reinterpret_cast<const uint16_t *>(reinterpret_cast<const uint8_t *>(P.codes) + row * (unsigned long long)m + g * 4 + team * 2);
            int idxs[2] = {0, 0};
            uint32_t marked = 0, done = 0;
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const int ss = team * 2 + h;
                if (pos_of(ss) == 15) continue;
                const uint32_t it = tile_iter * (uint32_t)nact + (uint32_t)pos_of(ss);
                if (!mbar_wait(&bars->tfull[team], uu & 1u, abort_flag, Q.error, 15)) break;
                ++uu;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)team * BN;
                uint32_t ra[32], rb[32];
                tmem_ld32_issue(taddr, ra);
                const float xh2 = xh_ring[(it & (XH_RING - 1)) * BM + 32 * q + lane];
                const float hmax2 = h ? hmax2_1 : hmax2_0;

                // pass 1: the smallest score (four independent 3-input min chains)
                float b0 = VQB_INF, b1 = VQB_INF, b2 = VQB_INF, b3 = VQB_INF;
                bool col0_nan = false;
                tmem_wait();
#pragma unroll 1
                for (int cb = 0; cb < nch; cb += 2) {
                    if (cb + 1 < nch) tmem_ld32_issue(taddr + (cb + 1) * 32, rb);
                    if (cb == 0) {
                        const float s0 = __uint_as_float(ra[0]);
                        col0_nan = !(s0 == s0);
                    }
#pragma unroll
                    for (int t = 0; t < 32; t += 8) {
                        b0 = min3f(b0, __uint_as_float(ra[t]), __uint_as_float(ra[t + 1]));
                        b1 = min3f(b1, __uint_as_float(ra[t + 2]), __uint_as_float(ra[t + 3]));
                        b2 = min3f(b2, __uint_as_float(ra[t + 4]), __uint_as_float(ra[t + 5]));
                        b3 = min3f(b3, __uint_as_float(ra[t + 6]), __uint_as_float(ra[t + 7]));
                    }
                    tmem_wait();
                    if (cb + 1 < nch) {
                        tmem_ld32_issue(taddr + (cb + 2 < nch ? cb + 2 : 0) * 32, ra); // past the end: the first chunk of pass 2
#pragma unroll
                        for (int t = 0; t < 32; t += 8) {
                            b0 = min3f(b0, __uint_as_float(rb[t]), __uint_as_float(rb[t + 1]));
                            b1 = min3f(b1, __uint_as_float(rb[t + 2]), __uint_as_float(rb[t + 3]));
                            b2 = min3f(b2, __uint_as_float(rb[t + 4]), __uint_as_float(rb[t + 5]));
                            b3 = min3f(b3, __uint_as_float(rb[t + 6]), __uint_as_float(rb[t + 7]));
                        }
                    } else {
                        tmem_ld32_issue(taddr, ra); // odd chunk count: the first chunk of pass 2
                    }
                    tmem_wait();
                }
                const float best = fminf(fminf(b0, b1), fminf(b2, b3));
                const float limit = best + (MARGIN_COEF * (xh2 + hmax2 + fabsf(best)) + 1e-36f);
                // rows the test below cannot rank: NaN / infinity anywhere that matters, or values too small to scale
                // (nor rows whose true distances could overflow f32: there the reference's own comparisons see infinities)
                const bool rankable = !col0_nan && (fabsf(limit) >= 8.6736174e-19f /* 2^-60 */) && (fabsf(limit) < VQB_INF) && (xh2 + hmax2 < 1e37f);
                const uint32_t eb = (__float_as_uint(limit) >> 23) & 0xFFu;
                const float nbig = __uint_as_float(0x80000000u | ((314u - eb) << 23)); // -2^(60 - exponent(limit))
                const float lb = -limit * nbig;                                       // exact scaling

                // pass 2: over the scores below the limit, total = sum (1 + t / 512) and offs = sum chunk * (1 + t / 512),
                // t = column within its 32-column chunk: exactly one score below the limit <=> 1 <= total < 1.07
                float total = 0.0f, offs = 0.0f; // chunk 0 was requested (and awaited) at the end of pass 1
#pragma unroll 1
                for (int cb = 0; cb < nch; cb += 2) {
                    if (cb + 1 < nch) tmem_ld32_issue(taddr + (cb + 1) * 32, rb);
                    {
                        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
                        for (int t = 0; t < 32; t += 4) {
                            a0 = fmaf(fma_sat(__uint_as_float(ra[t]), nbig, lb), 1.0f + (float)t * 0.001953125f, a0);
                            a1 = fmaf(fma_sat(__uint_as_float(ra[t + 1]), nbig, lb), 1.0f + (float)(t + 1) * 0.001953125f, a1);
                            a2 = fmaf(fma_sat(__uint_as_float(ra[t + 2]), nbig, lb), 1.0f + (float)(t + 2) * 0.001953125f, a2);
                            a3 = fmaf(fma_sat(__uint_as_float(ra[t + 3]), nbig, lb), 1.0f + (float)(t + 3) * 0.001953125f, a3);
                        }
                        const float cs = (a0 + a1) + (a2 + a3);
                        total += cs;
                        offs = fmaf(cs, (float)cb, offs);
                    }
                    tmem_wait();
                    if (cb + 1 < nch) {
                        if (cb + 2 < nch) tmem_ld32_issue(taddr + (cb + 2) * 32, ra);
                        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
                        for (int t = 0; t < 32; t += 4) {
                            a0 = fmaf(fma_sat(__uint_as_float(rb[t]), nbig, lb), 1.0f + (float)t * 0.001953125f, a0);
                            a1 = fmaf(fma_sat(__uint_as_float(rb[t + 1]), nbig, lb), 1.0f + (float)(t + 1) * 0.001953125f, a1);
                            a2 = fmaf(fma_sat(__uint_as_float(rb[t + 2]), nbig, lb), 1.0f + (float)(t + 2) * 0.001953125f, a2);
                            a3 = fmaf(fma_sat(__uint_as_float(rb[t + 3]), nbig, lb), 1.0f + (float)(t + 3) * 0.001953125f, a3);
                        }
                        const float cs = (a0 + a1) + (a2 + a3);
                        total += cs;
                        offs = fmaf(cs, (float)(cb + 1), offs);
                        tmem_wait();
                    }
                }
                if (Q.dbg_scores) { // diagnostic dump of the raw scores
                    for (int cb = 0; cb < nch; ++cb) {
                        tmem_ld32_issue(taddr + cb * 32, ra);
                        tmem_wait();
                        if (valid) {
                            float *o = Q.dbg_scores + ((size_t)row * m + g * 4 + ss) * BN + cb * 32;
#pragma unroll
                            for (int t = 0; t < 32; ++t) o[t] = __uint_as_float(ra[t]);
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->tempty[team]);

                const bool single = rankable && total >= 1.0f && total < 1.07f;
                const int idx = single ? ((int)offs) * 32 + (int)((total - 1.0f) * 512.0f + 0.5f) : 0;
                if (h == 0) idxs[0] = idx;
                else idxs[1] = idx;
                if (!single || idx >= k) marked |= 1u << h;
                done |= 1u << h;
            }

            if (valid && done) {
                if (marked) Q.marks[row * (unsigned long long)(m >> 1) + g * 2 + team] = (uint8_t)marked;
                if (TRAIN) {
                    uint8_t *cp = reinterpret_cast<uint8_t *>(P.codes) + row * (unsigned long long)m + g * 4 + team * 2;
                    if (done == 3u && marked == 0u) {
                        const uint32_t nw = (uint32_t)idxs[0] | ((uint32_t)idxs[1] << 8);
                        if (nw != old2) {
                            if ((nw ^ old2) & 0xFFu) moved_mask |= 1u << (team * 2);
                            if ((nw ^ old2) & 0xFF00u) moved_mask |= 1u << (team * 2 + 1);
                            *reinterpret_cast<uint16_t *>(cp) = (uint16_t)nw;
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            if ((done >> h & 1u) && !(marked >> h & 1u)) {
                                const uint32_t ob = (old2 >> (8 * h)) & 0xFFu;
                                if (ob != (uint32_t)idxs[h]) {
                                    moved_mask |= 1u << (team * 2 + h);
                                    cp[h] = (uint8_t)idxs[h];
                                }
                            }
                    }
                } else {
                    const int dim = m * SDW;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        if ((done >> h & 1u) && !(marked >> h & 1u)) {
                            const int ss = team * 2 + h, s = g * 4 + ss;
                            const int idx = idxs[h];
                            if (P.out_codes) P.out_codes[row * m + s] = (uint32_t)idx;
                            if (P.out_f16) // 16-byte aligned: dim % 8 == 0
                                *reinterpret_cast<uint4 *>(P.out_f16 + row * dim + (size_t)s * SDW) = c16_s[ss * BN + idx];
                            if (P.out_f32) {
                                const float4 *c = reinterpret_cast<const float4 *>(P.centroids + ((size_t)s * k + idx) * SDW);
                                float4 *o = reinterpret_cast<float4 *>(P.out_f32 + row * dim + (size_t)s * SDW);
                                o[0] = __ldg(c);
                                o[1] = __ldg(c + 1);
                            }
                        }
                }
            }
            {
                const uint32_t nm = __reduce_add_sync(0xffffffffu, (valid && done) ? (uint32_t)__popc(marked) : 0u);
                if (nm && lane == 0) atomicAdd(Q.stats, (unsigned long long)nm);
            }
        }
        if (TRAIN) {
            moved_mask = __reduce_or_sync(0xffffffffu, moved_mask);
            if (lane == 0)
                for (int ss = 0; ss < 4; ++ss)
                    if (moved_mask & (1u << ss)) atomicOr(P.changed + g * 4 + ss, VQB_MOVED_BITS);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Operand B of one sub-space per block (thread j = centroid j): 32 TF32 numbers per centroid
//   [-ch(8) | -cl(8) | -ch(8) | hn_h, hn_l, 0 ...]   (columns beyond k: zeros and a huge score),
// the binary16 image of the centroid (what an encode writes, src/pq.rs:176-180) and max_j hn_j.
__global__ void pq_operand_b_kernel(const float *cb, int k, float *bop, uint4 *c16, float *hnmax)
{
    __shared__ float smax[BN];
    const int s = blockIdx.x, j = threadIdx.x;
    float4 out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    float hn = 0.0f;
    uint4 img = make_uint4(0, 0, 0, 0);
    if (j < k) {
        const float4 *c = reinterpret_cast<const float4 *>(cb + ((size_t)s * k + j) * SDW);
        const float4 c0 = c[0], c1 = c[1];
        const float v[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float hi[8], lo[8], a = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            hi[i] = to_tf32(v[i]);
            lo[i] = to_tf32(v[i] - hi[i]);
            a = fmaf(v[i], v[i], a);
        }
        hn = 0.5f * a;
        const float hh = to_tf32(hn), hl = to_tf32(hn - hh);
        out[0] = out[4] = make_float4(-hi[0], -hi[1], -hi[2], -hi[3]);
        out[1] = out[5] = make_float4(-hi[4], -hi[5], -hi[6], -hi[7]);
        out[2] = make_float4(-lo[0], -lo[1], -lo[2], -lo[3]);
        out[3] = make_float4(-lo[4], -lo[5], -lo[6], -lo[7]);
        out[6] = make_float4(hh, hl, 0.f, 0.f);
        img.x = f32_to_f16_bits(v[0]) | ((uint32_t)f32_to_f16_bits(v[1]) << 16);
        img.y = f32_to_f16_bits(v[2]) | ((uint32_t)f32_to_f16_bits(v[3]) << 16);
        img.z = f32_to_f16_bits(v[4]) | ((uint32_t)f32_to_f16_bits(v[5]) << 16);
        img.w = f32_to_f16_bits(v[6]) | ((uint32_t)f32_to_f16_bits(v[7]) << 16);
    } else {
        out[6] = make_float4(to_tf32(PAD_SCORE), 0.f, 0.f, 0.f);
    }
    float4 *o = reinterpret_cast<float4 *>(bop + ((size_t)s * BN + j) * KOP);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = out[i];
    c16[(size_t)s * BN + j] = img;
    smax[j] = (j < k) ? fabsf(hn) : 0.0f;
    __syncthreads();
    for (int o2 = BN / 2; o2 > 0; o2 >>= 1) {
        if (j < o2) smax[j] = fmaxf(smax[j], smax[j + o2]); // a NaN half norm is dropped here; its column scores NaN and is never counted
        __syncthreads();
    }
    if (j == 0) hnmax[s] = smax[0];
}

// The marked (row, sub-space) pairs: one warp per pair scans all centroids with the reference's arithmetic
// (src/utils.rs:59-73, src/pq.rs:159-182): strict '<' in ascending index from centroid 0, so a NaN distance never wins
// unless it is centroid 0's, and equal distances keep the lowest index.
template <bool TRAIN, bool EUCLID> __global__ void __launch_bounds__(256) pq_marked_kernel(const PqTcParams Q)
{
    // Each step a CTA reads 256 x 16 mark bytes (all loads independent), collects the marked pairs in shared memory --
    // the list holds the worst case of a step -- and its eight warps then take the pairs in turn, so the work is balanced
    // whatever the distribution of the marks.
    __shared__ uint16_t s_list[256 * 16 * 2];
    __shared__ float s_x[256][SDW];
    __shared__ uint8_t s_old[256];
    __shared__ uint32_t s_count;
    const AssignParams &P = Q.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = P.m, k = P.k, half = m >> 1;
    const unsigned long long total = P.n * (unsigned long long)half; // mark bytes; the buffer is zero-padded to 16
    const unsigned long long total16 = (total + 15) / 16;
    uint32_t moved_lo = 0, moved_hi = 0;
    for (unsigned long long base = (unsigned long long)blockIdx.x * 256ull; base < total16; base += (unsigned long long)gridDim.x * 256ull) {
        if (threadIdx.x == 0) s_count = 0u;
        __syncthreads();
        const unsigned long long mine = base + threadIdx.x;
        if (mine < total16) {
            const uint4 f = reinterpret_cast<const uint4 *>(Q.marks)[mine];
            const uint32_t w[4] = {f.x, f.y, f.z, f.w};
            // the map is handed back all zero, so the next launch needs no memset
            if (f.x | f.y | f.z | f.w) reinterpret_cast<uint4 *>(Q.marks)[mine] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                uint32_t word = w[wi];
                while (word) {
                    const int bit = __ffs(word) - 1; // bit (8 byte + h): pair h of mark byte `byte`
                    word &= word - 1;
                    if ((bit & 7) < 2) s_list[atomicAdd(&s_count, 1u)] = (uint16_t)((threadIdx.x * 16u + (uint32_t)(wi * 4 + (bit >> 3))) * 2u + (uint32_t)(bit & 7));
                }
            }
        }
        __syncthreads();
        const uint32_t cnt = s_count;
        // rounds of up to 256 pairs: first every thread fetches one pair's row slice (and previous code) -- one trip to memory
        // for the whole round instead of one per pair and warp -- then the warps take the pairs in turn
        for (uint32_t r0 = 0; r0 < cnt; r0 += 256) {
            const uint32_t rc = min(256u, cnt - r0);
            if (threadIdx.x < rc) {
                const uint32_t ent = s_list[r0 + threadIdx.x];
                const unsigned long long e = base * 16ull + (ent >> 1);
                if (e < total) {
                    const unsigned long long row = e / half;
                    const int rem = (int)(e % half);
                    const int s = (rem >> 1) * 4 + (rem & 1) * 2 + (int)(ent & 1u);
                    float x[SDW];
                    load_slice<SDW>(x, P.x + row * P.ld + (size_t)s * SDW, P.x_vec4 != 0);
#pragma unroll
                    for (int i = 0; i < SDW; ++i) s_x[threadIdx.x][i] = x[i];
                    if (TRAIN) s_old[threadIdx.x] = reinterpret_cast<const uint8_t *>(P.codes)[row * (unsigned long long)m + s];
                }
            }
            __syncthreads();
            for (uint32_t i = warp; i < rc; i += 8) {
                const uint32_t ent = s_list[r0 + i];
                const unsigned long long e = base * 16ull + (ent >> 1);
                const int h = (int)(ent & 1u);
                if (e >= total) continue;
                const unsigned long long row = e / half;
                const int rem = (int)(e % half);
                const int s = (rem >> 1) * 4 + (rem & 1) * 2 + h;
                float x[SDW];
#pragma unroll
                for (int t = 0; t < SDW; ++t) x[t] = s_x[i][t];
                const float *cbs = P.centroids + (size_t)s * k * SDW;
                float bd = VQB_INF, d0 = 0.0f;
                int bi = 0x7fffffff;
                float c[BN / 32][SDW]; // this lane's centroids j = lane, lane + 32, ...: all requested before the first is used
#pragma unroll
                for (int u = 0; u < BN / 32; ++u) {
                    const int j = lane + 32 * u;
                    if (j < k) {
                        load_centroid<SDW>(c[u], cbs + (size_t)j * SDW);
                    } else {
#pragma unroll
                        for (int t = 0; t < SDW; ++t) c[u][t] = 0.0f;
                    }
                }
#pragma unroll
                for (int u = 0; u < BN / 32; ++u) {
                    const int j = lane + 32 * u;
                    float d = reg_dist<SDW, M_SQ>(x, c[u], 0.0f, 0.0f, 0.0f);
                    if (EUCLID) d = __fsqrt_rn(d);
                    if (j == 0) d0 = d;
                    if (j < k && d < bd) {
                        bd = d;
                        bi = j;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float od = __shfl_xor_sync(0xffffffffu, bd, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (od < bd || (od == bd && oi < bi)) {
                        bd = od;
                        bi = oi;
                    }
                }
                d0 = __shfl_sync(0xffffffffu, d0, 0);
                const int idx = (bi == 0x7fffffff || !(d0 == d0)) ? 0 : bi; // nothing below +inf, or the scan started at a NaN
                if (lane == 0) {
                    bool moved = false;
                    if (TRAIN) {
                        if (s_old[i] != (uint8_t)idx) {
                            moved = true;
                            reinterpret_cast<uint8_t *>(P.codes)[row * (unsigned long long)m + s] = (uint8_t)idx;
                        }
                    } else {
                        store_result<SDW, uint8_t, TRAIN>(P, row, s, idx, cbs, moved);
                    }
                    if (moved) {
                        if (s < 32) moved_lo |= 1u << s;
                        else moved_hi |= 1u << (s - 32);
                    }
                }
            }
            __syncthreads(); // the staged slices are rewritten by the next round
        }
        __syncthreads(); // the list is rewritten by the next step
    }
    if (TRAIN && lane == 0) {
        for (int s = 0; s < m; ++s)
            if ((s < 32 ? moved_lo >> s : moved_hi >> (s - 32)) & 1u) atomicOr(P.changed + s, VQB_MOVED_BITS);
    }
}

} // namespace

bool pq_tc_applicable(const AssignParams &p, int metric)
{
    return (metric == M_SQ || metric == M_EUCLID) && p.sd == SDW && p.m >= 4 && p.m <= MAXM && p.m % 4 == 0 && p.k >= 2 && p.k <= BN &&
           p.ld % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 && p.n >= 1 && (reinterpret_cast<uintptr_t>(p.codes) & 1u) == 0 &&
           (reinterpret_cast<uintptr_t>(p.centroids) & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.out_f16) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(p.out_f32) & 15u) == 0;
}

size_t pq_tc_scratch_floats() { return SCRATCH_FLOATS; }
size_t pq_tc_stats_offset_floats() { return OFF_STATS; }
size_t pq_tc_mark_bytes(size_t n, size_t m) { return (n * (m / 2) + 15) & ~(size_t)15; } // read 16 bytes at a time

template <bool TRAIN, bool EUCLID>
static void launch_t(CudaDevice &dev, const CUtensorMap &mb, const PqTcParams &q, unsigned grid)
{
    auto kernel = pq_tc_kernel<TRAIN, EUCLID>;
    constexpr size_t smem = PQ_TC_SMEM;
    static std::atomic<unsigned long long> configured{0}; // bit d: the attribute has been set on device d (it is per device and sticky)
    const unsigned long long bit = 1ull << (dev.device() & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    {
        KernelScope ks(dev, TRAIN ? "assign_train" : "pq_encode");
        kernel<<<grid, NTHREADS, smem, dev.stream()>>>(mb, q);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
    }
    {
        KernelScope ks(dev, TRAIN ? "assign_train_marked" : "pq_encode_marked");
        // one step (4 KiB of mark bytes) per CTA where the grid allows: the steps are latency-bound and independent
        const unsigned long long steps = ((q.a.n * (unsigned long long)(q.a.m / 2) + 15) / 16 + 255) / 256;
        const unsigned mgrid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>(steps, (unsigned long long)dev.sm_count() * 64));
        pq_marked_kernel<TRAIN, EUCLID><<<mgrid, 256, 0, dev.stream()>>>(q);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
    }
}

void launch_pq_operand_b(CudaDevice &dev, const float *centroids, int m, int k, float *scratch)
{
    KernelScope ks(dev, "pq_operand_b");
    pq_operand_b_kernel<<<m, BN, 0, dev.stream()>>>(centroids, k, scratch + OFF_BOP, reinterpret_cast<uint4 *>(scratch + OFF_C16), scratch + OFF_HMAX);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

void launch_pq_tc(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t code_bytes, const PqTcBuffers &b)
{
    if (train && code_bytes != 1) throw Error(100, "pq tensor path: one-byte codes expected for k <= 256");
    float *bop = b.scratch + OFF_BOP;
    if (b.prepare_operand) launch_pq_operand_b(dev, p.centroids, p.m, p.k, b.scratch);
    const CUtensorMap mb = make_tensor_map_2d(bop, KOP, (unsigned long long)p.m * BN, KOP, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    PqTcParams q;
    q.a = p;
    q.c16 = reinterpret_cast<uint4 *>(b.scratch + OFF_C16);
    q.hnmax = b.scratch + OFF_HMAX;
    q.marks = b.marks; // all zero between launches: the follow-up kernel clears what it reads
    q.stats = reinterpret_cast<unsigned long long *>(b.scratch + OFF_STATS);
    q.error = b.error_word;
    q.dbg_scores = b.dbg_scores;
    const unsigned long long tiles = (p.n + BM - 1) / BM;
    const unsigned ngroups = (unsigned)p.m / 4;
    const unsigned per = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>(tiles, (unsigned long long)dev.sm_count() / ngroups));
    const unsigned grid = per * ngroups;
    if (train) launch_t<true, false>(dev, mb, q, grid);
    else if (metric == M_EUCLID) launch_t<false, true>(dev, mb, q, grid);
    else launch_t<false, false>(dev, mb, q, grid);
}

// ------------------------------------------------------------------------------------------------
// Centroid update of one k-means iteration for the shapes this file serves, in one launch (one CTA per sub-space, thread j =
// cluster j): centroid = sum / count (src/vector.rs:315-316), the operand-B row, binary16 image and largest half norm the next
// assignment pass needs, the iteration's flags for the host, and the sums / counts / flags cleared for the next iteration.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(BN) pq_update_centroids_kernel(float *sums, uint32_t *counts, uint32_t *moved, int counts_f32, const uint32_t *active,
                                                                 int k, float *centroids, float *bop, uint4 *c16, float *hnmax, StatusPage sp,
                                                                 const PeerView pv)
{
    __shared__ float smax[BN];
    const int s = blockIdx.x, j = threadIdx.x;
    const bool act = !active || active[s] != 0;
    const bool direct = pv.world > 1; // the parts of all ranks are added here, in rank order (peer_exchange.cuh)
    peer_arrive_and_wait(pv);
    uint32_t mv_parts[VQB_MAX_PEERS]; // the ranks' "some row moved" words of this sub-space: requested now, used at the end
#pragma unroll
    for (int q = 0; q < VQB_MAX_PEERS; ++q) mv_parts[q] = (direct && j == 0 && q < pv.world) ? peer_ld(pv.words[q] + pv.off_moved + s) : 0u;
    bool empty = false;
    if (act) {
        float4 out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        float hn = 0.0f;
        uint4 img = make_uint4(0, 0, 0, 0);
        if (j < k) {
            const size_t cj = (size_t)s * k + j;
            float4 *cp = reinterpret_cast<float4 *>(centroids + cj * SDW);
            float4 *sp4 = reinterpret_cast<float4 *>(sums + cj * SDW);
            float4 a, b;
            float cf;
            if (direct) {
                // Every peer load is issued before the first one is used.  A warp stops at the first instruction that needs a
                // pending load, so "load rank q, add, load rank q + 1" pays one NVLink round trip (about 2 us) per rank:
                // 30 us of a 44 us kernel at eight ranks.  The parts are then added in rank order as before.
                float4 pa[VQB_MAX_PEERS], pb[VQB_MAX_PEERS];
                uint32_t pc[VQB_MAX_PEERS];
#pragma unroll
                for (int q = 0; q < VQB_MAX_PEERS; ++q) {
                    pa[q] = pb[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                    pc[q] = 0u;
                    if (q < pv.world) {
                        const uint32_t *w = pv.words[q];
                        pa[q] = peer_ld4(w + cj * SDW);
                        pb[q] = peer_ld4(w + cj * SDW + 4);
                        pc[q] = peer_ld(w + pv.off_counts + cj);
                    }
                }
                uint32_t cnt = pc[0];
                a = pa[0], b = pb[0];
#pragma unroll
                for (int q = 1; q < VQB_MAX_PEERS; ++q) {
                    if (q < pv.world) {
                        cnt += pc[q];
                        a.x = __fadd_rn(a.x, pa[q].x), a.y = __fadd_rn(a.y, pa[q].y), a.z = __fadd_rn(a.z, pa[q].z), a.w = __fadd_rn(a.w, pa[q].w);
                        b.x = __fadd_rn(b.x, pb[q].x), b.y = __fadd_rn(b.y, pb[q].y), b.z = __fadd_rn(b.z, pb[q].z), b.w = __fadd_rn(b.w, pb[q].w);
                    }
                }
                cf = __uint2float_rn(cnt);
                float4 *st4 = reinterpret_cast<float4 *>(pv.stale + cj * SDW);
                st4[0] = st4[1] = make_float4(0.f, 0.f, 0.f, 0.f);
                pv.stale[pv.off_counts + cj] = 0u;
            } else {
                const uint32_t cw = counts[cj];
                cf = counts_f32 ? __uint_as_float(cw) : __uint2float_rn(cw);
                a = sp4[0], b = sp4[1];
            }
            float4 c0, c1;
            if (cf != 0.0f) {
                c0 = make_float4(__fdiv_rn(a.x, cf), __fdiv_rn(a.y, cf), __fdiv_rn(a.z, cf), __fdiv_rn(a.w, cf));
                c1 = make_float4(__fdiv_rn(b.x, cf), __fdiv_rn(b.y, cf), __fdiv_rn(b.z, cf), __fdiv_rn(b.w, cf));
                cp[0] = c0;
                cp[1] = c1;
                if (!direct) {
                    sp4[0] = make_float4(0.f, 0.f, 0.f, 0.f);
                    sp4[1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    counts[cj] = 0u;
                }
            } else { // an empty cluster keeps its centroid until the host re-seeds it (src/utils.rs:99-101)
                empty = true;
                c0 = cp[0];
                c1 = cp[1];
            }
            const float v[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            float hi[8], lo[8], a2 = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hi[i] = to_tf32(v[i]);
                lo[i] = to_tf32(v[i] - hi[i]);
                a2 = fmaf(v[i], v[i], a2);
            }
            hn = 0.5f * a2;
            const float hh = to_tf32(hn), hl = to_tf32(hn - hh);
            out[0] = out[4] = make_float4(-hi[0], -hi[1], -hi[2], -hi[3]);
            out[1] = out[5] = make_float4(-hi[4], -hi[5], -hi[6], -hi[7]);
            out[2] = make_float4(-lo[0], -lo[1], -lo[2], -lo[3]);
            out[3] = make_float4(-lo[4], -lo[5], -lo[6], -lo[7]);
            out[6] = make_float4(hh, hl, 0.f, 0.f);
            img.x = f32_to_f16_bits(v[0]) | ((uint32_t)f32_to_f16_bits(v[1]) << 16);
            img.y = f32_to_f16_bits(v[2]) | ((uint32_t)f32_to_f16_bits(v[3]) << 16);
            img.z = f32_to_f16_bits(v[4]) | ((uint32_t)f32_to_f16_bits(v[5]) << 16);
            img.w = f32_to_f16_bits(v[6]) | ((uint32_t)f32_to_f16_bits(v[7]) << 16);
        } else {
            out[6] = make_float4(to_tf32(PAD_SCORE), 0.f, 0.f, 0.f);
        }
        float4 *o = reinterpret_cast<float4 *>(bop + ((size_t)s * BN + j) * KOP);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = out[i];
        c16[(size_t)s * BN + j] = img;
        smax[j] = (j < k) ? fabsf(hn) : 0.0f;
        __syncthreads();
        for (int o2 = BN / 2; o2 > 0; o2 >>= 1) {
            if (j < o2) smax[j] = fmaxf(smax[j], smax[j + o2]);
            __syncthreads();
        }
        if (j == 0) hnmax[s] = smax[0];
    }
    // flags of this sub-space for the host: 8 bitmap words (bit = cluster without rows) and the "some row moved" word
    const uint32_t bits = __ballot_sync(0xffffffffu, empty);
    if ((j & 31) == 0 && (uint32_t)(j >> 5) < sp.words_per_subspace) sp.put(sp.idx_bitmap(s, j >> 5), bits);
    if (j == 0) {
        uint32_t mv = 0u;
        if (direct) {
#pragma unroll
            for (int q = 0; q < VQB_MAX_PEERS; ++q) mv |= mv_parts[q];
            pv.stale[pv.off_moved + s] = 0u;
        } else {
            mv = moved[s];
            moved[s] = 0u;
        }
        sp.put(sp.idx_moved(s), act ? mv : 0u);
        if (s == 0) sp.put_error();
    }
}

void launch_pq_update_centroids(CudaDevice &dev, int m, int k, float *sums, uint32_t *counts, uint32_t *moved, bool counts_f32,
                                const uint32_t *active, float *centroids, float *scratch, const StatusPage &sp, const PeerView &pv)
{
    KernelScope ks(dev, "update_centroids");
    pq_update_centroids_kernel<<<m, BN, 0, dev.stream()>>>(sums, counts, moved, counts_f32 ? 1 : 0, active, k, centroids, scratch + OFF_BOP,
                                                            reinterpret_cast<uint4 *>(scratch + OFF_C16), scratch + OFF_HMAX, sp, pv);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

} // namespace vqb
