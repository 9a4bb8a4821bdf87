// pq_tc.cu -- product-quantizer nearest-centroid search (sub-space width 8) with the dot products on the tensor cores.
//
// Replaces the per-point scan of src/utils.rs:59-73 (training) and src/pq.rs:159-182 (encode) for the Euclidean metrics.
// For every 128-row tile and every sub-space one tcgen05.mma (M128 x N256 x K8, kind::tf32) writes the 128 x 256 dot
// products x.c_j into tensor memory; the epilogue turns them into scores S_j = |c_j|^2/2 - x.c_j, finds the smallest and
// marks every centroid whose score lies within a proven bound of it (the reasoning of dense_tc.cu with K = 8):
//     |dot_tc - x.c| <= 2.0e-3 |x| |c_j|,   limit = S_min + 2E + 1.05 (8 + 6) 2^-24 d + slack,   E = 2.0e-3 |x| max|c_j| (+ half-norm rounding)
// A single marked centroid is the answer; several are decided by the reference's exact f32 arithmetic in ascending index
// order with strict '<' (the row slice is re-read from L2, the centroids from the L1-cached codebook).  The result is the
// exact scan's, bit for bit; rows that cannot be ranked (NaN / infinity) are scanned exactly in full.
//
// CTA (1 per SM, persistent): warp 0 TMA producer (row tiles in 128-byte column chunks = 4 sub-spaces each, 5-stage ring;
// all codebooks once, 8 KiB per sub-space in the 32B-swizzled K-major layout), warp 1 MMA issuer + tensor-memory owner
// (two 256-column accumulators, one per sub-space parity), warps 2..9 epilogue in two teams of four (one row per lane;
// team t takes the sub-spaces of parity t).  All waits are bounded.
#include <algorithm>

#include "assign_reg.cuh"
#include "cuda_device.hpp"
#include "pq_tc.hpp"
#include "tma_host.hpp"
#include "umma.cuh"

namespace vqb {

namespace {

constexpr int BM = 128, BN = 256, SDW = 8, CHUNK = 32, NSTAGE = 5, MAXM = 16;
constexpr uint32_t X_STAGE_BYTES = BM * 128;
constexpr uint32_t CB_BYTES = BN * SDW * 4; // 8 KiB per sub-space

struct alignas(8) PqBarriers {
    unsigned long long full[NSTAGE], empty[NSTAGE], cfull, tfull[2], tempty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct PqTcParams {
    AssignParams a;
    const float *hn;   // [m][256] |c|^2/2, +inf beyond k
    const float *cmax; // [m]      max |c|
    int *error;
};

#define PQ_INF __int_as_float(0x7f800000)

template <typename CodeT, bool TRAIN, bool EUCLID>
__global__ void __launch_bounds__(320, 1) pq_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c, const PqTcParams Q)
{
    extern __shared__ unsigned char smem_raw[];
    const AssignParams &P = Q.a;
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *c_smem = base;                                     // m x 8 KiB
    unsigned char *x_smem = base + (size_t)MAXM * CB_BYTES;           // NSTAGE x 16 KiB
    float *hn_s = reinterpret_cast<float *>(x_smem + (size_t)NSTAGE * X_STAGE_BYTES); // [m][256]
    PqBarriers *bars = reinterpret_cast<PqBarriers *>(hn_s + (size_t)MAXM * BN + MAXM);
    volatile int *abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = P.m, k = P.k;
    const int nchunks = m / 4; // 4 sub-spaces per 128-byte chunk
    const unsigned long long n_tiles = (P.n + BM - 1) / BM;

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
    for (int t = threadIdx.x; t < m * BN; t += blockDim.x) hn_s[t] = Q.hn[t];
    float *cmax_s = hn_s + (size_t)MAXM * BN; // [m]
    if ((int)threadIdx.x < m) cmax_s[threadIdx.x] = Q.cmax[threadIdx.x];
    if (warp == 1) {
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
            mbar_expect_tx(&bars->cfull, (uint32_t)m * CB_BYTES);
            for (int s = 0; s < m; ++s) tma_load_2d(c_smem + (size_t)s * CB_BYTES, &map_c, 0, s * k, &bars->cfull);
            uint32_t it = 0;
            for (unsigned long long tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x) {
                for (int c = 0; c < nchunks; ++c, ++it) {
                    const int st = it % NSTAGE;
                    if (!mbar_wait(&bars->empty[st], ((it / NSTAGE) & 1u) ^ 1u, abort_flag, Q.error, 11)) break;
                    mbar_expect_tx(&bars->full[st], X_STAGE_BYTES);
                    tma_load_2d(x_smem + (size_t)st * X_STAGE_BYTES, &map_x, c * CHUNK, (int)(tile * BM), &bars->full[st]);
                }
            }
            if (*abort_flag) { // let copies in flight land before the CTA retires (bounded)
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
        // ------------------------------------------------ MMA issuer: one K=8 MMA per (tile, sub-space)
        if (lane == 0) {
            bool ok = mbar_wait(&bars->cfull, 0, abort_flag, Q.error, 12);
            uint32_t it = 0, uses[2] = {0, 0};
            for (unsigned long long tile = blockIdx.x; ok && tile < n_tiles && !*abort_flag; tile += gridDim.x) {
                for (int c = 0; ok && c < nchunks; ++c, ++it) {
                    const int st = it % NSTAGE;
                    if (!mbar_wait(&bars->full[st], (it / NSTAGE) & 1u, abort_flag, Q.error, 14)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = smem_desc_sw128(smem_u32(x_smem + (size_t)st * X_STAGE_BYTES));
                    for (int ss = 0; ss < 4; ++ss) {
                        const uint32_t b = (uint32_t)ss & 1u; // sub-space parity = epilogue team = accumulator
                        if (!mbar_wait(&bars->tempty[b], (uses[b] & 1u) ^ 1u, abort_flag, Q.error, 13)) {
                            ok = false;
                            break;
                        }
                        ++uses[b];
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t bdesc = smem_desc_sw32(smem_u32(c_smem + (size_t)(c * 4 + ss) * CB_BYTES));
                        umma_tf32(tmem_base + b * BN, adesc + (uint64_t)(2 * ss), bdesc, 0u); // sub-space ss = bytes [32 ss, 32 ss + 32) of the chunk rows
                        umma_commit(&bars->tfull[b]);
                    }
                    if (ok) umma_commit(&bars->empty[st]);
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue: two teams of four warps; team t owns accumulator t
        // and the sub-spaces s = t, t + 2, ...; within a team warp w reads the TMEM lane quadrant w & 3
        const int q = warp & 3;
        const int team = (warp - 2) >> 2;
        uint32_t moved_mask = 0; // bit s: some row of sub-space s changed its assignment (src/utils.rs:76-80)
        uint32_t uu = 0;         // uses of this team's accumulator so far
        mbar_wait(&bars->cfull, 0, abort_flag, Q.error, 16); // the codebooks are read from shared memory below
        for (unsigned long long tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x) {
            const unsigned long long row = tile * BM + 32ull * q + lane;
            const bool valid = row < P.n;
            // row slices are fetched one sub-space ahead (L2 hits: the tile was just streamed through it)
            float xnext[SDW];
#pragma unroll
            for (int i = 0; i < SDW; ++i) xnext[i] = 0.0f;
            if (valid && team < m) load_slice<SDW>(xnext, P.x + row * P.ld + (size_t)team * SDW, P.x_vec4 != 0);
            // previous assignments of this row (training): one byte per sub-space, fetched once per tile
            uint32_t oldc[4] = {0, 0, 0, 0};
            if (TRAIN && valid) {
                const uint8_t *oc = reinterpret_cast<const uint8_t *>(P.codes) + row * (unsigned long long)m;
                if (m == 16) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(oc);
                    oldc[0] = v.x, oldc[1] = v.y, oldc[2] = v.z, oldc[3] = v.w;
                } else {
                    for (int t = 0; t < m; ++t) oldc[t >> 2] |= (uint32_t)oc[t] << ((t & 3) * 8);
                }
            }
            for (int s = team; s < m && !*abort_flag; s += 2, ++uu) {
                const uint32_t b = (uint32_t)team;
                float x[SDW];
#pragma unroll
                for (int i = 0; i < SDW; ++i) x[i] = xnext[i];
                if (valid && s + 2 < m) load_slice<SDW>(xnext, P.x + row * P.ld + (size_t)(s + 2) * SDW, P.x_vec4 != 0);
                const float *hns = hn_s + (size_t)s * BN;
                if (!mbar_wait(&bars->tfull[b], uu & 1u, abort_flag, Q.error, 15)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + b * BN;
                if (TRAIN && P.active && P.active[s] == 0) { // retired sub-space: hand the accumulator back untouched
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->tempty[b]);
                    continue;
                }

                // pass 1: the smallest score (two independent 3-input min chains)
                float b0 = PQ_INF, b1 = PQ_INF;
                bool col0_nan = false;
                uint32_t ra[32], rb[32];
                tmem_ld32_issue(taddr, ra);
                tmem_wait();
#pragma unroll 1
                for (int cb = 0; cb < BN / 32; cb += 2) {
                    tmem_ld32_issue(taddr + (cb + 1) * 32, rb);
                    if (cb == 0) {
                        const float sc0 = hns[0] - __uint_as_float(ra[0]);
                        col0_nan = !(sc0 == sc0);
                    }
#pragma unroll
                    for (int t = 0; t < 32; t += 4) {
                        b0 = min3f(b0, hns[cb * 32 + t] - __uint_as_float(ra[t]), hns[cb * 32 + t + 1] - __uint_as_float(ra[t + 1]));
                        b1 = min3f(b1, hns[cb * 32 + t + 2] - __uint_as_float(ra[t + 2]), hns[cb * 32 + t + 3] - __uint_as_float(ra[t + 3]));
                    }
                    tmem_wait();
                    if (cb + 2 < BN / 32) tmem_ld32_issue(taddr + (cb + 2) * 32, ra);
#pragma unroll
                    for (int t = 0; t < 32; t += 4) {
                        b0 = min3f(b0, hns[(cb + 1) * 32 + t] - __uint_as_float(rb[t]), hns[(cb + 1) * 32 + t + 1] - __uint_as_float(rb[t + 1]));
                        b1 = min3f(b1, hns[(cb + 1) * 32 + t + 2] - __uint_as_float(rb[t + 2]), hns[(cb + 1) * 32 + t + 3] - __uint_as_float(rb[t + 3]));
                    }
                    tmem_wait();
                }
                const float best = fminf(b0, b1);
                float xn2 = 0.0f;
#pragma unroll
                for (int i = 0; i < SDW; ++i) xn2 = fmaf(x[i], x[i], xn2);
                xn2 *= 1.00001f;
                const float cmax = cmax_s[s];
                const float e2 = 2.0f * 2.0e-3f * sqrtf(xn2) * cmax + 1e-6f * cmax * cmax;
                const float d_a = fmaxf(xn2 + 2.0f * best + e2, 0.0f);
                const float limit = best + e2 + 1.05f * 14.0f * 5.9604645e-8f * d_a + 2.4e-7f * (fabsf(best) + e2) + 1e-36f;
                // rows the comparisons cannot rank (NaN / infinity, or centroid 0 not comparable) are scanned in full
                const bool scan_all = col0_nan || !(best < PQ_INF) || !(limit == limit) || !(fabsf(limit) < PQ_INF);

                // pass 2: candidate bits (sign of limit - S shifted in; reversed and inverted afterwards)
                uint32_t words[BN / 32];
                tmem_ld32_issue(taddr, ra);
                tmem_wait();
#pragma unroll
                for (int cb = 0; cb < BN / 32; cb += 2) {
                    tmem_ld32_issue(taddr + (cb + 1) * 32, rb);
                    uint32_t me = 0, mo = 0;
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        me = __funnelshift_l(__float_as_uint(limit - (hns[cb * 32 + t] - __uint_as_float(ra[t]))), me, 1);
                        mo = __funnelshift_l(__float_as_uint(limit - (hns[cb * 32 + t + 1] - __uint_as_float(ra[t + 1]))), mo, 1);
                    }
                    words[cb] = me | (mo << 16);
                    tmem_wait();
                    if (cb + 2 < BN / 32) tmem_ld32_issue(taddr + (cb + 2) * 32, ra);
                    me = 0, mo = 0;
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        me = __funnelshift_l(__float_as_uint(limit - (hns[(cb + 1) * 32 + t] - __uint_as_float(rb[t]))), me, 1);
                        mo = __funnelshift_l(__float_as_uint(limit - (hns[(cb + 1) * 32 + t + 1] - __uint_as_float(rb[t + 1]))), mo, 1);
                    }
                    words[cb + 1] = me | (mo << 16);
                    tmem_wait();
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->tempty[b]);

                if (valid) {
                    // decode: low half holds even columns, high half odd columns, each most-recent-first and inverted
                    int idx = 0, cnt = 0;
                    float bd = PQ_INF;
                    int bi = -1;
                    const unsigned char *cs = c_smem + (size_t)s * CB_BYTES; // 32B-swizzled: row j at (j/8)*256 + (j%8)*32, halves swapped when (j & 4)
                    auto exact = [&](int j) {
                        const unsigned char *rowp = cs + (size_t)(j >> 3) * 256 + (size_t)(j & 7) * 32;
                        const int sw = ((j >> 2) & 1) * 16;
                        const float4 lo = *reinterpret_cast<const float4 *>(rowp + sw), hi = *reinterpret_cast<const float4 *>(rowp + (16 - sw));
                        const float c[SDW] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                        float d = reg_dist<SDW, M_SQ>(x, c, 0.0f, 0.0f, 0.0f);
                        if (EUCLID) d = __fsqrt_rn(d);
                        if (j == 0) { // the reference's scan starts at centroid 0 whatever its value
                            bd = d;
                            bi = 0;
                        } else {
                            argmin_update(d, j, bd, bi);
                        }
                    };
#pragma unroll 1
                    for (int wd = 0; wd < BN / 32; ++wd) {
                        uint32_t cand = 0;
                        if (scan_all) {
                            cand = 0xFFFFFFFFu;
                        } else {
                            const uint32_t inv = ~words[wd];
                            uint32_t xe = __brev(inv << 16) & 0xFFFFu, xo = __brev(inv & 0xFFFF0000u) & 0xFFFFu; // bit i = column 2i (+1)
                            xe = (xe | (xe << 8)) & 0x00FF00FFu;
                            xe = (xe | (xe << 4)) & 0x0F0F0F0Fu;
                            xe = (xe | (xe << 2)) & 0x33333333u;
                            xe = (xe | (xe << 1)) & 0x55555555u;
                            xo = (xo | (xo << 8)) & 0x00FF00FFu;
                            xo = (xo | (xo << 4)) & 0x0F0F0F0Fu;
                            xo = (xo | (xo << 2)) & 0x33333333u;
                            xo = (xo | (xo << 1)) & 0x55555555u;
                            cand = xe | (xo << 1);
                        }
                        const int lo = wd * 32;
                        cand &= (k >= lo + 32) ? 0xFFFFFFFFu : ((k > lo) ? ((1u << (k - lo)) - 1u) : 0u);
                        while (cand) {
                            const int j = lo + __ffs(cand) - 1;
                            cand &= cand - 1;
                            ++cnt;
                            if (cnt == 1) idx = j;              // a lone candidate needs no arithmetic
                            if (cnt == 2) exact(idx);           // a second one: now the first needs its exact distance too
                            if (cnt >= 2) exact(j);
                        }
                    }
                    if (cnt >= 2) idx = bi < 0 ? 0 : bi;
                    if (cnt == 0) idx = 0;
                    if (TRAIN) {
                        const uint32_t old = (oldc[s >> 2] >> ((s & 3) * 8)) & 0xFFu;
                        if (old != (uint32_t)idx) moved_mask |= 1u << s;
                        reinterpret_cast<uint8_t *>(P.codes)[row * (unsigned long long)m + s] = (uint8_t)idx;
                    } else {
                        // the chosen centroid's values come from the shared-memory copy (src/pq.rs:176-180)
                        const unsigned char *rowp = cs + (size_t)(idx >> 3) * 256 + (size_t)(idx & 7) * 32;
                        const int sw = ((idx >> 2) & 1) * 16;
                        const float4 lo4 = *reinterpret_cast<const float4 *>(rowp + sw), hi4 = *reinterpret_cast<const float4 *>(rowp + (16 - sw));
                        const int dim = m * SDW;
                        if (P.out_codes) P.out_codes[row * m + s] = (uint32_t)idx;
                        if (P.out_f16) {
                            uint4 pk;
                            pk.x = f32_to_f16_bits(lo4.x) | ((uint32_t)f32_to_f16_bits(lo4.y) << 16);
                            pk.y = f32_to_f16_bits(lo4.z) | ((uint32_t)f32_to_f16_bits(lo4.w) << 16);
                            pk.z = f32_to_f16_bits(hi4.x) | ((uint32_t)f32_to_f16_bits(hi4.y) << 16);
                            pk.w = f32_to_f16_bits(hi4.z) | ((uint32_t)f32_to_f16_bits(hi4.w) << 16);
                            *reinterpret_cast<uint4 *>(P.out_f16 + row * dim + (size_t)s * SDW) = pk; // 16-byte aligned: dim % 8 == 0
                        }
                        if (P.out_f32) {
                            float4 *o = reinterpret_cast<float4 *>(P.out_f32 + row * dim + (size_t)s * SDW);
                            o[0] = lo4;
                            o[1] = hi4;
                        }
                    }
                }
            }
        }
        if (TRAIN) {
            moved_mask = __reduce_or_sync(0xffffffffu, moved_mask);
            if (lane == 0)
                for (int s = 0; s < m; ++s)
                    if (moved_mask & (1u << s)) atomicOr(P.changed + s, 1u);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// per sub-space: |c_j|^2/2 (+inf beyond k) and max_j |c_j|
__global__ void pq_codebook_norms_kernel(const float *cb, int m, int k, float *hn, float *cmax)
{
    __shared__ float smax[256];
    const int s = blockIdx.x, j = threadIdx.x;
    float a = 0.0f;
    if (j < k) {
        const float *c = cb + ((size_t)s * k + j) * SDW;
#pragma unroll
        for (int i = 0; i < SDW; ++i) a = fmaf(c[i], c[i], a);
    }
    hn[(size_t)s * BN + j] = (j < k) ? 0.5f * a : PQ_INF;
    smax[j] = (j < k) ? sqrtf(a) : 0.0f;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (j < o) smax[j] = fmaxf(smax[j], smax[j + o]);
        __syncthreads();
    }
    if (j == 0) cmax[s] = smax[0] * 1.000001f;
    (void)m;
}

} // namespace

bool pq_tc_applicable(const AssignParams &p, int metric)
{
    return (metric == M_SQ || metric == M_EUCLID) && p.sd == SDW && p.m >= 4 && p.m <= MAXM && p.m % 4 == 0 && p.k >= 2 && p.k <= BN &&
           p.ld == (unsigned long long)p.m * SDW && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 && p.n >= 1 &&
           (reinterpret_cast<uintptr_t>(p.codes) & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.out_f16) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(p.out_f32) & 15u) == 0;
}

size_t pq_tc_scratch_floats() { return (size_t)MAXM * BN + MAXM; }

template <typename CodeT, bool TRAIN, bool EUCLID>
static void launch_t(CudaDevice &dev, const CUtensorMap &mx, const CUtensorMap &mc, const PqTcParams &q, size_t smem, unsigned grid)
{
    auto kernel = pq_tc_kernel<CodeT, TRAIN, EUCLID>;
    VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KernelScope ks(dev, TRAIN ? "assign_train" : "pq_encode");
    kernel<<<grid, 320, smem, dev.stream()>>>(mx, mc, q);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

void launch_pq_tc(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t code_bytes, float *scratch, int *error_word)
{
    {
        KernelScope ks(dev, "codebook_norms");
        pq_codebook_norms_kernel<<<p.m, 256, 0, dev.stream()>>>(p.centroids, p.m, p.k, scratch, scratch + (size_t)MAXM * BN);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
    }
    const CUtensorMap mx = make_tensor_map_2d(p.x, (unsigned long long)p.ld, p.n, CHUNK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap mc = make_tensor_map_2d(p.centroids, SDW, (unsigned long long)p.m * p.k, SDW, BN, CU_TENSOR_MAP_SWIZZLE_32B);
    PqTcParams q;
    q.a = p;
    q.hn = scratch;
    q.cmax = scratch + (size_t)MAXM * BN;
    q.error = error_word;
    const size_t smem = 1024 + (size_t)MAXM * CB_BYTES + (size_t)NSTAGE * X_STAGE_BYTES + ((size_t)MAXM * BN + MAXM) * sizeof(float) + sizeof(PqBarriers) + 64;
    const unsigned long long tiles = (p.n + BM - 1) / BM;
    const unsigned grid = (unsigned)std::min<unsigned long long>(tiles, (unsigned long long)dev.sm_count());
    const bool eu = metric == M_EUCLID;
    if (train) {
        if (code_bytes == 1) launch_t<uint8_t, true, false>(dev, mx, mc, q, smem, grid);
        else if (code_bytes == 2) launch_t<uint16_t, true, false>(dev, mx, mc, q, smem, grid);
        else launch_t<uint32_t, true, false>(dev, mx, mc, q, smem, grid);
    } else if (eu) {
        launch_t<uint32_t, false, true>(dev, mx, mc, q, smem, grid);
    } else {
        launch_t<uint32_t, false, false>(dev, mx, mc, q, smem, grid);
    }
}

} // namespace vqb
