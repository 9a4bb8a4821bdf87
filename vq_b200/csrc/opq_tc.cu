// opq_tc.cu -- the two dense contractions of the optimized product quantizer on the 5th-generation tensor cores.
//
//   rotate:      y_r = R x_r for every row          (src/opq.rs:186-194 in fit, 232-234 in quantize)   Y = X R^T,  n x dim x dim
//   cross_cov:   A = Y X^T = sum_r y_r x_r^T        (src/opq.rs:172-179)                               dim x n x dim
//
// Both run as tcgen05.mma (kind::tf32, f32 accumulation in tensor memory) with SPLIT operands, so that the result keeps f32
// accuracy although TF32 carries 10 mantissa bits: every f32 number v is written as vh + vl with vh = tf32(v) and
// vl = tf32(v - vh), both exactly representable (what the hardware does with the low 13 bits of its inputs then does not
// matter), and a product a.b is accumulated as ah.bh + al.bh + ah.bl.  The dropped al.bl and the rounding of the low parts
// are below 3 * 2^-22 |a||b|; tests/test_gpu_opq_tensor.py measures the error against f64.
//
// Operand layouts (shared memory, 128-byte swizzle, canonical tcgen05 tiles):
//   rotate     A = X tile, K-major: 128 rows x 32 floats per K chunk (the row is the M index, dimensions are K);
//              B = R, K-major: dim rows (outputs) x 32 floats per K chunk, hi and lo copies resident for the whole launch,
//              loaded by TMA (tensor maps over this GPU's memory, no multicast).
//   cross_cov  the contraction runs over ROWS, so both operands are MN-major: a stage holds 32 rows (K) of Y and of X as
//              dim/32 column chunks of 32 rows x 128 bytes, which is how the rows lie in memory -- no transposition anywhere
//              (128-byte swizzle with 32-byte base, the one swizzled MN-major layout the tensor core takes for 32-bit elements).
// The split needs a pass through registers, so the row tiles are read from global memory by converter warps (coalesced 128-bit
// loads, one stage ahead) and written as hi / lo tiles with the swizzle applied; fence.proxy.async + mbarrier hand them to the
// MMA thread.  One persistent CTA per SM:
//   warp 0      operand B by TMA (rotate only)
//   warp 1      owns tensor memory (two accumulators) and issues the MMAs
//   warps 2-9   converters (three stages of global loads in flight per thread)
//   warps 10-13 epilogue: tcgen05.ld, one accumulator row per lane; rotate writes Y through a shared-memory transposition (whole
//               128-byte row pieces per store), cross_cov adds the accumulator to an f32 partial sum and, at the end, to the f64 result
// Every wait is bounded; on expiry the CTA records a code, stops issuing, frees tensor memory and the host raises an error.
#include <algorithm>
#include <atomic>

#include "cuda_device.hpp"
#include "kernels_common.cuh"
#include "opq_tc.hpp"
#include "tma_host.hpp"
#include "umma.cuh"

namespace vqb {

namespace {

constexpr int BM = 128;                    // rows per rotate tile = accumulator lanes
constexpr int CHUNK = 32;                  // f32 per 128-byte swizzle row
constexpr int NST = 2;                     // stage ring depth (rotate: hi + lo tile of one K chunk; cross_cov: four operand tiles)
constexpr int NCONV = 8;                   // converter warps
constexpr int PF = 3;                      // stages of global loads a converter thread keeps in flight (registers)
constexpr int NTHREADS = 32 * (2 + NCONV + 4);
constexpr uint32_t STAGE_ROW_BYTES = 144;  // epilogue staging: 32 floats of a row + 16 bytes, so that rows start in different banks
constexpr uint32_t TILE_BYTES = 128 * 128; // one 128 x 32-float operand tile
constexpr int XC_ROWS = 32;                // rows (K) per cross_cov stage
// The tensor core adds into its f32 accumulator with truncation, not round-to-nearest: over 1536 accumulator updates (4096 rows)
// the sums came out 1.5e-5 low.  So the accumulator is drained every 4 stages (128 rows, 48 updates, bias below 1.5e-6) into an
// f32 partial sum in shared memory with ordinary rounded additions, and that sum joins the f64 result once per CTA.
constexpr int XC_FLUSH_STAGES = 4;

struct alignas(8) OpqBarriers {
    unsigned long long afull[NST], aempty[NST], bfull, tfull[2], tempty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// kind::tf32, f32 accumulate, M = 128, N = n; a_mn / b_mn: operand is MN-major (transposed) instead of K-major
__host__ __device__ constexpr uint32_t idesc_tf32(int n, bool a_mn, bool b_mn)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32_d(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
}

// MN-major TF32 operand tile.  For 32-bit elements the tensor core takes exactly one swizzled MN-major layout, the 128-byte
// swizzle with a 32-byte base (layout type 1): rows of 32 floats along the M / N index, four rows of the K index per 512-byte
// atom, and inside every row the four 32-byte units are permuted by (unit ^ (row & 3)).  Column chunks (32 floats of M / N)
// are `chunk_bytes` apart (leading byte offset), the 4-row atoms along K 512 bytes (stride byte offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t chunk_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((chunk_bytes >> 4) & 0x3FFFu) << 16; // leading byte offset: between column chunks
    d |= (uint64_t)(512u >> 4) << 32;                    // stride byte offset: between 4-row atoms of K
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;                              // layout type: 128-byte swizzle, 32-byte base
    return d;
}

// byte offset of 16-byte unit e16 (0..7) of K row r inside its 128-byte row under that swizzle
__device__ __forceinline__ uint32_t mn_swizzle_unit(int e16, int r) { return (uint32_t)((((e16 >> 1) ^ (r & 3)) << 5) | ((e16 & 1) << 4)); }

__device__ __forceinline__ void split4(const float4 v, float4 &hi, float4 &lo)
{
    hi.x = tf32_round(v.x), hi.y = tf32_round(v.y), hi.z = tf32_round(v.z), hi.w = tf32_round(v.w);
    lo.x = tf32_round(v.x - hi.x), lo.y = tf32_round(v.y - hi.y), lo.z = tf32_round(v.z - hi.z), lo.w = tf32_round(v.w - hi.w);
}

__device__ __forceinline__ void common_setup(OpqBarriers *bars, int warp, uint32_t tmem_cols)
{
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bars->afull[s], NCONV);
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
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// rotate: Y = X R^T
// ------------------------------------------------------------------------------------------------
struct RotateParams {
    const float *x;
    float *y;
    unsigned long long n;
    int dim, kchunks;
    int *error;
};

__global__ void __launch_bounds__(NTHREADS, 1) opq_rotate_kernel(const __grid_constant__ CUtensorMap map_rh, const __grid_constant__ CUtensorMap map_rl,
                                                                 const RotateParams P)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int dim = P.dim, kchunks = P.kchunks;
    const uint32_t b_chunk = (uint32_t)dim * 128u;                 // bytes of one K chunk of R (dim rows x 128 bytes)
    unsigned char *bh_smem = base;                                 // kchunks x b_chunk
    unsigned char *bl_smem = base + (size_t)kchunks * b_chunk;     // kchunks x b_chunk
    unsigned char *a_smem = base + 2 * (size_t)kchunks * b_chunk;  // NST x (hi 16 KiB + lo 16 KiB)
    unsigned char *o_smem = a_smem + (size_t)NST * 2 * TILE_BYTES; // 4 epilogue warps x 32 rows x 144 bytes: output staging
    OpqBarriers *bars = reinterpret_cast<OpqBarriers *>(o_smem + 4 * 32 * STAGE_ROW_BYTES);
    volatile int *abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long n_tiles = (P.n + BM - 1) / BM;

    common_setup(bars, warp, 256u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t idesc = idesc_tf32(dim, false, false);

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars->bfull, 2u * (uint32_t)kchunks * b_chunk);
            for (int kc = 0; kc < kchunks; ++kc) {
                tma_load_2d(bh_smem + (size_t)kc * b_chunk, &map_rh, kc * CHUNK, 0, &bars->bfull);
                tma_load_2d(bl_smem + (size_t)kc * b_chunk, &map_rl, kc * CHUNK, 0, &bars->bfull);
            }
            mbar_wait(&bars->bfull, 0, abort_flag, P.error, 21); // the copies have landed before this warp retires
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(&bars->bfull, 0, abort_flag, P.error, 22);
            uint32_t it = 0, local = 0;
            for (unsigned long long tile = blockIdx.x; ok && tile < n_tiles && !*abort_flag; tile += gridDim.x, ++local) {
                const uint32_t b = local & 1u, buse = local >> 1;
                if (!mbar_wait(&bars->tempty[b], (buse & 1u) ^ 1u, abort_flag, P.error, 23)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + b * 128u;
                for (int kc = 0; kc < kchunks; ++kc, ++it) {
                    const int st = it % NST;
                    if (!mbar_wait(&bars->afull[st], (it / NST) & 1u, abort_flag, P.error, 24)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ah = smem_desc_sw128(smem_u32(a_smem + (size_t)st * 2 * TILE_BYTES));
                    const uint64_t al = smem_desc_sw128(smem_u32(a_smem + (size_t)st * 2 * TILE_BYTES + TILE_BYTES));
                    const uint64_t bh = smem_desc_sw128(smem_u32(bh_smem + (size_t)kc * b_chunk));
                    const uint64_t bl = smem_desc_sw128(smem_u32(bl_smem + (size_t)kc * b_chunk));
#pragma unroll
                    for (int k8 = 0; k8 < CHUNK / 8; ++k8) { // 8 f32 = 32 bytes = 2 descriptor units per step
                        const uint64_t o = (uint64_t)(2 * k8);
                        umma_tf32_d(d_tmem, ah + o, bh + o, idesc, (kc | k8) ? 1u : 0u);
                        umma_tf32_d(d_tmem, al + o, bh + o, idesc, 1u);
                        umma_tf32_d(d_tmem, ah + o, bl + o, idesc, 1u);
                    }
                    umma_commit(&bars->aempty[st]);
                }
                if (ok) umma_commit(&bars->tfull[b]);
            }
        }
    } else if (warp < 2 + NCONV) {
        // converters: 8 lanes per row (16 bytes each), 4 rows per warp instruction, rows cw*16 .. cw*16+15 of the tile per warp.
        // Stage g of this CTA is K chunk g % kchunks of its tile g / kchunks.  A thread keeps PF stages of loads in flight: with
        // one stage the kernel ran at the pace of one DRAM round trip per stage.
        const int cw = warp - 2, sub = lane >> 3, e16 = lane & 7;
        const unsigned long long my_tiles = (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
        const unsigned long long total = my_tiles * (unsigned long long)kchunks;
        auto fetch = [&](float4(&dst)[4], unsigned long long gidx) {
            const unsigned long long tile = blockIdx.x + (gidx / kchunks) * gridDim.x;
            const int kc = (int)(gidx % kchunks);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = cw * 16 + i * 4 + sub;
                const unsigned long long row = tile * BM + r;
                dst[i] = (gidx < total && row < P.n) ? __ldg(reinterpret_cast<const float4 *>(P.x + row * dim + kc * CHUNK) + e16)
                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        auto convert = [&](const float4(&src)[4], unsigned long long gidx) -> bool {
            const uint32_t it = (uint32_t)gidx;
            const int st = it % NST;
            if (!mbar_wait(&bars->aempty[st], ((it / NST) & 1u) ^ 1u, abort_flag, P.error, 25)) return false;
            unsigned char *hi_t = a_smem + (size_t)st * 2 * TILE_BYTES, *lo_t = hi_t + TILE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = cw * 16 + i * 4 + sub;
                float4 h, l;
                split4(src[i], h, l);
                const uint32_t off = (uint32_t)r * 128u + (uint32_t)((e16 ^ (r & 7)) << 4);
                *reinterpret_cast<float4 *>(hi_t + off) = h;
                *reinterpret_cast<float4 *>(lo_t + off) = l;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->afull[st]);
            return true;
        };
        float4 p0[4], p1[4], p2[4];
        static_assert(PF == 3, "the ring below is written out for three stages");
        fetch(p0, 0);
        fetch(p1, 1);
        fetch(p2, 2);
        for (unsigned long long gidx = 0; gidx < total && !*abort_flag; gidx += PF) {
            if (!convert(p0, gidx)) break;
            fetch(p0, gidx + 3);
            if (gidx + 1 < total) {
                if (!convert(p1, gidx + 1)) break;
                fetch(p1, gidx + 4);
            }
            if (gidx + 2 < total) {
                if (!convert(p2, gidx + 2)) break;
                fetch(p2, gidx + 5);
            }
        }
    } else {
        // epilogue: one accumulator row per lane, 32 outputs per tensor-memory load; the 32 x 32 block goes through shared memory
        // so that a store instruction writes four 128-byte row pieces instead of 32 scattered 16-byte pieces
        const int q = warp & 3;
        unsigned char *stg = o_smem + (size_t)q * 32 * STAGE_ROW_BYTES;
        const int rsub = lane >> 3, unit = lane & 7;
        uint32_t local = 0;
        for (unsigned long long tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x, ++local) {
            const uint32_t b = local & 1u, buse = local >> 1;
            if (!mbar_wait(&bars->tfull[b], buse & 1u, abort_flag, P.error, 26)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned long long row_base = tile * BM + 32ull * q;
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + b * 128u;
            uint32_t ra[32];
            for (int cb = 0; cb < kchunks; ++cb) {
                tmem_ld32_issue(taddr + cb * 32, ra);
                tmem_wait();
                float4 *mine = reinterpret_cast<float4 *>(stg + (size_t)lane * STAGE_ROW_BYTES);
#pragma unroll
                for (int t = 0; t < 8; ++t)
                    mine[t] = make_float4(__uint_as_float(ra[4 * t]), __uint_as_float(ra[4 * t + 1]), __uint_as_float(ra[4 * t + 2]), __uint_as_float(ra[4 * t + 3]));
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = i * 4 + rsub;
                    const float4 v = *reinterpret_cast<const float4 *>(stg + (size_t)r * STAGE_ROW_BYTES + unit * 16);
                    if (row_base + r < P.n) *reinterpret_cast<float4 *>(P.y + (row_base + r) * dim + cb * 32 + unit * 4) = v;
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tempty[b]);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
    }
}

// R (dim x dim, row-major) -> its TF32 high and low parts
__global__ void opq_split_matrix_kernel(const float *r, int count, float *hi, float *lo)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < count) {
        const float v = r[t], h = tf32_round(v);
        hi[t] = h;
        lo[t] = tf32_round(v - h);
    }
}

// ------------------------------------------------------------------------------------------------
// cross_cov: A += Y^T X over this CTA's rows
// ------------------------------------------------------------------------------------------------
struct CrossParams {
    const float *y, *x;
    unsigned long long n;
    int dim, kchunks;
    double *a; // [dim][dim], zero-filled by the caller
    int *error;
};

__global__ void __launch_bounds__(NTHREADS, 1) opq_cross_cov_kernel(const CrossParams P)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // a stage: Y hi | Y lo | X hi | X lo, each four column chunks of 32 rows x 128 bytes (the chunks beyond dim stay zero)
    constexpr uint32_t OPER_BYTES = 4 * XC_ROWS * 128; // 16 KiB
    constexpr uint32_t STAGE_BYTES = 4 * OPER_BYTES;   // 64 KiB
    unsigned char *s_smem = base;
    float *part = reinterpret_cast<float *>(s_smem + (size_t)NST * STAGE_BYTES); // [128 columns j][128 rows i]: this CTA's partial A
    OpqBarriers *bars = reinterpret_cast<OpqBarriers *>(part + 128 * 128);
    volatile int *abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dim = P.dim, kchunks = P.kchunks;
    const unsigned long long n_blocks = (P.n + XC_ROWS - 1) / XC_ROWS;       // stages of 32 rows in the whole input
    const unsigned long long per_cta = (n_blocks + gridDim.x - 1) / gridDim.x; // contiguous range per CTA
    const unsigned long long blk_begin = min(n_blocks, (unsigned long long)blockIdx.x * per_cta);
    const unsigned long long blk_end = min(n_blocks, blk_begin + per_cta);
    const unsigned long long my_blocks = blk_end - blk_begin;

    for (uint32_t t = threadIdx.x; t < (NST * STAGE_BYTES + 128 * 128 * 4) / 16; t += NTHREADS) reinterpret_cast<uint4 *>(s_smem)[t] = make_uint4(0, 0, 0, 0);
    common_setup(bars, warp, 256u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the zero fill is visible to the MMA's reads
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t idesc = idesc_tf32(dim, true, true);

    if (warp == 1) {
        if (lane == 0) {
            uint32_t flushes = 0;
            bool ok = true;
            for (unsigned long long j = 0; ok && j < my_blocks && !*abort_flag; ++j) {
                const uint32_t it = (uint32_t)j;
                const uint32_t in_acc = it % XC_FLUSH_STAGES;
                const uint32_t b = flushes & 1u, buse = flushes >> 1;
                if (in_acc == 0) {
                    if (!mbar_wait(&bars->tempty[b], (buse & 1u) ^ 1u, abort_flag, P.error, 31)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                const int st = it % NST;
                if (!mbar_wait(&bars->afull[st], (it / NST) & 1u, abort_flag, P.error, 32)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + b * 128u;
                const uint32_t sbase = smem_u32(s_smem + (size_t)st * STAGE_BYTES);
#pragma unroll
                for (int k8 = 0; k8 < XC_ROWS / 8; ++k8) { // 8 rows of K = one 1024-byte group of every column chunk
                    const uint32_t o = (uint32_t)k8 * 1024u;
                    const uint64_t yh = smem_desc_mn_sw128(sbase + o, XC_ROWS * 128), yl = smem_desc_mn_sw128(sbase + OPER_BYTES + o, XC_ROWS * 128);
                    const uint64_t xh = smem_desc_mn_sw128(sbase + 2 * OPER_BYTES + o, XC_ROWS * 128), xl = smem_desc_mn_sw128(sbase + 3 * OPER_BYTES + o, XC_ROWS * 128);
                    umma_tf32_d(d_tmem, yh, xh, idesc, (in_acc | (uint32_t)k8) ? 1u : 0u);
                    umma_tf32_d(d_tmem, yl, xh, idesc, 1u);
                    umma_tf32_d(d_tmem, yh, xl, idesc, 1u);
                }
                umma_commit(&bars->aempty[st]);
                if (in_acc == XC_FLUSH_STAGES - 1 || j + 1 == my_blocks) {
                    umma_commit(&bars->tfull[b]);
                    ++flushes;
                }
            }
        }
    } else if (warp >= 2 && warp < 2 + NCONV) {
        // converters: a warp instruction reads one whole row (lane l = floats 4l .. 4l+3); warp cw takes rows cw, cw+8, ... of the
        // stage; PF stages of loads in flight per thread
        const int cw = warp - 2;
        const int c = lane >> 3, e16 = lane & 7; // column chunk and 16-byte unit of this lane's float4
        const bool lane_in = lane * 4 < dim;
        constexpr int RPW = XC_ROWS / NCONV; // rows of a stage per warp
        auto fetch = [&](float4(&dy)[RPW], float4(&dx)[RPW], unsigned long long j) {
            const unsigned long long blk = blk_begin + j;
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const unsigned long long row = blk * XC_ROWS + (unsigned long long)(cw + NCONV * i);
                const bool in = lane_in && blk < blk_end && row < P.n;
                dy[i] = in ? __ldg(reinterpret_cast<const float4 *>(P.y + row * dim) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                dx[i] = in ? __ldg(reinterpret_cast<const float4 *>(P.x + row * dim) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        auto convert = [&](const float4(&sy)[RPW], const float4(&sx)[RPW], unsigned long long j) -> bool {
            const uint32_t it = (uint32_t)j;
            const int st = it % NST;
            if (!mbar_wait(&bars->aempty[st], ((it / NST) & 1u) ^ 1u, abort_flag, P.error, 33)) return false;
            unsigned char *sb = s_smem + (size_t)st * STAGE_BYTES;
            if (lane_in) {
#pragma unroll
                for (int i = 0; i < RPW; ++i) {
                    const int r = cw + NCONV * i;
                    const uint32_t off = (uint32_t)c * (XC_ROWS * 128u) + (uint32_t)r * 128u + mn_swizzle_unit(e16, r);
                    float4 h, l;
                    split4(sy[i], h, l);
                    *reinterpret_cast<float4 *>(sb + off) = h;
                    *reinterpret_cast<float4 *>(sb + OPER_BYTES + off) = l;
                    split4(sx[i], h, l);
                    *reinterpret_cast<float4 *>(sb + 2 * OPER_BYTES + off) = h;
                    *reinterpret_cast<float4 *>(sb + 3 * OPER_BYTES + off) = l;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->afull[st]);
            return true;
        };
        float4 y0[RPW], x0[RPW], y1[RPW], x1[RPW], y2[RPW], x2[RPW];
        fetch(y0, x0, 0);
        fetch(y1, x1, 1);
        fetch(y2, x2, 2);
        for (unsigned long long j = 0; j < my_blocks && !*abort_flag; j += PF) {
            if (!convert(y0, x0, j)) break;
            fetch(y0, x0, j + 3);
            if (j + 1 < my_blocks) {
                if (!convert(y1, x1, j + 1)) break;
                fetch(y1, x1, j + 4);
            }
            if (j + 2 < my_blocks) {
                if (!convert(y2, x2, j + 2)) break;
                fetch(y2, x2, j + 5);
            }
        }
    } else if (warp >= 2 + NCONV) {
        // epilogue: lane = dimension i of Y, columns = dimensions j of X
        const int q = warp & 3;
        const unsigned long long n_flush = (my_blocks + XC_FLUSH_STAGES - 1) / XC_FLUSH_STAGES;
        const int i = 32 * q + lane;
        for (unsigned long long f = 0; f < n_flush && !*abort_flag; ++f) {
            const uint32_t b = (uint32_t)f & 1u, buse = (uint32_t)f >> 1;
            if (!mbar_wait(&bars->tfull[b], buse & 1u, abort_flag, P.error, 34)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + b * 128u;
            uint32_t ra[32];
            for (int cb = 0; cb < kchunks; ++cb) {
                tmem_ld32_issue(taddr + cb * 32, ra);
                tmem_wait();
#pragma unroll
                for (int t = 0; t < 32; ++t) { // only this thread ever touches row i of the partial sum
                    float *pp = part + (size_t)(cb * 32 + t) * 128 + i;
                    *pp = __fadd_rn(*pp, __uint_as_float(ra[t]));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tempty[b]);
        }
        if (i < dim && my_blocks > 0 && !*abort_flag)
            for (int j = 0; j < dim; ++j) atomicAdd(P.a + (size_t)i * dim + j, (double)part[(size_t)j * 128 + i]);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
    }
}

template <typename K> void set_smem_once(K kernel, size_t smem, int device, std::atomic<unsigned long long> &configured)
{
    const unsigned long long bit = 1ull << (device & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
}

} // namespace

bool opq_tc_applicable(size_t dim, const float *x, const float *y)
{
    return dim >= 32 && dim <= 128 && dim % 32 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
}

size_t opq_tc_split_floats(size_t dim) { return 2 * dim * dim; }

void launch_opq_rotate(CudaDevice &dev, const float *rot, size_t dim, const float *x, size_t n, float *y, float *split, int *error_word)
{
    const int count = (int)(dim * dim);
    float *hi = split, *lo = split + dim * dim;
    {
        KernelScope ks(dev, "rotation_split");
        opq_split_matrix_kernel<<<(count + 255) / 256, 256, 0, dev.stream()>>>(rot, count, hi, lo);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
    }
    const CUtensorMap mh = make_tensor_map_2d(hi, dim, dim, CHUNK, (unsigned)dim, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap ml = make_tensor_map_2d(lo, dim, dim, CHUNK, (unsigned)dim, CU_TENSOR_MAP_SWIZZLE_128B);
    RotateParams p;
    p.x = x;
    p.y = y;
    p.n = n;
    p.dim = (int)dim;
    p.kchunks = (int)(dim / CHUNK);
    p.error = error_word;
    const size_t fixed = (size_t)NST * 2 * TILE_BYTES + 4 * 32 * STAGE_ROW_BYTES + sizeof(OpqBarriers) + 64;
    const size_t smem = 1024 + 2 * (size_t)p.kchunks * dim * 128 + fixed;
    static std::atomic<unsigned long long> configured{0};
    set_smem_once(opq_rotate_kernel, 1024 + 2 * (size_t)4 * 128 * 128 + fixed, dev.device(), configured);
    const unsigned long long tiles = (n + BM - 1) / BM;
    const unsigned grid = (unsigned)std::min<unsigned long long>(tiles, (unsigned long long)dev.sm_count());
    KernelScope ks(dev, "rotate_rows");
    opq_rotate_kernel<<<grid, NTHREADS, smem, dev.stream()>>>(mh, ml, p);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

void launch_opq_cross_cov(CudaDevice &dev, const float *y, const float *x, size_t n, size_t dim, double *a, int *error_word)
{
    CrossParams p;
    p.y = y;
    p.x = x;
    p.n = n;
    p.dim = (int)dim;
    p.kchunks = (int)(dim / CHUNK);
    p.a = a;
    p.error = error_word;
    const size_t smem = 1024 + (size_t)NST * 4 * 4 * XC_ROWS * 128 + 128 * 128 * sizeof(float) + sizeof(OpqBarriers) + 64;
    static std::atomic<unsigned long long> configured{0};
    set_smem_once(opq_cross_cov_kernel, smem, dev.device(), configured);
    const unsigned long long blocks = (n + XC_ROWS - 1) / XC_ROWS;
    const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>(blocks, (unsigned long long)dev.sm_count()));
    KernelScope ks(dev, "cross_cov");
    opq_cross_cov_kernel<<<grid, NTHREADS, smem, dev.stream()>>>(p);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

} // namespace vqb
