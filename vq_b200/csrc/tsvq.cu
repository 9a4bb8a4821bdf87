// tsvq.cu -- tree-structured vector quantizer (src/tsvq.rs) built level by level on the device.
//
// The reference recurses; here all nodes of one depth are processed together and numbered breadth-first (left child before
// right).  What fixes the result bit for bit is kept: the centroid of a node is the f32 sum of its rows divided by
// `len as f32` (mean_vector, src/vector.rs:282-318), added up as the sum of the sums of consecutive 1024-row chunks -- for
// up to 1024 rows the reference's serial order, above that one admissible order where the reference's own parallel
// reduction is unspecified, and one whose chunks can be added side by side; a dimension's spread is the serial f32 sum of
// (v - c)^2 in data order (src/tsvq.rs:86-98), which no reordering may touch; the
// split dimension is the last of equal maxima (max_by, 101-105); the median is taken from the sorted values (108-116); the
// partition is stable (119-122); children exist only when both sides are non-empty (127-141).
//
// Per level: chunk_sums_kernel + node_mean_kernel (centroids), node_spread_stream_kernel or node_spread_kernel (spreads of
// the nodes that split), pick_split_kernel, a 64-bit radix sort of (node, value) keys (CUB, library code off the hot path) from which the medians
// are read, a flag + exclusive scan (CUB) + scatter for the stable partition, and one small download of the left counts
// from which the host numbers the children.  The build is not sharded: every rank of a multi-GPU job builds the same tree.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <cstdlib>
#include <vector>

#include "cuda_device.hpp"
#include "kernels_common.cuh"
#include "tsvq.hpp"
#include "umma.cuh"

namespace vqb {

namespace {

struct NodeInfo {
    unsigned long long start, count;
    int split;       // 1: this node is being split at this level
    int split_dim;
    float median;
    unsigned long long sorted_start; // first key of this node in the sorted key array
    unsigned long long nleft;
    int child_left, child_right; // ids given by the host after the partition, -1 = none
    unsigned long long chunk0;   // first of this node's 1024-row chunks in the level's chunk table
    unsigned int nchunks;
};

constexpr unsigned MEAN_CHUNK = 1024;
struct ChunkInfo {
    unsigned long long start; // position of the chunk's first row in perm
    unsigned int rows;
};

constexpr uint32_t DEAD = 0xFFFFFFFFu;

// order-preserving map of f32 onto u32 (no NaN here)
__device__ __forceinline__ uint32_t f32_key(float v)
{
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_f32(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// ---- centroids: one warp per (1024-row chunk, 32 dimensions) adds the chunk's rows in data order (lane = dimension; the
// row numbers of the next 32 rows are requested while the current 32 rows are in flight), then one thread per (node,
// dimension) adds the node's chunk sums in order and divides.
__global__ void __launch_bounds__(128) chunk_sums_kernel(const float *__restrict__ x, size_t dim, const uint32_t *__restrict__ perm,
                                                         const ChunkInfo *chunks, float *partial)
{
    const ChunkInfo ch = chunks[blockIdx.x];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t d0 = ((size_t)blockIdx.y * 4 + warp) * 32;
    if (d0 >= dim) return;
    const size_t d = d0 + lane;
    const bool live = d < dim;
    const uint32_t *rows = perm + ch.start;
    float acc = 0.0f;
    uint32_t next = lane < (int)ch.rows ? rows[lane] : DEAD;
    for (unsigned r0 = 0; r0 < ch.rows; r0 += 32) {
        const uint32_t mine = next;
        next = r0 + 32 + lane < ch.rows ? rows[r0 + 32 + lane] : DEAD;
        float v[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) {
            const uint32_t idx = __shfl_sync(0xffffffffu, mine, u);
            v[u] = (idx != DEAD && live) ? x[(size_t)idx * dim + d] : 0.0f;
        }
        const int nrows = (int)min(32u, ch.rows - r0);
#pragma unroll
        for (int u = 0; u < 32; ++u)
            if (u < nrows) acc = __fadd_rn(acc, v[u]);
    }
    if (live) partial[(size_t)blockIdx.x * dim + d] = acc;
}

__global__ void node_mean_kernel(const NodeInfo *nodes, int first, int count, size_t dim, const float *partial, float *centroids)
{
    const size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (t >= (size_t)count * dim) return;
    const int node = first + (int)(t / dim);
    const size_t d = t % dim;
    const NodeInfo nd = nodes[node];
    float total = 0.0f;
    const float *p = partial + nd.chunk0 * dim + d;
#pragma unroll 8
    for (unsigned c = 0; c < nd.nchunks; ++c) total = __fadd_rn(total, p[(size_t)c * dim]);
    centroids[(size_t)node * dim + d] = __fdiv_rn(total, __ull2float_rn(nd.count)); // sum / (len as f32)
}

// ---- spreads, any width: one thread per (node, dimension) walks the node's rows in data order; the additions form one
// serial chain, so the loads are what can overlap: 48 rows are in flight while the previous 48 are consumed.
// grid.x = nodes of the level (ids first .. first + gridDim.x), grid.y x 32 threads over dimensions
__global__ void __launch_bounds__(32) node_spread_kernel(const float *x, size_t dim, const uint32_t *perm, const NodeInfo *nodes, int first,
                                                         const float *centroids, float *spread)
{
    const int node = first + blockIdx.x;
    const NodeInfo nd = nodes[node];
    if (!nd.split) return;
    const uint32_t *rows = perm + nd.start;
    constexpr int B = 48;
    for (size_t t = blockIdx.y * 32 + threadIdx.x; t < dim; t += (size_t)gridDim.y * 32) {
        const float c = centroids[(size_t)node * dim + t];
        float var = 0.0f;
        auto add = [&](float v) {
            const float d = __fsub_rn(v, c);
            var = __fadd_rn(var, __fmul_rn(d, d));
        };
        float cur[B], nxt[B];
        unsigned long long i = 0;
        if (nd.count >= (unsigned long long)B) {
#pragma unroll
            for (int u = 0; u < B; ++u) cur[u] = x[(size_t)rows[u] * dim + t];
        }
        for (; i + B <= nd.count; i += B) {
            const bool more = i + 2 * B <= nd.count;
            if (more) {
#pragma unroll
                for (int u = 0; u < B; ++u) nxt[u] = x[(size_t)rows[i + B + u] * dim + t];
            }
#pragma unroll
            for (int u = 0; u < B; ++u) add(cur[u]);
            if (more) {
#pragma unroll
                for (int u = 0; u < B; ++u) cur[u] = nxt[u];
            }
        }
        for (; i < nd.count; ++i) add(x[(size_t)rows[i] * dim + t]);
        spread[(size_t)blockIdx.x * dim + t] = var;
    }
}

// ---- spreads, rows whose 32-column pieces are whole 128-byte lines (dim a multiple of 32, 16-byte aligned base).  The sum
// stays one serial f32 chain per (node, dimension) in data order -- a dependent addition every 5.8 cycles at best -- so the
// kernel's job is to keep that chain fed: one CTA per (node, 32 dimensions); warp 0 is the consumer (lane = dimension) and
// does nothing but read stages from shared memory and add; eleven producer warps gather the node's rows (128-bit loads, 64
// rows per warp in flight, the next stage's row numbers requested meanwhile), form (v - c)^2 with each term rounded like the
// reference's (src/tsvq.rs:86-98) and store that into a ring of 64-row stages, so the consumer's work per row is a
// quarter of a shared-memory load and one addition.
//
// A stage is stored dimension-major, [32 dimensions][64 rows], so that the consumer fetches four consecutive rows of its
// dimension with one 128-bit load; the 16 four-row groups of a dimension are permuted by ns_swizzle(d), which keeps both
// the producers' 32-bit stores and the consumer's 128-bit loads free of bank conflicts.
//
// Hand-over.  A poll of an mbarrier costs the consumer 230 cycles even when the phase is complete (the instruction that
// reads the poll's predicate stalls the warp until the answer is back), as much as the 64 additions of a stage.  So the
// producers announce finished stages with a shared-memory counter per group of four stages, which the consumer reads
// with an ordinary load one group ahead -- the load is in flight during the additions and is looked at three stages
// later -- and the consumer hands a group back with one relaxed arrive.  Stage numbers are padded to a multiple of four
// (padding stages are announced without data) so that every group sees exactly four announcements.
constexpr int NS_STAGE_ROWS = 64, NS_GROUP = 4, NS_GROUPS = 6, NS_RING = NS_GROUP * NS_GROUPS, NS_PRODUCERS = 11, NS_THREADS = 32 * (1 + NS_PRODUCERS);
constexpr int NS_STAGE_BYTES = NS_STAGE_ROWS * 128;
constexpr int NS_SMEM = NS_RING * NS_STAGE_BYTES + NS_GROUPS * 8 + NS_GROUPS * 4;
// a producer may wait for the release of a group only when the release before that one has certainly happened (a parity
// wait cannot tell two phases apart); the same warp filled a stage NS_PRODUCERS stages earlier, so this holds while
// NS_PRODUCERS <= NS_RING - NS_GROUP
static_assert(NS_PRODUCERS <= NS_RING - NS_GROUP, "parity waits need the producers' lead to stay inside the ring");
constexpr int NS_ERR_WAIT = 190;
constexpr uint32_t NS_SPIN_LIMIT = 1u << 28;

__device__ __forceinline__ int ns_swizzle(int d) { return ((d & 7) ^ (d >> 3)) & 7; }

__global__ void __launch_bounds__(NS_THREADS) node_spread_stream_kernel(const float *__restrict__ x, size_t dim, const uint32_t *__restrict__ perm,
                                                                        const NodeInfo *nodes, int first, const float *centroids, float *spread, int *error)
{
    extern __shared__ __align__(128) unsigned char ns_smem[];
    float *ring = reinterpret_cast<float *>(ns_smem);
    uint64_t *empty = reinterpret_cast<uint64_t *>(ns_smem + NS_RING * NS_STAGE_BYTES);
    volatile uint32_t *filled = reinterpret_cast<volatile uint32_t *>(empty + NS_GROUPS);
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = first + blockIdx.x;
    const NodeInfo nd = nodes[node];
    if (!nd.split) return;
    const size_t col0 = (size_t)blockIdx.y * 32;
    const unsigned long long count = nd.count;
    const uint32_t S = (uint32_t)((count + NS_STAGE_ROWS - 1) / NS_STAGE_ROWS);      // stages with rows
    const uint32_t total = (S + NS_GROUP - 1) / NS_GROUP * NS_GROUP;                   // stage numbers
    if (threadIdx.x == 0) {
        for (int i = 0; i < NS_GROUPS; ++i) mbar_init(&empty[i], 1), filled[i] = 0;
        abort_flag = 0;
    }
    __syncthreads();
    if (warp == 0) {
        float4 a[16], b[16];
        float acc = 0.0f;
        bool ok = true;
        uint32_t ahead = 0; // filled[] of the group after the current one, as read at the start of the current group
        const int g = ns_swizzle(lane);
        auto group_ready = [&](uint32_t grp, uint32_t have) { // all four stages of group `grp` announced?
            const uint32_t need = NS_GROUP * (grp / NS_GROUPS + 1);
            if (have < need) {
                uint32_t i = 0;
                while (filled[grp % NS_GROUPS] < need) {
                    if (++i >= NS_SPIN_LIMIT || ((i & 4095u) == 0 && *(volatile int *)&abort_flag)) {
                        if (i >= NS_SPIN_LIMIT) abort_flag = 1, atomicCAS(error, 0, NS_ERR_WAIT);
                        ok = false;
                        return;
                    }
                }
            }
            __threadfence_block(); // the stages' values are read after their announcement
        };
        // shared-memory address of this lane's dimension in stage s; a four-row group q sits at + ((q ^ g) << 4) bytes
        auto stage_addr = [&](uint32_t s) { return smem_u32(ring + (size_t)(s % NS_RING) * (NS_STAGE_BYTES / 4) + lane * NS_STAGE_ROWS); };
        // volatile, so that the loads stay where they are written: between the additions, whose issue slots they fill
        auto load4 = [&](uint32_t addr, int q) {
            float4 r;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(addr + ((q ^ g) << 4)));
            return r;
        };
        auto request = [&](uint32_t s, float4(&buf)[16]) {
            const uint32_t addr = stage_addr(s);
#pragma unroll
            for (int q = 0; q < 16; ++q) buf[q] = load4(addr, q);
        };
        // cur holds stage s (s < S)
        auto step = [&](float4(&cur)[16], float4(&nxt)[16], uint32_t s) {
            const bool has_next = s + 1 < S;
            if (has_next && ((s + 1) & (NS_GROUP - 1)) == 0) {
                group_ready((s + 1) / NS_GROUP, ahead);
                if (!ok) return;
            }
            if ((s & (NS_GROUP - 1)) == 0) ahead = filled[(s / NS_GROUP + 1) % NS_GROUPS];
            const unsigned long long left = count - (unsigned long long)s * NS_STAGE_ROWS;
            if (left >= (unsigned long long)NS_STAGE_ROWS && has_next) {
                const uint32_t addr = stage_addr(s + 1);
#pragma unroll
                for (int q = 0; q < 16; ++q) { // one load of the next stage per four additions of this one
                    nxt[q] = load4(addr, q);
                    acc = __fadd_rn(acc, cur[q].x), acc = __fadd_rn(acc, cur[q].y);
                    acc = __fadd_rn(acc, cur[q].z), acc = __fadd_rn(acc, cur[q].w);
                }
            } else {
                if (has_next) request(s + 1, nxt);
                const int rows_here = left < (unsigned long long)NS_STAGE_ROWS ? (int)left : NS_STAGE_ROWS;
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    if (4 * q + 0 < rows_here) acc = __fadd_rn(acc, cur[q].x);
                    if (4 * q + 1 < rows_here) acc = __fadd_rn(acc, cur[q].y);
                    if (4 * q + 2 < rows_here) acc = __fadd_rn(acc, cur[q].z);
                    if (4 * q + 3 < rows_here) acc = __fadd_rn(acc, cur[q].w);
                }
            }
            if ((s & (NS_GROUP - 1)) == NS_GROUP - 1 || s + 1 == S) { // the group's last stage with rows: hand the group back
                __syncwarp();                                          // every lane has used its values
                if (lane == 0) mbar_arrive_relaxed(&empty[(s / NS_GROUP) % NS_GROUPS]);
            }
        };
        group_ready(0, 0);
        if (ok) request(0, a);
        for (uint32_t s = 0; s < S && ok; s += 2) {
            step(a, b, s);
            if (s + 1 < S && ok) step(b, a, s + 1);
        }
        if (ok) spread[(size_t)blockIdx.x * dim + col0 + lane] = acc;
    } else {
        const uint32_t *rows = perm + nd.start;
        const int sub = lane >> 3, piece = lane & 7;
        const float *xcol = x + col0 + piece * 4;
        const float4 cc = *reinterpret_cast<const float4 *>(centroids + (size_t)node * dim + col0 + piece * 4);
        // this lane's four dimensions 4 * piece + j: offset of (dimension, four-row group 0, position sub) in a stage
        int off[4], gj[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) gj[j] = ns_swizzle(4 * piece + j), off[j] = (4 * piece + j) * NS_STAGE_ROWS + sub;
        uint32_t idx[16];
        auto load_idx = [&](uint32_t s) { // stage numbers past the node's rows give no rows at all
            const unsigned long long r0 = (unsigned long long)s * NS_STAGE_ROWS + sub;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const unsigned long long r = r0 + 4 * i;
                idx[i] = r < count ? rows[r] : DEAD;
            }
        };
        uint32_t s = warp - 1;
        if (s < total) load_idx(s);
        for (; s < total; s += NS_PRODUCERS) {
            const bool padding = s >= S;
            float4 v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                v[i] = idx[i] != DEAD ? __ldg(reinterpret_cast<const float4 *>(xcol + (size_t)idx[i] * dim)) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (s + NS_PRODUCERS < total) load_idx(s + NS_PRODUCERS);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float d;
                d = __fsub_rn(v[i].x, cc.x), v[i].x = __fmul_rn(d, d);
                d = __fsub_rn(v[i].y, cc.y), v[i].y = __fmul_rn(d, d);
                d = __fsub_rn(v[i].z, cc.z), v[i].z = __fmul_rn(d, d);
                d = __fsub_rn(v[i].w, cc.w), v[i].w = __fmul_rn(d, d);
            }
            const uint32_t grp = s / NS_GROUP, gslot = grp % NS_GROUPS;
            if (!mbar_wait(&empty[gslot], ((grp / NS_GROUPS) & 1u) ^ 1u, &abort_flag, error, NS_ERR_WAIT, 100u)) break;
            if (!padding) {
                float *dst = ring + (size_t)(s % NS_RING) * (NS_STAGE_BYTES / 4);
#pragma unroll
                for (int i = 0; i < 16; ++i) { // row 4 i + sub of the stage: four-row group i, position sub
                    dst[off[0] + ((i ^ gj[0]) << 2)] = v[i].x;
                    dst[off[1] + ((i ^ gj[1]) << 2)] = v[i].y;
                    dst[off[2] + ((i ^ gj[2]) << 2)] = v[i].z;
                    dst[off[3] + ((i ^ gj[3]) << 2)] = v[i].w;
                }
            }
            __syncwarp();
            if (lane == 0) {
                __threadfence_block(); // the stage's values before its announcement
                atomicAdd(const_cast<uint32_t *>(&filled[gslot]), 1u);
            }
        }
    }
}

// one thread per node of the level: last of equal maxima; NaN is not comparable
__global__ void pick_split_kernel(NodeInfo *nodes, int first, int count, size_t dim, const float *spread, int *error)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= count) return;
    NodeInfo &nd = nodes[first + j];
    if (!nd.split) return;
    const float *v = spread + (size_t)j * dim;
    size_t best = 0;
    for (size_t t = 0; t < dim; ++t) {
        if (!(v[t] == v[t])) atomicExch(error, 105);
        if (t > 0 && !(v[t] < v[best])) best = t;
    }
    nd.split_dim = (int)best;
}

// key = (node << 32) | ordered value along the node's split dimension; positions outside splitting nodes sort last
__global__ void make_keys_kernel(const float *x, size_t n, size_t dim, const uint32_t *perm, const uint32_t *pos_node, const NodeInfo *nodes,
                                 unsigned long long *keys, int *error)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t node = pos_node[i];
        unsigned long long key = ~0ull;
        if (node != DEAD && nodes[node].split) {
            const float v = x[(size_t)perm[i] * dim + nodes[node].split_dim];
            if (!(v == v)) atomicExch(error, 105);
            key = ((unsigned long long)node << 32) | f32_key(v);
        }
        keys[i] = key;
    }
}

__global__ void median_kernel(NodeInfo *nodes, int first, int count, const unsigned long long *sorted)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= count) return;
    NodeInfo &nd = nodes[first + j];
    if (!nd.split) return;
    const unsigned long long *s = sorted + nd.sorted_start;
    const float hi = key_f32((uint32_t)s[nd.count / 2]);
    if (nd.count % 2 == 0) {
        const float lo = key_f32((uint32_t)s[nd.count / 2 - 1]);
        nd.median = __fdiv_rn(__fadd_rn(lo, hi), 2.0f);
    } else {
        nd.median = hi;
    }
}

__global__ void flag_kernel(const float *x, size_t n, size_t dim, const uint32_t *perm, const uint32_t *pos_node, const NodeInfo *nodes, uint32_t *flags)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i <= n; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t f = 0;
        if (i < n) {
            const uint32_t node = pos_node[i];
            if (node != DEAD && nodes[node].split) f = x[(size_t)perm[i] * dim + nodes[node].split_dim] <= nodes[node].median ? 1u : 0u;
        }
        flags[i] = f;
    }
}

__global__ void count_left_kernel(NodeInfo *nodes, int first, int count, const uint32_t *scan)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= count) return;
    NodeInfo &nd = nodes[first + j];
    if (nd.split) nd.nleft = scan[nd.start + nd.count] - scan[nd.start];
}

// stable partition of every splitting node's rows: the flagged rows first, both sides in their old order
__global__ void scatter_kernel(size_t n, const uint32_t *perm, const uint32_t *pos_node, const NodeInfo *nodes, const uint32_t *flags, const uint32_t *scan,
                               uint32_t *perm_out)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t node = pos_node[i];
        size_t dst = i;
        if (node != DEAD && nodes[node].split) {
            const NodeInfo &nd = nodes[node];
            const unsigned long long lr = scan[i] - scan[nd.start];
            dst = flags[i] ? nd.start + lr : nd.start + nd.nleft + (i - nd.start - lr);
        }
        perm_out[dst] = perm[i];
    }
}

// after the host has numbered the children: every position learns its new node (or none)
__global__ void relabel_kernel(size_t n, uint32_t *pos_node, const NodeInfo *nodes)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t node = pos_node[i];
        if (node == DEAD) continue;
        const NodeInfo &nd = nodes[node];
        uint32_t nn = DEAD;
        if (nd.split && nd.child_left >= 0) nn = (i < nd.start + nd.nleft) ? (uint32_t)nd.child_left : (uint32_t)nd.child_right;
        pos_node[i] = nn;
    }
}

template <int METRIC>
__global__ void tsvq_quantize_kernel(const float *x, size_t n, size_t dim, const float *centroids, const int32_t *left, const int32_t *right, float pv,
                                     uint16_t *out_f16, uint32_t *leaf_out)
{
    for (size_t row = blockIdx.x * (size_t)blockDim.x + threadIdx.x; row < n; row += (size_t)gridDim.x * blockDim.x) {
        const float *v = x + row * dim;
        float norm_a = 0.0f;
        if (METRIC == M_COSINE) norm_a = norm_chain(v, (int)dim, 1);
        int node = 0;
        for (;;) {
            const int l = left[node], r = right[node];
            if (l >= 0 && r >= 0) {
                const float *cl = centroids + (size_t)l * dim, *cr = centroids + (size_t)r * dim;
                DistAcc<METRIC> al, ar;
                al.init();
                ar.init();
                for (size_t t = 0; t < dim; ++t) {
                    const float xv = v[t];
                    al.step(xv, cl[t], pv);
                    ar.step(xv, cr[t], pv);
                }
                const float dl = al.finish(pv, norm_a), dr = ar.finish(pv, norm_a);
                node = (dl <= dr) ? l : r; // src/tsvq.rs:172: the left child on ties; a NaN distance sends the row right
            } else if (l >= 0) {
                node = l;
            } else if (r >= 0) {
                node = r;
            } else {
                break;
            }
        }
        if (leaf_out) leaf_out[row] = (uint32_t)node;
        if (out_f16) {
            const float *c = centroids + (size_t)node * dim;
            for (size_t t = 0; t < dim; ++t) out_f16[row * dim + t] = f32_to_f16_bits(c[t]);
        }
    }
}

// Tile variant of the lookup for rows in whole 16-byte pieces (dim a multiple of 8, aligned pointers): a CTA stages 128
// rows in shared memory with coalesced 128-bit loads (row stride dim + 4 floats, so the per-thread 128-bit reads of the
// walk are conflict-free), every thread walks the tree for its own row with the same serial distance chains as above but
// fetches both children's centroids 16 bytes at a time, and the f16 rows of the leaves are written by the whole CTA in
// 16-byte pieces.  One thread per row reading its row straight from global memory spends its time on 32 different lines
// per load instruction and 2-byte stores 2 * dim bytes apart.
constexpr int TQ_ROWS = 128;
template <int METRIC>
__global__ void __launch_bounds__(TQ_ROWS) tsvq_quantize_tile_kernel(const float *__restrict__ x, size_t n, int dim, const float *__restrict__ centroids,
                                                                     const int32_t *__restrict__ left, const int32_t *__restrict__ right, float pv,
                                                                     uint16_t *out_f16, uint32_t *leaf_out)
{
    extern __shared__ __align__(16) float tq_rows[];
    __shared__ int leaf_sh[TQ_ROWS];
    const int stride = dim + 4, chunks = dim / 4, octs = dim / 8;
    for (size_t tile = blockIdx.x; tile * TQ_ROWS < n; tile += gridDim.x) {
        const size_t row0 = tile * TQ_ROWS;
        const int rows = (int)(n - row0 < (size_t)TQ_ROWS ? n - row0 : (size_t)TQ_ROWS);
        __syncthreads(); // the previous tile's readers are done
        const float4 *src = reinterpret_cast<const float4 *>(x + row0 * dim);
        for (int i = threadIdx.x; i < rows * chunks; i += TQ_ROWS) {
            const int r = i / chunks, c = i - r * chunks;
            *reinterpret_cast<float4 *>(tq_rows + r * stride + 4 * c) = __ldcs(src + i);
        }
        __syncthreads();
        if ((int)threadIdx.x < rows) {
            const float *v = tq_rows + threadIdx.x * stride;
            float norm_a = 0.0f;
            if (METRIC == M_COSINE) norm_a = norm_chain(v, dim, 1);
            int node = 0;
            for (;;) {
                const int l = left[node], r = right[node];
                if (l >= 0 && r >= 0) {
                    const float4 *cl = reinterpret_cast<const float4 *>(centroids + (size_t)l * dim);
                    const float4 *cr = reinterpret_cast<const float4 *>(centroids + (size_t)r * dim);
                    DistAcc<METRIC> al, ar;
                    al.init();
                    ar.init();
#pragma unroll 2
                    for (int c = 0; c < chunks; ++c) {
                        const float4 xv = *reinterpret_cast<const float4 *>(v + 4 * c);
                        const float4 a = __ldg(cl + c), b = __ldg(cr + c);
                        al.step(xv.x, a.x, pv), ar.step(xv.x, b.x, pv);
                        al.step(xv.y, a.y, pv), ar.step(xv.y, b.y, pv);
                        al.step(xv.z, a.z, pv), ar.step(xv.z, b.z, pv);
                        al.step(xv.w, a.w, pv), ar.step(xv.w, b.w, pv);
                    }
                    const float dl = al.finish(pv, norm_a), dr = ar.finish(pv, norm_a);
                    node = (dl <= dr) ? l : r; // src/tsvq.rs:172: the left child on ties; a NaN distance sends the row right
                } else if (l >= 0) {
                    node = l;
                } else if (r >= 0) {
                    node = r;
                } else {
                    break;
                }
            }
            leaf_sh[threadIdx.x] = node;
            if (leaf_out) leaf_out[row0 + threadIdx.x] = (uint32_t)node;
        }
        __syncthreads();
        if (out_f16) {
            for (int i = threadIdx.x; i < rows * octs; i += TQ_ROWS) {
                const int r = i / octs, o = i - r * octs;
                const float4 *c = reinterpret_cast<const float4 *>(centroids + (size_t)leaf_sh[r] * dim) + 2 * o;
                const float4 p = __ldg(c), q = __ldg(c + 1);
                uint4 w;
                w.x = (uint32_t)f32_to_f16_bits(p.x) | ((uint32_t)f32_to_f16_bits(p.y) << 16);
                w.y = (uint32_t)f32_to_f16_bits(p.z) | ((uint32_t)f32_to_f16_bits(p.w) << 16);
                w.z = (uint32_t)f32_to_f16_bits(q.x) | ((uint32_t)f32_to_f16_bits(q.y) << 16);
                w.w = (uint32_t)f32_to_f16_bits(q.z) | ((uint32_t)f32_to_f16_bits(q.w) << 16);
                __stcs(reinterpret_cast<uint4 *>(out_f16 + (row0 + r) * dim + 8 * o), w);
            }
        }
    }
}

inline unsigned grid_for(size_t items, int threads, unsigned cap)
{
    return (unsigned)std::max<size_t>(1, std::min<size_t>((items + threads - 1) / threads, cap));
}

} // namespace

void tsvq_fit(CudaDevice &dev, const float *x, size_t n, size_t dim, size_t max_depth, TsvqTree &out)
{
    if (n == 0 || dim == 0) throw Error(1, "Empty input: at least one vector is required.");
    if (n >= 0x7FFFFFFFull) throw Error(103, "tsvq: more than 2^31 - 2 rows are not supported");
    cudaStream_t st = dev.stream();
    const size_t cap_nodes = std::min<size_t>(max_depth < 40 ? ((size_t)2 << max_depth) - 1 : 2 * n, 2 * n);
    std::vector<NodeInfo> h(1);
    std::vector<size_t> depth_left(1, max_depth);
    h[0] = NodeInfo{0, n, 0, 0, 0.0f, 0, 0, -1, -1, 0, 0};
    float *cent = static_cast<float *>(dev.alloc(sizeof(float) * cap_nodes * dim));
    NodeInfo *nodes_d = static_cast<NodeInfo *>(dev.alloc(sizeof(NodeInfo) * cap_nodes));
    uint32_t *perm = static_cast<uint32_t *>(dev.alloc(sizeof(uint32_t) * n)), *perm2 = static_cast<uint32_t *>(dev.alloc(sizeof(uint32_t) * n));
    uint32_t *pos_node = static_cast<uint32_t *>(dev.alloc(sizeof(uint32_t) * n));
    uint32_t *flags = static_cast<uint32_t *>(dev.alloc(sizeof(uint32_t) * (n + 1))), *scan = static_cast<uint32_t *>(dev.alloc(sizeof(uint32_t) * (n + 1)));
    unsigned long long *keys = static_cast<unsigned long long *>(dev.alloc(sizeof(unsigned long long) * n));
    unsigned long long *keys2 = static_cast<unsigned long long *>(dev.alloc(sizeof(unsigned long long) * n));
    int *error = static_cast<int *>(dev.alloc(sizeof(int)));
    size_t sort_bytes = 0, scan_bytes = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, sort_bytes, keys, keys2, (int)n, 0, 64, st);
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, flags, scan, (int)(n + 1), st);
    void *tmp = dev.alloc(std::max(sort_bytes, scan_bytes));
    size_t tmp_bytes = std::max(sort_bytes, scan_bytes);
    float *spread = nullptr, *partial = nullptr;
    ChunkInfo *chunks_d = nullptr;
    size_t spread_cap = 0, chunk_cap = 0;
    std::vector<ChunkInfo> chunks;
    // rows in whole 128-byte pieces of 32 columns: the streaming kernel; any other shape: one thread per (node, dimension)
    const bool stream_rows = dim % 32 == 0 && dim / 32 <= 65535 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && getenv("VQB_TSVQ_SERIAL_WALK") == nullptr;
    if (stream_rows) VQB_CUDA_CHECK(cudaFuncSetAttribute(node_spread_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, NS_SMEM));
    auto cleanup = [&] {
        dev.release(nodes_d), dev.release(perm), dev.release(perm2), dev.release(pos_node), dev.release(flags), dev.release(scan);
        dev.release(keys), dev.release(keys2), dev.release(error), dev.release(tmp), dev.release(spread), dev.release(partial), dev.release(chunks_d);
    };
    try {
        dev.zero(error, sizeof(int));
        dev.zero(pos_node, sizeof(uint32_t) * n); // every position belongs to node 0
        {
            std::vector<uint32_t> id(n);
            for (size_t i = 0; i < n; ++i) id[i] = (uint32_t)i;
            dev.upload(perm, id.data(), sizeof(uint32_t) * n);
        }
        size_t first = 0;
        while (first < h.size()) {
            const size_t level_count = h.size() - first;
            size_t n_split = 0, sorted = 0;
            chunks.clear();
            for (size_t j = first; j < h.size(); ++j) {
                h[j].chunk0 = chunks.size();
                h[j].nchunks = (unsigned)((h[j].count + MEAN_CHUNK - 1) / MEAN_CHUNK);
                for (unsigned long long r = 0; r < h[j].count; r += MEAN_CHUNK)
                    chunks.push_back(ChunkInfo{h[j].start + r, (unsigned)std::min<unsigned long long>(MEAN_CHUNK, h[j].count - r)});
                h[j].split = (depth_left[j] > 0 && h[j].count > 1) ? 1 : 0;
                h[j].sorted_start = sorted;
                if (h[j].split) {
                    sorted += h[j].count;
                    ++n_split;
                }
            }
            dev.upload(nodes_d + first, h.data() + first, sizeof(NodeInfo) * level_count);
            if (level_count > spread_cap) {
                dev.release(spread);
                spread = static_cast<float *>(dev.alloc(sizeof(float) * level_count * dim));
                spread_cap = level_count;
            }
            if (chunks.size() > chunk_cap) {
                dev.release(partial), dev.release(chunks_d);
                chunk_cap = chunks.size() + chunks.size() / 2;
                partial = static_cast<float *>(dev.alloc(sizeof(float) * chunk_cap * dim));
                chunks_d = static_cast<ChunkInfo *>(dev.alloc(sizeof(ChunkInfo) * chunk_cap));
            }
            dev.upload(chunks_d, chunks.data(), sizeof(ChunkInfo) * chunks.size());
            {
                KernelScope ks(dev, "tsvq_node_means");
                chunk_sums_kernel<<<dim3((unsigned)chunks.size(), (unsigned)((dim + 127) / 128)), 128, 0, st>>>(x, dim, perm, chunks_d, partial);
                node_mean_kernel<<<grid_for(level_count * dim, 128, 1u << 30), 128, 0, st>>>(nodes_d, (int)first, (int)level_count, dim, partial, cent);
                VQB_CUDA_CHECK(cudaGetLastError());
                dev.count_launch();
            }
            if (n_split == 0) break;
            {
                KernelScope ks(dev, "tsvq_node_spreads");
                if (stream_rows) {
                    const dim3 grid((unsigned)level_count, (unsigned)(dim / 32));
                    node_spread_stream_kernel<<<grid, NS_THREADS, NS_SMEM, st>>>(x, dim, perm, nodes_d, (int)first, cent, spread, error);
                } else {
                    const dim3 grid((unsigned)level_count, (unsigned)std::min<size_t>((dim + 31) / 32, 64));
                    node_spread_kernel<<<grid, 32, 0, st>>>(x, dim, perm, nodes_d, (int)first, cent, spread);
                }
                VQB_CUDA_CHECK(cudaGetLastError());
                dev.count_launch();
            }
            if (n_split == 0) break;
            {
                KernelScope ks(dev, "tsvq_split");
                pick_split_kernel<<<grid_for(level_count, 128, 1u << 20), 128, 0, st>>>(nodes_d, (int)first, (int)level_count, dim, spread, error);
                make_keys_kernel<<<grid_for(n, 256, (unsigned)dev.sm_count() * 8), 256, 0, st>>>(x, n, dim, perm, pos_node, nodes_d, keys, error);
                VQB_CUDA_CHECK(cudaGetLastError());
                VQB_CUDA_CHECK(cub::DeviceRadixSort::SortKeys(tmp, tmp_bytes, keys, keys2, (int)n, 0, 64, st));
                median_kernel<<<grid_for(level_count, 128, 1u << 20), 128, 0, st>>>(nodes_d, (int)first, (int)level_count, keys2);
                flag_kernel<<<grid_for(n + 1, 256, (unsigned)dev.sm_count() * 8), 256, 0, st>>>(x, n, dim, perm, pos_node, nodes_d, flags);
                VQB_CUDA_CHECK(cudaGetLastError());
                VQB_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, flags, scan, (int)(n + 1), st));
                count_left_kernel<<<grid_for(level_count, 128, 1u << 20), 128, 0, st>>>(nodes_d, (int)first, (int)level_count, scan);
                scatter_kernel<<<grid_for(n, 256, (unsigned)dev.sm_count() * 8), 256, 0, st>>>(n, perm, pos_node, nodes_d, flags, scan, perm2);
                VQB_CUDA_CHECK(cudaGetLastError());
                dev.count_launch();
            }
            std::swap(perm, perm2);
            int herr = 0;
            dev.download(&herr, error, sizeof(int));
            if (herr == NS_ERR_WAIT) throw Error(100, "tsvq: a wait inside the node statistics kernel ran out");
            if (herr) throw Error(herr, "values are not comparable (NaN in the training data)");
            dev.download(h.data() + first, nodes_d + first, sizeof(NodeInfo) * level_count);
            const size_t level_end = h.size();
            for (size_t j = first; j < level_end; ++j) {
                if (!h[j].split) continue;
                const unsigned long long nl = h[j].nleft, nr = h[j].count - nl;
                if (nl > 0 && nr > 0) { // otherwise neither side is a proper subset: no children (src/tsvq.rs:127-141)
                    h[j].child_left = (int)h.size();
                    h.push_back(NodeInfo{h[j].start, nl, 0, 0, 0.0f, 0, 0, -1, -1, 0, 0});
                    depth_left.push_back(depth_left[j] - 1);
                    h[j].child_right = (int)h.size();
                    h.push_back(NodeInfo{h[j].start + nl, nr, 0, 0, 0.0f, 0, 0, -1, -1, 0, 0});
                    depth_left.push_back(depth_left[j] - 1);
                }
            }
            if (h.size() > cap_nodes) throw Error(100, "tsvq: node capacity exceeded");
            dev.upload(nodes_d + first, h.data() + first, sizeof(NodeInfo) * level_count);
            relabel_kernel<<<grid_for(n, 256, (unsigned)dev.sm_count() * 8), 256, 0, st>>>(n, pos_node, nodes_d);
            VQB_CUDA_CHECK(cudaGetLastError());
            dev.count_launch();
            first = level_end;
        }
    } catch (...) {
        cudaStreamSynchronize(st);
        cleanup();
        dev.release(cent);
        throw;
    }
    out.dim = dim;
    out.nodes = h.size();
    out.h_left.resize(h.size());
    out.h_right.resize(h.size());
    for (size_t j = 0; j < h.size(); ++j) {
        out.h_left[j] = h[j].child_left;
        out.h_right[j] = h[j].child_right;
    }
    out.centroids = cent;
    out.left = static_cast<int32_t *>(dev.alloc(sizeof(int32_t) * h.size()));
    out.right = static_cast<int32_t *>(dev.alloc(sizeof(int32_t) * h.size()));
    dev.upload(out.left, out.h_left.data(), sizeof(int32_t) * h.size());
    dev.upload(out.right, out.h_right.data(), sizeof(int32_t) * h.size());
    cudaStreamSynchronize(st);
    cleanup();
}

template <int METRIC>
static void launch_quantize(CudaDevice &dev, const TsvqTree &t, double p, const float *x, size_t n, uint16_t *out_f16, uint32_t *leaf)
{
    KernelScope ks(dev, "tsvq_quantize");
    const size_t tile_smem = sizeof(float) * TQ_ROWS * (t.dim + 4);
    const bool aligned = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(out_f16) % 16 == 0;
    if (t.dim % 8 == 0 && tile_smem <= 200 * 1024 && aligned && getenv("VQB_TSVQ_SERIAL_WALK") == nullptr) {
        VQB_CUDA_CHECK(cudaFuncSetAttribute(tsvq_quantize_tile_kernel<METRIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem));
        const size_t tiles = (n + TQ_ROWS - 1) / TQ_ROWS;
        const unsigned per_sm = (unsigned)std::max<size_t>(1, std::min<size_t>(8, (220 * 1024) / (tile_smem + 1024)));
        const unsigned grid = (unsigned)std::min<size_t>(tiles, (size_t)dev.sm_count() * per_sm);
        tsvq_quantize_tile_kernel<METRIC><<<grid, TQ_ROWS, tile_smem, dev.stream()>>>(x, n, (int)t.dim, t.centroids, t.left, t.right, (float)p, out_f16, leaf);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
        return;
    }
    tsvq_quantize_kernel<METRIC><<<grid_for(n, 128, (unsigned)dev.sm_count() * 16), 128, 0, dev.stream()>>>(x, n, t.dim, t.centroids, t.left, t.right, (float)p,
                                                                                                     out_f16, leaf);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

void tsvq_quantize(CudaDevice &dev, const TsvqTree &t, int metric, double p, const float *x, size_t n, uint16_t *out_f16, uint32_t *leaf)
{
    if (n == 0) return;
    switch (metric) {
    case M_SQ: launch_quantize<M_SQ>(dev, t, p, x, n, out_f16, leaf); break;
    case M_EUCLID: launch_quantize<M_EUCLID>(dev, t, p, x, n, out_f16, leaf); break;
    case M_COSINE: launch_quantize<M_COSINE>(dev, t, p, x, n, out_f16, leaf); break;
    case M_MANHATTAN: launch_quantize<M_MANHATTAN>(dev, t, p, x, n, out_f16, leaf); break;
    case M_CHEBYSHEV: launch_quantize<M_CHEBYSHEV>(dev, t, p, x, n, out_f16, leaf); break;
    case M_MINKOWSKI: launch_quantize<M_MINKOWSKI>(dev, t, p, x, n, out_f16, leaf); break;
    case M_HAMMING: launch_quantize<M_HAMMING>(dev, t, p, x, n, out_f16, leaf); break;
    default: throw Error(90, "unknown metric");
    }
}

void tsvq_release(CudaDevice &dev, TsvqTree &t)
{
    dev.release(t.centroids), dev.release(t.left), dev.release(t.right);
    t.centroids = nullptr, t.left = nullptr, t.right = nullptr;
}

} // namespace vqb
