// tsvq.cu -- tree-structured vector quantizer (src/tsvq.rs) built level by level on the device.
//
// The reference recurses; here all nodes of one depth are processed together and numbered breadth-first (left child before
// right).  What fixes the result bit for bit is kept: the centroid of a node is the f32 sum of its rows in data order divided
// by `len as f32` (mean_vector, src/vector.rs:282-318; an admissible order for nodes above 1024 rows, where the reference's
// own order is unspecified); a dimension's spread is the serial f32 sum of (v - c)^2 in data order (src/tsvq.rs:86-98); the
// split dimension is the last of equal maxima (max_by, 101-105); the median is taken from the sorted values (108-116); the
// partition is stable (119-122); children exist only when both sides are non-empty (127-141).
//
// Per level: node_stats_kernel (one thread per (node, dimension) walks the node's rows in order, 32 loads in flight),
// pick_split_kernel, a 64-bit radix sort of (node, value) keys (CUB, library code off the hot path) from which the medians
// are read, a flag + exclusive scan (CUB) + scatter for the stable partition, and one small download of the left counts
// from which the host numbers the children.  The build is not sharded: every rank of a multi-GPU job builds the same tree.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <vector>

#include "cuda_device.hpp"
#include "kernels_common.cuh"
#include "tsvq.hpp"

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

// Calls f(value) for column t of the node's rows in data order.  The additions behind f form one serial chain, so the loads
// are what can overlap: 48 rows are in flight while the previous 48 are consumed (one warp per 32 dimensions, so that the
// 96 buffer registers per thread are affordable and a wide node spreads over several SMs).
template <typename F> __device__ __forceinline__ void walk_rows(const float *x, size_t dim, const uint32_t *rows, unsigned long long count, size_t t, F f)
{
    constexpr int B = 48;
    float cur[B], nxt[B];
    unsigned long long i = 0;
    if (count >= (unsigned long long)B) {
#pragma unroll
        for (int u = 0; u < B; ++u) cur[u] = x[(size_t)rows[u] * dim + t];
    }
    for (; i + B <= count; i += B) {
        const bool more = i + 2 * B <= count;
        if (more) {
#pragma unroll
            for (int u = 0; u < B; ++u) nxt[u] = x[(size_t)rows[i + B + u] * dim + t];
        }
#pragma unroll
        for (int u = 0; u < B; ++u) f(cur[u]);
        if (more) {
#pragma unroll
            for (int u = 0; u < B; ++u) cur[u] = nxt[u];
        }
    }
    for (; i < count; ++i) f(x[(size_t)rows[i] * dim + t]);
}

// grid.x = nodes of the level (ids first .. first + gridDim.x), grid.y x 32 threads over dimensions
__global__ void __launch_bounds__(32) node_stats_kernel(const float *x, size_t dim, const uint32_t *perm, NodeInfo *nodes, int first, float *centroids, float *spread)
{
    const int node = first + blockIdx.x;
    const NodeInfo nd = nodes[node];
    const uint32_t *rows = perm + nd.start;
    for (size_t t = blockIdx.y * 32 + threadIdx.x; t < dim; t += (size_t)gridDim.y * 32) {
        float sum = 0.0f;
        walk_rows(x, dim, rows, nd.count, t, [&](float v) { sum = __fadd_rn(sum, v); });
        const float c = __fdiv_rn(sum, __ull2float_rn(nd.count)); // sum / (len as f32)
        centroids[(size_t)node * dim + t] = c;
        if (nd.split) {
            float var = 0.0f;
            walk_rows(x, dim, rows, nd.count, t, [&](float v) {
                const float d = __fsub_rn(v, c);
                var = __fadd_rn(var, __fmul_rn(d, d));
            });
            spread[(size_t)blockIdx.x * dim + t] = var;
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
    h[0] = NodeInfo{0, n, 0, 0, 0.0f, 0, 0, -1, -1};
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
    float *spread = nullptr;
    size_t spread_cap = 0;
    auto cleanup = [&] {
        dev.release(nodes_d), dev.release(perm), dev.release(perm2), dev.release(pos_node), dev.release(flags), dev.release(scan);
        dev.release(keys), dev.release(keys2), dev.release(error), dev.release(tmp), dev.release(spread);
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
            for (size_t j = first; j < h.size(); ++j) {
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
            {
                KernelScope ks(dev, "tsvq_node_stats");
                const dim3 grid((unsigned)level_count, (unsigned)std::min<size_t>((dim + 31) / 32, 64));
                node_stats_kernel<<<grid, 32, 0, st>>>(x, dim, perm, nodes_d, (int)first, cent, spread);
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
            if (herr) throw Error(herr, "values are not comparable (NaN in the training data)");
            dev.download(h.data() + first, nodes_d + first, sizeof(NodeInfo) * level_count);
            const size_t level_end = h.size();
            for (size_t j = first; j < level_end; ++j) {
                if (!h[j].split) continue;
                const unsigned long long nl = h[j].nleft, nr = h[j].count - nl;
                if (nl > 0 && nr > 0) { // otherwise neither side is a proper subset: no children (src/tsvq.rs:127-141)
                    h[j].child_left = (int)h.size();
                    h.push_back(NodeInfo{h[j].start, nl, 0, 0, 0.0f, 0, 0, -1, -1});
                    depth_left.push_back(depth_left[j] - 1);
                    h[j].child_right = (int)h.size();
                    h.push_back(NodeInfo{h[j].start + nl, nr, 0, 0, 0.0f, 0, 0, -1, -1});
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
