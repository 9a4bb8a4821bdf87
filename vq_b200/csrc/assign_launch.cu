// assign_launch.cu -- picks and launches the nearest-centroid kernels (assign_reg.cuh, assign_generic.cuh).
#include <algorithm>

#include <cstdlib>
#include <mutex>

#include "assign_filter.cuh"
#include "assign_generic.cuh"
#include "assign_reg.cuh"
#include "cuda_device.hpp"

namespace vqb {

namespace {

// The opt-in to large dynamic shared memory is one attribute per kernel: it is only ever raised, and the resident
// CTAs per SM are looked up once per (kernel, device, size, threads) instead of on every launch (both are host round
// trips that show in short per-iteration launches).  The caches are shared by all kernels with the same signature,
// so the kernel's address is part of every key.
template <typename K> int configure(K kernel, int threads, size_t smem)
{
    struct Slot {
        const void *fn = nullptr;
        int device = -1, threads = 0, occ = 1;
        size_t smem = 0;
    };
    struct MaxSlot {
        const void *fn = nullptr;
        int device = -1;
        size_t smem = 0;
    };
    static std::mutex mu;
    static Slot slots[64];
    static MaxSlot maxes[64];
    static int next = 0, next_max = 0;
    int device = 0;
    cudaGetDevice(&device);
    const void *fn = reinterpret_cast<const void *>(kernel);
    std::lock_guard<std::mutex> lk(mu);
    MaxSlot *mx = nullptr;
    for (auto &m : maxes)
        if (m.fn == fn && m.device == device) mx = &m;
    if (!mx) {
        mx = &maxes[next_max++ % 64];
        mx->fn = fn;
        mx->device = device;
        mx->smem = 0;
    }
    if (smem > mx->smem) {
        VQB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        mx->smem = smem;
    }
    for (auto &s : slots)
        if (s.fn == fn && s.device == device && s.smem == smem && s.threads == threads) return s.occ;
    int occ = 1;
    VQB_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem));
    Slot &s = slots[next++ % 64];
    s.fn = fn;
    s.device = device;
    s.threads = threads;
    s.smem = smem;
    s.occ = std::max(1, occ);
    return s.occ;
}

// VQB_EXACT_SCAN=1 forces the plain exact scan (for A/B comparisons); results are identical either way.
bool use_filter()
{
    static const bool off = [] {
        const char *e = std::getenv("VQB_EXACT_SCAN");
        return e && *e && *e != '0';
    }();
    return !off;
}

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN, bool FILTER>
void launch_reg_t(CudaDevice &dev, const AssignParams &p, size_t smem);

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN>
void launch_reg_t(CudaDevice &dev, const AssignParams &p, size_t smem)
{
    if ((METRIC == M_SQ || METRIC == M_EUCLID) && use_filter())
        launch_reg_t<SD, V, (METRIC == M_EUCLID ? M_EUCLID : M_SQ), CodeT, TRAIN, true>(dev, p, smem);
    else
        launch_reg_t<SD, V, METRIC, CodeT, TRAIN, false>(dev, p, smem);
}

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN, bool FILTER> struct KernelPick {
    static auto get() { return assign_reg_kernel<SD, V, METRIC, CodeT, TRAIN>; }
};
template <int SD, int V, typename CodeT, bool TRAIN> struct KernelPick<SD, V, M_SQ, CodeT, TRAIN, true> {
    static auto get() { return assign_filter_kernel<SD, V, M_SQ, CodeT, TRAIN>; }
};
template <int SD, int V, typename CodeT, bool TRAIN> struct KernelPick<SD, V, M_EUCLID, CodeT, TRAIN, true> {
    static auto get() { return assign_filter_kernel<SD, V, M_EUCLID, CodeT, TRAIN>; }
};

template <int SD, int V, int METRIC, typename CodeT, bool TRAIN, bool FILTER>
void launch_reg_t(CudaDevice &dev, const AssignParams &p, size_t smem)
{
    auto kernel = KernelPick<SD, V, METRIC, CodeT, TRAIN, FILTER>::get();
    const int threads = (FILTER && SD == 8 && V == 2) ? 1024 : 512; // the two-rows-per-lane filter variant runs 32 warps per CTA
    const int occ = configure(kernel, threads, smem);
    const unsigned long long rbw = (threads / 32) / p.group;
    const unsigned long long n_blocks = (p.n + 32ull * V - 1) / (32ull * V);
    const unsigned long long chunks = (n_blocks + rbw - 1) / rbw;
    const unsigned gx = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>(chunks, (unsigned long long)dev.sm_count() * occ));
    const unsigned gy = (unsigned)((p.m + p.group - 1) / p.group);
    KernelScope ks(dev, TRAIN ? "assign_train" : "pq_encode");
    kernel<<<dim3(gx, gy), threads, smem, dev.stream()>>>(p);
    VQB_CUDA_CHECK(cudaGetLastError());
    dev.count_launch();
}

template <int SD, int V, typename CodeT> void launch_reg_train(CudaDevice &dev, const AssignParams &p, size_t smem)
{
    launch_reg_t<SD, V, M_SQ, CodeT, true>(dev, p, smem);
}

template <int SD, int V> bool launch_reg_sd(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t cb, size_t smem)
{
    if (train) {
        if (cb == 1) launch_reg_train<SD, V, uint8_t>(dev, p, smem);
        else if (cb == 2) launch_reg_train<SD, V, uint16_t>(dev, p, smem);
        else launch_reg_train<SD, V, uint32_t>(dev, p, smem);
        return true;
    }
    switch (metric) {
    case M_SQ: launch_reg_t<SD, V, M_SQ, uint32_t, false>(dev, p, smem); return true;
    case M_EUCLID: launch_reg_t<SD, V, M_EUCLID, uint32_t, false>(dev, p, smem); return true;
    case M_COSINE: launch_reg_t<SD, V, M_COSINE, uint32_t, false>(dev, p, smem); return true;
    case M_MANHATTAN: launch_reg_t<SD, V, M_MANHATTAN, uint32_t, false>(dev, p, smem); return true;
    default: return false;
    }
}

} // namespace

bool launch_assign_reg(CudaDevice &dev, const AssignParams &p_in, int metric, bool train, size_t cb)
{
    if (p_in.n == 0) return true;
    if (!(p_in.sd == 4 || p_in.sd == 8 || p_in.sd == 16)) return false;
    const int met = train ? (int)M_SQ : metric;
    if (!(met == M_SQ || met == M_EUCLID || met == M_COSINE || met == M_MANHATTAN)) return false;
    AssignParams p = p_in;
    // subspaces per CTA: a power of two dividing the 16 warps, as many as fit in shared memory
    // codebook + one float per centroid (cosine: norm; Euclidean filter: half squared norm) + one float per subspace
    const size_t per_sub = (size_t)p.k * p.sd * sizeof(float) + (met == M_MANHATTAN ? 0 : (size_t)p.k * sizeof(float)) + sizeof(float);
    const size_t budget = dev.smem_limit() - 1024;
    int g = 16;
    while (g > 1 && (g / 2 >= p.m || (size_t)g * per_sub > budget)) g /= 2;
    if ((size_t)g * per_sub > budget) return false;
    p.group = g;
    const size_t smem = (size_t)g * per_sub;
    if (p.sd == 4) return launch_reg_sd<4, 4>(dev, p, met, train, cb, smem);
    if (p.sd == 8) {
        static const bool v2 = [] {
            const char *e = std::getenv("VQB_FILTER_V2"); // experiment: 2 rows per lane, 1024 threads per CTA
            return e && *e == '1';
        }();
        return v2 ? launch_reg_sd<8, 2>(dev, p, met, train, cb, smem) : launch_reg_sd<8, 4>(dev, p, met, train, cb, smem);
    }
    return launch_reg_sd<16, 2>(dev, p, met, train, cb, smem);
}

namespace {

template <int METRIC, int MODE, typename CodeT> void launch_gen_t(CudaDevice &dev, GenericParams &p)
{
    const int sd = p.sd;
    const size_t tile_bytes = (size_t)sd * VQB_XS_STRIDE * sizeof(float) * (MODE == G_RVQ_QUANT ? 2 : 1);
    const size_t budget = dev.smem_limit() - 1024;
    int w = 8;
    while (w > 1 && (size_t)w * tile_bytes > budget * 6 / 10) w /= 2;
    if ((size_t)w * tile_bytes + 4 * (size_t)sd * sizeof(float) + 16 > budget)
        throw Error(103, "vector width too large for the nearest-centroid kernel");
    const size_t left = budget - (size_t)w * tile_bytes - 16;
    long long jc = (long long)(left / ((size_t)sd * sizeof(float)));
    jc = std::min<long long>(jc, p.k);
    if (jc >= 4) jc &= ~3ll;
    p.jc = (int)std::max<long long>(1, jc);
    p.resident = (p.jc >= p.k) && (MODE != G_RVQ_QUANT || p.stages == 1) ? 1 : 0;
    const size_t smem = (size_t)w * tile_bytes + 16 + (size_t)p.jc * sd * sizeof(float);
    const bool vec4 = (sd % 4 == 0);
    const int threads = 32 * w;
    const unsigned long long n_tiles = (p.n + 32ull * w - 1) / (32ull * w);
    auto go = [&](auto kernel) {
        const int occ = configure(kernel, threads, smem);
        const unsigned gx = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>(n_tiles, (unsigned long long)dev.sm_count() * occ));
        KernelScope ks(dev, MODE == G_TRAIN ? "assign_train" : (MODE == G_ENCODE ? "pq_encode" : (MODE == G_RVQ_UPDATE ? "rvq_update" : "rvq_quantize")));
        kernel<<<dim3(gx, (unsigned)p.m), threads, smem, dev.stream()>>>(p);
        VQB_CUDA_CHECK(cudaGetLastError());
        dev.count_launch();
    };
    if (vec4) go(assign_generic_kernel<METRIC, MODE, CodeT, true>);
    else go(assign_generic_kernel<METRIC, MODE, CodeT, false>);
}

template <int MODE> void launch_gen_metric(CudaDevice &dev, GenericParams &p, int metric)
{
    switch (metric) {
    case M_SQ: launch_gen_t<M_SQ, MODE, uint32_t>(dev, p); break;
    case M_EUCLID: launch_gen_t<M_EUCLID, MODE, uint32_t>(dev, p); break;
    case M_COSINE: launch_gen_t<M_COSINE, MODE, uint32_t>(dev, p); break;
    case M_MANHATTAN: launch_gen_t<M_MANHATTAN, MODE, uint32_t>(dev, p); break;
    case M_CHEBYSHEV: launch_gen_t<M_CHEBYSHEV, MODE, uint32_t>(dev, p); break;
    case M_MINKOWSKI: launch_gen_t<M_MINKOWSKI, MODE, uint32_t>(dev, p); break;
    case M_HAMMING: launch_gen_t<M_HAMMING, MODE, uint32_t>(dev, p); break;
    default: throw Error(90, "unknown metric");
    }
}

} // namespace

void launch_assign_generic(CudaDevice &dev, GenericParams &p, int metric, int mode, size_t cb)
{
    if (p.n == 0) return;
    switch (mode) {
    case G_TRAIN:
        if (cb == 1) launch_gen_t<M_SQ, G_TRAIN, uint8_t>(dev, p);
        else if (cb == 2) launch_gen_t<M_SQ, G_TRAIN, uint16_t>(dev, p);
        else launch_gen_t<M_SQ, G_TRAIN, uint32_t>(dev, p);
        break;
    case G_ENCODE: launch_gen_metric<G_ENCODE>(dev, p, metric); break;
    case G_RVQ_UPDATE: launch_gen_metric<G_RVQ_UPDATE>(dev, p, metric); break;
    case G_RVQ_QUANT: launch_gen_metric<G_RVQ_QUANT>(dev, p, metric); break;
    default: throw Error(90, "unknown mode");
    }
}

} // namespace vqb
