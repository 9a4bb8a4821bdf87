// nccl_comm.cpp -- vqb::Comm over NCCL (one process per GPU; all-reduces travel over NVLink/NVSwitch).
//
// NCCL is opened with dlopen at communicator creation so that the library itself loads on machines
// without NCCL, and so that a process that already holds an NCCL (e.g. through PyTorch) shares it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "cuda_device.hpp"

namespace vqb {

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi &api()
{
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {std::getenv("VQB_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char *nm : names) {
            if (!nm || !*nm) continue;
            a.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
            if (a.handle) break;
        }
        if (!a.handle) return;
        a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.handle, "ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.handle, "ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.handle, "ncclCommDestroy");
        a.AllReduce = (decltype(a.AllReduce))dlsym(a.handle, "ncclAllReduce");
        a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.handle, "ncclGetErrorString");
        a.GroupStart = (decltype(a.GroupStart))dlsym(a.handle, "ncclGroupStart");
        a.GroupEnd = (decltype(a.GroupEnd))dlsym(a.handle, "ncclGroupEnd");
    });
    if (!a.handle || !a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce)
        throw Error(101, "NCCL library (libnccl.so.2) could not be loaded");
    return a;
}

void check(ncclResult_t r, const char *what)
{
    if (r != ncclSuccess) {
        const char *msg = api().GetErrorString ? api().GetErrorString(r) : "?";
        throw Error(101, std::string("NCCL error in ") + what + ": " + msg);
    }
}

class NcclComm : public Comm {
  public:
    NcclComm(CudaDevice &dev, const uint8_t *id_bytes, int rank, int world) : dev_(dev), rank_(rank), world_(world)
    {
        static_assert(sizeof(ncclUniqueId) <= 128, "unique id larger than the ABI's buffer");
        ncclUniqueId id;
        std::memcpy(&id, id_bytes, sizeof id);
        dev_.make_current();
        check(api().CommInitRank(&comm_, world, id, rank), "ncclCommInitRank");
    }
    ~NcclComm() override
    {
        for (Window &w : windows_) close_window(w);
        if (comm_) api().CommDestroy(comm_);
    }
    int rank() const override { return rank_; }
    int world() const override { return world_; }
    void allreduce_sum_f32(float *b, size_t n) override { run(b, n, ncclFloat32, ncclSum); }
    void allreduce_sum_f64(double *b, size_t n) override { run(b, n, ncclFloat64, ncclSum); }
    void allreduce_sum_u32(uint32_t *b, size_t n) override { run(b, n, ncclUint32, ncclSum); }
    void allreduce_max_u32(uint32_t *b, size_t n) override { run(b, n, ncclUint32, ncclMax); }
    void allreduce_sum_u64(uint64_t *b, size_t n) override { run(b, n, ncclUint64, ncclSum); }
    void group_begin() override
    {
        if (api().GroupStart) check(api().GroupStart(), "ncclGroupStart");
    }
    void group_end() override
    {
        if (api().GroupEnd) check(api().GroupEnd(), "ncclGroupEnd");
    }

    // ---- iteration buffers every GPU of the node can read (CUDA IPC; protocol in peer_exchange.cuh) ----
    bool peer_window(size_t words, uint32_t *local[2]) override
    {
        if (peer_off_ || world_ < 2 || world_ > MAX_PEERS) return false;
        if (windows_.empty() || windows_.back().cap_words < words) {
            if (!open_window(words)) { // every rank takes the same decision: it follows from all-reduced flags
                peer_off_ = true;
                return false;
            }
        }
        Window &w = windows_.back();
        dev_.make_current();
        local[0] = w.local + FLAG_WORDS;
        local[1] = local[0] + w.cap_words;
        if (cudaMemsetAsync(local[0], 0, sizeof(uint32_t) * 2 * w.cap_words, dev_.stream()) != cudaSuccess) throw Error(100, "cudaMemsetAsync failed");
        return true;
    }
    PeerExchange peer_exchange(int which) override
    {
        const Window &w = windows_.back();
        PeerExchange px;
        px.world = world_;
        px.rank = rank_;
        px.epoch = ++epoch_;
        for (int r = 0; r < world_; ++r) {
            px.flags[r] = w.peer[r];
            px.words[r] = w.peer[r] + FLAG_WORDS + (size_t)(which & 1) * w.cap_words;
        }
        px.stale = w.local + FLAG_WORDS + (size_t)((which & 1) ^ 1) * w.cap_words;
        return px;
    }
    uint64_t peer_exchanges() const override { return epoch_; }

  private:
    static constexpr size_t FLAG_WORDS = 64; // arrival flags, one word per rank, ahead of the two buffers
    struct Window {
        size_t cap_words = 0;
        uint32_t *local = nullptr;       // this rank's allocation: flags | buffer 0 | buffer 1
        uint32_t *peer[MAX_PEERS] = {};  // the same allocation of every rank as mapped here (peer[rank] == local)
    };
    void close_window(Window &w)
    {
        for (int r = 0; r < world_; ++r)
            if (r != rank_ && w.peer[r]) cudaIpcCloseMemHandle(w.peer[r]);
        if (w.local) cudaFree(w.local);
        w = Window();
    }
    // Collective.  Allocates this rank's window, passes its IPC handle around (an all-reduce over slots that only the
    // owner fills) and maps the others.  An older, smaller window stays mapped until the communicator goes: a peer may
    // still be reading it.
    bool open_window(size_t words)
    {
        // Measured on B200s (1M x 128 rows in total, 132 KiB per rank and iteration): against one NCCL all-reduce per iteration
        // the direct exchange wins with two ranks (6.92 against 7.03 ms per fit + encode) and with four (3.93 against 4.07 ms);
        // with eight it runs at 2.61 ms.  VQB_PEER_EXCHANGE=0 selects NCCL.
        const char *env = std::getenv("VQB_PEER_EXCHANGE");
        const bool wanted = !(env && env[0] == '0');
        dev_.make_current();
        Window w;
        w.cap_words = (words + 63) / 64 * 64;
        const size_t bytes = sizeof(uint32_t) * (FLAG_WORDS + 2 * w.cap_words);
        constexpr size_t HW = sizeof(cudaIpcMemHandle_t) / sizeof(uint32_t);
        static_assert(sizeof(cudaIpcMemHandle_t) % sizeof(uint32_t) == 0, "handle size");
        std::vector<uint32_t> slots((size_t)world_ * (HW + 1), 0u);
        uint32_t *mine = slots.data() + (size_t)rank_ * (HW + 1);
        cudaIpcMemHandle_t handle;
        bool ok = wanted && cudaMalloc(reinterpret_cast<void **>(&w.local), bytes) == cudaSuccess;
        ok = ok && cudaMemset(w.local, 0, bytes) == cudaSuccess;
        ok = ok && cudaIpcGetMemHandle(&handle, w.local) == cudaSuccess;
        if (ok) {
            mine[0] = 1u;
            std::memcpy(mine + 1, &handle, sizeof handle);
        }
        cudaGetLastError();
        share(slots);
        bool all = true;
        for (int r = 0; r < world_; ++r) all = all && slots[(size_t)r * (HW + 1)] == 1u;
        uint32_t mapped = 0;
        if (all) {
            mapped = 1;
            for (int r = 0; r < world_ && mapped; ++r) {
                if (r == rank_) {
                    w.peer[r] = w.local;
                    continue;
                }
                cudaIpcMemHandle_t h;
                std::memcpy(&h, slots.data() + (size_t)r * (HW + 1) + 1, sizeof h);
                void *p = nullptr;
                if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) mapped = 0;
                w.peer[r] = static_cast<uint32_t *>(p);
            }
            cudaGetLastError();
        }
        std::vector<uint32_t> votes((size_t)world_, 0u);
        votes[rank_] = mapped;
        share(votes);
        for (int r = 0; r < world_; ++r) all = all && votes[r] == 1u;
        if (!all) {
            close_window(w);
            return false;
        }
        windows_.push_back(w);
        return true;
    }
    // all-reduce (sum) of a host vector whose entries are zero except where this rank owns them
    void share(std::vector<uint32_t> &v)
    {
        uint32_t *d = static_cast<uint32_t *>(dev_.alloc(sizeof(uint32_t) * v.size()));
        try {
            dev_.upload(d, v.data(), sizeof(uint32_t) * v.size());
            allreduce_sum_u32(d, v.size());
            dev_.download(v.data(), d, sizeof(uint32_t) * v.size());
        } catch (...) {
            dev_.release(d);
            throw;
        }
        dev_.release(d);
    }
    void run(void *b, size_t n, ncclDataType_t t, ncclRedOp_t op)
    {
        if (n == 0) return;
        check(api().AllReduce(b, b, n, t, op, comm_, dev_.stream()), "ncclAllReduce");
    }
    CudaDevice &dev_;
    ncclComm_t comm_ = nullptr;
    int rank_, world_;
    std::vector<Window> windows_;
    bool peer_off_ = false;
    uint32_t epoch_ = 0;
};

} // namespace

void nccl_unique_id(uint8_t *out128)
{
    ncclUniqueId id;
    check(api().GetUniqueId(&id), "ncclGetUniqueId");
    std::memset(out128, 0, 128);
    std::memcpy(out128, &id, sizeof id);
}

Comm *make_nccl_comm(CudaDevice &dev, const uint8_t *id_bytes, int rank, int world)
{
    return new NcclComm(dev, id_bytes, rank, world);
}

} // namespace vqb
