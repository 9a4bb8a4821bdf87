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

  private:
    void run(void *b, size_t n, ncclDataType_t t, ncclRedOp_t op)
    {
        if (n == 0) return;
        check(api().AllReduce(b, b, n, t, op, comm_, dev_.stream()), "ncclAllReduce");
    }
    CudaDevice &dev_;
    ncclComm_t comm_ = nullptr;
    int rank_, world_;
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
