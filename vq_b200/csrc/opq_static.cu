// opq_static.cu -- OPQ encode for hosts that cannot let the library allocate device memory.
//
// Some embedders hand every byte of HBM to their own pool at start-up (so a cudaMalloc from inside a library
// fails or fragments their budget), and some call from a request loop where the driver's allocator lock and the
// implicit synchronisation of cudaMalloc/cudaFree are not acceptable.  vqb_opq_quantize needs one piece of scratch
// -- the rotated rows y = R x that sit between the rotation kernel and the nearest-centroid kernel -- and normally
// takes it from the stream-ordered pool.  The entry point below keeps that scratch in a fixed array that is part
// of the library image instead, and runs the nearest-centroid step on the CUDA-core kernels, which need no device
// memory of their own (the tensor-core kernel vqb_opq_quantize prefers works through operand tiles and a mark map
// that the context allocates on first use and grows with the batch).  Nothing on this path calls an allocator or
// creates an event, whether or not the context has been used before.
#include <mutex>

#include "../../include/vqb.h"
#include "opq_parts.hpp"

namespace {

// The rotated rows of one call.  Every GPU that loads the library holds this array until the process exits.
static __device__ __align__(256) float g_rotated_rows[VQB_OPQ_STATIC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
float *g_scratch_addr[kMaxDevices] = {};

// In host code `g_rotated_rows` is only a stand-in for the symbol, not an address a kernel may be given: the
// device address has to be asked for, once per device, while that device is current.
float *scratch_for_current_device(int device)
{
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (device < 0 || device >= kMaxDevices) throw vqb::Error(VQB_ERR_UNSUPPORTED, "device index beyond the static scratch table");
    if (!g_scratch_addr[device]) {
        float *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_rotated_rows);
        if (e != cudaSuccess || !ptr)
            throw vqb::Error(VQB_ERR_CUDA, std::string("cudaGetSymbolAddress failed for the static OPQ scratch: ") + cudaGetErrorString(e));
        g_scratch_addr[device] = ptr;
    }
    return g_scratch_addr[device];
}

} // namespace

extern "C" int vqb_opq_quantize_static(vqb_opq *oq, const float *x, size_t n, size_t dim, uint16_t *out_f16, uint32_t *codes)
{
    if (!oq) return VQB_ERR_BAD_ARGUMENT;
    vqb::OpqParts P = vqb::opq_parts(oq);
    std::lock_guard<std::mutex> lk(*P.mu);
    try {
        vqb::CudaDevice &dev = *P.dev;
        dev.make_current();
        if (dim != P.dim)
            throw vqb::Error(VQB_ERR_DIMENSION_MISMATCH,
                             "Dimension mismatch: expected " + std::to_string(P.dim) + ", got " + std::to_string(dim));
        if (P.empty) return VQB_OK; // no codebooks: empty result, as vqb_opq_quantize
        if (P.metric == VQB_MINKOWSKI && P.p <= 0.0)
            throw vqb::Error(VQB_ERR_INVALID_METRIC_PARAMETER, "Invalid metric parameter for Minkowski: p must be positive");
        if (n == 0) return VQB_OK;
        if (n > VQB_OPQ_STATIC_MAX_FLOATS / dim)
            throw vqb::Error(VQB_ERR_UNSUPPORTED, "vqb_opq_quantize_static: n * dim = " + std::to_string(n) + " * " + std::to_string(dim) +
                                                      " exceeds the static scratch of " + std::to_string((size_t)VQB_OPQ_STATIC_MAX_FLOATS) +
                                                      " floats; split the batch or use vqb_opq_quantize");
        if (!x || (!out_f16 && !codes)) throw vqb::Error(VQB_ERR_BAD_ARGUMENT, "NULL data pointer");
        if (!dev.is_device_pointer(x) || (out_f16 && !dev.is_device_pointer(out_f16)) || (codes && !dev.is_device_pointer(codes)))
            throw vqb::Error(VQB_ERR_BAD_ARGUMENT, "vqb_opq_quantize_static takes device pointers only (staging host memory would allocate)");
        if (dev.timing())
            throw vqb::Error(VQB_ERR_UNSUPPORTED, "vqb_opq_quantize_static: switch per-kernel timing off first (timing creates events)");
        float *y = scratch_for_current_device(dev.device());
        dev.rotate_rows(P.rotation, dim, x, n, y); // overwrites y[0 .. n*dim): nothing has to start at zero
        vqb::Shape sh;
        sh.n_local = n;
        sh.ld = dim;
        sh.m = P.m;
        sh.sd = P.sd;
        sh.k = P.k;
        // the CUDA-core nearest-centroid kernels: codebooks in shared memory, rows in registers, nothing else -- the tensor-core
        // kernel vqb_opq_quantize uses keeps operand tiles and a mark map in device memory that the context allocates
        dev.pq_encode_no_scratch(sh, y, P.codebooks, P.metric, P.p, out_f16, codes);
        return VQB_OK;
    } catch (const vqb::Error &e) {
        *P.err = e.what();
        return e.code;
    } catch (const std::exception &e) {
        *P.err = e.what();
        return VQB_ERR_BAD_ARGUMENT;
    }
}
