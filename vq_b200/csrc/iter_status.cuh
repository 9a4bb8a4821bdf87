// iter_status.cuh -- how the centroid-update kernels hand one k-means iteration's flags to the host.
//
// The host needs, once per iteration, the "some row moved" word of every sub-space and the set of clusters that received
// no row (src/utils.rs:76-80,95-106).  The update kernels write them straight into a page of mapped pinned host memory,
// which the host polls, so no copy is queued and no stream is synchronised.  Every entry of the page is one aligned 64-bit
// word (sequence number of the update << 32) | value, stored with a single instruction: the host accepts an entry when
// it carries the number it is waiting for, so the kernels need neither fences nor a "last CTA" count.
//   entry 0            the tensor-core kernels' error word (0 = no bounded wait expired)
//   entries 1 .. m     moved[s]
//   then m x wps       bitmap, bit j of sub-space s = cluster j is empty   (wps = ceil(k / 32))
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vqb {

struct StatusPage {
    unsigned long long *host_words; // device-side address of the mapped page
    const int *tc_error;            // device memory, may be null
    uint32_t seq;                   // number of this update
    uint32_t m, words_per_subspace;
    __host__ __device__ size_t idx_error() const { return 0; }
    __host__ __device__ size_t idx_moved(size_t s) const { return 1 + s; }
    __host__ __device__ size_t idx_bitmap(size_t s, size_t w) const { return 1 + m + s * words_per_subspace + w; }
    static size_t words(size_t m, size_t k) { return 1 + m + m * ((k + 31) / 32); }
#ifdef __CUDACC__
    __device__ __forceinline__ void put(size_t idx, uint32_t value) const
    {
        *reinterpret_cast<volatile unsigned long long *>(host_words + idx) = ((unsigned long long)seq << 32) | value;
    }
    // one thread of the launch, after its own work: the error word as it stands
    __device__ __forceinline__ void put_error() const { put(idx_error(), tc_error ? (uint32_t)*reinterpret_cast<const volatile int *>(tc_error) : 0u); }
#endif
};

} // namespace vqb
