// iter_status.cuh -- how the centroid-update kernels hand one k-means iteration's flags to the host.
//
// The host needs, once per iteration, the "some row moved" word of every sub-space and the set of clusters that received
// no row (src/utils.rs:76-80,95-106).  The update kernels write them straight into a page of mapped pinned host memory and
// then publish a sequence number; the host polls that word, so no copy is queued and no stream is synchronised:
//   word 0            sequence number of the last finished update
//   word 1            the tensor-core kernels' error word at that time (0 = no bounded wait expired)
//   words 4 .. 4+m    moved[s]
//   then m x wps      bitmap, bit j of sub-space s = cluster j is empty   (wps = ceil(k / 32))
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vqb {

struct StatusPage {
    uint32_t *host_words;       // device-side address of the mapped page
    unsigned int *done_counter; // device memory, zero between launches
    const int *tc_error;        // device memory, may be null
    uint32_t seq;               // value to publish
    uint32_t total_blocks;      // CTAs of the publishing launch
    uint32_t m, words_per_subspace;
    __host__ __device__ uint32_t *host_moved() const { return host_words + 4; }
    __host__ __device__ uint32_t *host_bitmap() const { return host_words + 4 + m; }
    static size_t words(size_t m, size_t k) { return 4 + m + m * ((k + 31) / 32); }
};

#ifdef __CUDACC__
// Every thread of every CTA calls this at the end of the kernel; `wrote` = this thread stored something into the page.  Only
// those threads pay for a system-scope fence (the others may have a hundred bytes of ordinary global stores in flight, which
// the next kernel on the stream sees anyway).  The last CTA to arrive publishes the sequence number.
__device__ __forceinline__ void status_publish(const StatusPage &sp, bool wrote)
{
    if (wrote) __threadfence_system(); // this thread's page writes are visible to the host before anything that follows
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0) {
        __threadfence_system(); // orders what the barrier made visible to this thread before the arrival below
        if (atomicAdd(sp.done_counter, 1u) == sp.total_blocks - 1u) {
            *sp.done_counter = 0u; // the next launch on the stream starts from zero again
            sp.host_words[1] = sp.tc_error ? (uint32_t)*sp.tc_error : 0u;
            __threadfence_system();
            *reinterpret_cast<volatile uint32_t *>(sp.host_words) = sp.seq;
        }
    }
}
#endif

} // namespace vqb
