// peer_exchange.cuh -- the centroid-update kernels' own all-reduce over the peer memory of one node.
//
// With one process per GPU every rank gathers sums, counts and moved flags of its rows in an iteration buffer.  Instead of
// an NCCL all-reduce followed by the update kernel, the update kernel of every rank reads the same slice of EVERY rank's
// buffer straight over NVLink (plain peer loads, no multicast), adds the parts in rank order -- so all ranks compute
// bit-identical centroids -- and goes on with the division.  One launch and one NVLink round trip instead of a collective
// plus a launch; the data is 132 KiB per rank, so latency is all that matters.
//
// Hand-shake (flags live in every rank's exchange window, one word per peer, carrying the number of the last exchange that
// peer announced):
//   * at its start the update kernel of rank r stores the exchange number e into flags[p][r] of every rank p (its own rows
//     were accumulated by earlier kernels of the same stream) and waits until flags[r][q] >= e for every q;
//   * it then reads window buffer e mod 2 of every rank and clears its OWN buffer (e - 1) mod 2: a rank announces e only
//     after its update kernel of exchange e - 1 has finished, so by then nobody reads that buffer any more.
// Every wait is bounded (about four seconds); on expiry the kernel records an error, finishes with whatever it read, and
// the host raises at its next synchronisation.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vqb {

constexpr int VQB_MAX_PEERS = 8;
constexpr int PEER_ERR_WAIT = 170;

struct PeerView {
    int world = 0, rank = 0;                 // world <= 1: no exchange, the local buffer is final
    uint32_t epoch = 0;                      // number of this exchange
    const uint32_t *words[VQB_MAX_PEERS];    // rank q's iteration buffer of this exchange: sums | counts (u32) | moved
    uint32_t *flags[VQB_MAX_PEERS];          // rank p's arrival flags, one word per rank
    uint32_t *stale = nullptr;               // this rank's buffer of the previous exchange
    unsigned long long off_counts = 0, off_moved = 0; // word offsets inside a buffer
    int *error = nullptr;                    // device error word, may be null
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long peer_now_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Called by all threads of every CTA (blockDim.x >= world) before the first peer load.
__device__ __forceinline__ void peer_arrive_and_wait(const PeerView &pv)
{
    if (pv.world <= 1) return;
    const int t = threadIdx.x + threadIdx.y * blockDim.x;
    if (blockIdx.x == 0 && blockIdx.y == 0 && t < pv.world) {
        // release at system scope: what earlier kernels of this stream wrote into the buffer is visible to whoever
        // acquires this flag
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pv.flags[t] + pv.rank), "r"(pv.epoch) : "memory");
    }
    if (t < pv.world && t != pv.rank) {
        const uint32_t *f = pv.flags[pv.rank] + t;
        const unsigned long long t0 = peer_now_ns();
        for (uint32_t i = 0;; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int32_t)(v - pv.epoch) >= 0) break;
            if ((i & 255u) == 255u && peer_now_ns() - t0 > 4000000000ull) {
                if (pv.error) atomicCAS(pv.error, 0, PEER_ERR_WAIT);
                break;
            }
        }
    }
    __syncthreads();
}

// Loads that go to another GPU's memory every time (never from a local cache line of an earlier exchange).
__device__ __forceinline__ float4 peer_ld4(const uint32_t *p) { return __ldcv(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ uint32_t peer_ld(const uint32_t *p) { return __ldcv(p); }
#endif

} // namespace vqb
