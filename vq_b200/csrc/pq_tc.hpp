// pq_tc.hpp -- tensor-core product-quantizer assignment (pq_tc.cu).
#pragma once
#include <cstddef>
#include <cstdint>

#include "iter_status.cuh"
#include "peer_exchange.cuh"

namespace vqb {

class CudaDevice;
struct AssignParams;

// sub-space width 8, 4 <= m <= 64 (multiple of 4), 2 <= k <= 256, 16-byte aligned row slices, Euclidean metrics
bool pq_tc_applicable(const AssignParams &p, int metric);
size_t pq_tc_scratch_floats();
// bytes of the (row, sub-space pair) mark map for n rows of m sub-spaces
size_t pq_tc_mark_bytes(size_t n, size_t m);

// Device memory one launch works with besides its inputs and outputs.
struct PqTcBuffers {
    float *scratch = nullptr;     // pq_tc_scratch_floats() floats, zero-filled once: operand B, binary16 images, half-norm maxima, statistics
    uint8_t *marks = nullptr;     // pq_tc_mark_bytes(n, m) bytes, zero-filled once; every launch hands it back zero-filled
    int *error_word = nullptr;    // set when a bounded wait expires
    bool prepare_operand = true;  // false: scratch already holds operand B of p.centroids (written by launch_pq_update_centroids)
    float *dbg_scores = nullptr;  // optional: n x m x 256 raw scores
};
void launch_pq_tc(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t code_bytes, const PqTcBuffers &b);
// number of (row, sub-space) pairs the tensor kernel has handed to the exact scan so far (first u64 of the statistics)
size_t pq_tc_stats_offset_floats();
// centroid update + operand B of the next pass + the iteration's flags, one launch (m CTAs)
void launch_pq_update_centroids(CudaDevice &dev, int m, int k, float *sums, uint32_t *counts, uint32_t *moved, bool counts_f32,
                                const uint32_t *active, float *centroids, float *scratch, const StatusPage &sp, const PeerView &pv);

} // namespace vqb
