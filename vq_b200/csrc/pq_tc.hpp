// pq_tc.hpp -- tensor-core product-quantizer assignment (pq_tc.cu).
#pragma once
#include <cstddef>

namespace vqb {

class CudaDevice;
struct AssignParams;

// sub-space width 8, 4 <= m <= 64 (multiple of 4), 2 <= k <= 256, 16-byte aligned row slices, Euclidean metrics
bool pq_tc_applicable(const AssignParams &p, int metric);
size_t pq_tc_scratch_floats();
// scratch: pq_tc_scratch_floats() floats, zero-filled once; dbg_scores (optional): n x m x 256 raw scores
void launch_pq_tc(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t code_bytes, float *scratch, int *error_word,
                  float *dbg_scores = nullptr);
// number of (row, sub-space) pairs the tensor kernel has handed to the exact scan so far (first u64 of the statistics)
size_t pq_tc_stats_offset_floats();

} // namespace vqb
