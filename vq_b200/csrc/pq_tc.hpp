// pq_tc.hpp -- tensor-core product-quantizer assignment (pq_tc.cu).
#pragma once
#include <cstddef>

namespace vqb {

class CudaDevice;
struct AssignParams;

// sub-space width 8, 4 <= m <= 16 (multiple of 4), 2 <= k <= 256, contiguous 16-byte aligned rows, Euclidean metrics
bool pq_tc_applicable(const AssignParams &p, int metric);
size_t pq_tc_scratch_floats();
void launch_pq_tc(CudaDevice &dev, const AssignParams &p, int metric, bool train, size_t code_bytes, float *scratch, int *error_word);

} // namespace vqb
