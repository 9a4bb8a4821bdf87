// opq_tc.hpp -- rotation and cross-covariance of the optimized product quantizer on tcgen05 (opq_tc.cu).
#pragma once
#include <cstddef>

namespace vqb {

class CudaDevice;

// 32 <= dim <= 128 in steps of 32, 16-byte aligned row matrices
bool opq_tc_applicable(size_t dim, const float *x, const float *y);
// floats of scratch launch_opq_rotate needs for the two TF32 parts of the rotation matrix
size_t opq_tc_split_floats(size_t dim);
// y[r] = R x[r]   (src/opq.rs:186-194, 232-234); rot: device, dim x dim row-major
void launch_opq_rotate(CudaDevice &dev, const float *rot, size_t dim, const float *x, size_t n, float *y, float *split, int *error_word);
// a[i][j] += sum_r y[r][i] x[r][j]   (src/opq.rs:172-179); a: device f64, zero-filled by the caller
void launch_opq_cross_cov(CudaDevice &dev, const float *y, const float *x, size_t n, size_t dim, double *a, int *error_word);

} // namespace vqb
