// tsvq.hpp -- tree-structured vector quantizer on the device (tsvq.cu).
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

namespace vqb {

class CudaDevice;

struct TsvqTree {
    size_t dim = 0, nodes = 0;
    float *centroids = nullptr; // device, nodes x dim
    int32_t *left = nullptr;    // device, -1 = no child
    int32_t *right = nullptr;   // device
    std::vector<int32_t> h_left, h_right;
};

// TSVQNode::fit (src/tsvq.rs:71-148), breadth-first; x: n x dim on the device.  Throws Error(105, ..) on NaN.
void tsvq_fit(CudaDevice &dev, const float *x, size_t n, size_t dim, size_t max_depth, TsvqTree &out);
// TSVQ::quantize (src/tsvq.rs:162-181, 231-249) for n rows; out_f16 / leaf may be null.
void tsvq_quantize(CudaDevice &dev, const TsvqTree &t, int metric, double p, const float *x, size_t n, uint16_t *out_f16, uint32_t *leaf);
void tsvq_release(CudaDevice &dev, TsvqTree &t);

} // namespace vqb
