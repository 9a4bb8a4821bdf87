// opq_parts.hpp -- read-only view of a trained OPQ handle for translation units other than api.cpp.
#pragma once
#include <mutex>
#include <string>

#include "cuda_device.hpp"

struct vqb_opq;

namespace vqb {

struct OpqParts {
    CudaDevice *dev;
    std::mutex *mu;
    std::string *err;
    const float *rotation; // device, dim x dim row-major
    const float *codebooks; // device, m x k x sd
    size_t m, k, sd, dim;
    int metric;
    double p;
    bool empty;
};

OpqParts opq_parts(vqb_opq *oq);

} // namespace vqb
