// dense_tc.hpp -- tensor-core shortlist + exact resolve for full-width nearest-centroid search (dense_tc.cu, resolve.cu).
#pragma once
#include <cstddef>
#include <cstdint>

namespace vqb {

class CudaDevice;

#define DENSE_MASK_WORDS 8 /* 256 candidate bits per row (32 bytes) */
#define VQB_DENSE_INF __int_as_float(0x7f800000)

// Squared-Euclidean / Euclidean, 32 <= dim <= 128 in steps of 32, 2 <= k <= 256, 16-byte aligned rows.
bool dense_tc_applicable(size_t n, size_t dim, size_t k, int metric, const float *x);
size_t dense_tc_smem_bytes();
// out[r] >= |x_r|^2 (tight upper bound)
void dense_row_norms(CudaDevice &dev, const float *x, size_t n, size_t dim, float *out);
// cand[r][0..8): 256-bit mask, bit j set for every centroid that can be the reference's choice for row r; rows that
// cannot be ranked (NaN / infinity) come back with all k bits set.
// With `train` (k-means passes; assignments are one byte here, k <= 256) the kernel also decides every row that has a single
// candidate -- codes[r] is rewritten, train->changed gets VQB_MOVED_BITS when a row moved -- and appends the other rows to
// train->list (count in *train->list_count, zero on entry); only those rows get their mask written.
struct ShortlistTrain {
    uint8_t *codes;
    uint32_t *changed;
    uint32_t *list;
    uint32_t *list_count;
};
void dense_shortlist(CudaDevice &dev, const float *x, size_t n, size_t dim, const float *codebook, size_t k, const float *xnorm2,
                     float *hn_scratch /* 257 floats */, uint32_t *cand, unsigned long long *stats, int *error_word, float *debug_dots,
                     const ShortlistTrain *train = nullptr);

enum : int { R_TRAIN = 0, R_RVQ_UPDATE = 1, R_RVQ_STAGE = 2 };

struct ResolveParams {
    const float *x; // n rows of dim floats (R_RVQ_UPDATE / R_RVQ_STAGE: the residuals, updated in place through `res`)
    unsigned long long n;
    int dim, k;
    const float *codebook; // [k][dim]
    const uint32_t *cand;  // [n][DENSE_MASK_WORDS]
    int euclid;            // compare square roots (Distance::Euclidean) instead of squared sums
    // R_TRAIN: only the rows in list[0 .. *list_count) are looked at (the shortlist kernel decided the others)
    void *codes;
    uint32_t *changed;
    const uint32_t *list;
    const uint32_t *list_count;
    // R_RVQ_UPDATE, R_RVQ_STAGE
    float *res;
    double *norm_sum;
    // R_RVQ_STAGE
    float *qsum;         // [n][dim] running sum of chosen centroids
    uint8_t *done;       // [n] row stopped early (src/rvq.rs:204-207)
    uint32_t *out_codes; // [n][stages] or null
    int stage, stages;
    float epsilon;
};

void launch_resolve(CudaDevice &dev, const ResolveParams &p, int mode, size_t code_bytes);

} // namespace vqb
