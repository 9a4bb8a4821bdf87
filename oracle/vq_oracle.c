/*
 * vq_oracle.c -- CPU restatement of the habedi/vq quantizer hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker and the timed CPU
 * baseline for the CUDA library; it is never linked into, loaded by, or used as
 * a fallback for the product library (libvqb.so).
 *
 * Every function follows the reference's operation order exactly (f32, separate
 * multiply and add roundings, serial left folds from 0.0, strict '<' argmin).
 * It must be compiled with  -ffp-contract=off  and without -ffast-math.
 *
 * Parity status:
 *   - distances, distance2, mean, SQ, BQ, single-point LBG: pinned against the
 *     known answers in the reference's own tests (see tests/test_oracle_*.py).
 *   - which rows the seeded RNG draws (rand 0.9 StdRng / choose_multiple /
 *     choose, source not available): PARITY UNPINNED.  Row indices are inputs
 *     here (init_idx + a draw callback), never generated.
 *   - OPQ rotation (nalgebra 0.33 SVD / product order): PARITY UNPINNED; the
 *     rotation update lives in the Python part of the oracle (numpy SVD).
 *
 * Reference citations are "file:line" inside the habedi/vq source tree.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define VQO_OK 0
#define VQO_EMPTY_INPUT 1
#define VQO_INVALID_PARAMETER 2
#define VQO_DIMENSION_MISMATCH 3
#define VQO_INVALID_METRIC_PARAMETER 4

enum {
    VQO_SQUARED_EUCLIDEAN = 0,
    VQO_EUCLIDEAN = 1,
    VQO_COSINE = 2,
    VQO_MANHATTAN = 3,
    VQO_CHEBYSHEV = 4,
    VQO_MINKOWSKI = 5,
    VQO_HAMMING = 6
};

/* uint64_t draw(user, stream, n): index in [0, n) of the row that re-seeds an
 * empty cluster -- stands for `data.choose(&mut rng)` (src/utils.rs:100).
 * `stream` identifies the per-call RNG (PQ subspace / RVQ stage). */
typedef uint64_t (*vqo_draw_fn)(void *user, size_t stream, uint64_t n);

static __thread char g_err[256];

const char *vqo_last_error(void) { return g_err; }

static int fail(int code, const char *msg)
{
    snprintf(g_err, sizeof g_err, "%s", msg);
    return code;
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline wants all host threads. */
void vqo_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int vqo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* f32 -> IEEE binary16 bits, round to nearest even (half::f16::from_f32,     */
/* used at src/pq.rs:179, src/rvq.rs:212, src/opq.rs:260).                    */
/* ------------------------------------------------------------------------ */
uint16_t vqo_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xffu;
    uint32_t man = x & 0x7fffffu;
    if (exp == 0xff) { /* inf / nan */
        if (man == 0) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | 0x7c00u | 0x0200u | (man >> 13));
    }
    int e = (int)exp - 127 + 15;
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u); /* overflow -> inf */
    if (e <= 0) {                                     /* subnormal or zero */
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e; /* 14..24 */
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++; /* may carry into exp: correct */
    return (uint16_t)(sign | half);
}

/* ------------------------------------------------------------------------ */
/* Vector::distance2 -- src/vector.rs:214-220: diff = a - b (Sub, 247-267),   */
/* then dot(diff, diff) as a serial fold `acc + a*b` from 0 (198-201).        */
/* ------------------------------------------------------------------------ */
float vqo_distance2(const float *a, const float *b, size_t d)
{
    float acc = 0.0f;
    for (size_t i = 0; i < d; ++i) {
        float diff = a[i] - b[i];
        float prod = diff * diff;
        acc = acc + prod;
    }
    return acc;
}

/* ------------------------------------------------------------------------ */
/* Distance::compute -- src/distances.rs:115-172, serial helpers 27-30,       */
/* 47-50, 66-69 (inputs here never exceed the 1024-element parallel switch;   */
/* for longer inputs the reference's order is unspecified and this serial     */
/* order is one admissible result).                                           */
/* ------------------------------------------------------------------------ */
int vqo_distance(int metric, double p, const float *a, size_t na, const float *b, size_t nb,
                 float *out)
{
    if (na != nb) {
        snprintf(g_err, sizeof g_err, "Dimension mismatch: expected %zu, got %zu", na, nb);
        return VQO_DIMENSION_MISMATCH;
    }
    size_t d = na;
    switch (metric) {
    case VQO_SQUARED_EUCLIDEAN: { /* 130-133 */
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float diff = a[i] - b[i];
            float v = diff * diff;
            acc = acc + v;
        }
        *out = acc;
        return VQO_OK;
    }
    case VQO_EUCLIDEAN: { /* 134-140 */
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float diff = a[i] - b[i];
            float v = diff * diff;
            acc = acc + v;
        }
        *out = sqrtf(acc);
        return VQO_OK;
    }
    case VQO_COSINE: { /* 141-151 */
        float dot = 0.0f, sa = 0.0f, sb = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float v = a[i] * b[i];
            dot = dot + v;
        }
        for (size_t i = 0; i < d; ++i) {
            float v = a[i] * a[i];
            sa = sa + v;
        }
        for (size_t i = 0; i < d; ++i) {
            float v = b[i] * b[i];
            sb = sb + v;
        }
        float norm_a = sqrtf(sa), norm_b = sqrtf(sb);
        if (norm_a == 0.0f || norm_b == 0.0f) {
            *out = 1.0f;
        } else {
            float den = norm_a * norm_b;
            float q = dot / den;
            *out = 1.0f - q;
        }
        return VQO_OK;
    }
    case VQO_MANHATTAN: { /* 152 */
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float v = fabsf(a[i] - b[i]);
            acc = acc + v;
        }
        *out = acc;
        return VQO_OK;
    }
    case VQO_CHEBYSHEV: { /* 153, fold-max from 0 (47-50) */
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float v = fabsf(a[i] - b[i]);
            if (v > acc) acc = v;
        }
        *out = acc;
        return VQO_OK;
    }
    case VQO_MINKOWSKI: { /* 154-167 */
        if (p <= 0.0)
            return fail(VQO_INVALID_METRIC_PARAMETER,
                        "Invalid metric parameter for Minkowski: p must be positive");
        float pv = (float)p;
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float v = powf(fabsf(a[i] - b[i]), pv);
            acc = acc + v;
        }
        *out = powf(acc, 1.0f / pv);
        return VQO_OK;
    }
    case VQO_HAMMING: { /* 168-170 */
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) {
            float v = (a[i] == b[i]) ? 0.0f : 1.0f;
            acc = acc + v;
        }
        *out = acc;
        return VQO_OK;
    }
    default:
        return fail(VQO_INVALID_PARAMETER, "Invalid parameter: unknown metric");
    }
}

static inline float dist_nocheck(int metric, double p, const float *a, const float *b, size_t d)
{
    float r = 0.0f;
    (void)vqo_distance(metric, p, a, d, b, d, &r);
    return r;
}

/* ------------------------------------------------------------------------ */
/* mean_vector -- src/vector.rs:282-318.  Members are added in ascending data */
/* order (the <=1024-member branch, 305-313); the reference's >1024-member    */
/* branch (298-304) is an unordered tree sum, for which this order is one     */
/* admissible result.  Division by `len as f32` (315-316).                    */
/* rows: n x ld floats, members picked by `assign[i] == cluster`.             */
/* ------------------------------------------------------------------------ */
int vqo_mean_rows(const float *rows, size_t n, size_t ld, size_t d, float *mean)
{
    if (n == 0) return fail(VQO_EMPTY_INPUT, "Empty input: at least one vector is required.");
    for (size_t c = 0; c < d; ++c) mean[c] = 0.0f;
    for (size_t i = 0; i < n; ++i)
        for (size_t c = 0; c < d; ++c) mean[c] = mean[c] + rows[i * ld + c];
    float len = (float)(double)n;
    for (size_t c = 0; c < d; ++c) mean[c] = mean[c] / len;
    return VQO_OK;
}

/* ------------------------------------------------------------------------ */
/* Nearest centroid under squared Euclidean for a block of points, written    */
/* so the compiler can vectorise ACROSS centroids while each centroid's sum   */
/* keeps the reference's serial order over dimensions (src/utils.rs:59-73 +   */
/* src/vector.rs:214-220).  ct = centroids transposed, d x kp (kp >= k).      */
/* ------------------------------------------------------------------------ */
static inline uint32_t argmin_sq_t(const float *x, const float *ct, size_t d, size_t k, size_t kp,
                                   float *acc /* kp scratch */, int take_root)
{
    for (size_t j = 0; j < k; ++j) acc[j] = 0.0f;
    for (size_t i = 0; i < d; ++i) {
        const float xi = x[i];
        const float *row = ct + i * kp;
        for (size_t j = 0; j < k; ++j) {
            float diff = xi - row[j];
            float prod = diff * diff;
            acc[j] = acc[j] + prod;
        }
    }
    if (take_root) /* Euclidean compares the roots (src/distances.rs:134-140) */
        for (size_t j = 0; j < k; ++j) acc[j] = sqrtf(acc[j]);
    uint32_t best = 0;
    float best_dist = acc[0];
    for (size_t j = 1; j < k; ++j) {
        if (acc[j] < best_dist) { /* strict '<': lowest index wins ties (utils.rs:66) */
            best = (uint32_t)j;
            best_dist = acc[j];
        }
    }
    return best;
}

static void transpose_codebook(const float *c, size_t k, size_t d, size_t kp, float *ct)
{
    for (size_t i = 0; i < d; ++i)
        for (size_t j = 0; j < kp; ++j) ct[i * kp + j] = (j < k) ? c[j * d + i] : 0.0f;
}

/* ------------------------------------------------------------------------ */
/* lbg_quantize -- src/utils.rs:32-109.                                       */
/*   data      : n rows, row i at data + i*ld + col0, d columns used          */
/*   init_idx  : k row indices = the `choose_multiple(k)` draw (line 54)      */
/*   draw      : `data.choose(&mut rng)` for each empty cluster, ascending j  */
/*   centroids : out, k x d                                                   */
/*   assign_out: optional, n entries, last assignments                        */
/*   iters_out : optional, iterations executed                                */
/* ------------------------------------------------------------------------ */
int vqo_lbg(const float *data, size_t n, size_t ld, size_t col0, size_t d, size_t k,
            size_t max_iters, const uint64_t *init_idx, vqo_draw_fn draw, void *user, size_t stream,
            float *centroids, uint32_t *assign_out, size_t *iters_out)
{
    if (k == 0) /* 39-44 */
        return fail(VQO_INVALID_PARAMETER, "Invalid parameter: k must be greater than 0");
    if (n < k) /* 45-50 */
        return fail(VQO_INVALID_PARAMETER,
                    "Invalid parameter: Not enough data points for k clusters");
    for (size_t j = 0; j < k; ++j) { /* 54 */
        if (init_idx[j] >= n) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: init index out of range");
        memcpy(centroids + j * d, data + init_idx[j] * ld + col0, d * sizeof(float));
    }
    size_t kp = (k + 15) & ~(size_t)15;
    uint32_t *assign = (uint32_t *)calloc(n ? n : 1, sizeof(uint32_t)); /* 55: all zeros */
    float *ct = (float *)malloc(sizeof(float) * d * kp);
    float *sums = (float *)malloc(sizeof(float) * k * d);
    uint64_t *counts = (uint64_t *)malloc(sizeof(uint64_t) * k);
    size_t iters = 0;
    for (size_t it = 0; it < max_iters; ++it) { /* 57 */
        ++iters;
        transpose_codebook(centroids, k, d, kp, ct);
        int changed = 0;
        /* assignment, parallel over points (59-73); order-independent */
#pragma omp parallel
        {
            float *acc = (float *)malloc(sizeof(float) * kp);
            int local_changed = 0;
#pragma omp for schedule(static)
            for (size_t i = 0; i < n; ++i) {
                uint32_t b = argmin_sq_t(data + i * ld + col0, ct, d, k, kp, acc, 0);
                if (b != assign[i]) local_changed = 1; /* 76-80 */
                assign[i] = b;
            }
            if (local_changed) {
#pragma omp atomic write
                changed = 1;
            }
            free(acc);
        }
        /* gather + mean (83-99): one ascending pass adds every member to its  */
        /* cluster's sum in data order, which is the order mean_vector uses.   */
        memset(sums, 0, sizeof(float) * k * d);
        memset(counts, 0, sizeof(uint64_t) * k);
        for (size_t i = 0; i < n; ++i) {
            float *s = sums + (size_t)assign[i] * d;
            const float *x = data + i * ld + col0;
            for (size_t c = 0; c < d; ++c) s[c] = s[c] + x[c];
            counts[assign[i]]++;
        }
        for (size_t j = 0; j < k; ++j) { /* 95-102, ascending j */
            if (counts[j] != 0) {
                float len = (float)(double)counts[j];
                for (size_t c = 0; c < d; ++c) centroids[j * d + c] = sums[j * d + c] / len;
            } else {
                uint64_t r = draw ? draw(user, stream, (uint64_t)n) : 0;
                if (r >= n) r = n - 1;
                memcpy(centroids + j * d, data + r * ld + col0, d * sizeof(float));
            }
        }
        if (!changed) break; /* 104-106 */
    }
    if (assign_out) memcpy(assign_out, assign, n * sizeof(uint32_t));
    if (iters_out) *iters_out = iters;
    free(assign);
    free(ct);
    free(sums);
    free(counts);
    return VQO_OK;
}

/* ------------------------------------------------------------------------ */
/* ProductQuantizer::fit -- src/pq.rs:79-129.  init_idx is m x k; stream =    */
/* subspace index (the reference seeds subspace i with seed+i, line 119).     */
/* The `distance` argument of the reference is not used during training.      */
/* ------------------------------------------------------------------------ */
int vqo_pq_fit(const float *data, size_t n, size_t dim, size_t m, size_t k, size_t max_iters,
               const uint64_t *init_idx, vqo_draw_fn draw, void *user, float *codebooks,
               size_t *iters_out /* m or NULL */)
{
    if (n == 0) return fail(VQO_EMPTY_INPUT, "Empty input: at least one vector is required.");
    if (m == 0) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: m must be greater than 0");
    if (dim < m) /* 91-96 */
        return fail(VQO_INVALID_PARAMETER, "Invalid parameter: Data dimension must be at least m");
    if (dim % m != 0) /* 97-102 */
        return fail(VQO_INVALID_PARAMETER,
                    "Invalid parameter: Data dimension must be divisible by m");
    size_t sd = dim / m;
    for (size_t s = 0; s < m; ++s) { /* 106-121 */
        int rc = vqo_lbg(data, n, dim, s * sd, sd, k, max_iters, init_idx + s * k, draw, user, s,
                         codebooks + s * k * sd, NULL, iters_out ? iters_out + s : NULL);
        if (rc) return rc;
    }
    return VQO_OK;
}

/* ------------------------------------------------------------------------ */
/* The same fit with the reference's MEMORY BEHAVIOUR, for timing only: the     */
/* "faithful" CPU baseline.  Results equal vqo_pq_fit's bit for bit.            */
/*   - every row of a subspace is its own heap allocation (src/pq.rs:110-117   */
/*     builds a Vec<Vector<f32>> of slices; src/vector.rs:150-152)             */
/*   - distance2 allocates the difference vector on every call                 */
/*     (src/vector.rs:214-220 via Sub, 259-265)                                */
/*   - the gather scans all n assignments once per cluster and clones the      */
/*     members (src/utils.rs:83-92), then mean_vector (95-99)                  */
/*   - rayon's decomposition: points for the assignment, clusters for the      */
/*     gather; subspaces outermost and serial (src/pq.rs:106-121)              */
/* ------------------------------------------------------------------------ */
static float distance2_alloc(const float *a, const float *b, size_t d)
{
    float *diff = (float *)malloc(sizeof(float) * d); /* the `self - other` temporary */
    for (size_t i = 0; i < d; ++i) diff[i] = a[i] - b[i];
    float acc = 0.0f;
    for (size_t i = 0; i < d; ++i) acc = acc + diff[i] * diff[i];
    free(diff);
    return acc;
}

static int lbg_faithful(float **rows, size_t n, size_t d, size_t k, size_t max_iters, const uint64_t *init_idx,
                        vqo_draw_fn draw, void *user, size_t stream, float *centroids_out)
{
    if (k == 0) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: k must be greater than 0");
    if (n < k) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: Not enough data points for k clusters");
    float **cent = (float **)malloc(sizeof(float *) * k);
    for (size_t j = 0; j < k; ++j) {
        cent[j] = (float *)malloc(sizeof(float) * d);
        memcpy(cent[j], rows[init_idx[j]], sizeof(float) * d);
    }
    size_t *assign = (size_t *)calloc(n ? n : 1, sizeof(size_t));
    for (size_t it = 0; it < max_iters; ++it) {
        int changed = 0;
#pragma omp parallel for schedule(static) reduction(| : changed)
        for (size_t i = 0; i < n; ++i) {
            size_t best = 0;
            float bd = distance2_alloc(rows[i], cent[0], d);
            for (size_t j = 1; j < k; ++j) {
                float dist = distance2_alloc(rows[i], cent[j], d);
                if (dist < bd) {
                    bd = dist;
                    best = j;
                }
            }
            if (best != assign[i]) changed = 1;
            assign[i] = best;
        }
        /* per cluster: scan every assignment, clone the members, mean in data order (serial over j for the draws) */
        for (size_t j0 = 0; j0 < k; j0 += 64) {
            size_t j1 = j0 + 64 < k ? j0 + 64 : k;
            size_t counts[64];
#pragma omp parallel for schedule(dynamic, 1)
            for (size_t j = j0; j < j1; ++j) {
                size_t cnt = 0, cap = 16;
                float **members = (float **)malloc(sizeof(float *) * cap);
                for (size_t i = 0; i < n; ++i)
                    if (assign[i] == j) {
                        if (cnt == cap) {
                            cap *= 2;
                            members = (float **)realloc(members, sizeof(float *) * cap);
                        }
                        members[cnt] = (float *)malloc(sizeof(float) * d); /* the clone */
                        memcpy(members[cnt], rows[i], sizeof(float) * d);
                        ++cnt;
                    }
                if (cnt) {
                    float *sum = (float *)calloc(d, sizeof(float));
                    for (size_t t = 0; t < cnt; ++t)
                        for (size_t c = 0; c < d; ++c) sum[c] = sum[c] + members[t][c];
                    float len = (float)(double)cnt;
                    for (size_t c = 0; c < d; ++c) cent[j][c] = sum[c] / len;
                    free(sum);
                }
                for (size_t t = 0; t < cnt; ++t) free(members[t]);
                free(members);
                counts[j - j0] = cnt;
            }
            for (size_t j = j0; j < j1; ++j)
                if (counts[j - j0] == 0) {
                    uint64_t r = draw ? draw(user, stream, (uint64_t)n) : 0;
                    if (r >= n) r = n - 1;
                    memcpy(cent[j], rows[r], sizeof(float) * d);
                }
        }
        if (!changed) break;
    }
    for (size_t j = 0; j < k; ++j) {
        memcpy(centroids_out + j * d, cent[j], sizeof(float) * d);
        free(cent[j]);
    }
    free(cent);
    free(assign);
    return VQO_OK;
}

int vqo_pq_fit_faithful(const float *data, size_t n, size_t dim, size_t m, size_t k, size_t max_iters,
                        const uint64_t *init_idx, vqo_draw_fn draw, void *user, float *codebooks)
{
    if (n == 0) return fail(VQO_EMPTY_INPUT, "Empty input: at least one vector is required.");
    if (m == 0 || dim < m || dim % m != 0) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: bad m");
    size_t sd = dim / m;
    float **rows = (float **)malloc(sizeof(float *) * n);
    for (size_t s = 0; s < m; ++s) {
        for (size_t i = 0; i < n; ++i) { /* src/pq.rs:110-117: a fresh Vector per row and subspace */
            rows[i] = (float *)malloc(sizeof(float) * sd);
            memcpy(rows[i], data + i * dim + s * sd, sizeof(float) * sd);
        }
        int rc = lbg_faithful(rows, n, sd, k, max_iters, init_idx + s * k, draw, user, s, codebooks + s * k * sd);
        for (size_t i = 0; i < n; ++i) free(rows[i]);
        if (rc) {
            free(rows);
            return rc;
        }
    }
    free(rows);
    return VQO_OK;
}

/* argmin with the stored metric, strict '<' (src/pq.rs:166-174 and the same  */
/* loop at rvq.rs:117-124,190-197; opq.rs:154-161,250-257).                   */
static uint32_t argmin_metric(int metric, double p, const float *x, const float *cb, size_t k,
                              size_t d)
{
    uint32_t best = 0;
    float best_dist = dist_nocheck(metric, p, x, cb, d);
    for (size_t j = 1; j < k; ++j) {
        float dist = dist_nocheck(metric, p, x, cb + j * d, d);
        if (dist < best_dist) {
            best_dist = dist;
            best = (uint32_t)j;
        }
    }
    return best;
}

/* ------------------------------------------------------------------------ */
/* ProductQuantizer::quantize for a batch -- src/pq.rs:146-187 applied to     */
/* each row.  out_f16 (n x dim, binary16 bits) and codes (n x m) are optional.*/
/* Squared-Euclidean and Euclidean use the vectorisable exact form; for       */
/* Euclidean the comparison is still made on sqrtf() values.                  */
/* ------------------------------------------------------------------------ */
int vqo_pq_quantize(const float *codebooks, size_t m, size_t k, size_t sd, int metric, double p,
                    const float *x, size_t n, uint16_t *out_f16, uint32_t *codes,
                    float *out_f32 /* optional n x dim reconstruction in f32 */)
{
    if (metric == VQO_MINKOWSKI && p <= 0.0)
        return fail(VQO_INVALID_METRIC_PARAMETER,
                    "Invalid metric parameter for Minkowski: p must be positive");
    size_t dim = m * sd;
    size_t kp = (k + 15) & ~(size_t)15;
    float *ct = NULL;
    if (metric == VQO_SQUARED_EUCLIDEAN || metric == VQO_EUCLIDEAN) {
        ct = (float *)malloc(sizeof(float) * m * sd * kp);
        for (size_t s = 0; s < m; ++s) transpose_codebook(codebooks + s * k * sd, k, sd, kp, ct + s * sd * kp);
    }
#pragma omp parallel
    {
        float *acc = (float *)malloc(sizeof(float) * kp);
#pragma omp for schedule(static)
        for (size_t i = 0; i < n; ++i) {
            for (size_t s = 0; s < m; ++s) {
                const float *sub = x + i * dim + s * sd;
                const float *cb = codebooks + s * k * sd;
                uint32_t b = ct ? argmin_sq_t(sub, ct + s * sd * kp, sd, k, kp, acc, metric == VQO_EUCLIDEAN)
                                : argmin_metric(metric, p, sub, cb, k, sd);
                if (codes) codes[i * m + s] = b;
                if (out_f16)
                    for (size_t c = 0; c < sd; ++c)
                        out_f16[i * dim + s * sd + c] = vqo_f32_to_f16(cb[b * sd + c]);
                if (out_f32)
                    for (size_t c = 0; c < sd; ++c) out_f32[i * dim + s * sd + c] = cb[b * sd + c];
            }
        }
        free(acc);
    }
    free(ct);
    return VQO_OK;
}

/* ------------------------------------------------------------------------ */
/* ResidualQuantizer::fit -- src/rvq.rs:87-154.                               */
/*   init(user, stage, n, k, out): the stage's `choose_multiple` draw.        */
/*   residuals: n x dim scratch owned by the caller; starts as a copy of the  */
/*   data (103) and ends as the final residuals.                              */
/*   Returns the number of codebooks produced in *stages_out (145).           */
/* The mean residual norm (131-138) is an f32 sum in unspecified order in the */
/* reference; here it is summed in f64 and rounded once.                      */
/* ------------------------------------------------------------------------ */
typedef void (*vqo_init_fn)(void *user, size_t stage, uint64_t n, size_t k, uint64_t *out);

int vqo_rvq_fit(float *residuals, size_t n, size_t dim, size_t stages, size_t k, size_t max_iters,
                float epsilon, int metric, double p, vqo_init_fn init, vqo_draw_fn draw, void *user,
                float *codebooks /* stages x k x dim */, size_t *stages_out, float *avg_norms /* stages or NULL */)
{
    if (n == 0) return fail(VQO_EMPTY_INPUT, "Empty input: at least one vector is required.");
    if (metric == VQO_MINKOWSKI && p <= 0.0)
        return fail(VQO_INVALID_METRIC_PARAMETER,
                    "Invalid metric parameter for Minkowski: p must be positive");
    size_t done = 0;
    uint64_t *idx = (uint64_t *)malloc(sizeof(uint64_t) * (k ? k : 1));
    for (size_t stage = 0; stage < stages; ++stage) { /* 105 */
        float *cb = codebooks + stage * k * dim;
        if (k > 0 && n >= k) init(user, stage, (uint64_t)n, k, idx);
        int rc = vqo_lbg(residuals, n, dim, 0, dim, k, max_iters, idx, draw, user, stage, cb, NULL, NULL);
        if (rc) {
            free(idx);
            return rc;
        }
        ++done;
        double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
        for (size_t i = 0; i < n; ++i) { /* 111-128 */
            float *res = residuals + i * dim;
            uint32_t b = (k < 2) ? 0u : argmin_metric(metric, p, res, cb, k, dim);
            const float *c = cb + (size_t)b * dim;
            float nsq = 0.0f;
            for (size_t t = 0; t < dim; ++t) {
                res[t] = res[t] - c[t];
            }
            for (size_t t = 0; t < dim; ++t) { /* 133-135 */
                float v = res[t] * res[t];
                nsq = nsq + v;
            }
            total += (double)sqrtf(nsq);
        }
        float avg = (float)(total / (double)n);
        if (avg_norms) avg_norms[stage] = avg;
        if (avg < epsilon) break; /* 139-141 */
    }
    free(idx);
    *stages_out = done;
    return VQO_OK;
}

/* ------------------------------------------------------------------------ */
/* ResidualQuantizer::quantize for a batch -- src/rvq.rs:171-215.             */
/* ------------------------------------------------------------------------ */
int vqo_rvq_quantize(const float *codebooks, size_t stages, size_t k, size_t dim, float epsilon,
                     int metric, double p, const float *x, size_t n, uint16_t *out_f16,
                     uint32_t *codes /* n x stages, 0xFFFFFFFF where the early exit skipped */,
                     float *out_f32)
{
    if (metric == VQO_MINKOWSKI && p <= 0.0)
        return fail(VQO_INVALID_METRIC_PARAMETER,
                    "Invalid metric parameter for Minkowski: p must be positive");
#pragma omp parallel
    {
        float *res = (float *)malloc(sizeof(float) * (dim ? dim : 1));
        float *sum = (float *)malloc(sizeof(float) * (dim ? dim : 1));
#pragma omp for schedule(static)
        for (size_t i = 0; i < n; ++i) {
            memcpy(res, x + i * dim, sizeof(float) * dim);
            for (size_t t = 0; t < dim; ++t) sum[t] = 0.0f;
            if (codes)
                for (size_t s = 0; s < stages; ++s) codes[i * stages + s] = 0xFFFFFFFFu;
            for (size_t s = 0; s < stages; ++s) {
                const float *cb = codebooks + s * k * dim;
                uint32_t b = (k < 2) ? 0u : argmin_metric(metric, p, res, cb, k, dim);
                const float *c = cb + (size_t)b * dim;
                if (codes) codes[i * stages + s] = b;
                for (size_t t = 0; t < dim; ++t) sum[t] = sum[t] + c[t]; /* 200-201 */
                for (size_t t = 0; t < dim; ++t) res[t] = res[t] - c[t]; /* 202 */
                float nsq = 0.0f;
                for (size_t t = 0; t < dim; ++t) {
                    float v = res[t] * res[t];
                    nsq = nsq + v;
                }
                if (sqrtf(nsq) < epsilon) break; /* 204-207 */
            }
            if (out_f16)
                for (size_t t = 0; t < dim; ++t) out_f16[i * dim + t] = vqo_f32_to_f16(sum[t]);
            if (out_f32) memcpy(out_f32 + i * dim, sum, sizeof(float) * dim);
        }
        free(res);
        free(sum);
    }
    return VQO_OK;
}

/* ------------------------------------------------------------------------ */
/* y = R * x for each row -- src/opq.rs:186-194, 232-234.  The reference's    */
/* product is nalgebra's (accumulation order unspecified); f32 ascending-j    */
/* accumulation here, compared to the device result with a tolerance.         */
/* rot is row-major dim x dim: y[i] = sum_j rot[i*dim+j] * x[j].              */
/* ------------------------------------------------------------------------ */
void vqo_rotate_rows(const float *rot, size_t dim, const float *x, size_t n, float *y)
{
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n; ++r)
        for (size_t i = 0; i < dim; ++i) {
            float acc = 0.0f;
            for (size_t j = 0; j < dim; ++j) acc += rot[i * dim + j] * x[r * dim + j];
            y[r * dim + i] = acc;
        }
}

/* A = Y * X^T with X, Y dim x n column-major (column j = vector j), i.e.     */
/* A[i][j] = sum_r y_r[i] * x_r[j] -- src/opq.rs:172-179.  f64 accumulation.  */
void vqo_cross_cov(const float *y, const float *x, size_t n, size_t dim, double *a /* dim x dim row-major */)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < dim; ++i)
        for (size_t j = 0; j < dim; ++j) {
            double acc = 0.0;
            for (size_t r = 0; r < n; ++r) acc += (double)y[r * dim + i] * (double)x[r * dim + j];
            a[i * dim + j] = acc;
        }
}

/* ------------------------------------------------------------------------ */
/* ScalarQuantizer -- src/sq.rs:50-76 (fit), 117-127 (quantize_scalar).       */
/* ------------------------------------------------------------------------ */
int vqo_sq_fit(float min, float max, size_t levels, float *step)
{
    if (max <= min) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: max must be greater than min");
    if (levels < 2) return fail(VQO_INVALID_PARAMETER, "Invalid parameter: levels must be at least 2");
    if (levels > 256)
        return fail(VQO_INVALID_PARAMETER, "Invalid parameter: levels must be no more than 256");
    *step = (max - min) / (float)(levels - 1); /* 69 */
    return VQO_OK;
}

static inline size_t f32_as_usize_saturating(float v)
{
    /* Rust `as usize`: NaN -> 0, negative -> 0, too large -> usize::MAX */
    if (!(v == v)) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 18446744073709551616.0f) return (size_t)-1;
    return (size_t)v;
}

void vqo_sq_quantize(float min, float max, size_t levels, float step, const float *x, size_t n,
                     uint8_t *out)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        float v = x[i];
        float clamped = (v < min) ? min : ((v > max) ? max : v); /* 118-124: NaN passes through */
        float q = (clamped - min) / step;
        size_t index = f32_as_usize_saturating(roundf(q)); /* f32::round = half away from zero */
        if (index > levels - 1) index = levels - 1;        /* 126 */
        out[i] = (uint8_t)index;                           /* sq.rs:95,102 `as u8` */
    }
}

/* ------------------------------------------------------------------------ */
/* BinaryQuantizer -- src/bq.rs:46-60 (fit), 94-100 (element rule).           */
/* ------------------------------------------------------------------------ */
int vqo_bq_fit(uint8_t low, uint8_t high)
{
    if (low >= high)
        return fail(VQO_INVALID_PARAMETER,
                    "Invalid parameter: Low quantization level must be less than high quantization level");
    return VQO_OK;
}

void vqo_bq_quantize(float threshold, uint8_t low, uint8_t high, const float *x, size_t n, uint8_t *out)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = (x[i] >= threshold) ? high : low;
}

/* ------------------------------------------------------------------------ */
/* Reconstruction error as the eval harness defines it --                     */
/* src/bin/utils.rs:50-67: mean over vectors of (sum of squared differences / */
/* dim).  f64 accumulation (the reference sums f32 in unspecified order).     */
/* ------------------------------------------------------------------------ */
double vqo_mse_f16(const float *x, const uint16_t *q_f16, size_t n, size_t dim)
{
    double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (size_t i = 0; i < n; ++i) {
        double s = 0.0;
        for (size_t t = 0; t < dim; ++t) {
            uint16_t h = q_f16[i * dim + t];
            uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1f, mnt = h & 0x3ffu, bits;
            if (e == 0) {
                if (mnt == 0) bits = sign;
                else {
                    int sh = 0;
                    while (!(mnt & 0x400u)) { mnt <<= 1; ++sh; }
                    mnt &= 0x3ffu;
                    bits = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | (mnt << 13);
                }
            } else if (e == 0x1f) bits = sign | 0x7f800000u | (mnt << 13);
            else bits = sign | ((e + 112u) << 23) | (mnt << 13);
            float f;
            memcpy(&f, &bits, 4);
            double dd = (double)x[i * dim + t] - (double)f;
            s += dd * dd;
        }
        total += s / (double)dim;
    }
    return total / (double)n;
}

/* ------------------------------------------------------------------------ */
/* Tree-structured VQ -- src/tsvq.rs.                                         */
/* TSVQNode::fit (71-148): centroid = mean_vector of the node's rows: the sum */
/* of the sums of consecutive 1024-row chunks, each chunk added up in data    */
/* order from 0.0.  Up to 1024 rows that is exactly the reference's serial    */
/* branch (src/vector.rs:305-313); above, where the reference reduces in      */
/* parallel in an unspecified order (298-304), it is one admissible order;    */
/* leaf when max_depth == 0 or <= 1 row; variance per dimension = serial f32  */
/* sum of (v - c)^2 in data order (86-98); split dimension = max_by with      */
/* partial_cmp, i.e. the LAST of equal maxima (101-105); median of the sorted */
/* values, mean of the two middle ones for an even count (108-116); stable    */
/* partition v <= median / v > median (119-122); a child exists only when its */
/* side is non-empty and smaller than the node (127-141).  Nodes are numbered */
/* breadth-first, the left child before the right one.                        */
/* A NaN among the values being compared makes the reference panic on         */
/* `partial_cmp(..).unwrap()`; here that is status 105.                       */
/* ------------------------------------------------------------------------ */
#define VQO_NOT_COMPARABLE 105
#define VQO_MEAN_CHUNK 1024

static int cmp_f32(const void *a, const void *b)
{
    const float x = *(const float *)a, y = *(const float *)b;
    return (x > y) - (x < y);
}

int vqo_tsvq_fit(const float *x, size_t n, size_t dim, size_t max_depth, size_t cap_nodes, float *centroids,
                 int32_t *left, int32_t *right, size_t *n_nodes_out)
{
    if (n == 0) return fail(VQO_EMPTY_INPUT, "Empty input: at least one vector is required.");
    typedef struct { size_t start, count, depth; } Seg;
    uint32_t *perm = (uint32_t *)malloc(n * sizeof(uint32_t)), *tmp = (uint32_t *)malloc(n * sizeof(uint32_t));
    Seg *segs = (Seg *)malloc(cap_nodes * sizeof(Seg));
    float *var = (float *)malloc(dim * sizeof(float)), *vals = (float *)malloc(n * sizeof(float));
    int rc = VQO_OK;
    for (size_t i = 0; i < n; ++i) perm[i] = (uint32_t)i;
    size_t n_nodes = 1;
    segs[0].start = 0, segs[0].count = n, segs[0].depth = max_depth;
    for (size_t node = 0; node < n_nodes && rc == VQO_OK; ++node) {
        const Seg sg = segs[node];
        const uint32_t *rows = perm + sg.start;
        float *c = centroids + node * dim;
        left[node] = right[node] = -1;
        for (size_t t = 0; t < dim; ++t) c[t] = 0.0f;
        for (size_t i0 = 0; i0 < sg.count; i0 += VQO_MEAN_CHUNK) {
            const size_t i1 = i0 + VQO_MEAN_CHUNK < sg.count ? i0 + VQO_MEAN_CHUNK : sg.count;
            for (size_t t = 0; t < dim; ++t) var[t] = 0.0f; /* the chunk's sums (var is free until the spreads below) */
            for (size_t i = i0; i < i1; ++i)
                for (size_t t = 0; t < dim; ++t) var[t] = var[t] + x[(size_t)rows[i] * dim + t];
            for (size_t t = 0; t < dim; ++t) c[t] = c[t] + var[t];
        }
        const float len = (float)(double)sg.count;
        for (size_t t = 0; t < dim; ++t) c[t] = c[t] / len;
        if (sg.depth == 0 || sg.count <= 1) continue;
        for (size_t t = 0; t < dim; ++t) var[t] = 0.0f;
        for (size_t i = 0; i < sg.count; ++i)
            for (size_t t = 0; t < dim; ++t) {
                const float diff = x[(size_t)rows[i] * dim + t] - c[t];
                const float sq = diff * diff;
                var[t] = var[t] + sq;
            }
        size_t split = 0;
        for (size_t t = 0; t < dim; ++t) {
            if (var[t] != var[t]) rc = fail(VQO_NOT_COMPARABLE, "values are not comparable (NaN)");
            if (t > 0 && !(var[t] < var[split])) split = t; /* max_by keeps the last of equal maxima */
        }
        if (rc != VQO_OK) break;
        for (size_t i = 0; i < sg.count; ++i) {
            vals[i] = x[(size_t)rows[i] * dim + split];
            if (vals[i] != vals[i]) rc = fail(VQO_NOT_COMPARABLE, "values are not comparable (NaN)");
        }
        if (rc != VQO_OK) break;
        qsort(vals, sg.count, sizeof(float), cmp_f32);
        const float median = (sg.count % 2 == 0) ? (vals[sg.count / 2 - 1] + vals[sg.count / 2]) / 2.0f : vals[sg.count / 2];
        size_t nl = 0, nr = 0;
        for (size_t i = 0; i < sg.count; ++i) {
            if (x[(size_t)rows[i] * dim + split] <= median) tmp[nl++] = rows[i];
        }
        for (size_t i = 0; i < sg.count; ++i) {
            if (!(x[(size_t)rows[i] * dim + split] <= median)) tmp[nl + nr++] = rows[i];
        }
        memcpy(perm + sg.start, tmp, sg.count * sizeof(uint32_t));
        if (nl > 0 && nl < sg.count) {
            if (n_nodes >= cap_nodes) { rc = fail(VQO_INVALID_PARAMETER, "node capacity too small"); break; }
            left[node] = (int32_t)n_nodes;
            segs[n_nodes].start = sg.start, segs[n_nodes].count = nl, segs[n_nodes].depth = sg.depth - 1;
            ++n_nodes;
        }
        if (nr > 0 && nr < sg.count) {
            if (n_nodes >= cap_nodes) { rc = fail(VQO_INVALID_PARAMETER, "node capacity too small"); break; }
            right[node] = (int32_t)n_nodes;
            segs[n_nodes].start = sg.start + nl, segs[n_nodes].count = nr, segs[n_nodes].depth = sg.depth - 1;
            ++n_nodes;
        }
    }
    if (n_nodes_out) *n_nodes_out = n_nodes;
    free(perm), free(tmp), free(segs), free(var), free(vals);
    return rc;
}

/* TSVQ::quantize (src/tsvq.rs:231-249) with quantize_with_distance (162-181): descend towards the child whose centroid is */
/* nearer under the metric, the left one on ties (`<=`), an only child unconditionally; the leaf's centroid as f16.        */
int vqo_tsvq_quantize(const float *centroids, const int32_t *left, const int32_t *right, size_t dim, int metric, double p,
                      const float *x, size_t n, uint16_t *out_f16, uint32_t *leaf_out)
{
    int rc = VQO_OK;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float *v = x + i * dim;
        int32_t node = 0;
        for (;;) {
            const int32_t l = left[node], r = right[node];
            if (l >= 0 && r >= 0) {
                const float dl = dist_nocheck(metric, p, v, centroids + (size_t)l * dim, dim);
                const float dr = dist_nocheck(metric, p, v, centroids + (size_t)r * dim, dim);
                node = (dl <= dr) ? l : r;
            } else if (l >= 0) node = l;
            else if (r >= 0) node = r;
            else break;
        }
        if (leaf_out) leaf_out[i] = (uint32_t)node;
        if (out_f16)
            for (size_t t = 0; t < dim; ++t) out_f16[i * dim + t] = vqo_f32_to_f16(centroids[(size_t)node * dim + t]);
    }
    return rc;
}
