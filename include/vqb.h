/*
 * vqb.h -- C ABI of libvqb.so: the B200 (sm_100a) implementation of the
 * quantizer hot path of the Rust crate `vq` (habedi/vq).
 *
 * The reference has no FFI of its own; its boundary is the public Rust API.
 * Each entry point below names the reference item it stands behind
 * ("file:line" inside the reference source tree).  A Rust facade keeps the
 * reference signatures (`fit(&[Vector<f32>], ..., Distance, seed)`,
 * `quantize(&Vector<f32>) -> Vector<f16|u8>`), packs rows into one contiguous
 * row-major buffer, draws row indices with its own `StdRng`, and maps the
 * status codes back to the reference's panics.
 *
 * Conventions
 *   - every function returns an int status (0 = success) and never throws or
 *     aborts; vqb_last_error() gives the message, which for codes 1..4 is the
 *     reference's `VqError` Display text (src/exceptions.rs:9-25);
 *   - data pointers (`x`, outputs) may be HOST or DEVICE pointers of the
 *     context's GPU; the library detects which and copies when needed;
 *   - one context per (process, GPU); multi-GPU runs use one process per GPU,
 *     each holding the rows of its shard (contiguous blocks in rank order);
 *   - there is no CPU fallback: without a usable GPU vqb_ctx_create fails.
 *   - a context (and the quantizers made from it) may be used from several
 *     host threads, one call at a time per context (calls are serialised by an
 *     internal lock), matching the reference's `Send + Sync` plain-data types.
 */
#ifndef VQB_H
#define VQB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define VQB_OK 0
#define VQB_ERR_EMPTY_INPUT 1              /* VqError::EmptyInput              exceptions.rs:15-16 */
#define VQB_ERR_INVALID_PARAMETER 2        /* VqError::InvalidParameter        exceptions.rs:19-20 */
#define VQB_ERR_DIMENSION_MISMATCH 3       /* VqError::DimensionMismatch       exceptions.rs:11-12 */
#define VQB_ERR_INVALID_METRIC_PARAMETER 4 /* VqError::InvalidMetricParameter  exceptions.rs:23-24 */
#define VQB_ERR_BAD_ARGUMENT 90            /* NULL handle / pointer, bad enum value */
#define VQB_ERR_CUDA 100
#define VQB_ERR_NCCL 101
#define VQB_ERR_NO_DEVICE 102
#define VQB_ERR_UNSUPPORTED 103
#define VQB_ERR_CALLBACK 104
#define VQB_ERR_NOT_COMPARABLE 105         /* a NaN where the reference calls partial_cmp(..).unwrap() (src/tsvq.rs:104,109) */

/* ---- Distance (src/distances.rs:73-88) --------------------------------- */
enum vqb_metric {
    VQB_SQUARED_EUCLIDEAN = 0,
    VQB_EUCLIDEAN = 1,
    VQB_COSINE = 2,
    VQB_MANHATTAN = 3,
    VQB_CHEBYSHEV = 4,
    VQB_MINKOWSKI = 5, /* uses the `p` argument; result agrees with the reference to powf rounding only */
    VQB_HAMMING = 6
};

/* ---- fit flags --------------------------------------------------------- */
#define VQB_ACCUM_AUTO 0    /* ordered when the global row count is <= 65536, else fast */
#define VQB_ACCUM_ORDERED 1 /* cluster sums in ascending row order == src/vector.rs:305-313 (bit-exact on one GPU) */
#define VQB_ACCUM_FAST 2    /* shared-memory atomics; order unspecified, like src/vector.rs:298-304 */

typedef struct vqb_ctx vqb_ctx;
typedef struct vqb_pq vqb_pq;
typedef struct vqb_rvq vqb_rvq;
typedef struct vqb_opq vqb_opq;

/* Row index in [0, n) that re-seeds an empty cluster: `data.choose(&mut rng)`
 * (src/utils.rs:100).  `stream` = PQ/OPQ subspace or RVQ stage, i.e. which of
 * the reference's per-call RNGs (`seed + i`) is asked.  Called in ascending
 * cluster order within an iteration.  In a multi-process run every rank is
 * called identically and must return identical values. */
typedef uint64_t (*vqb_draw_fn)(void *user, size_t stream, uint64_t n);

/* The k distinct row indices of `data.choose_multiple(&mut rng, k)`
 * (src/utils.rs:54) for RVQ stage `stage`, written to out[0..k). */
typedef void (*vqb_init_fn)(void *user, size_t stage, uint64_t n, size_t k, uint64_t *out);

/* ---- context ----------------------------------------------------------- */
const char *vqb_version(void);
/* Creates the context on CUDA device `device` (streams, scratch). */
int vqb_ctx_create(int device, vqb_ctx **out);
int vqb_ctx_destroy(vqb_ctx *ctx);
/* Message of the last failing call on `ctx` (or of the last failing call on
 * this thread that had no context, when ctx == NULL). */
const char *vqb_last_error(const vqb_ctx *ctx);
/* Run all work of `ctx` on the caller's CUDA stream (cudaStream_t).  NULL is the
 * CUDA default stream (what a framework's "current stream" usually is), NOT "no
 * stream": work is then ordered with everything else on that stream. */
int vqb_ctx_set_stream(vqb_ctx *ctx, void *cuda_stream);
/* Back to the context's own (non-blocking) stream, the state after creation. */
int vqb_ctx_reset_stream(vqb_ctx *ctx);
/* Waits for the context's stream.  Also the place where a caller that passes DEVICE outputs (and therefore never
 * triggers a download) learns that a tensor-core kernel gave up on one of its bounded waits: VQB_ERR_CUDA with a message. */
int vqb_ctx_synchronize(vqb_ctx *ctx);
/* Number of kernels this context has launched so far. */
int vqb_ctx_launch_count(const vqb_ctx *ctx, uint64_t *out);
/* How many times this context has asked CUDA for device or pinned memory so far (cudaMalloc, cudaMallocAsync,
 * cudaHostAlloc).  No counterpart in the reference; lets an embedder (and the tests) check that a call allocated nothing. */
int vqb_ctx_alloc_count(const vqb_ctx *ctx, uint64_t *out);

/* Per-kernel timing with CUDA events on the launching stream (off by default; the reference times
 * with std::time::Instant around whole calls, src/bin/eval_pq.rs:42-44,50-60).  The report is JSON:
 * {"kernel name": {"launches": L, "ms": total}, ...}; reading it clears the record. */
int vqb_ctx_timing(vqb_ctx *ctx, int enable);
int vqb_ctx_timing_report(vqb_ctx *ctx, char *buf, size_t cap);

/* ---- multi-GPU (one process per GPU; the reference has no counterpart, it is a single-process rayon program).
 * Once per LBG iteration the centroid sums, counts and moved flags of all ranks are added.  Ranks of one node that can
 * map each other's memory (up to 8; CUDA IPC over NVLink) do this inside the centroid-update kernel, which reads every
 * rank's part with peer loads and adds them in rank order; otherwise one NCCL all-reduce runs before that kernel.
 * VQB_PEER_EXCHANGE=0 in the environment selects NCCL.  Either way all ranks end with bit-identical codebooks. */
#define VQB_UNIQUE_ID_BYTES 128
int vqb_comm_unique_id(uint8_t *out /* VQB_UNIQUE_ID_BYTES */);
int vqb_comm_init(vqb_ctx *ctx, const uint8_t *unique_id, int rank, int world);
int vqb_comm_destroy(vqb_ctx *ctx);
/* Number of iterations so far whose parts were added by the update kernel itself (0: NCCL did all of them). */
int vqb_comm_exchange_count(const vqb_ctx *ctx, uint64_t *out);

/* ---- Distance::compute, row-wise on the GPU (src/distances.rs:115-172):
 * out[i] = distance(a[i*d .. ), b[i*d .. )) for i < n.  da != db reproduces
 * the reference's DimensionMismatch. ------------------------------------- */
int vqb_distance_rows(vqb_ctx *ctx, int metric, double p, const float *a, size_t da, const float *b,
                      size_t db, size_t n, float *out);

/* ---- TSVQ (src/tsvq.rs) --------------------------------------------------------------------------------------
 * vqb_tsvq_fit: TSVQ::new (205-211) -> TSVQNode::fit (71-148), nodes numbered breadth-first (left child before right).
 * vqb_tsvq_quantize: TSVQ::quantize (231-249): n x dim binary16 leaf centroids; leaf_out (optional): the leaf's node id.
 * vqb_tsvq_tree: centroids nodes x dim, left / right child ids (-1 = none).  The tree is built on one GPU. */
typedef struct vqb_tsvq vqb_tsvq;
int vqb_tsvq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t max_depth, int metric, double p, vqb_tsvq **out);
int vqb_tsvq_quantize(vqb_tsvq *t, const float *x, size_t n, size_t dim, uint16_t *out_f16, uint32_t *leaf_out);
int vqb_tsvq_shape(const vqb_tsvq *t, size_t *nodes, size_t *dim);
int vqb_tsvq_tree(const vqb_tsvq *t, float *centroids_out, int32_t *left_out, int32_t *right_out);
int vqb_tsvq_destroy(vqb_tsvq *t);

/* ---- evaluation metrics of the reference's harness, computed on the device --------------------------------
 * mse_out: mean squared reconstruction error, calculate_reconstruction_error (src/bin/utils.rs:50-67);
 * recall_out: recall@k over at most 1000 evenly spaced queries, each searched in a 5000-row window when n > 10000,
 * calculate_recall (src/bin/utils.rs:70-127).  q_f16: the n x dim binary16 output of a quantize call.  1 <= k <= 32. */
int vqb_evaluate_f16(vqb_ctx *ctx, const float *x, const uint16_t *q_f16, size_t n, size_t dim, size_t k,
                     float *mse_out, float *recall_out);

/* Diagnostic for the tensor-core path used by full-width k-means (residual quantizer): the raw tcgen05 TF32 dot
 * products x_r . c_j (dots_out: n x 256, columns >= k are 0; may be NULL) and shortlist statistics
 * stats_out[3] = {rows, shortlisted candidates, rows that needed a full exact scan}.  Requires 32 <= dim <= 128,
 * dim % 32 == 0, 2 <= k <= 256.  No counterpart in the reference. */
int vqb_dense_dots(vqb_ctx *ctx, const float *x, size_t n, size_t dim, const float *codebook, size_t k,
                   float *dots_out, unsigned long long *stats_out);

/* The two dense contractions of OptimizedProductQuantizer::fit as calls of their own (they run inside vqb_opq_fit and
 * vqb_opq_quantize; exposed so that their accuracy can be checked against f64):
 *   vqb_opq_rotate_rows   y[r] = R x[r]                  src/opq.rs:186-194, 232-234   rot: dim x dim row-major
 *   vqb_opq_cross_cov     a = sum_r y[r] x[r]^T (f64)     src/opq.rs:172-179            a_out: dim x dim row-major
 * For 32 <= dim <= 128 in steps of 32 both run on the tensor cores with split-TF32 operands (f32-level accuracy); other
 * widths take the FP32 kernels.  Pointers may be host or device. */
int vqb_opq_rotate_rows(vqb_ctx *ctx, const float *rot, size_t dim, const float *x, size_t n, float *y_out);
int vqb_opq_cross_cov(vqb_ctx *ctx, const float *y, const float *x, size_t n, size_t dim, double *a_out);

/* Diagnostic for the tensor-core path of the product quantizer (sub-space width 8): the raw split-TF32 scores
 * |c_j|^2/2 - x.c_j (scores_out: n x m x 256, may be NULL), the codes the path produces (codes_out: n x m) and the number
 * of (row, sub-space) pairs it left to the exact scan.  Requires m % 4 == 0, 4 <= m <= 64, 2 <= k <= 256.
 * No counterpart in the reference. */
int vqb_pq_tensor_scores(vqb_ctx *ctx, const float *x, size_t n, size_t m, const float *codebooks, size_t k,
                         float *scores_out, uint32_t *codes_out, unsigned long long *marked_out);

/* ---- lbg_quantize (src/utils.rs:32-109) on `n` rows of width d:
 * init_idx = k row indices, centroids_out = k x d (host or device). ------- */
int vqb_lbg_fit(vqb_ctx *ctx, const float *x, size_t n, size_t d, size_t k, size_t max_iters,
                const uint64_t *init_idx, vqb_draw_fn draw, void *user, int flags,
                float *centroids_out, size_t *iterations_out /* may be NULL */);

/* ---- ProductQuantizer (src/pq.rs) -------------------------------------- */
/* ProductQuantizer::fit, src/pq.rs:79-129.  x: this rank's n x dim rows.
 * init_idx: m x k GLOBAL row indices (subspace-major).  `metric`/`p` are only
 * stored, as in the reference. */
int vqb_pq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t m, size_t k,
               size_t max_iters, int metric, double p, const uint64_t *init_idx, vqb_draw_fn draw,
               void *user, int flags, vqb_pq **out);
/* A quantizer over given codebooks (m x k x sub_dim, f32) -- what the fields
 * of `ProductQuantizer` hold after fit (src/pq.rs:52-61). */
int vqb_pq_from_codebooks(vqb_ctx *ctx, const float *codebooks, size_t m, size_t k, size_t sub_dim,
                          int metric, double p, vqb_pq **out);
/* ProductQuantizer::quantize for n rows, src/pq.rs:146-187.  `dim` is the row
 * width the caller has (checked against m*sub_dim, 147-156).  out_f16: n x dim
 * IEEE binary16 bits (may be NULL); codes: n x m chosen centroid indices (may
 * be NULL; not returned by the reference, exposed for parity checks). */
int vqb_pq_quantize(vqb_pq *pq, const float *x, size_t n, size_t dim, uint16_t *out_f16,
                    uint32_t *codes);
int vqb_pq_shape(const vqb_pq *pq, size_t *m, size_t *k, size_t *sub_dim);
int vqb_pq_codebooks(const vqb_pq *pq, float *out /* m x k x sub_dim */);
/* LBG iterations each subspace ran (<= max_iters), out[m]. */
int vqb_pq_iterations(const vqb_pq *pq, size_t *out);
int vqb_pq_destroy(vqb_pq *pq);

/* ---- ResidualQuantizer (src/rvq.rs) ------------------------------------ */
/* ResidualQuantizer::fit, src/rvq.rs:87-154. */
int vqb_rvq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t stages, size_t k,
                size_t max_iters, float epsilon, int metric, double p, vqb_init_fn init,
                vqb_draw_fn draw, void *user, int flags, vqb_rvq **out);
int vqb_rvq_from_codebooks(vqb_ctx *ctx, const float *codebooks, size_t stages, size_t k, size_t dim,
                           float epsilon, int metric, double p, vqb_rvq **out);
/* ResidualQuantizer::quantize for n rows, src/rvq.rs:171-215.  codes: n x
 * stages, 0xFFFFFFFF for stages skipped by the per-row early exit (204-207). */
int vqb_rvq_quantize(vqb_rvq *rvq, const float *x, size_t n, size_t dim, uint16_t *out_f16,
                     uint32_t *codes);
int vqb_rvq_shape(const vqb_rvq *rvq, size_t *stages, size_t *k, size_t *dim);
int vqb_rvq_codebooks(const vqb_rvq *rvq, float *out /* stages x k x dim */);
int vqb_rvq_destroy(vqb_rvq *rvq);

/* ---- OptimizedProductQuantizer (src/opq.rs) ---------------------------- */
/* OptimizedProductQuantizer::fit, src/opq.rs:90-205.  init_idx (m x k) and the
 * draw streams are re-used by every outer iteration, as the reference re-seeds
 * with `seed + i` each time (opq.rs:140); `restart(user)` (may be NULL) is
 * called at the start of each outer iteration so the host can reset its RNGs. */
typedef void (*vqb_restart_fn)(void *user);
int vqb_opq_fit(vqb_ctx *ctx, const float *x, size_t n, size_t dim, size_t m, size_t k,
                size_t max_iters, size_t opq_iters, int metric, double p, const uint64_t *init_idx,
                vqb_draw_fn draw, vqb_restart_fn restart, void *user, int flags, vqb_opq **out);
int vqb_opq_from_parts(vqb_ctx *ctx, const float *rotation /* dim x dim row-major */,
                       const float *codebooks, size_t m, size_t k, size_t sub_dim, int metric, double p,
                       vqb_opq **out);
/* OptimizedProductQuantizer::quantize for n rows, src/opq.rs:222-264. */
int vqb_opq_quantize(vqb_opq *opq, const float *x, size_t n, size_t dim, uint16_t *out_f16,
                     uint32_t *codes);
/* OPQ encode that allocates nothing.  No counterpart in the reference (which has no device memory to manage).
 * For embedders that own all of HBM through their own pool, or that must not enter the CUDA allocator from a
 * request loop: the rotated rows that vqb_opq_quantize keeps in pool memory live here in a fixed array inside
 * the library image (VQB_OPQ_STATIC_MAX_FLOATS floats = 4 MiB, resident on every GPU that loads the library,
 * for the life of the process), and the nearest-centroid step runs on the CUDA-core kernels, which work out of
 * shared memory and registers (the tensor-core kernel of vqb_opq_quantize needs operand tiles and a mark map in
 * device memory).  The call makes no cudaMalloc / cudaMallocAsync / cudaFree and creates no event, on its first
 * use of a context as on any later one (vqb_ctx_alloc_count stays unchanged across it).
 *   - x, out_f16 and codes must be DEVICE pointers (either output may be NULL, not both); host pointers are
 *     refused because staging them would allocate;
 *   - n * dim must not exceed VQB_OPQ_STATIC_MAX_FLOATS, otherwise VQB_ERR_UNSUPPORTED with a message;
 *   - per-kernel timing (vqb_ctx_timing) must be off;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress); make that first
 *     call before starting any stream capture;
 *   - all calls, from all quantizers of the process, share the one array per GPU and it keeps whatever the last
 *     call wrote; each call overwrites the part it reads, so nothing needs clearing, but two calls whose GPU work
 *     overlaps (different streams or contexts on one GPU) race on it -- keep them on one stream.
 * Results are identical to vqb_opq_quantize. */
#define VQB_OPQ_STATIC_MAX_FLOATS (1u << 20)
int vqb_opq_quantize_static(vqb_opq *opq, const float *x, size_t n, size_t dim, uint16_t *out_f16,
                            uint32_t *codes);
int vqb_opq_shape(const vqb_opq *opq, size_t *m, size_t *k, size_t *sub_dim);
int vqb_opq_rotation(const vqb_opq *opq, float *out /* dim x dim row-major */);
int vqb_opq_codebooks(const vqb_opq *opq, float *out /* m x k x sub_dim */);
int vqb_opq_destroy(vqb_opq *opq);

/* ---- ScalarQuantizer (src/sq.rs) --------------------------------------- */
/* ScalarQuantizer::fit, src/sq.rs:50-76: validates and returns `step`. */
int vqb_sq_fit(float min, float max, size_t levels, float *step_out);
/* ScalarQuantizer::quantize over n_elems contiguous f32 values (any number of
 * vectors back to back), src/sq.rs:89-106 + quantize_scalar 117-127. */
int vqb_sq_quantize(vqb_ctx *ctx, float min, float max, size_t levels, float step, const float *x,
                    size_t n_elems, uint8_t *out);

/* ---- BinaryQuantizer (src/bq.rs) --------------------------------------- */
/* BinaryQuantizer::fit, src/bq.rs:46-60: validates low < high. */
int vqb_bq_fit(float threshold, uint8_t low, uint8_t high);
/* BinaryQuantizer::quantize over n_elems contiguous values, src/bq.rs:75-104. */
int vqb_bq_quantize(vqb_ctx *ctx, float threshold, uint8_t low, uint8_t high, const float *x,
                    size_t n_elems, uint8_t *out);

#ifdef __cplusplus
}
#endif
#endif /* VQB_H */
