// backend.hpp -- the device operations and the collective the training loops are written against.
//
// The LBG / RVQ / OPQ loops (driver.cpp) hold the control flow of the reference
// (src/utils.rs:32-109, src/rvq.rs:87-154, src/opq.rs:90-205) and call the
// operations below for everything that touches rows of data.  The shipped
// library implements `Device` with sm_100a kernels (cuda_device.cu) and `Comm`
// with NCCL (nccl_comm.cpp).  There is no other implementation in the library.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace vqb {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &msg) : std::runtime_error(msg), code(c) {}
};

// One (subspace, cluster) slot that takes the bits of one data row: the initial
// sample (src/utils.rs:54) and the empty-cluster re-seed (src/utils.rs:100).
struct RowPatch {
    uint32_t subspace;
    uint32_t cluster;
    uint64_t row; // GLOBAL row index
};

// n_local rows of `ld` floats; subspace s covers columns [s*sd, (s+1)*sd); k centroids per subspace.
struct Shape {
    size_t n_local = 0, ld = 0, m = 0, sd = 0, k = 0;
};

// What one k-means iteration gathers on the device, in ONE allocation so that one all-reduce covers it:
//   sums[m][k][sd] f32 | counts[m][k] | moved[m]
// counts hold u32 values, or f32 values when counts_f32 is set (exact below 2^24 rows, which lets the three parts
// travel as a single f32 all-reduce).  moved[s] is zero or has the bits of 1.0f OR-ed in (non-zero either way; a sum of
// such words over ranks read as f32 stays non-zero).  The buffer starts zero-filled; update_centroids hands it back
// zero-filled.
struct IterBuffers {
    float *sums = nullptr;
    uint32_t *counts = nullptr;
    uint32_t *moved = nullptr;
    bool counts_f32 = false;
    size_t words(const Shape &sh) const { return sh.m * sh.k * sh.sd + sh.m * sh.k + sh.m; }
};

// What the host learns from one iteration (src/utils.rs:76-80,95-106): which subspaces saw a row move and which
// (subspace, cluster) slots received no row.
struct IterStatus {
    std::vector<uint8_t> moved;          // [m]
    std::vector<uint8_t> has_empty;      // [m]
    std::vector<uint32_t> empty_bits;    // [m][ceil(k / 32)], bit j of subspace s = cluster j is empty
};

// One direct exchange of iteration buffers between the GPUs of a node (peer_exchange.cuh has the protocol): where every
// rank's buffer of this exchange and every rank's arrival flags are mapped in this process.
constexpr int MAX_PEERS = 8;
struct PeerExchange {
    int world = 0, rank = 0;
    uint32_t epoch = 0;
    const uint32_t *words[MAX_PEERS] = {};
    uint32_t *flags[MAX_PEERS] = {};
    uint32_t *stale = nullptr; // this rank's buffer of the previous exchange
};

class Comm {
  public:
    virtual ~Comm() {}
    virtual int rank() const = 0;
    virtual int world() const = 0;
    // In-place all-reduce over device buffers, ordered on the device's stream.
    virtual void allreduce_sum_f32(float *buf, size_t n) = 0;
    virtual void allreduce_sum_f64(double *buf, size_t n) = 0;
    virtual void allreduce_sum_u32(uint32_t *buf, size_t n) = 0;
    virtual void allreduce_max_u32(uint32_t *buf, size_t n) = 0;
    virtual void allreduce_sum_u64(uint64_t *buf, size_t n) = 0;
    // Optional: iteration buffers that every GPU of the node can read, so that the centroid-update kernel does the
    // all-reduce itself.  peer_window (collective; every rank passes the same size) returns two zero-filled buffers of
    // `words` 32-bit words in this rank's window, or false when the ranks cannot map each other's memory.
    // peer_exchange(which) (same call order on every rank) numbers the next exchange, whose data every rank gathered in
    // its buffer `which`.
    virtual bool peer_window(size_t words, uint32_t *local[2])
    {
        (void)words;
        (void)local;
        return false;
    }
    virtual PeerExchange peer_exchange(int which)
    {
        (void)which;
        return PeerExchange();
    }
    virtual uint64_t peer_exchanges() const { return 0; } // direct exchanges numbered so far
    // Collectives issued between group_begin() and group_end() may be fused into one launch.
    virtual void group_begin() {}
    virtual void group_end() {}
};

class Device {
  public:
    virtual ~Device() {}
    // ---- memory (device side of the boundary) ----
    virtual void *alloc(size_t bytes) = 0;
    virtual void release(void *p) = 0;
    virtual void upload(void *dst, const void *src, size_t bytes) = 0;   // host -> device, complete on return
    virtual void download(void *dst, const void *src, size_t bytes) = 0; // device -> host, complete on return
    virtual void copy(void *dst, const void *src, size_t bytes) = 0;     // device -> device
    virtual void zero(void *dst, size_t bytes) = 0;
    virtual size_t code_bytes(size_t k) const = 0; // bytes per stored assignment for k centroids

    // centroids[patch.subspace][patch.cluster][:] = x[patch.row - row_begin][subspace columns] for
    // every patch; rows outside [row_begin, row_begin + n_local) come from the rank that owns them
    // (bit patterns are exchanged with a max-reduce over zero-filled slots, so -0.0 and NaN payloads survive).
    virtual void patch_centroids(const Shape &sh, const float *x, uint64_t row_begin, const RowPatch *patches,
                                 size_t n_patches, float *centroids, Comm *comm) = 0;
    // Called once per lbg_fit before the first assignment: `x` stays unchanged until the next call, so the device
    // may precompute per-row data (the tensor-core path keeps row norms).  Default: nothing.
    virtual void prepare_rows(const Shape &sh, const float *x)
    {
        (void)sh;
        (void)x;
    }
    // Rows that are still being copied in from the caller's host buffer when the fit starts.  arriving_pieces(x) is the
    // number of pieces in which the rows at `x` arrive (0: they are all there).  await_piece(x, i) makes the device's queue
    // wait for piece i and returns the row at which that piece ends; the first iteration of lbg_fit then works through the
    // rows piece by piece behind the copies.  Pieces arrive in order.  Default: nothing is ever in flight.
    virtual size_t arriving_pieces(const float *x)
    {
        (void)x;
        return 0;
    }
    virtual size_t await_piece(const float *x, size_t piece)
    {
        (void)x, (void)piece;
        return 0;
    }
    // One-sided Jacobi sweeps on the device, until no pair of columns rotates.  gt / vt (host, n x n, f64) hold the
    // working matrix G = A V and V TRANSPOSED (row p = column p), and are updated in place.  Returns false when the
    // device does not take the shape; the caller then runs the sweeps on the host.  Default: host.
    virtual bool svd_sweeps(double *gt, double *vt, size_t n)
    {
        (void)gt;
        (void)vt;
        (void)n;
        return false;
    }
    // rot_dev (device, n x n row-major f32) = V U^T of the SVD a = U S V^T (src/opq.rs:180-183), computed on the device from
    // a_dev (device, n x n row-major f64) as the orthogonal polar factor of a^T.  Returns false when the device does not take
    // the shape or the iteration did not converge (rank-deficient a); the caller then runs the Jacobi SVD.  Default: false.
    virtual bool polar_rotation(const double *a_dev, size_t n, float *rot_dev)
    {
        (void)a_dev;
        (void)n;
        (void)rot_dev;
        return false;
    }
    // Nearest centroid under squared Euclidean (src/utils.rs:59-73); codes are read as the previous
    // assignment and overwritten; buf.moved[s] becomes non-zero if any row of subspace s moved (76-80).
    // Subspaces with active[s] == 0 are left untouched.
    virtual void assign_train(const Shape &sh, const float *x, const float *centroids, void *codes,
                              const uint32_t *active, const IterBuffers &buf) = 0;
    // buf.sums[s][j][:] += the rows assigned to (s, j), buf.counts[s][j] += how many (src/utils.rs:83-92,
    // src/vector.rs:297-314); the buffer comes in zero-filled.  ordered = ascending row order per cluster.
    virtual void accumulate(const Shape &sh, const float *x, const void *codes, const uint32_t *active,
                            bool ordered, const IterBuffers &buf) = 0;
    // Optional short cut for all but the first iteration: `local` holds the sums and counts of THIS rank's rows under the
    // assignment codes_prev; bring it up to date with `codes` by moving only the rows whose code changed (add to the new
    // cluster, subtract from the old one; counts likewise).  After a few iterations a small part of the rows still moves,
    // so this touches a fraction of what a full pass adds up.  The order of the additions is as unspecified as in the full
    // pass (src/vector.rs:298-304 for the clusters this mode is used on).  On return codes_prev equals codes in every active
    // subspace, so the next iteration needs no copy of the assignments.  Returns false, having changed nothing, when the device
    // does not take the shape; the caller then clears `local` and accumulates all rows.
    virtual bool accumulate_moved(const Shape &sh, const float *x, void *codes_prev, const void *codes, const uint32_t *active,
                                  const IterBuffers &local)
    {
        (void)sh, (void)x, (void)codes_prev, (void)codes, (void)active, (void)local;
        return false;
    }
    // centroids = sums / (counts as f32) where counts > 0 (src/vector.rs:315-316), active subspaces only; reports
    // the iteration's flags to the host (complete on return) and clears the buffer for the next iteration.
    // With `px` the buffer holds this rank's part only (u32 counts) and the kernel adds the parts of all ranks itself; it
    // then clears px->stale instead of `buf`.
    virtual void update_centroids(const Shape &sh, const IterBuffers &buf, const uint32_t *active, float *centroids,
                                  IterStatus &status, const PeerExchange *px = nullptr) = 0;
    // Residual update of one RVQ stage (src/rvq.rs:111-138): argmin with `metric`, res -= centroid in place,
    // *norm_sum += sum over rows of sqrt(sum res^2) (f64, device scalar, not cleared here).
    virtual void rvq_update(float *res, size_t n, size_t dim, const float *centroids, size_t k, int metric,
                            double p, double *norm_sum) = 0;
    // PQ encode (src/pq.rs:159-186 per row; also the OPQ reconstruction src/opq.rs:146-168 via out_f32).
    virtual void pq_encode(const Shape &sh, const float *x, const float *codebooks, int metric, double p,
                           uint16_t *out_f16, uint32_t *out_codes, float *out_f32) = 0;
    // y[r] = R * x[r] (src/opq.rs:186-194, 232-234); R row-major dim x dim.
    virtual void rotate_rows(const float *rot, size_t dim, const float *x, size_t n, float *y) = 0;
    // a[i][j] += sum_r y[r][i] * x[r][j]  (A = Y * X^T, src/opq.rs:172-179), f64 dim x dim, cleared here.
    virtual void cross_cov(const float *y, const float *x, size_t n, size_t dim, double *a) = 0;
};

// ---- training loops (driver.cpp) ------------------------------------------------------------

typedef uint64_t (*DrawFn)(void *user, size_t stream, uint64_t n);
typedef void (*InitFn)(void *user, size_t stage, uint64_t n, size_t k, uint64_t *out);
typedef void (*RestartFn)(void *user);

struct LbgResult {
    size_t iterations[1];
};

// Batched lbg_quantize over the m subspaces of `sh` (m == 1, sd == ld for a full-width run).
// init_idx: m x k global row indices.  stream0: draw-stream id of subspace 0 (subspace s asks stream0 + s).
// centroids: device, m x k x sd, written.  iterations: host, m entries (may be null).
void lbg_fit(Device &dev, Comm *comm, const Shape &sh, const float *x, size_t max_iters, const uint64_t *init_idx,
             DrawFn draw, void *user, size_t stream0, int flags, float *centroids, size_t *iterations);

// src/rvq.rs:87-154.  res: device copy of the data, overwritten with the final residuals.
// codebooks: device, stages x k x dim.  Returns the number of stages produced.
size_t rvq_fit(Device &dev, Comm *comm, float *res, size_t n_local, size_t dim, size_t stages, size_t k,
               size_t max_iters, float epsilon, int metric, double p, InitFn init, DrawFn draw, void *user,
               int flags, float *codebooks);

// src/opq.rs:90-205.  x: device original rows; rotation: HOST dim x dim row-major out; codebooks: device m x k x sd.
// Returns false when opq_iters == 0 (identity rotation, no codebooks).
bool opq_fit(Device &dev, Comm *comm, const float *x, size_t n_local, size_t dim, size_t m, size_t k,
             size_t max_iters, size_t opq_iters, int metric, double p, const uint64_t *init_idx, DrawFn draw,
             RestartFn restart, void *user, int flags, float *rotation_host, float *codebooks);

// Thin one-sided Jacobi SVD of a square matrix (f64): a = u * diag(s) * v^T, all row-major n x n.
// With a device the sweeps run there (Device::svd_sweeps) when it takes the shape.
// v0 (optional, orthogonal n x n): where the sweeps start; the factors satisfy a = u diag(s) v^T either way.
void jacobi_svd(const double *a, size_t n, double *u, double *s, double *v, Device *dev = nullptr, const double *v0 = nullptr);

} // namespace vqb
