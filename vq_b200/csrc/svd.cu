// svd.cu -- the sweeps of the one-sided (Hestenes) Jacobi SVD behind OPQ's Procrustes step (src/opq.rs:180-183, where the
// reference calls nalgebra's SVD) on the device.
//
// One CTA of 1024 threads.  A sweep visits all n(n-1)/2 column pairs in the round-robin (tournament) order: n - 1 steps of n/2
// disjoint pairs, one team of 1024 / (n/2) threads per pair (n = 64 or 128).  The working matrices G = A V and V are held transposed (row p =
// column p) in global memory and read / written past the L1 cache, so a step sees what the previous step wrote after one
// __syncthreads.  The sweeps end when no pair rotated (|g_p . g_q| <= 1e-15 |g_p| |g_q| for all pairs) or after 60 sweeps;
// singular values, U and the completion of a rank-deficient U are computed by the caller from the converged G.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "cuda_device.hpp"

namespace vqb {

namespace {

template <int EPT> // elements of a row per thread = n / (threads per pair)
__global__ void __launch_bounds__(1024, 1) jacobi_sweeps_kernel(double *gt, double *vt, int n, int *sweeps_out)
{
    __shared__ int rotated_any;
    const int pairs = n / 2;
    const int team = 1024 / pairs;            // threads per pair: a power of two between 8 and 32 (and at most a warp)
    const int pr = threadIdx.x / team, tl = threadIdx.x % team;
    const unsigned lane = threadIdx.x & 31u;
    const unsigned team_mask = (team == 32) ? 0xffffffffu : (((1u << team) - 1u) << (lane & ~(unsigned)(team - 1)));
    const double eps = 1e-15;
    int sweep = 0;
    for (; sweep < 60; ++sweep) {
        if (threadIdx.x == 0) rotated_any = 0;
        __syncthreads();
        for (int step = 0; step < n - 1; ++step) {
            // round-robin pairing of 0 .. n-1: player n-1 stays, the others rotate
            int p, q;
            if (pr == 0) {
                p = n - 1;
                q = step;
            } else {
                p = (step + pr) % (n - 1);
                q = (step - pr + (n - 1)) % (n - 1);
            }
            if (p > q) {
                const int t = p;
                p = q;
                q = t;
            }
            double *gp = gt + (size_t)p * n, *gq = gt + (size_t)q * n;
            double *vp = vt + (size_t)p * n, *vq = vt + (size_t)q * n;
            // this thread's elements of the two G rows stay in registers from the dot products to the rotation
            double ga[EPT], gb[EPT];
#pragma unroll
            for (int e = 0; e < EPT; ++e) {
                const int i = tl + e * team;
                ga[e] = __ldcg(gp + i), gb[e] = __ldcg(gq + i);
            }
            double alpha = 0.0, beta = 0.0, gamma = 0.0;
#pragma unroll
            for (int e = 0; e < EPT; ++e) {
                alpha += ga[e] * ga[e];
                beta += gb[e] * gb[e];
                gamma += ga[e] * gb[e];
            }
            for (int o = team >> 1; o > 0; o >>= 1) {
                alpha += __shfl_xor_sync(team_mask, alpha, o);
                beta += __shfl_xor_sync(team_mask, beta, o);
                gamma += __shfl_xor_sync(team_mask, gamma, o);
            }
            // the rotation's parameters: f64 square roots and divisions are slow, so one thread of the team computes them
            double c = 1.0, sn = 0.0;
            int rot = 0;
            if (tl == 0 && !(fabs(gamma) <= eps * sqrt(alpha * beta) || gamma == 0.0)) {
                rot = 1;
                const double zeta = (beta - alpha) / (2.0 * gamma);
                const double t = (zeta >= 0 ? 1.0 : -1.0) / (fabs(zeta) + sqrt(1.0 + zeta * zeta));
                c = 1.0 / sqrt(1.0 + t * t);
                sn = c * t;
            }
            const int src = (int)(lane & ~(unsigned)(team - 1));
            rot = __shfl_sync(team_mask, rot, src);
            c = __shfl_sync(team_mask, c, src);
            sn = __shfl_sync(team_mask, sn, src);
            if (rot) {
                if (tl == 0) rotated_any = 1;
#pragma unroll
                for (int e = 0; e < EPT; ++e) {
                    const int i = tl + e * team;
                    const double va = __ldcg(vp + i), vb = __ldcg(vq + i);
                    __stcg(gp + i, c * ga[e] - sn * gb[e]);
                    __stcg(gq + i, sn * ga[e] + c * gb[e]);
                    __stcg(vp + i, c * va - sn * vb);
                    __stcg(vq + i, sn * va + c * vb);
                }
            }
            __syncthreads(); // the rows written in this step are read by other teams in the next
        }
        if (!rotated_any) break;
        __syncthreads();
    }
    if (threadIdx.x == 0) *sweeps_out = sweep;
}

} // namespace

bool CudaDevice::svd_sweeps(double *gt, double *vt, size_t n)
{
    // n = 64 or 128: n/2 pairs, teams of 32 or 16 threads inside one warp, 2 or 8 elements of each row per thread
    if (n != 64 && n != 128) return false;
    const size_t bytes = sizeof(double) * n * n;
    double *g_d = static_cast<double *>(alloc(bytes)), *v_d = static_cast<double *>(alloc(bytes));
    int *sw_d = static_cast<int *>(alloc(sizeof(int)));
    upload(g_d, gt, bytes);
    upload(v_d, vt, bytes);
    {
        KernelScope ks(*this, "jacobi_sweeps");
        if (n == 64) jacobi_sweeps_kernel<2><<<1, 1024, 0, stream_>>>(g_d, v_d, (int)n, sw_d);
        else jacobi_sweeps_kernel<8><<<1, 1024, 0, stream_>>>(g_d, v_d, (int)n, sw_d);
        VQB_CUDA_CHECK(cudaGetLastError());
        count_launch();
    }
    download(gt, g_d, bytes);
    download(vt, v_d, bytes);
    release(g_d), release(v_d), release(sw_d);
    return true;
}

} // namespace vqb

// ------------------------------------------------------------------------------------------------
// The rotation without the SVD.  src/opq.rs:180-183 takes A = U S V^T and sets R = V U^T.  Since A^T = (V U^T)(U S U^T), that R
// is the orthogonal polar factor of A^T, which is unique when A has full rank and does not depend on how an SVD orders or signs
// its vectors.  The Newton-Schulz iteration
//        X_0 = A^T / sqrt(|A|_1 |A|_inf),      X_{k+1} = X_k (1.5 I - 0.5 X_k^T X_k)
// drives every singular value of X (all in (0, 1] at the start) to 1 and leaves the singular vectors alone, so it converges to
// that factor: linearly (x 1.5 per step) while a singular value is small, then quadratically.  All of it is 128 x 128 x 128 f64
// products on the device: no download of A, no sweeps on one SM.
//
// polar_iterate_kernel runs the whole iteration in ONE cooperative launch (one CTA per 16 x 16 tile, all resident; its own
// bounded barrier between the two products of a step; the residual max|X^T X - I| is looked at on the device after every
// step).  While the singular values are spread it uses, instead of (1.5, 0.5), the odd cubic a x - b x^3 that maps the current
// interval [l, 1] of singular values into the narrowest interval [l', 1] (l' is known in closed form, so every CTA follows the
// same sequence); small singular values then grow by up to 2.6 instead of 1.5 per step.  The interval starts at l = 1e-4, a
// guess: a smaller true value only means the last steps run with the plain coefficients.  One launch and about 16 steps
// replace some 25 steps of three stream operations each and a host round trip every eighth step (1.23 -> 0.37 ms at n = 128).
// The step-by-step kernels below remain for matrices whose tiles cannot all be resident.  If the iteration has not converged
// after 96 steps (rank-deficient or extremely ill-conditioned A) the caller falls back to the Jacobi SVD, which also
// completes a null space.
// ------------------------------------------------------------------------------------------------
namespace vqb {

namespace {

constexpr int POLAR_TILE = 16;
constexpr double POLAR_TOL = 1e-13;

// scale^2 = |a|_1 |a|_inf (largest column sum times largest row sum of |a|), an upper bound of the largest singular value squared
// that is within a small factor of it
__global__ void polar_scale_kernel(const double *a, int n, double *scale2)
{
    __shared__ double red[256];
    double best_row = 0.0, best_col = 0.0;
    for (int t = threadIdx.x; t < n; t += 256) {
        double r = 0.0, c = 0.0;
        for (int u = 0; u < n; ++u) {
            r += fabs(a[(size_t)t * n + u]);
            c += fabs(a[(size_t)u * n + t]);
        }
        best_row = fmax(best_row, r);
        best_col = fmax(best_col, c);
    }
    red[threadIdx.x] = best_row;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    const double rmax = red[0];
    __syncthreads();
    red[threadIdx.x] = best_col;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    if (threadIdx.x == 0) *scale2 = rmax * red[0];
}

// x[i][j] = a[j][i] / sqrt(scale2)
__global__ void polar_init_kernel(const double *a, int n, const double *scale2, double *x)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n * n) return;
    const int i = t / n, j = t % n;
    const double f = sqrt(*scale2);
    x[t] = (f > 0.0 && f == f) ? a[(size_t)j * n + i] / f : 0.0;
}

// b = x^T x, and *resid = max |b - I| (bits of a non-negative double, so an integer max orders them)
__global__ void __launch_bounds__(POLAR_TILE *POLAR_TILE) polar_gram_kernel(const double *x, int n, double *b, unsigned long long *resid)
{
    __shared__ double xa[POLAR_TILE][POLAR_TILE + 1], xb[POLAR_TILE][POLAR_TILE + 1];
    const int tx = threadIdx.x % POLAR_TILE, ty = threadIdx.x / POLAR_TILE;
    const int i = blockIdx.y * POLAR_TILE + ty, j = blockIdx.x * POLAR_TILE + tx; // b[i][j] = sum_r x[r][i] x[r][j]
    double acc = 0.0;
    for (int r0 = 0; r0 < n; r0 += POLAR_TILE) {
        xa[ty][tx] = x[(size_t)(r0 + ty) * n + blockIdx.y * POLAR_TILE + tx]; // rows r0.., columns of the i block
        xb[ty][tx] = x[(size_t)(r0 + ty) * n + blockIdx.x * POLAR_TILE + tx]; // rows r0.., columns of the j block
        __syncthreads();
#pragma unroll
        for (int r = 0; r < POLAR_TILE; ++r) acc = fma(xa[r][ty], xb[r][tx], acc);
        __syncthreads();
    }
    b[(size_t)i * n + j] = acc;
    const double dev = fabs(acc - (i == j ? 1.0 : 0.0));
    atomicMax(resid, (unsigned long long)__double_as_longlong(dev == dev ? dev : 1e300));
}

// y = 1.5 x - 0.5 x b    (y = x once the residual of this step's b is below the tolerance)
__global__ void __launch_bounds__(POLAR_TILE *POLAR_TILE) polar_update_kernel(const double *x, const double *b, int n, const unsigned long long *resid, double *y)
{
    __shared__ double xs[POLAR_TILE][POLAR_TILE + 1], bs[POLAR_TILE][POLAR_TILE + 1];
    const int tx = threadIdx.x % POLAR_TILE, ty = threadIdx.x / POLAR_TILE;
    const int i = blockIdx.y * POLAR_TILE + ty, j = blockIdx.x * POLAR_TILE + tx;
    if (__longlong_as_double((long long)*resid) < POLAR_TOL) {
        y[(size_t)i * n + j] = x[(size_t)i * n + j];
        return;
    }
    double acc = 0.0;
    for (int r0 = 0; r0 < n; r0 += POLAR_TILE) {
        xs[ty][tx] = x[(size_t)i * n + r0 + tx];
        bs[ty][tx] = b[(size_t)(r0 + ty) * n + j];
        __syncthreads();
#pragma unroll
        for (int r = 0; r < POLAR_TILE; ++r) acc = fma(xs[ty][r], bs[r][tx], acc);
        __syncthreads();
    }
    y[(size_t)i * n + j] = 1.5 * x[(size_t)i * n + j] - 0.5 * acc;
}

// ---- the whole iteration in one cooperative launch ---------------------------------------------
struct PolarWork {
    double *x0, *x1, *b;             // n x n each
    unsigned long long *resid;       // [max_steps + 1] bits of max |X^T X - I| per step, zero on entry
    unsigned int *arrivals;          // grid barrier counter, zero on entry
    int *status;                     // [0] 1 = converged, 0 = not, -1 = a barrier wait ran out; [1] steps taken
};

// All threads of all CTAs call this the same number of times; `round` counts the calls from 1.  Bounded: a CTA that does not
// see the others arrive gives up, records -1 and every later call returns false at once.
__device__ __forceinline__ bool polar_grid_barrier(const PolarWork &w, unsigned int round, unsigned int ctas, int *failed_sh)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(w.arrivals, 1u);
        const unsigned int target = round * ctas;
        unsigned int i = 0;
        while ((int)(*reinterpret_cast<volatile unsigned int *>(w.arrivals) - target) < 0) {
            if (++i > (1u << 26) || *reinterpret_cast<volatile int *>(w.status) < 0) {
                *reinterpret_cast<volatile int *>(w.status) = -1;
                *failed_sh = 1;
                break;
            }
        }
        __threadfence();
    }
    __syncthreads();
    return *failed_sh == 0;
}

__global__ void __launch_bounds__(POLAR_TILE *POLAR_TILE) polar_iterate_kernel(const double *a, int n, PolarWork w, float *rot, int max_steps, double l0)
{
    __shared__ double sa[POLAR_TILE][POLAR_TILE + 1], sb[POLAR_TILE][POLAR_TILE + 1];
    __shared__ double red[POLAR_TILE * POLAR_TILE];
    __shared__ int failed_sh;
    const int tx = threadIdx.x % POLAR_TILE, ty = threadIdx.x / POLAR_TILE;
    const int i = blockIdx.y * POLAR_TILE + ty, j = blockIdx.x * POLAR_TILE + tx;
    const unsigned int ctas = gridDim.x * gridDim.y;
    unsigned int round = 0;
    if (threadIdx.x == 0) failed_sh = 0;
    // scale^2 = |a|_1 |a|_inf, computed by every CTA for itself (the same value everywhere)
    double best_row = 0.0, best_col = 0.0;
    for (int t = threadIdx.x; t < n; t += POLAR_TILE * POLAR_TILE) {
        double r = 0.0, c = 0.0;
        for (int u = 0; u < n; ++u) {
            r += fabs(__ldcg(a + (size_t)t * n + u));
            c += fabs(__ldcg(a + (size_t)u * n + t));
        }
        best_row = fmax(best_row, r);
        best_col = fmax(best_col, c);
    }
    red[threadIdx.x] = best_row;
    __syncthreads();
    for (int o = POLAR_TILE * POLAR_TILE / 2; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    const double rmax = red[0];
    __syncthreads();
    red[threadIdx.x] = best_col;
    __syncthreads();
    for (int o = POLAR_TILE * POLAR_TILE / 2; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    const double f = sqrt(rmax * red[0]);
    __syncthreads();
    double *cur = w.x0, *nxt = w.x1;
    cur[(size_t)i * n + j] = (f > 0.0 && f == f) ? __ldcg(a + (size_t)j * n + i) / f : 0.0; // X_0 = A^T / f
    if (!polar_grid_barrier(w, ++round, ctas, &failed_sh)) return;
    double l = l0, resid = 1.0;
    int step = 0;
    for (; step <= max_steps; ++step) {
        // b = cur^T cur, tile (i-block, j-block), and the step's residual
        double acc = 0.0;
        for (int r0 = 0; r0 < n; r0 += POLAR_TILE) {
            sa[ty][tx] = __ldcg(cur + (size_t)(r0 + ty) * n + blockIdx.y * POLAR_TILE + tx);
            sb[ty][tx] = __ldcg(cur + (size_t)(r0 + ty) * n + blockIdx.x * POLAR_TILE + tx);
            __syncthreads();
#pragma unroll
            for (int r = 0; r < POLAR_TILE; ++r) acc = fma(sa[r][ty], sb[r][tx], acc);
            __syncthreads();
        }
        w.b[(size_t)i * n + j] = acc;
        const double dev = fabs(acc - (i == j ? 1.0 : 0.0));
        red[threadIdx.x] = dev == dev ? dev : 1e300;
        __syncthreads();
        for (int o = POLAR_TILE * POLAR_TILE / 2; o > 0; o >>= 1) {
            if ((int)threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
            __syncthreads();
        }
        if (threadIdx.x == 0) atomicMax(w.resid + step, (unsigned long long)__double_as_longlong(red[0]));
        if (!polar_grid_barrier(w, ++round, ctas, &failed_sh)) return;
        resid = __longlong_as_double((long long)__ldcg(w.resid + step));
        if (resid < POLAR_TOL || step == max_steps) break; // the same value in every CTA
        // coefficients: the cubic that maps [l, 1] into the narrowest [l', 1]; (1.5, 0.5) once l has reached 1
        double ca = 1.5, cb = 0.5;
        if (l < 0.999) {
            const double s = 1.0 + l + l * l, xs = sqrt(s / 3.0);
            const double pa = 2.0 / ((2.0 / 3.0) * xs + 1.0 - 1.0 / s), pe = (2.0 * pa / 3.0) * xs - 1.0;
            ca = pa / (1.0 + pe);
            cb = pa / s / (1.0 + pe);
            l = (1.0 - pe) / (1.0 + pe);
        }
        // nxt = ca cur - cb cur b, tile (i-block, j-block)
        acc = 0.0;
        for (int r0 = 0; r0 < n; r0 += POLAR_TILE) {
            sa[ty][tx] = __ldcg(cur + (size_t)i * n + r0 + tx);
            sb[ty][tx] = __ldcg(w.b + (size_t)(r0 + ty) * n + j);
            __syncthreads();
#pragma unroll
            for (int r = 0; r < POLAR_TILE; ++r) acc = fma(sa[ty][r], sb[r][tx], acc);
            __syncthreads();
        }
        nxt[(size_t)i * n + j] = ca * __ldcg(cur + (size_t)i * n + j) - cb * acc;
        if (!polar_grid_barrier(w, ++round, ctas, &failed_sh)) return;
        double *t = cur;
        cur = nxt;
        nxt = t;
    }
    rot[(size_t)i * n + j] = (float)__ldcg(cur + (size_t)i * n + j);
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
        w.status[0] = resid < 1e-11 ? 1 : 0;
        w.status[1] = step;
    }
}

__global__ void polar_finish_kernel(const double *x, int count, float *rot)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < count) rot[t] = (float)x[t];
}

} // namespace

bool CudaDevice::polar_rotation(const double *a_dev, size_t n, float *rot_dev)
{
    if (n == 0 || n % POLAR_TILE != 0 || n > 512) return false;
    const size_t bytes = sizeof(double) * n * n;
    const int max_steps = 96;
    {
        // one cooperative launch when every tile's CTA can be resident at once
        int per_sm = 0, coop = 0, dev_id = 0;
        cudaGetDevice(&dev_id);
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev_id);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, polar_iterate_kernel, POLAR_TILE * POLAR_TILE, 0);
        const size_t ctas = (n / POLAR_TILE) * (n / POLAR_TILE);
        if (coop && (size_t)per_sm * (size_t)sm_count() >= ctas && std::getenv("VQB_POLAR_STEPWISE") == nullptr) {
            const size_t extra = sizeof(unsigned long long) * (max_steps + 2) + 64;
            unsigned char *blk = static_cast<unsigned char *>(alloc(3 * bytes + extra));
            PolarWork w;
            w.x0 = reinterpret_cast<double *>(blk);
            w.x1 = w.x0 + n * n;
            w.b = w.x1 + n * n;
            w.resid = reinterpret_cast<unsigned long long *>(blk + 3 * bytes);
            w.arrivals = reinterpret_cast<unsigned int *>(w.resid + max_steps + 2);
            w.status = reinterpret_cast<int *>(w.arrivals + 2);
            int status[2] = {0, 0};
            {
                KernelScope ks(*this, "polar_rotation");
                VQB_CUDA_CHECK(cudaMemsetAsync(w.resid, 0, extra, stream_));
                const dim3 grid((unsigned)(n / POLAR_TILE), (unsigned)(n / POLAR_TILE));
                int n_i = (int)n, steps_i = max_steps;
                double l0 = 1e-4;
                void *args[] = {(void *)&a_dev, (void *)&n_i, (void *)&w, (void *)&rot_dev, (void *)&steps_i, (void *)&l0};
                VQB_CUDA_CHECK(cudaLaunchCooperativeKernel((const void *)polar_iterate_kernel, grid, dim3(POLAR_TILE * POLAR_TILE), args, 0, stream_));
                count_launch();
            }
            download(status, w.status, sizeof status);
            release(blk);
            if (status[0] < 0) throw Error(100, "polar rotation: a wait between the steps ran out");
            return status[0] == 1;
        }
    }
    double *x0 = static_cast<double *>(alloc(bytes)), *x1 = static_cast<double *>(alloc(bytes)), *b = static_cast<double *>(alloc(bytes));
    double *fro2 = static_cast<double *>(alloc(sizeof(double)));
    unsigned long long *resid = static_cast<unsigned long long *>(alloc(sizeof(unsigned long long) * 2));
    const int count = (int)(n * n);
    const dim3 grid((unsigned)(n / POLAR_TILE), (unsigned)(n / POLAR_TILE));
    const int batch = 8; // x 1.5 per step while a singular value is small: down to 1e-16 of the largest
    double *cur = x0, *nxt = x1;
    double r = 1.0;
    {
        KernelScope ks(*this, "polar_rotation");
        polar_scale_kernel<<<1, 256, 0, stream_>>>(a_dev, (int)n, fro2);
        polar_init_kernel<<<(count + 255) / 256, 256, 0, stream_>>>(a_dev, (int)n, fro2, cur);
        count_launch(2);
        for (int s0 = 0; s0 < max_steps && !(r < 1e-11); s0 += batch) {
            for (int s = 0; s < batch; ++s) {
                VQB_CUDA_CHECK(cudaMemsetAsync(resid, 0, sizeof(unsigned long long), stream_));
                polar_gram_kernel<<<grid, POLAR_TILE * POLAR_TILE, 0, stream_>>>(cur, (int)n, b, resid);
                polar_update_kernel<<<grid, POLAR_TILE * POLAR_TILE, 0, stream_>>>(cur, b, (int)n, resid, nxt);
                count_launch(2);
                std::swap(cur, nxt);
            }
            // the residual of the current iterate; the host looks at it once per batch of steps
            VQB_CUDA_CHECK(cudaMemsetAsync(resid, 0, sizeof(unsigned long long), stream_));
            polar_gram_kernel<<<grid, POLAR_TILE * POLAR_TILE, 0, stream_>>>(cur, (int)n, b, resid);
            count_launch();
            unsigned long long bits = 0;
            download(&bits, resid, sizeof bits);
            std::memcpy(&r, &bits, sizeof r);
        }
        polar_finish_kernel<<<(count + 255) / 256, 256, 0, stream_>>>(cur, count, rot_dev);
        count_launch();
        VQB_CUDA_CHECK(cudaGetLastError());
    }
    release(x0), release(x1), release(b), release(fro2), release(resid);
    return r < 1e-11;
}

} // namespace vqb
