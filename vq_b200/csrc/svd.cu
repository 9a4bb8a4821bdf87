// svd.cu -- the sweeps of the one-sided (Hestenes) Jacobi SVD behind OPQ's Procrustes step (src/opq.rs:180-183, where the
// reference calls nalgebra's SVD) on the device.
//
// One CTA of 1024 threads.  A sweep visits all n(n-1)/2 column pairs in the round-robin (tournament) order: n - 1 steps of n/2
// disjoint pairs, one team of 1024 / (n/2) threads per pair (n = 64 or 128).  The working matrices G = A V and V are held transposed (row p =
// column p) in global memory and read / written past the L1 cache, so a step sees what the previous step wrote after one
// __syncthreads.  The sweeps end when no pair rotated (|g_p . g_q| <= 1e-15 |g_p| |g_q| for all pairs) or after 60 sweeps;
// singular values, U and the completion of a rank-deficient U are computed by the caller from the converged G.
#include <algorithm>

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
