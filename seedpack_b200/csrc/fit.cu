// Deterministic float64 reductions and small solves behind the importance fit (seedpack/imxfit.py:36-75) and other
// decisions the reference wants identical on every machine (seedpack/detmath.py:76-153): sums of a float64 matrix
// along its rows, batched Gram matrices X X^T and products X y with float64 accumulation in index order, and batched
// linear systems of at most 16 unknowns by Gaussian elimination with partial pivoting.  One thread per output, the
// terms of a sum added one after the other in index order (a float64 sum depends on its order; the fit's eigenvectors
// and the blocks they then reproduce depend on these sums).
#include "api_util.h"
#include "common.cuh"

namespace sg {
namespace fit {

// sum over t of f(t), t = 0 .. n - 1, strictly in that order
template <class F> SG_DEVINL double ordered_sum(long long n, F term) {
    double acc = 0.0;
    for (long long t = 0; t < n; ++t) acc = acc + term(t);
    return acc;
}

__global__ void __launch_bounds__(256) k_rows_f64(const double* __restrict__ x, long long nr, long long nc, int square, double* __restrict__ out) {
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nr) return;
    const double* p = x + r * nc;
    out[r] = square ? ordered_sum(nc, [&](long long j) { return p[j] * p[j]; }) : ordered_sum(nc, [&](long long j) { return p[j]; });
}

// out[c][a][b] = sum_t X[c][a][t] X[c][b][t]
__global__ void __launch_bounds__(256) k_gram(const float* __restrict__ X, long long nb, int k, long long d, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nb * k * k) return;
    const long long c = i / ((long long)k * k);
    const int a = (int)((i / k) % k), b = (int)(i % k);
    const float* xa = X + (c * k + a) * d;
    const float* xb = X + (c * k + b) * d;
    out[i] = (float)ordered_sum(d, [&](long long t) { return (double)xa[t] * (double)xb[t]; });
}

// out[c][a] = sum_t X[c][a][t] y[c][t]
__global__ void __launch_bounds__(256) k_bdot(const float* __restrict__ X, const float* __restrict__ y, long long nb, int k, long long d,
                                              float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nb * k) return;
    const float* xa = X + i * d;
    const float* yc = y + (i / k) * d;
    out[i] = (float)ordered_sum(d, [&](long long t) { return (double)xa[t] * (double)yc[t]; });
}

// A[c] x = b[c], k <= 16: the augmented matrix in float64, pivot = the largest magnitude of the column (the first
// such row on ties), elimination row by row from the pivot's column on, back substitution from the last row up
__global__ void __launch_bounds__(64) k_solve(const float* __restrict__ A, const float* __restrict__ b, long long nb, int k, float* __restrict__ x) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nb) return;
    double m[16][17];
    for (int r = 0; r < k; ++r) {
        for (int q = 0; q < k; ++q) m[r][q] = (double)A[(c * k + r) * k + q];
        m[r][k] = (double)b[c * k + r];
    }
    for (int col = 0; col < k; ++col) {
        int best = col;
        for (int r = col + 1; r < k; ++r) if (fabs(m[r][col]) > fabs(m[best][col])) best = r;
        if (best != col)
            for (int q = 0; q <= k; ++q) { const double t = m[col][q]; m[col][q] = m[best][q]; m[best][q] = t; }
        const double pivot = m[col][col];
        for (int r = col + 1; r < k; ++r) {
            const double f = m[r][col] / pivot;
            for (int q = col; q <= k; ++q) m[r][q] = m[r][q] - f * m[col][q];
        }
    }
    for (int r = k - 1; r >= 0; --r) {
        double s = m[r][k];
        for (int q = r + 1; q < k; ++q) s = s - m[r][q] * m[q][k];
        m[r][k] = s / m[r][r];
    }
    for (int r = 0; r < k; ++r) x[c * k + r] = (float)m[r][k];
}

}  // namespace fit
}  // namespace sg

using namespace sg;

static unsigned grid_of(long long n, int tpb) { return (unsigned)((n + tpb - 1) / tpb); }

extern "C" int sg_dm_rows_f64(int device, void* stream, const double* x, long long nr, long long nc, int square, double* out) {
    if (nr < 0 || nc < 0 || (nr && (!x || !out))) return SG_ERR_ARG;
    if (nr == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    fit::k_rows_f64<<<grid_of(nr, 256), 256, 0, (cudaStream_t)stream>>>(x, nr, nc, square, out);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_dm_gram(int device, void* stream, const float* X, long long nb, int k, long long d, float* out) {
    if (nb < 0 || k < 0 || d < 0 || (nb && k && (!X || !out))) return SG_ERR_ARG;
    if (nb == 0 || k == 0) return SG_OK;
    if (nb * k * k > 0x7fffffffLL * 256) return SG_ERR_LIMIT;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    fit::k_gram<<<grid_of(nb * k * k, 256), 256, 0, (cudaStream_t)stream>>>(X, nb, k, d, out);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_dm_bdot(int device, void* stream, const float* X, const float* y, long long nb, int k, long long d, float* out) {
    if (nb < 0 || k < 0 || d < 0 || (nb && k && (!X || !y || !out))) return SG_ERR_ARG;
    if (nb == 0 || k == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    fit::k_bdot<<<grid_of(nb * k, 256), 256, 0, (cudaStream_t)stream>>>(X, y, nb, k, d, out);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_dm_solve(int device, void* stream, const float* A, const float* b, long long nb, int k, float* x) {
    if (nb < 0 || k < 0 || (nb && k && (!A || !b || !x))) return SG_ERR_ARG;
    if (k > 16) return SG_ERR_LIMIT;
    if (nb == 0 || k == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    fit::k_solve<<<grid_of(nb, 64), 64, 0, (cudaStream_t)stream>>>(A, b, nb, k, x);
    return cuda_ok(cudaGetLastError());
}
