// M30, sibling quantisations of one model without the model itself (seedpack/siblings.py:51-77): the three element-wise
// kernels behind its precision-weighted estimate of a weight from the versions coded so far.  A version gives a value x
// and half a code step h per weight; the estimate is sum(x / h^2) / sum(1 / h^2) with uncertainty sum(1 / h^2)^-1/2,
// handed to the QR coder as an explicit (x, h) seed.  One thread per weight; every operation an explicit IEEE one in the
// reference's order (the estimate decides coded bytes).
#include "api_util.h"

namespace sg {
namespace sib {

// half the interval a weight's code stands for; one infinite side: the distance to the finite one; none: -1 (no information)
__global__ void __launch_bounds__(256) k_half_step(const float* __restrict__ x, const float* __restrict__ lo, const float* __restrict__ hi,
                                                   long long n, float* __restrict__ h) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float l = lo[i], u = hi[i], v = x[i];
    const bool fl = isfinite(l), fu = isfinite(u);
    h[i] = fl && fu ? __fmul_rn(0.5f, __fsub_rn(u, l)) : fu ? __fsub_rn(u, v) : fl ? __fsub_rn(v, l) : -1.f;
}
// one more version into the running sums: ws += 1 / max(h^2, 1e-30), wx += x * that weight; h < 0: the version says nothing
__global__ void __launch_bounds__(256) k_est_add(const float* __restrict__ x, const float* __restrict__ h, long long n, float* ws, float* wx) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float hv = h[i];
    if (hv < 0.f) return;
    const float w = __fdiv_rn(1.f, fmaxf(__fmul_rn(hv, hv), 1e-30f));
    ws[i] = __fadd_rn(ws[i], w);
    wx[i] = __fadd_rn(wx[i], __fmul_rn(x[i], w));
}
// the explicit seed (x, h) pairs; a weight no version told anything about: the first version's value with h = 0
__global__ void __launch_bounds__(256) k_est_seed(const float* __restrict__ ws, const float* __restrict__ wx, const float* __restrict__ x0,
                                                  long long n, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float s = ws[i];
    if (s > 0.f) { out[2 * i] = __fdiv_rn(wx[i], s); out[2 * i + 1] = __fdiv_rn(1.f, __fsqrt_rn(s)); }
    else { out[2 * i] = x0[i]; out[2 * i + 1] = 0.f; }
}

static unsigned grid_for(long long n) { return (unsigned)((n + 255) / 256); }

}  // namespace sib
}  // namespace sg

using namespace sg;

extern "C" int sg_sib_half_step(int device, void* stream, const float* x, const float* lo, const float* hi, long long n, float* h) {
    if (n < 0 || (n && (!x || !lo || !hi || !h))) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    if (n > 0x7fffffffLL * 256) return SG_ERR_LIMIT;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    sib::k_half_step<<<sib::grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, lo, hi, n, h);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_sib_est_add(int device, void* stream, const float* x, const float* h, long long n, float* ws, float* wx) {
    if (n < 0 || (n && (!x || !h || !ws || !wx))) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    if (n > 0x7fffffffLL * 256) return SG_ERR_LIMIT;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    sib::k_est_add<<<sib::grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, h, n, ws, wx);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_sib_est_seed(int device, void* stream, const float* ws, const float* wx, const float* x0, long long n, float* out) {
    if (n < 0 || (n && (!ws || !wx || !x0 || !out))) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    if (n > 0x7fffffffLL * 256) return SG_ERR_LIMIT;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    sib::k_est_seed<<<sib::grid_for(n), 256, 0, (cudaStream_t)stream>>>(ws, wx, x0, n, out);
    return cuda_ok(cudaGetLastError());
}
