// Small per-block / per-weight kernels around the QR model, used where a quantised tensor is coded without a BF16 seed
// (from a sibling quant, or from nothing but its own statistics): the reference's block_fields, blocks_from_fields,
// intervals, weq and grid_h (seedpack/qr.py:811-878).  One thread per block or weight; they share the block accessors of
// qr_model.cuh with the coder, so a field or a code means the same thing everywhere.
#include "api_util.h"
#include "qr_model.cuh"

namespace sg {
namespace qr {

// the scale fields of every block as integers, nfield(T) per block
__global__ void __launch_bounds__(256) k_block_fields(int T, const uchar* __restrict__ F, long long nblk, int* __restrict__ out) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblk) return;
    int v[34];
    unpack_fields(T, F + b * bs_of(T), v);
    const int nf = nfield(T);
    for (int k = 0; k < nf; ++k) out[b * nf + k] = v[k];
}

// blocks that hold the given fields and all-zero codes
__global__ void __launch_bounds__(32) k_blocks_from_fields(int T, const int* __restrict__ fields, int n, uchar* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n) return;
    uchar* o = out + (long long)k * bs_of(T);
    for (int i = 0; i < bs_of(T); ++i) o[i] = 0;
    int v[34];
    const int nf = nfield(T);
    for (int i = 0; i < nf; ++i) v[i] = fields[(long long)k * nf + i];
    pack_fields(T, o, v);
}

// per weight: the interval of original values that rounds to its code (open towards infinity at the ends of the code range)
__global__ void __launch_bounds__(256) k_intervals(int T, const uchar* __restrict__ F, long long nw, float* __restrict__ lo, float* __restrict__ hi) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nw) return;
    const float INF = __int_as_float(0x7f800000);
    const int qk = qk_of(T), w = (int)(i % qk);
    const uchar* b = F + (i / qk) * bs_of(T);
    int v[34];
    unpack_fields(T, b, v);
    float a, c;
    wscale(T, v, w / sublen_of(T), a, c);
    const int q = get_code(T, b, w);
    float l, h;
    if (nonlin(T)) {
        l = q > 0 ? __fmul_rn(a, 0.5f * (kv(q - 1) + kv(q))) : -INF;
        h = q < 15 ? __fmul_rn(a, 0.5f * (kv(q) + kv(q + 1))) : INF;
        if (a < 0.f) { const float t = l; l = q < 15 ? h : -INF; h = q > 0 ? t : INF; }
        if (a == 0.f) { l = -INF; h = INF; }
    } else {
        const float val = __fadd_rn(__fmul_rn(a, (float)q), c), e = __fmul_rn(fabsf(a), 0.5f);
        l = __fsub_rn(val, e); h = __fadd_rn(val, e);
        const bool lowend = q == qmin_of(T), highend = q == qmax_of(T);
        if (a > 0.f) { if (lowend) l = -INF; if (highend) h = INF; }
        else if (a < 0.f) { if (highend) l = -INF; if (lowend) h = INF; }
        else { l = -INF; h = INF; }
    }
    lo[i] = l; hi[i] = h;
}

// per weight: 1 where its code and its sub-block's integer scale (and min) are the same in both tensors
__global__ void __launch_bounds__(256) k_weight_equal(int T, const uchar* __restrict__ F, const uchar* __restrict__ P, long long nw, uchar* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nw) return;
    const int qk = qk_of(T), w = (int)(i % qk), sub = w / sublen_of(T);
    const uchar* f = F + (i / qk) * bs_of(T);
    const uchar* p = P + (i / qk) * bs_of(T);
    int eq = get_code(T, f, w) == get_code(T, p, w);
    int vf[34], vp[34];
    unpack_fields(T, f, vf); unpack_fields(T, p, vp);
    switch (T) {
        case 10: eq &= vf[2 + sub] == vp[2 + sub] && vf[18 + sub] == vp[18 + sub]; break;
        case 11: case 14: case 23: eq &= vf[1 + sub] == vp[1 + sub]; break;
        case 12: case 13: eq &= vf[2 + sub] == vp[2 + sub] && vf[10 + sub] == vp[10 + sub]; break;
    }
    out[i] = (uchar)eq;
}

// per weight of lattice-type blocks: half the step between the lattice's levels around it
__global__ void __launch_bounds__(256) k_grid_half_step(int T, const uchar* __restrict__ F, long long nw, float* __restrict__ h) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nw) return;
    const uchar* b = F + (i / 256) * bs_of(T);
    int v[34];
    unpack_fields(T, b, v);
    float s, dl;
    gscale(T, b, v, (int)(i % 256) / 8, s, dl);
    h[i] = (T == 19 || T == 29) ? 0.5f * fabsf(s) : fabsf(s);
}

}  // namespace qr
}  // namespace sg

using namespace sg;
using namespace sg::qr;

static bool scalar_type(int T) {
    switch (T) { case 2: case 3: case 6: case 7: case 8: case 10: case 11: case 12: case 13: case 14: case 20: case 23: case 42: return true; }
    return false;
}
static unsigned blocks_for(long long n, int tpb) { return (unsigned)((n + tpb - 1) / tpb); }

extern "C" int sg_qr_block_fields(int device, void* stream, int T, const unsigned char* F, long long nblocks, int* out) {
    if (!(scalar_type(T) || is_grid(T))) return SG_ERR_TYPE;
    if (nblocks < 0 || (nblocks && (!F || !out))) return SG_ERR_ARG;
    if (nblocks == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_block_fields<<<blocks_for(nblocks, 256), 256, 0, (cudaStream_t)stream>>>(T, F, nblocks, out);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_blocks_from_fields(int device, void* stream, int T, const int* fields, int nblocks, unsigned char* out) {
    if (!(scalar_type(T) || is_grid(T))) return SG_ERR_TYPE;
    if (nblocks < 0 || (nblocks && (!fields || !out))) return SG_ERR_ARG;
    if (nblocks == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_blocks_from_fields<<<blocks_for(nblocks, 32), 32, 0, (cudaStream_t)stream>>>(T, fields, nblocks, out);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_intervals(int device, void* stream, int T, const unsigned char* F, long long nweights, float* lo, float* hi) {
    if (!scalar_type(T)) return SG_ERR_TYPE;
    if (nweights < 0 || (nweights && (!F || !lo || !hi))) return SG_ERR_ARG;
    if (nweights == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_intervals<<<blocks_for(nweights, 256), 256, 0, (cudaStream_t)stream>>>(T, F, nweights, lo, hi);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_weight_equal(int device, void* stream, int T, const unsigned char* F, const unsigned char* P, long long nweights,
                                  unsigned char* out) {
    if (!scalar_type(T)) return SG_ERR_TYPE;
    if (nweights < 0 || (nweights && (!F || !P || !out))) return SG_ERR_ARG;
    if (nweights == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_weight_equal<<<blocks_for(nweights, 256), 256, 0, (cudaStream_t)stream>>>(T, F, P, nweights, out);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_grid_half_step(int device, void* stream, int T, const unsigned char* F, long long nweights, float* h) {
    if (!is_grid(T)) return SG_ERR_TYPE;
    if (nweights < 0 || (nweights && (!F || !h))) return SG_ERR_ARG;
    if (nweights == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_grid_half_step<<<blocks_for(nweights, 256), 256, 0, (cudaStream_t)stream>>>(T, F, nweights, h);
    return cuda_ok(cudaGetLastError());
}
