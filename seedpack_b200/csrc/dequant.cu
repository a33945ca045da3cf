// Dequantisers: ggml blocks -> float32, the arithmetic of dequantize_row_<type> (ggml-quants.c:419-589, 961-1968,
// 2489-2766), one thread per weight.  Replaces k_dq_<type> (seedpack/gpuquant.py:215-219).  Used where a quantised
// tensor stands in for missing weights (seeds) and by the importance-matrix fit; a minor, write-bound path
// (4 bytes out per weight).  The bit layouts come from the same locators the residual coder uses.
#include "api_util.h"
#include "qr_model.cuh"
#include "quant_extra.cuh"
#include "quant_iq.cuh"

namespace sg {

using namespace qr;

SG_DEVINL float iq4_level(int i) { return kv(i); }
SG_DEVINL float lattice_value(int T, int level) {          // dequantisation value of a lattice coordinate
    switch (T) {
        case 16: case 17: case 22: return level == 0 ? 8.f : level == 1 ? 25.f : 43.f;
        case 18: return level == 7 ? 62.f : (float)(4 + 8 * level);
        case 21: return (float)(2 * level + 1);
    }
    return (float)(level - 1);                              // IQ1_S / IQ1_M
}

__global__ void __launch_bounds__(256) k_dequant(int T, const uchar* __restrict__ y, float* __restrict__ x, long long n,
                                                 const uint16_t* __restrict__ gk) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int qk = qk_of(T), bs = bs_of(T);
    const uchar* b = y + (i / qk) * bs;
    const int w = (int)(i % qk);
    int v[MAXF];
    unpack_fields(T, b, v);
    const float d = f16_to_f32((uint16_t)v[0]);
    float out;
    if (!is_grid(T)) {
        const int c = get_code(T, b, w);
        switch (T) {
            case 2: out = fmul((float)(c - 8), d); break;
            case 3: out = fadd(fmul((float)c, d), f16_to_f32((uint16_t)v[1])); break;
            case 6: out = fmul((float)(c - 16), d); break;
            case 7: out = fadd(fmul((float)c, d), f16_to_f32((uint16_t)v[1])); break;
            case 8: out = fmul((float)c, d); break;
            case 42: out = fmul((float)(c - 1), d); break;
            case 10: { const int s = w >> 4; out = fsub(fmul(fmul(d, (float)v[2 + s]), (float)c), fmul(f16_to_f32((uint16_t)v[1]), (float)v[18 + s])); break; }
            case 11: { const int s = w >> 4; out = fmul(fmul(d, (float)(v[1 + s] - 32)), (float)(c - 4)); break; }
            case 12: case 13: { const int s = w >> 5; out = fsub(fmul(fmul(d, (float)v[2 + s]), (float)c), fmul(f16_to_f32((uint16_t)v[1]), (float)v[10 + s])); break; }
            case 14: { const int s = w >> 4; out = fmul(fmul(d, (float)v[1 + s]), (float)(c - 32)); break; }
            case 20: out = fmul(d, iq4_level(c)); break;
            case 23: out = fmul(fmul(d, (float)(v[1 + (w >> 5)] - 32)), iq4_level(c)); break;
            default: out = 0.f;
        }
    } else {
        const int B = (T == 18 || T == 21) ? 3 : 2, N = (T == 18 || T == 21) ? 4 : 8;
        const int g = w / N;                                                    // lattice group of the weight
        const int level = (gk[get_gidx(T, b, g)] >> (B * (w % N))) & ((1 << B) - 1);
        const float gv = lattice_value(T, level);
        const float sign = get_neg(T, b, w) ? -1.f : 1.f;
        switch (T) {
            case 16: out = fmul(fmul(fmul(fmul(d, fadd(0.5f, (float)v[1 + (w >> 5)])), 0.25f), gv), sign); break;
            case 17: case 22: out = fmul(fmul(fmul(fmul(d, fadd(0.5f, (float)v[1 + (w >> 4)])), 0.25f), gv), sign); break;
            case 18: out = fmul(fmul(fmul(fmul(d, fadd(0.5f, (float)v[1 + (w >> 5)])), 0.5f), gv), sign); break;
            case 21: out = fmul(fmul(fmul(d, (float)(1 + 2 * v[1 + (w >> 5)])), gv), sign); break;
            case 19: { const int f = v[1 + (w >> 5)]; out = fmul(fmul(d, (float)(2 * (f & 7) + 1)), fadd(gv, (f & 8) ? -0.125f : 0.125f)); break; }
            default: { const int f = v[1 + (w >> 4)];                           // IQ1_M
                       out = fmul(fmul(d, (float)(2 * f + 1)), fadd(gv, get_shift(b, w >> 3) ? -0.125f : 0.125f)); break; }
        }
    }
    x[i] = out;
}

// the five types outside the reference's own table: dequantize_row_q1_0 / mxfp4 / nvfp4 (ggml-quants.c:419-437, 569-612)
// and dequantize_row_tq1_0 / tq2_0 (2429-2487)
__global__ void __launch_bounds__(256) k_dequant_extra(int T, const uchar* __restrict__ y, float* __restrict__ x, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float kvf[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};
    const unsigned pow3[5] = {1, 3, 9, 27, 81};
    float out = 0.f;
    if (T == SG_Q1_0) {
        const uchar* b = y + (i / 128) * 18;
        const int w = (int)(i % 128);
        const float d = f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        out = ((b[2 + (w >> 3)] >> (w & 7)) & 1) ? d : -d;
    } else if (T == SG_TQ2_0) {
        const uchar* b = y + (i / 256) * 66;
        const int w = (int)(i % 256);
        const float d = f16_to_f32((uint16_t)(b[64] | (b[65] << 8)));
        const int q = (b[32 * (w >> 7) + (w & 31)] >> (2 * ((w >> 5) & 3))) & 3;
        out = fmul((float)(q - 1), d);
    } else if (T == SG_TQ1_0) {
        const uchar* b = y + (i / 256) * 54;
        const int w = (int)(i % 256);
        const float d = f16_to_f32((uint16_t)(b[52] | (b[53] << 8)));
        unsigned byte, n;
        if (w < 160) { byte = b[w & 31]; n = w >> 5; }
        else if (w < 240) { byte = b[32 + ((w - 160) & 15)]; n = (w - 160) >> 4; }
        else { byte = b[48 + ((w - 240) & 3)]; n = (w - 240) >> 2; }
        const unsigned q = (byte * pow3[n]) & 0xffu;
        out = fmul((float)((int)((q * 3) >> 8) - 1), d);
    } else if (T == SG_MXFP4) {
        const uchar* b = y + (i / 32) * 17;
        const int w = (int)(i % 32);
        const float d = e8m0_half(b[0]);
        out = fmul(kvf[w < 16 ? b[1 + w] & 15 : b[1 + w - 16] >> 4], d);
    } else {
        const uchar* b = y + (i / 64) * 36;
        const int w = (int)(i % 64), sb = w >> 4, j = w & 15;
        const float d = ue4m3_to_f32(b[sb]);
        out = fmul(kvf[j < 8 ? b[4 + 8 * sb + j] & 15 : b[4 + 8 * sb + j - 8] >> 4], d);
    }
    x[i] = out;
}

// BF16 / F16 / F32 conversions of unquantised tensors (norms, embeddings kept in float): replaces
// M28RepoGPU._float_dev (seedpack/repo3.py:673-689).  To BF16: round to nearest even by integer add on the bits.
__global__ void __launch_bounds__(256) k_convert_float(const void* __restrict__ src, int st, void* __restrict__ dst, int dt, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float f;
    if (st == SG_DT_BF16) f = bf16_to_f32(static_cast<const uint16_t*>(src)[i]);
    else if (st == SG_DT_F16) f = f16_to_f32(static_cast<const uint16_t*>(src)[i]);
    else f = static_cast<const float*>(src)[i];
    if (dt == SG_DT_F32) static_cast<float*>(dst)[i] = f;
    else if (dt == SG_DT_F16) static_cast<uint16_t*>(dst)[i] = f32_to_f16(f);
    else { const unsigned u = __float_as_uint(f); static_cast<uint16_t*>(dst)[i] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16); }
}

const uint16_t* device_grid_keys(int device, int which);

}  // namespace sg

using namespace sg;

extern "C" int sg_dequantize(int device, void* stream, int T, const unsigned char* y, float* x, long long n_weights) {
    int qk, bs;
    if (sg_type_info(T, &qk, &bs) != SG_OK) return SG_ERR_TYPE;
    if (n_weights < 0 || (n_weights && (!y || !x))) return SG_ERR_ARG;
    if (n_weights % qk) return SG_ERR_SHAPE;
    if (n_weights == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    const uint16_t* gk = nullptr;
    if (T == 16 || T == 17 || T == 18 || T == 19 || T == 21 || T == 22 || T == 29) {
        const int gi = T == 16 ? 0 : T == 17 ? 1 : (T == 19 || T == 29) ? 2 : T == 22 ? 3 : T == 18 ? 4 : 5;
        gk = device_grid_keys(device, gi);
        if (!gk) return SG_ERR_TABLES;
    }
    const long long grid = (n_weights + 255) / 256;
    if (grid > 0x7fffffffLL) return SG_ERR_LIMIT;
    if (T == SG_Q1_0 || T == SG_TQ1_0 || T == SG_TQ2_0 || T == SG_MXFP4 || T == SG_NVFP4)
        k_dequant_extra<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(T, y, x, n_weights);
    else
        k_dequant<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(T, y, x, n_weights, gk);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_convert_float(int device, void* stream, const void* src, int src_dtype, void* dst, int dst_dtype, long long n) {
    if (n < 0 || (n && (!src || !dst))) return SG_ERR_ARG;
    if (src_dtype < 0 || src_dtype > 2 || dst_dtype < 0 || dst_dtype > 2) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long grid = (n + 255) / 256;
    if (grid > 0x7fffffffLL) return SG_ERR_LIMIT;
    k_convert_float<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(src, src_dtype, dst, dst_dtype, n);
    return cuda_ok(cudaGetLastError());
}

// nearest_int of every element: the rounding helper of all quantisers, exposed so that it can be swept on its own
__global__ void __launch_bounds__(256) k_nearest_int(const float* __restrict__ x, int* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = sg::nearest_int(x[i]);
}

extern "C" int sg_selftest_nearest_int(int device, void* stream, const float* x, int* out, long long n) {
    if (n < 0 || (n && (!x || !out))) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long grid = (n + 255) / 256;
    if (grid > 0x7fffffffLL) return SG_ERR_LIMIT;
    k_nearest_int<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(x, out, n);
    return cuda_ok(cudaGetLastError());
}
