// Shared device helpers for the re-quantiser kernels (sm_100a).
//
// Everything here is arithmetic whose result is fixed by llama.cpp's scalar C code
// (ggml-quants.c as vendored by the reference): plain IEEE single precision, no FMA
// contraction (the library is built with -fmad=false), correctly rounded division and
// square root, denormals kept.  Every float operation that matters is spelled with an
// explicit round-to-nearest intrinsic so that the expression tree is the reference's.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/seedgrow.h"

#define SG_DEVINL __device__ __forceinline__

namespace sg {

// ---------------------------------------------------------------------------------------------
// Exact division by a literal.  ptxas may turn `div.rn.f32 x, <immediate>` into a multiplication by
// the rounded reciprocal, which differs from the IEEE quotient in a few percent of cases
// (the reference works around the same rewrite, seedpack/ptxfix.py:1-7).  Divisors therefore come
// from constant memory, which the assembler cannot fold.
enum DivK { DIV_15 = 0, DIV_31, DIV_127, DIV_63, DIV_5, DIV_6, DIV_COUNT };
static __constant__ float c_div[DIV_COUNT] = {15.f, 31.f, 127.f, 63.f, 5.f, 6.f};

SG_DEVINL float fdiv(float a, float b) { return __fdiv_rn(a, b); }
SG_DEVINL float fmul(float a, float b) { return __fmul_rn(a, b); }
SG_DEVINL float fadd(float a, float b) { return __fadd_rn(a, b); }
SG_DEVINL float fsub(float a, float b) { return __fsub_rn(a, b); }
SG_DEVINL float fsqrt(float a) { return __fsqrt_rn(a); }
SG_DEVINL float frcp(float a) { return __fdiv_rn(1.0f, a); }

// nearest_int (ggml-quants.c:621-626): add 1.5 * 2^23, read the mantissa.  Out-of-range inputs give
// the same garbage as the C code; no assertion.
SG_DEVINL int nearest_int(float f) {
    float v = __fadd_rn(f, 12582912.f);
    return (__float_as_int(v) & 0x007fffff) - 0x00400000;
}

// fp32 -> fp16 bits, the integer/float construction of ggml-impl.h:417-443 (round to nearest even,
// NaN -> 0x7e00, overflow -> infinity); needs denormals, hence no -ftz.
SG_DEVINL uint16_t f32_to_f16(float f) {
    float base = __fmul_rn(__fmul_rn(fabsf(f), __uint_as_float(0x77800000u)), __uint_as_float(0x08800000u));
    const uint32_t w = __float_as_uint(f);
    const uint32_t shl1_w = w + w;
    const uint32_t sign = w & 0x80000000u;
    uint32_t bias = shl1_w & 0xFF000000u;
    if (bias < 0x71000000u) bias = 0x71000000u;
    base = __fadd_rn(__uint_as_float((bias >> 1) + 0x07800000u), base);
    const uint32_t bits = __float_as_uint(base);
    const uint32_t exp_bits = (bits >> 13) & 0x00007C00u;
    const uint32_t mantissa_bits = bits & 0x00000FFFu;
    const uint32_t nonsign = exp_bits + mantissa_bits;
    return (uint16_t)((sign >> 16) | (shl1_w > 0xFF000000u ? 0x7E00u : nonsign));
}

// fp16 bits -> fp32 (ggml-impl.h:396-415); exact for every input.
SG_DEVINL float f16_to_f32(uint16_t h) {
    const uint32_t w = (uint32_t)h << 16;
    const uint32_t sign = w & 0x80000000u;
    const uint32_t two_w = w + w;
    const float normalized = __fmul_rn(__uint_as_float((two_w >> 4) + (0xE0u << 23)), __uint_as_float(0x07800000u));
    const float denormalized = __fsub_rn(__uint_as_float((two_w >> 17) | (126u << 23)), 0.5f);
    const uint32_t r = sign | (two_w < (1u << 27) ? __float_as_uint(denormalized) : __float_as_uint(normalized));
    return __uint_as_float(r);
}

SG_DEVINL float bf16_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// ---------------------------------------------------------------------------------------------
// Source element types.  Loads are 16-byte vectors; a "group" is 8 consecutive weights.
template <int DT> struct Src;
template <> struct Src<SG_DT_BF16> {
    static constexpr int BYTES = 2;
    static SG_DEVINL void load8(const void* p, long long idx, float* o) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + idx)), o);
    }
    static SG_DEVINL void unpack8(const uint4 v, float* o) {
        o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
        o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
        o[4] = __uint_as_float(v.z << 16); o[5] = __uint_as_float(v.z & 0xffff0000u);
        o[6] = __uint_as_float(v.w << 16); o[7] = __uint_as_float(v.w & 0xffff0000u);
    }
};
template <> struct Src<SG_DT_F16> {
    static constexpr int BYTES = 2;
    static SG_DEVINL void load8(const void* p, long long idx, float* o) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + idx)), o);
    }
    static SG_DEVINL void unpack8(const uint4 v, float* o) {
        o[0] = f16_to_f32((uint16_t)v.x); o[1] = f16_to_f32((uint16_t)(v.x >> 16));
        o[2] = f16_to_f32((uint16_t)v.y); o[3] = f16_to_f32((uint16_t)(v.y >> 16));
        o[4] = f16_to_f32((uint16_t)v.z); o[5] = f16_to_f32((uint16_t)(v.z >> 16));
        o[6] = f16_to_f32((uint16_t)v.w); o[7] = f16_to_f32((uint16_t)(v.w >> 16));
    }
};
template <> struct Src<SG_DT_F32> {
    static constexpr int BYTES = 4;
    static SG_DEVINL void load8(const void* p, long long idx, float* o) {
        const float4* q = reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx);
        const float4 a = __ldg(q), b = __ldg(q + 1);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
};

template <int DT, int N> SG_DEVINL void load_vals(const void* p, long long idx, float* o) {
#pragma unroll
    for (int i = 0; i < N; i += 8) Src<DT>::load8(p, idx + i, o + i);
}
template <int N> SG_DEVINL void load_f32(const float* p, long long idx, float* o) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p + idx + i));
        o[i] = a.x; o[i + 1] = a.y; o[i + 2] = a.z; o[i + 3] = a.w;
    }
}

// ---------------------------------------------------------------------------------------------
// Work decomposition.  A launch covers up to SG_MAX_TENSORS tensors laid out in one source and one
// destination buffer.  The unit of work is a "slab": SLAB consecutive weights of one row (a K/IQ
// super-block, or 8 legacy blocks); rows whose length is not a multiple of SLAB end in a short slab.
struct Tensor {
    long long xoff;    // first weight of the tensor, in elements of the source buffer
    long long yoff;    // first output byte
    long long woff;    // first importance weight (floats), < 0: none
    long long slab0;   // index of the tensor's first slab within the launch
    long long row0;    // index of the tensor's first row within the launch (for per-row scratch)
    int nrows, npr;    // rows, weights per row
    int spr;           // slabs per row
    int pad;
};
#define SG_MAX_TENSORS 16
struct Job {
    const void* x;
    uint8_t* y;
    const float* w;
    float* rowstat;     // per-row scratch (row-wide sigma2 of the legacy importance paths) or null
    int* status;        // device status word, OR-ed with SG_ST_* bits by kernels that detect trouble
    long long nslabs;
    int ntens;
    Tensor t[SG_MAX_TENSORS];
};

struct Slab {
    long long x;       // element index of the slab's first weight in the source buffer
    long long w;       // index of its first importance weight, < 0: none
    long long grow;    // launch-wide row index (index into Job::rowstat)
    long long yrow;    // output byte offset of the tensor (add row and block offsets with out_offset())
    long long lrow;    // row index within its tensor
    int u;             // slab index within the row
    int n;             // weights in this slab (SLAB, or fewer at a ragged row end)
    int npr;           // weights per row
};

template <int SLAB> SG_DEVINL Slab locate(const Job& job, long long s) {
    int ti = 0;
#pragma unroll 1
    for (int i = 1; i < job.ntens; ++i) if (s >= job.t[i].slab0) ti = i;
    const Tensor& t = job.t[ti];
    const long long ls = s - t.slab0;
    const long long r = ls / t.spr;
    const int u = (int)(ls - r * t.spr);
    Slab o;
    o.x = t.xoff + r * t.npr + (long long)u * SLAB;
    o.w = t.woff < 0 ? -1 : t.woff + (long long)u * SLAB;
    o.grow = t.row0 + r;
    o.yrow = t.yoff;
    o.lrow = r;
    o.u = u;
    o.npr = t.npr;
    o.n = min(SLAB, t.npr - u * SLAB);
    return o;
}

// byte offset of block `b` (counted within the slab) for a type with QK weights / BS bytes per block
template <int SLAB, int QK, int BS> SG_DEVINL long long out_offset(const Slab& s, int b) {
    return s.yrow + (s.lrow * (long long)(s.npr / QK) + (long long)s.u * (SLAB / QK) + b) * BS;
}

}  // namespace sg
