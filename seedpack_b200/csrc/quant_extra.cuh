// The five quantisers of ggml-quants.c outside the reference's own type table: Q1_0 (sign bits + mean magnitude,
// ggml-quants.c:40-72), TQ1_0 / TQ2_0 (ternary, 2317-2413), MXFP4 and NVFP4 (4-bit floats with a shared E8M0 / per-16
// UE4M3 scale, 336-417).  None of them uses an importance matrix.  All are bound by memory traffic.
//
// Mapping: a CTA of 128 threads takes 8 slabs of 256 consecutive weights, 16 threads per slab.  The weights come in
// with 16-byte loads and are spread out as floats in shared memory, because the block layouts gather weights that
// lie far apart (a TQ1_0 byte holds weights m, m + 32, ... m + 128); the slab's output bytes are put together in
// shared memory and written out side by side.
#pragma once
#include "quant_k.cuh"

namespace sg {

template <int TYPE> struct Extra;
template <> struct Extra<SG_Q1_0>  { static constexpr int QK = 128, BS = 18; };
template <> struct Extra<SG_TQ1_0> { static constexpr int QK = 256, BS = 54; };
template <> struct Extra<SG_TQ2_0> { static constexpr int QK = 256, BS = 66; };
template <> struct Extra<SG_MXFP4> { static constexpr int QK = 32, BS = 17; };
template <> struct Extra<SG_NVFP4> { static constexpr int QK = 64, BS = 36; };

// lroundf(v) + 1 for the ternary types: round half away from zero
SG_DEVINL int trit(float x, float id) { return (int)roundf(fmul(x, id)) + 1; }
// five trits, most significant first, as a byte: ceil(value * 256 / 243)   (ggml-quants.c:2343-2346)
SG_DEVINL unsigned pack_trits(unsigned q) { return ((q & 0xffu) * 256u + 242u) / 243u & 0xffu; }

// index of the 4-bit float closest to x at scale e (ggml-quants.c:336-348): first strictly smaller error wins
SG_DEVINL unsigned best_fp4(float x, float e) {
    const float kv[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};
    unsigned best = 0;
    float err = fabsf(fsub(fmul(kv[0], e), x));
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        const float d = fabsf(fsub(fmul(kv[i], e), x));
        if (d < err) { err = d; best = i; }
    }
    return best;
}
// E8M0 exponent byte -> half its value as a float (ggml-impl.h:489-507)
SG_DEVINL float e8m0_half(unsigned e) { return __uint_as_float(e < 2 ? 0x00200000u << e : (e - 1) << 23); }
// float -> UE4M3 byte and back, the integer constructions of ggml-impl.h:514-565
SG_DEVINL unsigned f32_to_ue4m3(float x) {
    if (!(x > 0.f)) return 0;
    if (x > 448.f) x = 448.f;
    const unsigned bits = __float_as_uint(x);
    int ex = (int)((bits >> 23) & 0xff) - 127 + 7;
    if (ex <= 0) {
        int man = (int)fadd(fmul(x, 512.f), 0.5f);
        if (man > 7) man = 7;
        return man < 1 ? 0u : (unsigned)man;
    }
    if (ex >= 15) return 0x7e;
    int man = (int)((bits >> 20) & 7) + (int)((bits >> 19) & 1);
    if (man > 7) { man = 0; if (++ex >= 15) return 0x7e; }
    return (unsigned)((ex << 3) | man);
}
SG_DEVINL float ue4m3_to_f32(unsigned x) {
    if (x == 0 || x == 0x7f) return 0.f;
    const int ex = (int)(x >> 3) & 15, man = (int)(x & 7);
    const float raw = ex == 0 ? ldexpf((float)man, -9) : ldexpf(fadd(1.0f, fmul((float)man, 0.125f)), ex - 7);
    return fmul(raw, 0.5f);
}

constexpr int EX_SLABS = 8, EX_TPB = EX_SLABS * 16;

template <int TYPE, int DT>
__global__ void __launch_bounds__(EX_TPB) k_quant_extra(const __grid_constant__ Job job) {
    using E = Extra<TYPE>;
    constexpr int QK = E::QK, BS = E::BS, NBLK = 256 / QK, OUT = NBLK * BS;
    __shared__ float xs[EX_SLABS][256];
    __shared__ float red[EX_SLABS][16];
    __shared__ __align__(4) unsigned char out[EX_SLABS][(OUT + 3) / 4 * 4];
    const int g = threadIdx.x >> 4, t = threadIdx.x & 15;
    long long s = (long long)blockIdx.x * EX_SLABS + g;
    const bool valid = s < job.nslabs;
    if (!valid) s = job.nslabs - 1;
    const Slab sl = locate<256>(job, s);
    {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
        if (t * 16 < sl.n) load_vals<DT, 16>(job.x, sl.x + t * 16, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) xs[g][t * 16 + i] = v[i];
    }
    __syncthreads();
    const float* x = xs[g];
    unsigned char* o = out[g];
    if (TYPE == SG_TQ1_0 || TYPE == SG_TQ2_0) {
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(x[t * 16 + i]));
        red[g][t] = m;
        __syncthreads();
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, red[g][i]);
        const float id = amax != 0.f ? frcp(amax) : 0.f;
        if (TYPE == SG_TQ2_0) {
            // byte j = 32 a + m: weights 128 a + m + 32 n, n = 0..3, two bits each
            for (int j = t; j < 64; j += 16) {
                const int a = j >> 5, mm = j & 31;
                unsigned q = 0;
#pragma unroll
                for (int n = 0; n < 4; ++n) q += (unsigned)(trit(x[128 * a + mm + 32 * n], id) & 3) << (2 * n);
                o[j] = (unsigned char)q;
            }
            if (t == 0) { const unsigned h = f32_to_f16(amax); o[64] = (unsigned char)h; o[65] = (unsigned char)(h >> 8); }
        } else {
            // qs[0..31]: weights m + 32 n (n < 5); qs[32..47]: weights 160 + m + 16 n; qh[j]: weights 240 + j + 4 m, then a zero trit
            for (int j = t; j < 52; j += 16) {
                unsigned q = 0;
                if (j < 32) { for (int n = 0; n < 5; ++n) q = q * 3 + (unsigned)trit(x[j + 32 * n], id); }
                else if (j < 48) { for (int n = 0; n < 5; ++n) q = q * 3 + (unsigned)trit(x[160 + (j - 32) + 16 * n], id); }
                else { for (int n = 0; n < 4; ++n) q = q * 3 + (unsigned)trit(x[240 + (j - 48) + 4 * n], id); q *= 3; }
                o[j] = (unsigned char)pack_trits(q);
            }
            if (t == 0) { const unsigned h = f32_to_f16(amax); o[52] = (unsigned char)h; o[53] = (unsigned char)(h >> 8); }
        }
    } else if (TYPE == SG_Q1_0) {
        // mean magnitude: a float sum in index order, one thread per block of 128
        if (t < 2) {
            float sum = 0.f;
            for (int j = 0; j < 128; ++j) sum = fadd(sum, fabsf(x[128 * t + j]));
            const unsigned h = f32_to_f16(fmul(sum, 1.0f / 128.f));
            o[18 * t] = (unsigned char)h; o[18 * t + 1] = (unsigned char)(h >> 8);
        }
        {   // 16 sign bits per thread
            unsigned bits = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) if (x[16 * t + i] >= 0.f) bits |= 1u << i;
            const int b = t >> 3, k = t & 7;
            o[18 * b + 2 + 2 * k] = (unsigned char)bits; o[18 * b + 3 + 2 * k] = (unsigned char)(bits >> 8);
        }
    } else if (TYPE == SG_MXFP4) {
        // 8 blocks of 32, two threads per block; the exponent byte from the block's largest magnitude
        const int b = t >> 1, hf = t & 1;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) { const float a = fabsf(x[32 * b + j]); if (amax < a) amax = a; }
        unsigned e = 0;
        if (amax > 0.f) e = (unsigned)(int)fadd(fsub(floorf((float)log2((double)amax)), 2.f), 127.f) & 0xffu;
        const float d = e8m0_half(e);
        if (hf == 0) o[17 * b] = (unsigned char)e;
        for (int j = 8 * hf; j < 8 * hf + 8; ++j)
            o[17 * b + 1 + j] = (unsigned char)(best_fp4(x[32 * b + j], d) | (best_fp4(x[32 * b + 16 + j], d) << 4));
    } else {
        // NVFP4: 4 blocks of 64, each 4 sub-blocks of 16 with their own UE4M3 scale; one thread per sub-block
        const int b = t >> 2, sb = t & 3;
        const float* xb = x + 64 * b + 16 * sb;
        float amax = 0.f;
        for (int j = 0; j < 16; ++j) { const float a = fabsf(xb[j]); if (amax < a) amax = a; }
        const unsigned ue = f32_to_ue4m3(fdiv(amax, c_div[DIV_6]));
        const float d = ue4m3_to_f32(ue);
        o[36 * b + sb] = (unsigned char)ue;
        for (int j = 0; j < 8; ++j) o[36 * b + 4 + 8 * sb + j] = (unsigned char)(best_fp4(xb[j], d) | (best_fp4(xb[8 + j], d) << 4));
    }
    __syncthreads();
    if (!valid) return;
    const int nbytes = (sl.n / QK) * BS;                       // a ragged row end holds fewer blocks
    unsigned char* y = job.y + out_offset<256, QK, BS>(sl, 0);
    for (int i = t; i < nbytes; i += 16) y[i] = o[i];
}

template <int TYPE>
static int launch_extra(const Job& job, int dt, cudaStream_t st) {
    const unsigned grid = (unsigned)((job.nslabs + EX_SLABS - 1) / EX_SLABS);
    if (grid == 0) return SG_OK;
    switch (dt) {
        case SG_DT_BF16: k_quant_extra<TYPE, SG_DT_BF16><<<grid, EX_TPB, 0, st>>>(job); break;
        case SG_DT_F16:  k_quant_extra<TYPE, SG_DT_F16><<<grid, EX_TPB, 0, st>>>(job); break;
        case SG_DT_F32:  k_quant_extra<TYPE, SG_DT_F32><<<grid, EX_TPB, 0, st>>>(job); break;
        default: return SG_ERR_ARG;
    }
    return cuda_ok(cudaGetLastError());
}

}  // namespace sg
