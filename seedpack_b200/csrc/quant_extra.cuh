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
// The same choice from seven thresholds.  The candidates' magnitudes are 0, e, 2e, 3e, 4e, 6e, 8e, 12e; a candidate of the
// other sign than x, or two places away, is never the first strictly smaller one (its error is larger by at least e, far
// above the rounding of a difference below 16 e), and between the two neighbours of |x| both differences are exact
// (each is a difference of floats within a factor of two, or of 0), so the loop picks the upper neighbour exactly when
// |x| lies strictly above the midpoint: the index is the number of midpoints 0.5e, 1.5e, 2.5e, 3.5e, 5e, 7e, 10e below
// |x|.  Holds while the products are exact and the errors stay far from fp32's last bit: the caller checks
// 2^-100 <= e and |x| < 2^20 e for the block and uses best_fp4 otherwise.
struct Fp4Mid {
    float m[7];
    SG_DEVINL void set(float e) {
        const float k[7] = {0.5f, 1.5f, 2.5f, 3.5f, 5.f, 7.f, 10.f};
#pragma unroll
        for (int i = 0; i < 7; ++i) m[i] = fmul(k[i], e);
    }
    SG_DEVINL unsigned pick(float x) const {
        const float ax = fabsf(x);
        const bool b2 = ax > m[3];                                 // binary search over the ordered midpoints
        const bool b1 = ax > (b2 ? m[5] : m[1]);
        const float last = b2 ? (b1 ? m[6] : m[4]) : (b1 ? m[2] : m[0]);
        const unsigned idx = (b2 ? 4u : 0u) + (b1 ? 2u : 0u) + (ax > last ? 1u : 0u);
        return idx | ((x < 0.f && idx) ? 8u : 0u);
    }
};
SG_DEVINL bool fp4_fast_ok(float e, float amax) { return e >= 7.888609052e-31f && amax < fmul(e, 1048576.f); }

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

// the 16 trits of a thread's weights as 2-bit fields, weight i in bits 2i..2i+1
SG_DEVINL unsigned trit_word(const float (&v)[16], float id) {
    unsigned w = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) w |= (unsigned)(trit(v[i], id) & 3) << (2 * i);
    return w;
}

template <int TYPE, int DT>
__global__ void __launch_bounds__(EX_TPB) k_quant_extra(const __grid_constant__ Job job) {
    using E = Extra<TYPE>;
    constexpr int QK = E::QK, BS = E::BS, NBLK = 256 / QK, OUT = NBLK * BS;
    __shared__ __align__(16) unsigned char out[EX_SLABS * OUT];       // the slabs' bytes back to back, as they lie in the file
    __shared__ unsigned long long dst[EX_SLABS];
    // 16 lanes per slab of 256 weights, lane t holding weights 16 t .. 16 t + 15 in registers; what a block's bytes need
    // from other lanes' weights (the layouts gather weights that lie 16, 32 or 4 apart) comes through shuffles
    const int g = threadIdx.x >> 4, t = threadIdx.x & 15;
    long long s = (long long)blockIdx.x * EX_SLABS + g;
    const bool valid = s < job.nslabs;
    if (!valid) s = job.nslabs - 1;
    const Slab sl = locate<256>(job, s);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
    if (t * 16 < sl.n) load_vals<DT, 16>(job.x, sl.x + t * 16, v);
    if (t == 0) dst[g] = valid ? (unsigned long long)(job.y + out_offset<256, QK, BS>(sl, 0)) : 0ull;
    unsigned char* o = out + g * OUT;
    if (TYPE == SG_TQ1_0 || TYPE == SG_TQ2_0) {
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int m = 1; m < 16; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        const float id = amax != 0.f ? frcp(amax) : 0.f;
        const unsigned tw = trit_word(v, id);
        const int lane0 = threadIdx.x & 16;                       // first lane of this slab inside the warp
        if (TYPE == SG_TQ2_0) {
            // byte 32 a + m: weights 128 a + m + 32 n, n = 0..3, two bits each = lanes 8 a + 2 n + (m >> 4), element m & 15.
            // Lane 8 a + 2 k + h writes the four bytes m = 16 h + 4 k .. + 3.
            const int a = t >> 3, k = (t >> 1) & 3, h = t & 1;
            unsigned src[4];
#pragma unroll
            for (int n = 0; n < 4; ++n) src[n] = __shfl_sync(0xffffffffu, tw, lane0 + 8 * a + 2 * n + h);
            unsigned word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int el = 4 * k + b;                         // m & 15
                unsigned q = 0;
#pragma unroll
                for (int n = 0; n < 4; ++n) q |= (src[n] >> (2 * el) & 3u) << (2 * n);
                word |= q << (8 * b);
            }
            unsigned short* o2 = reinterpret_cast<unsigned short*>(o + 32 * a + 16 * h + 4 * k);   // 66 g + ...: 2-byte aligned
            o2[0] = (unsigned short)word; o2[1] = (unsigned short)(word >> 16);
            if (t == 0) { const unsigned hh = f32_to_f16(amax); o[64] = (unsigned char)hh; o[65] = (unsigned char)(hh >> 8); }
        } else {
            // qs[m], m < 32: weights m + 32 n (n < 5) = lanes 2 n + (m >> 4), element m & 15; lane t writes m = 2 t, 2 t + 1
            {
                const int h = t >> 3;                             // (2 t) >> 4
                unsigned src[5];
#pragma unroll
                for (int n = 0; n < 5; ++n) src[n] = __shfl_sync(0xffffffffu, tw, lane0 + 2 * n + h);
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const int el = (2 * t + b) & 15;
                    unsigned q = 0;
#pragma unroll
                    for (int n = 0; n < 5; ++n) q = q * 3 + (src[n] >> (2 * el) & 3u);
                    o[2 * t + b] = (unsigned char)pack_trits(q);
                }
            }
            // qs[32 + m], m < 16: weights 160 + m + 16 n (n < 5) = lanes 10 + n, element m; lane t writes m = t
            {
                unsigned q = 0;
#pragma unroll
                for (int n = 0; n < 5; ++n) q = q * 3 + (__shfl_sync(0xffffffffu, tw, lane0 + 10 + n) >> (2 * t) & 3u);
                o[32 + t] = (unsigned char)pack_trits(q);
            }
            // qh[j], j < 4: weights 240 + j + 4 n (n < 4) = lane 15, elements j + 4 n, then a zero trit; lanes 0..3 write j = t
            {
                const unsigned last = __shfl_sync(0xffffffffu, tw, lane0 + 15);
                if (t < 4) {
                    unsigned q = 0;
#pragma unroll
                    for (int n = 0; n < 4; ++n) q = q * 3 + (last >> (2 * (t + 4 * n)) & 3u);
                    o[48 + t] = (unsigned char)pack_trits(q * 3);
                }
            }
            if (t == 0) { const unsigned hh = f32_to_f16(amax); o[52] = (unsigned char)hh; o[53] = (unsigned char)(hh >> 8); }
        }
    } else if (TYPE == SG_Q1_0) {
        // mean magnitude: a float sum in index order over the block's 128 weights - one chain, handed from lane to lane:
        // the eight lanes of a block add their sixteen weights in turn
        float sum = 0.f;
#pragma unroll
        for (int step = 0; step < 8; ++step) {
            if ((t & 7) == step) {
#pragma unroll
                for (int i = 0; i < 16; ++i) sum = fadd(sum, fabsf(v[i]));
            }
            sum = __shfl_sync(0xffffffffu, sum, (threadIdx.x & 24) + step);       // every lane of the block carries the chain on
        }
        if ((t & 7) == 7) {
            const unsigned h = f32_to_f16(fmul(sum, 1.0f / 128.f));
            o[18 * (t >> 3)] = (unsigned char)h; o[18 * (t >> 3) + 1] = (unsigned char)(h >> 8);
        }
        {   // 16 sign bits per thread
            unsigned bits = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) if (v[i] >= 0.f) bits |= 1u << i;
            const int b = t >> 3, k = t & 7;
            o[18 * b + 2 + 2 * k] = (unsigned char)bits; o[18 * b + 3 + 2 * k] = (unsigned char)(bits >> 8);
        }
    } else if (TYPE == SG_MXFP4) {
        // 8 blocks of 32 = two lanes each; the exponent byte from the block's largest magnitude
        const int b = t >> 1, hf = t & 1;
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { const float a = fabsf(v[j]); if (amax < a) amax = a; }
        { const float other = __shfl_xor_sync(0xffffffffu, amax, 1); if (amax < other) amax = other; }
        unsigned e = 0;
        if (amax > 0.f) {
            // floorf(log2f(amax)) is the float's exponent unless its mantissa is within 2^-15 of the next power of two
            // (there log2f may round up to the integer): those, subnormals and non-finite values take the long way
            const unsigned bits = __float_as_uint(amax), ex = bits >> 23 & 0xffu;
            const float fl = (ex != 0 && ex != 255 && (bits & 0x7fffffu) < 0x7fff00u) ? (float)((int)ex - 127)
                                                                                       : floorf((float)log2((double)amax));
            e = (unsigned)(int)fadd(fsub(fl, 2.f), 127.f) & 0xffu;
        }
        const float d = e8m0_half(e);
        // this lane's sixteen codes, weight j in bits 4j..4j+3; byte j of the block = code j of the even lane | code j of the odd lane << 4
        unsigned codes[2] = {0, 0};                               // weights 0..7, 8..15
        if (fp4_fast_ok(d, amax)) {
            Fp4Mid mid; mid.set(d);
#pragma unroll
            for (int j = 0; j < 16; ++j) codes[j >> 3] |= mid.pick(v[j]) << (4 * (j & 7));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) codes[j >> 3] |= best_fp4(v[j], d) << (4 * (j & 7));
        }
        // the even lane writes bytes 0..7, the odd lane bytes 8..15: each needs that half of the other lane's codes
        const unsigned mine = hf ? codes[1] : codes[0];
        const unsigned give = hf ? codes[0] : codes[1];
        const unsigned got = __shfl_xor_sync(0xffffffffu, give, 1);
        const unsigned lo = hf ? got : mine, hi = hf ? mine : got;           // low nibbles come from the even lane
        if (hf == 0) o[17 * b] = (unsigned char)e;
#pragma unroll
        for (int j = 0; j < 8; ++j) o[17 * b + 1 + 8 * hf + j] = (unsigned char)((lo >> (4 * j) & 15u) | (hi >> (4 * j) & 15u) << 4);
    } else {
        // NVFP4: 4 blocks of 64, each 4 sub-blocks of 16 with their own UE4M3 scale; a lane's weights are one sub-block
        const int b = t >> 2, sb = t & 3;
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { const float a = fabsf(v[j]); if (amax < a) amax = a; }
        const unsigned ue = f32_to_ue4m3(fdiv(amax, c_div[DIV_6]));
        const float d = ue4m3_to_f32(ue);
        o[36 * b + sb] = (unsigned char)ue;
        unsigned q[2] = {0, 0};
        if (fp4_fast_ok(d, amax)) {
            Fp4Mid mid; mid.set(d);
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j >> 2] |= (mid.pick(v[j]) | mid.pick(v[8 + j]) << 4) << (8 * (j & 3));
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j >> 2] |= (best_fp4(v[j], d) | best_fp4(v[8 + j], d) << 4) << (8 * (j & 3));
        }
        *reinterpret_cast<unsigned*>(o + 36 * b + 4 + 8 * sb) = q[0];        // 144 g + 36 b + 4 + 8 sb: a multiple of 4
        *reinterpret_cast<unsigned*>(o + 36 * b + 8 + 8 * sb) = q[1];
    }
    // a CTA whose eight slabs are whole and lie back to back in the output (the rule inside a row) writes them as one
    // run of 16-byte words between a byte-wise head and tail; any other CTA writes slab by slab
    const bool whole = valid && sl.n == 256 && dst[g] == dst[0] + (unsigned long long)g * OUT;
    if (__syncthreads_and(whole)) {
        unsigned char* y0 = reinterpret_cast<unsigned char*>(dst[0]);
        constexpr int TOTAL = EX_SLABS * OUT;
        const int head = (int)((16 - (dst[0] & 15)) & 15);            // TOTAL >= 288: always longer than the head
        const int nvec = (TOTAL - head) / 16;
        for (int i = threadIdx.x; i < head; i += EX_TPB) y0[i] = out[i];
        for (int i = threadIdx.x; i < nvec; i += EX_TPB) {
            const unsigned char* sp = out + head + 16 * i;
            uint4 w;
            if (head == 0) w = *reinterpret_cast<const uint4*>(sp);
            else {                                                    // shared-memory side not aligned: put the word together
                unsigned q[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) q[k] = sp[4 * k] | sp[4 * k + 1] << 8 | sp[4 * k + 2] << 16 | (unsigned)sp[4 * k + 3] << 24;
                w = make_uint4(q[0], q[1], q[2], q[3]);
            }
            *reinterpret_cast<uint4*>(y0 + head + 16 * i) = w;
        }
        for (int i = head + 16 * nvec + threadIdx.x; i < TOTAL; i += EX_TPB) y0[i] = out[i];
        return;
    }
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
