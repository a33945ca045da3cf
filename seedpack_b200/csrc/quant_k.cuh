// K-quants: Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, with and without an importance matrix.
//
// Mapping: one thread per sub-block (16 or 32 weights, held in registers), the 16 or 8 threads of a
// 256-weight super-block are neighbouring lanes of one warp.  Sub-block searches run independently
// (search.cuh); everything that spans the super-block - the in-order sum of squares, the maxima with
// llama.cpp's first-wins rule, the second-level quantisation of the 8/16 sub-scales, the interleaved
// bit packing - is done with width-limited warp shuffles.  No shared memory, no global scratch.
//
// Reference arithmetic: ggml-quants.c:891-959 / 1150-1210 (Q2_K), 1230-1304 / 1356-1438 (Q3_K),
// 1458-1528 / 1554-1625 (Q4_K), 1645-1730 / 1759-1850 (Q5_K), 1870-1938 / 1971-2053 (Q6_K).
#pragma once
#include "search.cuh"

namespace sg {

#define SG_FULL 0xffffffffu

template <int LANES> SG_DEVINL float gshfl(float v, int j) { return __shfl_sync(SG_FULL, v, j, LANES); }
template <int LANES> SG_DEVINL int gshfl(int v, int j) { return __shfl_sync(SG_FULL, v, j, LANES); }
template <int LANES> SG_DEVINL unsigned gshfl(unsigned v, int j) { return __shfl_sync(SG_FULL, v, j, LANES); }

// In-order sum of x[i]^2 over the whole super-block (ggml-quants.c:1167, 1369, 1570, 1775): the chain
// starts in lane 0 and is handed from lane to lane, so the additions happen in index order.
template <int SUB, int LANES> SG_DEVINL float ordered_sumsq(const float (&x)[SUB], int sub) {
    float s = 0.f;
#pragma unroll 1
    for (int stage = 0; stage < LANES; ++stage) {
        float t = s;
        if (sub == stage) {
#pragma unroll
            for (int i = 0; i < SUB; ++i) t = fadd(t, fmul(x[i], x[i]));
        }
        s = gshfl<LANES>(t, stage);
    }
    return s;
}

// all LANES values of the group, in lane order
template <int LANES> SG_DEVINL void gather(float v, float (&out)[LANES]) {
#pragma unroll
    for (int j = 0; j < LANES; ++j) out[j] = gshfl<LANES>(v, j);
}

SG_DEVINL void st16(uint8_t* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    *reinterpret_cast<uint4*>(p) = make_uint4(a, b, c, d);
}
SG_DEVINL void st2(uint8_t* p, uint32_t v) { *reinterpret_cast<uint16_t*>(p) = (uint16_t)v; }
SG_DEVINL void st4(uint8_t* p, uint32_t v) { *reinterpret_cast<uint32_t*>(p) = v; }
// 4 bytes at a 2-byte aligned address
SG_DEVINL void st4_a2(uint8_t* p, uint32_t v) { st2(p, v & 0xffff); st2(p + 2, v >> 16); }

// 2-bit planes of Q2_K / Q3_K (ggml-quants.c:951-955, 1296-1300): byte l of a 128-weight half holds the
// codes of weights l, l+32, l+64, l+96.  `codes` = this lane's 16 two-bit codes, code i at bits 2i.
// Lanes q = 0,1 of each half assemble 16 bytes from lanes q, q+2, q+4, q+6 and return true.
SG_DEVINL bool pack_2bit_planes(unsigned codes, int sub, uint32_t (&out)[4]) {
    const int half = sub >> 3, q = sub & 7;
    unsigned c[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = gshfl<16>(codes, half * 8 + (q & 1) + 2 * k);
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = 4 * m + k;
            const uint32_t b = ((c[0] >> (2 * i)) & 3) | (((c[1] >> (2 * i)) & 3) << 2) |
                               (((c[2] >> (2 * i)) & 3) << 4) | (((c[3] >> (2 * i)) & 3) << 6);
            word |= b << (8 * k);
        }
        out[m] = word;
    }
    return q < 2;
}

// ================================================================================================
struct Q2K {
    static constexpr int SLAB = 256, SUB = 16, LANES = 16, QK = 256, BS = 84;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid) {
        float x[16], wt[16];
        load_vals<DT, 16>(job.x, sl.x + sub * 16, x);
        QkxBest b;
        float sw = 0.f;
        if (IMX) {
            const float sumx2 = ordered_sumsq<16, 16>(x, sub);
            const float sigma2 = fmul(sumx2, 1.0f / 256);        // power of two: exact either way
            float qw[16];
            load_f32<16>(job.w, sl.w + sub * 16, qw);
#pragma unroll
            for (int l = 0; l < 16; ++l) wt[l] = fmul(qw[l], fsqrt(fadd(sigma2, fmul(x[l], x[l]))));
#pragma unroll
            for (int l = 0; l < 16; ++l) sw = fadd(sw, wt[l]);
            b = make_qkx_quants<16, true>(3, x, wt, -0.9f, 0.05f, 36, false);
        } else {
#pragma unroll
            for (int l = 0; l < 16; ++l) wt[l] = fabsf(x[l]);
            b = make_qkx_quants<16, false>(3, x, wt, -0.5f, 0.1f, 15, true);
        }
        float scales[16], mins[16];
        gather<16>(b.scale, scales);
        gather<16>(b.the_min, mins);
        int ls, lm;
        uint16_t dh, dmh;
        if (IMX) {
            float sws[16];
            gather<16>(sw, sws);
            int Ls[16], Lm[16];
            const float dm = make_qp_quants<16>(15, scales, Ls, sws);
            const float mm = make_qp_quants<16>(15, mins, Lm, sws);
            dh = f32_to_f16(dm); dmh = f32_to_f16(mm);
            ls = 0; lm = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) if (j == sub) { ls = Ls[j]; lm = Lm[j]; }
        } else {
            float max_scale = 0.f, max_min = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (scales[j] > max_scale) max_scale = scales[j];
                if (mins[j] > max_min) max_min = mins[j];
            }
            if (max_scale > 0.f) {
                const float iscale = fdiv(15.f, max_scale);
                ls = nearest_int(fmul(iscale, b.scale));
                dh = f32_to_f16(fdiv(max_scale, c_div[DIV_15]));
            } else { ls = 0; dh = f32_to_f16(0.f); }
            if (max_min > 0.f) {
                const float iscale = fdiv(15.f, max_min);
                lm = nearest_int(fmul(iscale, b.the_min));
                dmh = f32_to_f16(fdiv(max_min, c_div[DIV_15]));
            } else { lm = 0; dmh = f32_to_f16(0.f); }
        }
        const uint32_t sc = ((uint32_t)ls | ((uint32_t)lm << 4)) & 0xff;   // uint8_t scales[j]
        const float d = fmul(f16_to_f32(dh), (float)(sc & 0xF));
        unsigned codes = 0;
        if (d != 0.f) {
            const float dm = fmul(f16_to_f32(dmh), (float)(sc >> 4));
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int l = clampi(nearest_int(fdiv(fadd(x[i], dm), d)), 0, 3);
                codes |= (unsigned)l << (2 * i);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                codes |= (unsigned)(IMX ? qkx_code<16, true>(b, 3, x[i]) : qkx_code<16, false>(b, 3, x[i])) << (2 * i);
        }
        // block_q2_K: scales[16], qs[64], d, dmin
        uint32_t q[4];
        const bool writer = pack_2bit_planes(codes, sub, q);
        unsigned scw[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            unsigned wv = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) wv |= gshfl<16>(sc, 4 * m + k) << (8 * k);
            scw[m] = wv;
        }
        if (!valid) return;
        uint8_t* y = job.y + out_offset<256, 256, 84>(sl, 0);
        if (writer) {
            uint8_t* p = y + 16 + (sub >> 3) * 32 + (sub & 1) * 16;
            st4(p, q[0]); st4(p + 4, q[1]); st4(p + 8, q[2]); st4(p + 12, q[3]);
        }
        if (sub == 2) { st4(y, scw[0]); st4(y + 4, scw[1]); st4(y + 8, scw[2]); st4(y + 12, scw[3]); }
        if (sub == 3) st4(y + 80, (uint32_t)dh | ((uint32_t)dmh << 16));
    }
};

// ================================================================================================
struct Q3K {
    static constexpr int SLAB = 256, SUB = 16, LANES = 16, QK = 256, BS = 110;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid) {
        float x[16];
        load_vals<DT, 16>(job.x, sl.x + sub * 16, x);
        float myscale;
        int L0[16];            // codes from the sub-block search, kept for the d == 0 case
        float scales[16];
        int l6;                // this sub-block's 6-bit scale, 0..63
        uint16_t dh;
        if (IMX) {
            const float sumx2 = ordered_sumsq<16, 16>(x, sub);
            const float sigma2 = fmul(fmul(2.f, sumx2), 1.0f / 256);
            float qw[16], wt[16];
            load_f32<16>(job.w, sl.w + sub * 16, qw);
#pragma unroll
            for (int l = 0; l < 16; ++l) wt[l] = fmul(qw[l], fsqrt(fadd(sigma2, fmul(x[l], x[l]))));
            float sumw = 0.f;
#pragma unroll
            for (int l = 0; l < 16; ++l) sumw = fadd(sumw, wt[l]);
            const QxBest b = make_qx_quants<16, true>(4, x, wt);
#pragma unroll
            for (int i = 0; i < 16; ++i) L0[i] = qx_code(b, 4, x[i]);
            myscale = b.scale;
            gather<16>(myscale, scales);
            float sws[16];
            gather<16>(sumw, sws);
            const QxBest bb = make_qx_quants<16, true>(32, scales, sws);
            l6 = qx_code(bb, 32, myscale);
            dh = f32_to_f16(bb.scale);
        } else {
            myscale = make_q3_quants<16>(4, x, L0);
            gather<16>(myscale, scales);
            float max_scale = 0.f, amax = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float a = fabsf(scales[j]);
                if (a > amax) { amax = a; max_scale = scales[j]; }
            }
            if (max_scale != 0.f) {
                const float iscale = fdiv(-32.f, max_scale);
                int l = (int)(int8_t)nearest_int(fmul(iscale, myscale));
                l6 = clampi(l, -32, 31) + 32;
                dh = f32_to_f16(frcp(iscale));
            } else { l6 = 0; dh = f32_to_f16(0.f); }
        }
        // the 6-bit scale goes through its packed form and back (ggml-quants.c:1268-1272): same value - 32
        const int sc = l6 - 32;
        const float d = fmul(f16_to_f32(dh), (float)sc);
        unsigned lo = 0, hi = 0;            // 2 low bits per weight, 1 high bit per weight
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int l;
            if (d != 0.f) l = clampi(nearest_int(fdiv(x[i], d)), -4, 3) + 4;
            else l = L0[i];
            if (l > 3) { hi |= 1u << i; l -= 4; }
            lo |= (unsigned)l << (2 * i);
        }
        uint32_t q[4];
        const bool qwriter = pack_2bit_planes(lo, sub, q);
        // hmask[m] bit b = high bit of weight 32*b + m  (ggml-quants.c:1283-1295): lanes 0,1 build 16 bytes each
        unsigned hb[8];
#pragma unroll
        for (int bq = 0; bq < 8; ++bq) hb[bq] = gshfl<16>(hi, 2 * bq + (sub & 1));
        uint32_t hm[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t word = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = 4 * m + k;
                uint32_t byte = 0;
#pragma unroll
                for (int bq = 0; bq < 8; ++bq) byte |= ((hb[bq] >> i) & 1) << bq;
                word |= byte << (8 * k);
            }
            hm[m] = word;
        }
        // scales[12] (ggml-quants.c:1252-1262)
        int l6s[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) l6s[j] = gshfl<16>(l6, j);
        uint32_t s12[3] = {0, 0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t l = (uint32_t)l6s[j];
            const int bi = j < 8 ? j : j - 8;
            s12[bi >> 2] |= (j < 8 ? (l & 0xF) : ((l & 0xF) << 4)) << (8 * (bi & 3));
            const int hi_b = 8 + (j & 3);
            s12[hi_b >> 2] |= ((l >> 4) << (2 * (j >> 2))) << (8 * (hi_b & 3));
        }
        if (!valid) return;
        // block_q3_K: hmask[32], qs[64], scales[12], d        (2-byte aligned)
        uint8_t* y = job.y + out_offset<256, 256, 110>(sl, 0);
        if (sub < 2) {
            uint8_t* p = y + sub * 16;
            st4_a2(p, hm[0]); st4_a2(p + 4, hm[1]); st4_a2(p + 8, hm[2]); st4_a2(p + 12, hm[3]);
        }
        if (qwriter) {
            uint8_t* p = y + 32 + (sub >> 3) * 32 + (sub & 1) * 16;
            st4_a2(p, q[0]); st4_a2(p + 4, q[1]); st4_a2(p + 8, q[2]); st4_a2(p + 12, q[3]);
        }
        if (sub == 2) { st4_a2(y + 96, s12[0]); st4_a2(y + 100, s12[1]); st4_a2(y + 104, s12[2]); }
        if (sub == 3) st2(y + 108, dh);
    }
};

// ================================================================================================
// Q4_K and Q5_K share everything but the code range and the fifth bit plane.
template <int BITS> struct Q45K {
    static constexpr int SLAB = 256, SUB = 32, LANES = 8, QK = 256, BS = BITS == 4 ? 144 : 176;
    static constexpr int NMAX = BITS == 4 ? 15 : 31;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid) {
        float x[32], wt[32];
        load_vals<DT, 32>(job.x, sl.x + sub * 32, x);
        QkxBest b;
        float sw = 0.f;
        if (IMX) {
            const float sum_x2 = ordered_sumsq<32, 8>(x, sub);
            const float sigma2 = fmul(fmul(2.f, sum_x2), 1.0f / 256);
            float qw[32];
            load_f32<32>(job.w, sl.w + sub * 32, qw);
#pragma unroll
            for (int l = 0; l < 32; ++l) wt[l] = fmul(qw[l], fsqrt(fadd(sigma2, fmul(x[l], x[l]))));
#pragma unroll
            for (int l = 0; l < 32; ++l) sw = fadd(sw, wt[l]);
            b = make_qkx_quants<32, true>(NMAX, x, wt, -0.9f, 0.05f, 36, false);
        } else {
            float sum_x2 = 0.f;
#pragma unroll
            for (int l = 0; l < 32; ++l) sum_x2 = fadd(sum_x2, fmul(x[l], x[l]));
            const float av_x = fsqrt(fmul(sum_x2, 1.0f / 32));
#pragma unroll
            for (int l = 0; l < 32; ++l) wt[l] = fadd(av_x, fabsf(x[l]));
            if (BITS == 4) b = make_qkx_quants<32, false>(15, x, wt, -1.f, 0.1f, 20, false);
            else           b = make_qkx_quants<32, false>(31, x, wt, -0.5f, 0.1f, 15, false);
        }
        float scales[8], mins[8];
        gather<8>(b.scale, scales);
        gather<8>(b.the_min, mins);
        int ls, lm;
        uint16_t dh, dmh;
        if (IMX) {
            float sws[8];
            gather<8>(sw, sws);
            int Ls[8], Lm[8];
            const float d_block = make_qp_quants<8>(63, scales, Ls, sws);
            const float m_block = make_qp_quants<8>(63, mins, Lm, sws);
            ls = 0; lm = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) if (j == sub) { ls = Ls[j]; lm = Lm[j]; }
            if (BITS == 5) { ls = min(63, ls); lm = min(63, lm); }
            dh = f32_to_f16(d_block); dmh = f32_to_f16(m_block);
        } else {
            float max_scale = 0.f, max_min = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (scales[j] > max_scale) max_scale = scales[j];
                if (mins[j] > max_min) max_min = mins[j];
            }
            const float inv_scale = max_scale > 0.f ? fdiv(63.f, max_scale) : 0.f;
            const float inv_min = max_min > 0.f ? fdiv(63.f, max_min) : 0.f;
            ls = nearest_int(fmul(inv_scale, b.scale)) & 0xff;    // uint8_t ls
            lm = nearest_int(fmul(inv_min, b.the_min)) & 0xff;
            ls = min(63, ls); lm = min(63, lm);
            dh = f32_to_f16(fdiv(max_scale, c_div[DIV_63]));
            dmh = f32_to_f16(fdiv(max_min, c_div[DIV_63]));
        }
        ls &= 0xff; lm &= 0xff;
        // get_scale_min_k4 returns the 6-bit values that were packed: sc = ls & 63 ... the packing
        // keeps only 6 bits of each (ggml-quants.c:1495-1502), so mask here.
        const int sc = ls & 63, mq = lm & 63;
        const float d = fmul(f16_to_f32(dh), (float)sc);
        uint32_t lo[4] = {0, 0, 0, 0};     // 4-bit codes, 8 per word
        unsigned hi = 0;                   // fifth bits (Q5_K)
        const float dm = fmul(f16_to_f32(dmh), (float)mq);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            int l;
            if (d != 0.f) l = clampi(nearest_int(fdiv(fadd(x[i], dm), d)), 0, NMAX);
            else l = IMX ? qkx_code<32, true>(b, NMAX, x[i]) : qkx_code<32, false>(b, NMAX, x[i]);
            if (BITS == 5 && l > 15) { l -= 16; hi |= 1u << i; }
            lo[i >> 3] |= (uint32_t)l << (4 * (i & 7));
        }
        // qs: byte l of pair k = code(sub 2k, l) | code(sub 2k+1, l) << 4.  Lane pairs swap halves: the even
        // lane emits bytes 0..15, the odd lane bytes 16..31.
        const bool odd = sub & 1;
        uint32_t mine[2], theirs[2];
        // what I keep: my codes for the half I emit; what I send: my codes for the half the partner emits
        mine[0] = odd ? lo[2] : lo[0]; mine[1] = odd ? lo[3] : lo[1];
        uint32_t send0 = odd ? lo[0] : lo[2], send1 = odd ? lo[1] : lo[3];
        theirs[0] = __shfl_xor_sync(SG_FULL, send0, 1);
        theirs[1] = __shfl_xor_sync(SG_FULL, send1, 1);
        const uint32_t low0 = odd ? theirs[0] : mine[0], low1 = odd ? theirs[1] : mine[1];   // low nibbles: even lane's codes
        const uint32_t hig0 = odd ? mine[0] : theirs[0], hig1 = odd ? mine[1] : theirs[1];
        uint32_t qs[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t word = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = 4 * m + k;                    // code index within the 16 this lane emits
                const uint32_t a = ((i < 8 ? low0 : low1) >> (4 * (i & 7))) & 0xF;
                const uint32_t c = ((i < 8 ? hig0 : hig1) >> (4 * (i & 7))) & 0xF;
                word |= (a | (c << 4)) << (8 * k);
            }
            qs[m] = word;
        }
        // scales[12] (ggml-quants.c:1495-1502)
        int lss[8], lms[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { lss[j] = gshfl<8>(ls, j); lms[j] = gshfl<8>(lm, j); }
        uint32_t s12[3] = {0, 0, 0};
        {
            uint8_t sb[12];
#pragma unroll
            for (int j = 0; j < 12; ++j) sb[j] = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint8_t a = (uint8_t)lss[j], c = (uint8_t)lms[j];
                if (j < 4) { sb[j] = a; sb[j + 4] = c; }
                else {
                    sb[j + 4] = (a & 0xF) | ((c & 0xF) << 4);
                    sb[j - 4] |= (uint8_t)((a >> 4) << 6);
                    sb[j] |= (uint8_t)((c >> 4) << 6);
                }
            }
#pragma unroll
            for (int j = 0; j < 12; ++j) s12[j >> 2] |= (uint32_t)sb[j] << (8 * (j & 3));
        }
        uint32_t qh = 0;
        if (BITS == 5) {
            // qh[j] bit s = fifth bit of weight j of sub-block s (ggml-quants.c:1711-1726); lane s builds qh[4s..4s+3]
            unsigned his[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) his[j] = gshfl<8>(hi, j);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t byte = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) byte |= ((his[j] >> (4 * sub + k)) & 1) << j;
                qh |= byte << (8 * k);
            }
        }
        if (!valid) return;
        uint8_t* y = job.y + out_offset<256, 256, BS>(sl, 0);
        if (sub == 0) st16(y, (uint32_t)dh | ((uint32_t)dmh << 16), s12[0], s12[1], s12[2]);
        if (BITS == 5) st4(y + 16 + 4 * sub, qh);
        uint8_t* p = y + (BITS == 4 ? 16 : 48) + (sub >> 1) * 32 + (odd ? 16 : 0);
        st16(p, qs[0], qs[1], qs[2], qs[3]);
    }
};

// ================================================================================================
struct Q6K {
    static constexpr int SLAB = 256, SUB = 16, LANES = 16, QK = 256, BS = 210;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid) {
        float x[16], qw[16];
        load_vals<DT, 16>(job.x, sl.x + sub * 16, x);
        QxBest b;
        if (IMX) {
            load_f32<16>(job.w, sl.w + sub * 16, qw);
            b = make_qx_quants<16, true>(32, x, qw);
        } else {
            b = make_qx_quants<16, false>(32, x, x);
        }
        float scales[16];
        gather<16>(b.scale, scales);
        float max_scale = 0.f, max_abs_scale = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float a = fabsf(scales[j]);
            if (a > max_abs_scale) { max_abs_scale = a; max_scale = scales[j]; }
        }
        uint8_t* y = job.y + out_offset<256, 256, 210>(sl, 0);
        // an all-zero super-block is stored as 210 zero bytes (ggml-quants.c:1895-1900); the test is uniform
        // over the 16 lanes of the group, but the other group of the warp still needs this one's shuffles
        const bool zero = max_abs_scale < SG_GROUP_MAX_EPS;
        if (zero) max_scale = 1.f;
        const float iscale = fdiv(-128.f, max_scale);
        const uint16_t dh = f32_to_f16(frcp(iscale));
        const int sc = (int)(int8_t)min(127, nearest_int(fmul(iscale, b.scale)));
        const float d = fmul(f16_to_f32(dh), (float)sc);
        uint32_t lo[2] = {0, 0};      // low nibbles, 8 per word
        unsigned hi = 0;              // upper two bits, 2 per weight
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int l;
            if (d != 0.f) l = clampi(nearest_int(fdiv(x[i], d)), -32, 31) + 32;
            else l = qx_code(b, 32, x[i]);
            lo[i >> 3] |= (uint32_t)(l & 0xF) << (4 * (i & 7));
            hi |= (unsigned)(l >> 4) << (2 * i);
        }
        // ql / qh layout (ggml-quants.c:1922-1934).  Within a 128-weight half (8 lanes, q = 0..7, weights
        // 16q..16q+15): ql[l] = w[l] | w[l+64] << 4, ql[l+32] = w[l+32] | w[l+96] << 4 for l < 32, i.e. ql byte
        // group g (16 bytes, g = 0..3) pairs lane g with lane g + 4.  qh[l] = hi(w[l]) | hi(w[l+32]) << 2 |
        // hi(w[l+64]) << 4 | hi(w[l+96]) << 6: qh byte group g (g = 0,1) combines lanes g, g+2, g+4, g+6.
        const int half = sub >> 3, q = sub & 7;
        const uint32_t p0 = gshfl<16>(lo[0], half * 8 + (q & 3) + 4), p1 = gshfl<16>(lo[1], half * 8 + (q & 3) + 4);
        unsigned h4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) h4[k] = gshfl<16>(hi, half * 8 + (q & 1) + 2 * k);
        int scs[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) scs[j] = gshfl<16>(sc, j);
        if (!valid) return;
        if (zero) {
#pragma unroll
            for (int k = 0; k < 6; ++k) st2(y + sub * 12 + 2 * k, 0);
            if (sub < 9) st2(y + 192 + 2 * sub, 0);
            return;
        }
        if (q < 4) {          // 16 bytes of ql
            uint8_t* p = y + half * 64 + q * 16;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                uint32_t word = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = 4 * m + k;
                    const uint32_t a = (lo[i >> 3] >> (4 * (i & 7))) & 0xF;
                    const uint32_t c = ((i < 8 ? p0 : p1) >> (4 * (i & 7))) & 0xF;
                    word |= (a | (c << 4)) << (8 * k);
                }
                st4_a2(p + 4 * m, word);
            }
        } else if (q < 6) {   // 16 bytes of qh
            uint8_t* p = y + 128 + half * 32 + (q & 1) * 16;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                uint32_t word = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = 4 * m + k;
                    const uint32_t byte = ((h4[0] >> (2 * i)) & 3) | (((h4[1] >> (2 * i)) & 3) << 2) |
                                          (((h4[2] >> (2 * i)) & 3) << 4) | (((h4[3] >> (2 * i)) & 3) << 6);
                    word |= byte << (8 * k);
                }
                st4_a2(p + 4 * m, word);
            }
        } else if (q == 6) {  // 8 of the 16 scales
#pragma unroll
            for (int k = 0; k < 4; ++k)
                st2(y + 192 + half * 8 + 2 * k,
                    (uint32_t)(scs[half * 8 + 2 * k] & 0xff) | ((uint32_t)(scs[half * 8 + 2 * k + 1] & 0xff) << 8));
        } else if (half == 0) {
            st2(y + 208, dh);
        }
    }
};

}  // namespace sg
