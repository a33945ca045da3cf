// Context model of the quantiser-aware residual coder ("QR"): which symbols a stored block turns into, given
// its prediction and the BF16 seed, and in which context each is coded.  The symbol and context definitions are
// the reference's (seedpack/qr.py:136-377) - they fix the archive bytes - restated here per component:
//
//   fields   the block's scale fields as integers (fp16 d / dmin / m, 4-6-8 bit sub-scales), each coded as a
//            delta against the predicted block's field; model 2 first rescales predicted sub-scales to the
//            true super-scale (qr.py:203-283)
//   codes    per weight: residual of the stored code against round((seed - c) / a) computed with the TRUE
//            scales, mirrored so that the likely side is positive; context = uncertainty bin x margin bin, or
//            (model 2, exact seed) row-position bin x finer margin (qr.py:295-377)
//
// Floating point follows the reference exactly: explicit round-to-nearest intrinsics where it uses them, plain
// IEEE operations (no contraction: the library is built with -fmad=false) elsewhere.
#pragma once
#include "common.cuh"

namespace sg {
namespace qr {

constexpr int NSB_MAX = 20;
constexpr int NTAB = NSB_MAX + 64 + 2;      // field contexts, (uncertainty x margin) code contexts, block flag
constexpr int FLAG = NSB_MAX + 64;          // + previous block's flag
constexpr int CODE2 = NTAB;                 // model 2: position (8) x margin (16)
constexpr int GRANK2 = NTAB + 128;          // grid rank: clearness (4) x position (4)
constexpr int GSIGN2 = NTAB + 144;          // grid signs: (level 0, |u| bin) (16) x position (4)
constexpr int NTAB2 = NTAB + 208;           // 294
constexpr int FESC_LO = 8, FESC_HI = 9;
constexpr int GRID_RANK = NSB_MAX, GRID_SIGN = NSB_MAX + 8, GRID_SHIFT = NSB_MAX + 24;
constexpr int HBOFF_COL = 3;
constexpr int MAXF = 34;

typedef unsigned char uchar;

struct TM { long long blk0, seed_off; int seed_type, cols; long long imx_off; };   // per tensor (qr.py:898)
struct SG { int t, nb; long long b0; };                                           // per segment (qr.py:900)

SG_DEVINL float kv(int i) {      // IQ4 levels
    switch (i) { case 0: return -127.f; case 1: return -104.f; case 2: return -83.f; case 3: return -65.f; case 4: return -49.f;
                 case 5: return -35.f; case 6: return -22.f; case 7: return -10.f; case 8: return 1.f; case 9: return 13.f;
                 case 10: return 25.f; case 11: return 38.f; case 12: return 53.f; case 13: return 69.f; case 14: return 89.f; }
    return 113.f;
}

// fp16 bits -> float, by cases (qr.py:76-85)
SG_DEVINL float h2fv(unsigned h) {
    unsigned s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023, f;
    if (e == 0) {
        if (m == 0) f = s << 31;
        else { int ee = 113; while (!(m & 1024)) { m <<= 1; ee--; } m &= 1023; f = (s << 31) | ((unsigned)ee << 23) | (m << 13); }
    } else if (e == 31) f = (s << 31) | 0x7f800000u | (m << 13);
    else f = (s << 31) | ((e + 112) << 23) | (m << 13);
    return __uint_as_float(f);
}
SG_DEVINL int u16(const uchar* b) { return b[0] | (b[1] << 8); }
SG_DEVINL unsigned u32(const uchar* b) { return b[0] | (b[1] << 8) | (b[2] << 16) | ((unsigned)b[3] << 24); }
SG_DEVINL float h2f(const uchar* p) { return h2fv((unsigned)u16(p)); }

__host__ SG_DEVINL int qk_of(int T) { return (T == 2 || T == 3 || T == 6 || T == 7 || T == 8 || T == 20) ? 32 : T == 42 ? 64 : 256; }
SG_DEVINL int bs_of(int T) {
    switch (T) { case 2: return 18; case 3: return 20; case 6: return 22; case 7: return 24; case 8: return 34; case 10: return 84;
                 case 11: return 110; case 12: return 144; case 13: return 176; case 14: return 210; case 20: return 18;
                 case 23: return 136; case 42: return 18; case 16: return 66; case 17: return 74; case 18: return 98;
                 case 19: return 50; case 21: return 110; case 22: return 82; case 29: return 56; }
    return 1;
}
__host__ SG_DEVINL bool is_grid(int T) { return T == 16 || T == 17 || T == 18 || T == 19 || T == 21 || T == 22 || T == 29; }
SG_DEVINL int qmin_of(int T) { return T == 8 ? -128 : 0; }
SG_DEVINL int qmax_of(int T) {
    switch (T) { case 10: case 42: return 3; case 11: return 7; case 6: case 7: case 13: return 31; case 14: return 63; case 8: return 127; }
    return 15;
}
SG_DEVINL bool nonlin(int T) { return T == 20 || T == 23; }
SG_DEVINL int sublen_of(int T) { return (T == 10 || T == 11 || T == 14) ? 16 : 32; }

SG_DEVINL void scale_min_k4(int j, const uchar* q, int& sc, int& m) {
    if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}
// 6-bit scale `is` of a Q3_K block, as a signed byte (the value before the -32 offset)
SG_DEVINL int q3k_scale(const uchar* s, int is) {
    const int lo = is < 8 ? (s[is] & 15) : (s[is - 8] >> 4);
    const int hi = (s[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
    return (int)(signed char)(lo | (hi << 4));
}

// ---- codes ------------------------------------------------------------------------------------------------
// Where the code of weight w lives: `lo_bits` bits at (lo_byte, lo_shift) and, for the 5/6-bit types and Q3_K,
// `hi_bits` more at (hi_byte, hi_shift).  One locator serves reading and writing.
struct CodeLoc { int lo_byte, lo_shift, lo_bits, hi_byte, hi_shift, hi_bits; };
SG_DEVINL CodeLoc code_loc(int T, int w) {
    CodeLoc L = {0, 0, 4, 0, 0, 0};
    const int half = (w >> 4) & 1, l16 = w & 15;             // legacy 32-blocks: low nibbles = first 16 weights
    const int n128 = w >> 7, plane = (w & 127) >> 5, l32 = w & 31;
    switch (T) {
        case 2: case 20: L.lo_byte = 2 + l16; L.lo_shift = 4 * half; break;
        case 3: L.lo_byte = 4 + l16; L.lo_shift = 4 * half; break;
        case 6: L.lo_byte = 6 + l16; L.lo_shift = 4 * half; L.hi_byte = 2 + (w >> 3); L.hi_shift = w & 7; L.hi_bits = 1; break;
        case 7: L.lo_byte = 8 + l16; L.lo_shift = 4 * half; L.hi_byte = 4 + (w >> 3); L.hi_shift = w & 7; L.hi_bits = 1; break;
        case 8: L.lo_byte = 2 + w; L.lo_bits = 8; break;
        case 10: L.lo_byte = 16 + 32 * n128 + l32; L.lo_shift = 2 * plane; L.lo_bits = 2; break;
        case 11: L.lo_byte = 32 + 32 * n128 + l32; L.lo_shift = 2 * plane; L.lo_bits = 2;
                 L.hi_byte = l32; L.hi_shift = 4 * n128 + plane; L.hi_bits = 1; break;
        case 12: L.lo_byte = 16 + 32 * (w >> 6) + l32; L.lo_shift = 4 * ((w >> 5) & 1); break;
        case 13: L.lo_byte = 48 + 32 * (w >> 6) + l32; L.lo_shift = 4 * ((w >> 5) & 1);
                 L.hi_byte = 16 + l32; L.hi_shift = w >> 5; L.hi_bits = 1; break;
        case 14: L.lo_byte = 64 * n128 + l32 + 32 * (plane & 1); L.lo_shift = 4 * (plane >> 1);
                 L.hi_byte = 128 + 32 * n128 + l32; L.hi_shift = 2 * plane; L.hi_bits = 2; break;
        case 23: L.lo_byte = 8 + 16 * (w >> 5) + l16; L.lo_shift = 4 * half; break;
        case 42: L.lo_byte = 2 + (w >> 2); L.lo_shift = 2 * (w & 3); L.lo_bits = 2; break;
    }
    return L;
}
SG_DEVINL int get_code(int T, const uchar* b, int w) {
    const CodeLoc L = code_loc(T, w);
    if (T == 8) return (int)(signed char)b[L.lo_byte];
    int q = (b[L.lo_byte] >> L.lo_shift) & ((1 << L.lo_bits) - 1);
    if (L.hi_bits) q |= ((b[L.hi_byte] >> L.hi_shift) & ((1 << L.hi_bits) - 1)) << L.lo_bits;
    return q;
}
// bits are OR-ed in: the code bytes must be zero before
SG_DEVINL void put_code(int T, uchar* b, int w, int q) {
    const CodeLoc L = code_loc(T, w);
    if (T == 8) { b[L.lo_byte] = (uchar)q; return; }
    if (L.hi_bits) {
        b[L.lo_byte] |= (uchar)((q & ((1 << L.lo_bits) - 1)) << L.lo_shift);
        b[L.hi_byte] |= (uchar)(((q >> L.lo_bits) & ((1 << L.hi_bits) - 1)) << L.hi_shift);
    } else if (L.lo_bits == 2) b[L.lo_byte] |= (uchar)((q & 3) << L.lo_shift);
    else b[L.lo_byte] |= (uchar)(q << L.lo_shift);           // 4-bit single-part codes are OR-ed in unmasked (qr.py:156-175)
}

// ---- scale fields ------------------------------------------------------------------------------------------
// A block's scale fields as an integer vector: [0] fp16 scale (bits), [1] fp16 min where the type has one, then
// the sub-block scales (and sub-block mins).  unpack_fields / pack_fields are inverse on every valid block.
__host__ SG_DEVINL int nfield(int T) {
    switch (T) { case 2: case 6: case 8: case 20: case 42: return 1; case 3: case 7: return 2; case 10: return 34;
                 case 11: case 14: return 17; case 12: case 13: return 18; case 23: return 9;
                 case 16: case 18: case 19: case 21: return 9; case 17: case 22: case 29: return 17; }
    return 0;
}
// 0 fp16 scale, 1 fp16 min, 2 sub-scale, 3 sub-min
SG_DEVINL int fkind(int T, int k) {
    if (k == 0) return 0;
    const bool has_min = T == 3 || T == 7 || T == 10 || T == 12 || T == 13;
    if (k == 1 && has_min) return 1;
    if (T == 10) return k < 18 ? 2 : 3;
    if (T == 12 || T == 13) return k < 10 ? 2 : 3;
    return 2;
}
SG_DEVINL void unpack_fields(int T, const uchar* b, int* v) {
    switch (T) {
        case 2: case 6: case 8: case 20: case 42: v[0] = u16(b); return;
        case 3: case 7: v[0] = u16(b); v[1] = u16(b + 2); return;
        case 10: v[0] = u16(b + 80); v[1] = u16(b + 82);
                 for (int j = 0; j < 16; ++j) { v[2 + j] = b[j] & 15; v[18 + j] = b[j] >> 4; }
                 return;
        case 11: v[0] = u16(b + 108); for (int j = 0; j < 16; ++j) v[1 + j] = q3k_scale(b + 96, j); return;
        case 12: case 13: v[0] = u16(b); v[1] = u16(b + 2);
                 for (int j = 0; j < 8; ++j) scale_min_k4(j, b + 4, v[2 + j], v[10 + j]);
                 return;
        case 14: v[0] = u16(b + 208); for (int j = 0; j < 16; ++j) v[1 + j] = (int)(signed char)b[192 + j]; return;
        case 23: { v[0] = u16(b); const int sh = u16(b + 2);
                   for (int j = 0; j < 8; ++j) v[1 + j] = ((b[4 + j / 2] >> (4 * (j & 1))) & 15) | (((sh >> (2 * j)) & 3) << 4);
                   return; }
        case 16: v[0] = u16(b); for (int j = 0; j < 8; ++j) v[1 + j] = b[2 + 8 * j + 7] >> 4; return;
        case 18: v[0] = u16(b); for (int j = 0; j < 8; ++j) v[1 + j] = b[66 + 4 * j + 3] >> 4; return;
        case 17: v[0] = u16(b); for (int j = 0; j < 16; ++j) v[1 + j] = (b[66 + j / 2] >> (4 * (j & 1))) & 15; return;
        case 22: v[0] = u16(b); for (int j = 0; j < 16; ++j) v[1 + j] = (b[74 + j / 2] >> (4 * (j & 1))) & 15; return;
        case 21: v[0] = u16(b); for (int j = 0; j < 8; ++j) v[1 + j] = (b[106 + j / 2] >> (4 * (j & 1))) & 15; return;
        case 19: v[0] = u16(b); for (int j = 0; j < 8; ++j) v[1 + j] = b[34 + 2 * j + 1] >> 4; return;     // 3-bit scale + shift bit
        case 29: v[0] = (u16(b + 48) >> 12) | ((u16(b + 50) >> 8) & 0xf0) | ((u16(b + 52) >> 4) & 0xf00) | (u16(b + 54) & 0xf000);
                 for (int j = 0; j < 16; ++j) v[1 + j] = (u16(b + 48 + 2 * (j >> 2)) >> (3 * (j & 3))) & 7;
                 return;
    }
}
SG_DEVINL void put16(uchar* b, int v) { b[0] = (uchar)(v & 255); b[1] = (uchar)((v >> 8) & 255); }
// writes every scale field; the bytes that hold them must be zero before (the grid types share bytes with
// grid indices and signs, which are OR-ed in separately)
SG_DEVINL void pack_fields(int T, uchar* b, const int* v) {
    switch (T) {
        case 2: case 6: case 8: case 20: case 42: put16(b, v[0]); return;
        case 3: case 7: put16(b, v[0]); put16(b + 2, v[1]); return;
        case 10: put16(b + 80, v[0]); put16(b + 82, v[1]);
                 for (int j = 0; j < 16; ++j) b[j] = (uchar)((v[2 + j] & 15) | ((v[18 + j] & 15) << 4));
                 return;
        case 11: put16(b + 108, v[0]);
                 for (int j = 0; j < 16; ++j) {
                     b[96 + (j & 7)] |= (uchar)((v[1 + j] & 15) << (4 * (j >> 3)));
                     b[104 + (j & 3)] |= (uchar)(((v[1 + j] >> 4) & 3) << (2 * (j >> 2)));
                 }
                 return;
        case 12: case 13: put16(b, v[0]); put16(b + 2, v[1]);
                 for (int j = 0; j < 4; ++j) {
                     b[4 + j] = (uchar)(v[2 + j] | ((v[6 + j] >> 4) << 6));
                     b[8 + j] = (uchar)(v[10 + j] | ((v[14 + j] >> 4) << 6));
                     b[12 + j] = (uchar)((v[6 + j] & 15) | ((v[14 + j] & 15) << 4));
                 }
                 return;
        case 14: put16(b + 208, v[0]); for (int j = 0; j < 16; ++j) b[192 + j] = (uchar)v[1 + j]; return;
        case 23: { put16(b, v[0]); int sh = 0;
                   for (int j = 0; j < 8; ++j) { b[4 + j / 2] |= (uchar)((v[1 + j] & 15) << (4 * (j & 1))); sh |= ((v[1 + j] >> 4) & 3) << (2 * j); }
                   put16(b + 2, sh); return; }
        case 16: put16(b, v[0]); for (int j = 0; j < 8; ++j) b[2 + 8 * j + 7] |= (uchar)((v[1 + j] & 15) << 4); return;
        case 18: put16(b, v[0]); for (int j = 0; j < 8; ++j) b[66 + 4 * j + 3] |= (uchar)((v[1 + j] & 15) << 4); return;
        case 17: put16(b, v[0]); for (int j = 0; j < 16; ++j) b[66 + j / 2] |= (uchar)((v[1 + j] & 15) << (4 * (j & 1))); return;
        case 22: put16(b, v[0]); for (int j = 0; j < 16; ++j) b[74 + j / 2] |= (uchar)((v[1 + j] & 15) << (4 * (j & 1))); return;
        case 21: put16(b, v[0]); for (int j = 0; j < 8; ++j) b[106 + j / 2] |= (uchar)((v[1 + j] & 15) << (4 * (j & 1))); return;
        case 19: put16(b, v[0]); for (int j = 0; j < 8; ++j) b[34 + 2 * j + 1] |= (uchar)((v[1 + j] & 15) << 4); return;
        case 29: for (int j = 0; j < 16; ++j) {
                     const int s = (v[1 + j] & 7) << (3 * (j & 3));
                     b[48 + 2 * (j >> 2)] |= (uchar)(s & 255); b[49 + 2 * (j >> 2)] |= (uchar)(s >> 8);
                 }
                 for (int i = 0; i < 4; ++i) b[49 + 2 * i] |= (uchar)(((v[0] >> (4 * i)) & 15) << 4);
                 return;
    }
}
// What field k is coded against, given the true fp16 fields t0 (and t1) that were coded before it.  Model 1: the
// predicted block's field.  Model 2 rescales the predicted sub-scales (K-quants: and sub-mins) to the true
// super-scale, so that sub-scale x super-scale stays the prediction's (qr.py:264-283).  pv = unpacked prediction.
SG_DEVINL int fpred(int T, int mv, const int* pv, int k, int t0, int t1) {
    const int pr = pv[k];
    const bool grid = is_grid(T), two = T == 10 || T == 12 || T == 13;
    if (mv < 2 || !(grid || two || T == 11 || T == 14 || T == 23) || k < (two ? 2 : 1)) return pr;
    const int ref = two && k >= (T == 10 ? 18 : 10) ? 1 : 0;
    const float tv = h2fv((unsigned)(ref ? t1 : t0)), pf = h2fv((unsigned)pv[ref]);
    if (tv == 0.f || !isfinite(tv) || !isfinite(pf)) return pr;
    if (grid) {                                   // value d (2 ls + 1); IQ1_S keeps its shift bit
        const int hi = (T == 19 || T == 29) ? 7 : 15, ls = T == 19 ? (pr & 7) : pr;
        const float v = rintf(__fmul_rn(__fsub_rn(__fdiv_rn(__fmul_rn((float)(2 * ls + 1), pf), tv), 1.f), 0.5f));
        const int q = (int)fminf(fmaxf(v, 0.f), (float)hi);
        return T == 19 ? (pr & 8) | q : q;
    }
    if (T == 11 || T == 23) {                     // value d (ls - 32)
        const float v = rintf(__fdiv_rn(__fmul_rn((float)(pr - 32), pf), tv));
        return (int)fminf(fmaxf(v, -32.f), 31.f) + 32;
    }
    const float v = rintf(__fdiv_rn(__fmul_rn((float)pr, pf), tv));
    return T == 14 ? (int)fminf(fmaxf(v, -128.f), 127.f) : (int)fminf(fmaxf(v, 0.f), T == 10 ? 15.f : 63.f);
}
SG_DEVINL int pos8(long long col, int cols) { return cols <= 0 || col < 256 ? 0 : 1 + min(6, (int)(col * 7 / cols)); }
SG_DEVINL int pos4(long long col, int cols) { return cols <= 0 || col < 256 ? 0 : 1 + min(2, (int)(col * 3 / cols)); }
SG_DEVINL int fctx(int kind, int any) { return kind * 2 + any; }

// value = a * code + c (IQ4 types: a * level[code]) for the sub-block `sub` (= w / sublen) of a block whose
// unpacked fields are v (qr.py:295-316)
SG_DEVINL void wscale(int T, const int* v, int sub, float& a, float& c) {
    const float d = h2fv((unsigned)v[0]);
    c = 0.f;
    switch (T) {
        case 2: a = d; c = __fmul_rn(-8.f, a); return;
        case 3: case 7: a = d; c = h2fv((unsigned)v[1]); return;
        case 6: a = d; c = __fmul_rn(-16.f, a); return;
        case 8: case 20: a = d; return;
        case 42: a = d; c = -a; return;                                     // codes 0..3 are -1..2 x d
        case 10: a = __fmul_rn(d, (float)v[2 + sub]); c = -__fmul_rn(h2fv((unsigned)v[1]), (float)v[18 + sub]); return;
        case 11: a = __fmul_rn(d, (float)(v[1 + sub] - 32)); c = __fmul_rn(-4.f, a); return;
        case 12: case 13: a = __fmul_rn(d, (float)v[2 + sub]); c = -__fmul_rn(h2fv((unsigned)v[1]), (float)v[10 + sub]); return;
        case 14: a = __fmul_rn(d, (float)v[1 + sub]); c = __fmul_rn(-32.f, a); return;
        case 23: a = __fmul_rn(d, (float)(v[1 + sub] - 32)); return;
    }
    a = 0.f;
}

// The seed's value of weight gw of the tensor and its half uncertainty (qr.py:323-344).  Seed types: 30 BF16, 0 F32,
// 1 F16 (exact: h = 0), 98 no seed (x = 0, h = the column's RMS), 99 explicit (x, h) pairs, or a scalar-code quant type
// (a sibling quant standing in for a missing BF16 file: x = its dequantised weight a code + c, h = half a code step;
// the IQ4 level types: half the gap to the next level).  The host refuses every other type before a launch.
SG_DEVINL bool seed_is_quant(int ST) {
    switch (ST) { case 2: case 3: case 6: case 7: case 8: case 10: case 11: case 12: case 13: case 14: case 20: case 23: case 42: return true; }
    return false;
}
SG_DEVINL bool seed_known(int ST) { return ST == 30 || ST == 0 || ST == 1 || ST == 98 || ST == 99 || seed_is_quant(ST); }
SG_DEVINL void unpack_fields(int T, const uchar* b, int* v);
SG_DEVINL void wscale(int T, const int* v, int sub, float& a, float& c);
SG_DEVINL void seed_val(int ST, const uchar* sb, long long gw, float& x, float& h, int cols) {
    h = 0.f;
    if (ST == 30) { x = __uint_as_float((unsigned)reinterpret_cast<const unsigned short*>(sb)[gw] << 16); return; }
    if (ST == 0) { x = reinterpret_cast<const float*>(sb)[gw]; return; }
    if (ST == 1) { x = h2fv(reinterpret_cast<const unsigned short*>(sb)[gw]); return; }
    if (ST == 98) { x = 0.f; h = reinterpret_cast<const float*>(sb)[gw % cols]; return; }
    if (ST == 99) { const float* f = reinterpret_cast<const float*>(sb); x = f[2 * gw]; h = f[2 * gw + 1]; return; }
    const int qk = qk_of(ST), w = (int)(gw % qk);
    const uchar* blk = sb + (gw / qk) * bs_of(ST);
    int v[34];
    unpack_fields(ST, blk, v);
    float a, c;
    wscale(ST, v, w / sublen_of(ST), a, c);
    const int q = get_code(ST, blk, w);
    if (nonlin(ST)) {
        x = __fmul_rn(a, kv(q));
        const float g = q < 15 ? kv(q + 1) - kv(q) : kv(15) - kv(14);
        h = __fmul_rn(fabsf(a), 0.5f * g);
    } else {
        x = __fadd_rn(__fmul_rn(a, (float)q), c);
        h = __fmul_rn(fabsf(a), 0.5f);
    }
}

// predicted code r, mirror sign s and context of weight w from the TRUE block scales (qr.py:348-377)
SG_DEVINL void predict_code(int T, float a, float c, const uchar* pblk, int w, float x, float h, int hboff, int& r, int& s, int& ctx,
                            int mv, int p8) {
    float u, hu;
    if (nonlin(T)) {
        const float t = __fdiv_rn(x, a);
        int i = 0;
        while (i < 14 && t >= kv(i + 1)) i++;
        const float g = kv(i + 1) - kv(i);
        u = __fadd_rn((float)i, __fdiv_rn(__fsub_rn(t, kv(i)), g));
        hu = __fdiv_rn(h, __fmul_rn(fabsf(a), g));
    } else {
        u = __fdiv_rn(__fsub_rn(x, c), a);
        // exact seeds carry h = 0: 0 / |a| is 0 unless a is 0 or NaN, where it is NaN - no division needed to know that
        hu = h == 0.f ? ((a == 0.f || a != a) ? __int_as_float(0x7fc00000) : 0.f) : __fdiv_rn(h, fabsf(a));
    }
    if (!isfinite(u) || !isfinite(hu)) { r = get_code(T, pblk, w); s = 1; ctx = NSB_MAX + 63; return; }
    const float ru = rintf(u), fr = __fsub_rn(u, ru);
    const int q = (int)fmaxf(fminf(ru, (float)qmax_of(T)), (float)qmin_of(T));
    r = q; s = fr >= 0.f ? 1 : -1;
    int mb = min(7, (int)__fmul_rn(fabsf(fr), 16.f));
    if (hboff == HBOFF_COL) {
        s = 1;
        mb = min(7, max(0, (q - qmin_of(T)) * 8 / (qmax_of(T) - qmin_of(T) + 1)));
    }
    int hb = 0;
    if (hu > 0.f) { const int e = ilogbf(hu); hb = max(1, min(7, e + hboff)); }
    ctx = NSB_MAX + hb * 8 + mb;
    if (mv >= 2 && hu == 0.f && hboff != HBOFF_COL) ctx = CODE2 + p8 * 16 + min(15, (int)__fmul_rn(fabsf(fr), 32.f));
}

// ==== grid (IQ) types ===========================================================================================
// A unit = 8 consecutive weights: one lattice point (IQ3: two points of 4), one sign group, one scale.
SG_DEVINL int grid_size(int T) {
    switch (T) { case 16: case 18: return 256; case 17: case 21: return 512; case 22: return 1024; }
    return 2048;
}
SG_DEVINL bool parity_type(int T) { return T == 16 || T == 17 || T == 18; }      // 7 stored sign bits + parity

// where the index of lattice group g is kept: 8 low bits in a byte, the rest (1-3 bits) elsewhere
struct GidxLoc { int lo_byte, hi_byte, hi_shift, hi_bits; };
SG_DEVINL GidxLoc gidx_loc(int T, int g) {
    GidxLoc L = {2 + g, 0, 0, 0};
    switch (T) {
        case 16: L.lo_byte = 2 + 8 * (g >> 2) + (g & 3); break;
        case 17: L.lo_byte = 2 + 2 * g; L.hi_byte = 3 + 2 * g; L.hi_bits = 1; break;
        case 22: L.hi_byte = 66 + (g >> 2); L.hi_shift = 2 * (g & 3); L.hi_bits = 2; break;
        case 21: L.hi_byte = 66 + (g >> 3); L.hi_shift = g & 7; L.hi_bits = 1; break;
        case 19: L.hi_byte = -1; break;                                   // 3 bits inside the 16-bit qh word, below
        case 29: L.lo_byte = g; L.hi_byte = 32 + (g >> 1); L.hi_shift = 4 * (g & 1); L.hi_bits = 3; break;
    }
    return L;
}
SG_DEVINL int get_gidx(int T, const uchar* b, int g) {
    const GidxLoc L = gidx_loc(T, g);
    if (T == 19) return b[L.lo_byte] | (((u16(b + 34 + 2 * (g >> 2)) >> (3 * (g & 3))) & 7) << 8);
    int k = b[L.lo_byte];
    if (L.hi_bits) k |= ((b[L.hi_byte] >> L.hi_shift) & ((1 << L.hi_bits) - 1)) << 8;
    return k;
}
SG_DEVINL void put_gidx(int T, uchar* b, int g, int k) {
    const GidxLoc L = gidx_loc(T, g);
    if (T == 16 || T == 18) { b[L.lo_byte] |= (uchar)k; return; }
    b[L.lo_byte] |= (uchar)(k & 255);
    if (T == 19) {
        const int v = ((k >> 8) & 7) << (3 * (g & 3));
        b[34 + 2 * (g >> 2)] |= (uchar)(v & 255); b[35 + 2 * (g >> 2)] |= (uchar)(v >> 8);
        return;
    }
    b[L.hi_byte] |= (uchar)(((k >> 8) & ((1 << L.hi_bits) - 1)) << L.hi_shift);
}
// bit position (from the start of the block) of the stored sign of weight w; -1: the type stores no signs
SG_DEVINL int sign_bit_pos(int T, int w) {
    const int j = w & 7;
    switch (T) {
        case 16: return 8 * (2 + 8 * (w >> 5) + 4) + 7 * ((w >> 3) & 3) + j;
        case 17: return 8 * (2 + 2 * (w >> 3)) + 9 + j;
        case 18: return 8 * (66 + 4 * (w >> 5)) + 7 * ((w >> 3) & 3) + j;
        case 22: return 8 * (34 + (w >> 3)) + j;
        case 21: return 8 * (74 + (w >> 3)) + j;
    }
    return -1;
}
// 1 = weight w is stored negative.  Parity types keep 7 bits per group of 8; the eighth makes the count even.
SG_DEVINL int get_neg(int T, const uchar* b, int w) {
    if (sign_bit_pos(T, w) < 0) return 0;
    if (!parity_type(T)) { const int p = sign_bit_pos(T, w); return (b[p >> 3] >> (p & 7)) & 1; }
    const int p0 = sign_bit_pos(T, w & ~7);
    int s7 = 0;
    for (int i = 0; i < 7; ++i) s7 |= ((b[(p0 + i) >> 3] >> ((p0 + i) & 7)) & 1) << i;
    const int j = w & 7;
    return j < 7 ? (s7 >> j) & 1 : __popc(s7) & 1;
}
SG_DEVINL void put_neg(int T, uchar* b, int w) {         // parity types: only for w % 8 < 7
    const int p = sign_bit_pos(T, w);
    if (p >= 0) b[p >> 3] |= (uchar)(1 << (p & 7));
}
// IQ1_M: shift bit of unit u (bit 3 or 7 of the qh byte of its pair of units)
SG_DEVINL int get_shift(const uchar* b, int u) { return (b[32 + (u >> 1)] >> ((u & 1) ? 7 : 3)) & 1; }
SG_DEVINL void put_shift(uchar* b, int u) { b[32 + (u >> 1)] |= (u & 1) ? 0x80 : 0x08; }

// scale of unit u and the IQ1 shift: value = s (2 l + 1), IQ1: s (l - 1 + dl).  The quantisers' fudge factors on
// the stored fp16 are undone by multiplying with the rounded reciprocal (what the reference's GPU build does
// for a division by a literal, seedpack/cpukernels.py:254-264).  v = the block's unpacked fields.
SG_DEVINL void gscale(int T, const uchar* b, const int* v, int u, float& s, float& dl) {
    float d = h2fv((unsigned)v[0]);
    int ls;
    dl = 0.f;
    switch (T) {
        case 16: case 18: ls = v[1 + (u >> 2)]; break;
        case 17: ls = v[1 + (u >> 1)]; break;
        case 22: d = d * (1.0f / 0.9875f); ls = v[1 + (u >> 1)]; break;
        case 21: d = d * (1.0f / 1.033f); ls = v[1 + (u >> 2)]; break;
        case 19: d = d * (1.0f / 1.125f); ls = v[1 + (u >> 2)] & 7; dl = (v[1 + (u >> 2)] & 8) ? -0.125f : 0.125f; break;
        case 29: d = d * (1.0f / 1.1125f); ls = v[1 + (u >> 1)]; dl = get_shift(b, u) ? -0.125f : 0.125f; break;
        default: d = 0.f; ls = 0;
    }
    s = d * (float)(2 * ls + 1);
}
SG_DEVINL int gapctx(float d1, float d2) {
    const float g = (d2 - d1) / (d1 + 1e-30f);
    return (g >= 0.05f) + (g >= 0.2f) + (g >= 0.6f);
}

}  // namespace qr
}  // namespace sg
