/* TEST INFRASTRUCTURE - plain-C restatement of the reference quantisers (CPU checker, never shipped).
 *
 * Scalar, one row at a time, written from the algorithm descriptions in llama.cpp's ggml-quants.c as
 * vendored by the reference (seedpack/ggml/ggml-quants.c); each routine names the lines it follows.
 * Pinned against the reference's own compiled code (oracle/_ref, tests/test_oracle.py) on seeded inputs
 * and against the golden vectors in tests/golden/.  Compile with -ffp-contract=off -fno-fast-math.
 *
 * Covered here: fp16 conversions, nearest_int, the legacy block types Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q2_0
 * (plain and importance-weighted), make_qx_quants, make_qkx2/3_quants, make_qp_quants, make_q3_quants and
 * the K-quants Q2_K..Q6_K.  The IQ types are checked against oracle/_ref only.
 */
#include <math.h>
#include <string.h>

#include "oracle_port.h"

/* ---- helpers -------------------------------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ggml-impl.h:417-443 */
uint16_t op_f32_to_f16(float f) {
    float base = (fabsf(f) * u2f(0x77800000u)) * u2f(0x08800000u);
    const uint32_t w = f2u(f), shl1 = w + w, sign = w & 0x80000000u;
    uint32_t bias = shl1 & 0xFF000000u;
    if (bias < 0x71000000u) bias = 0x71000000u;
    base = u2f((bias >> 1) + 0x07800000u) + base;
    const uint32_t bits = f2u(base);
    const uint32_t nonsign = ((bits >> 13) & 0x7C00u) + (bits & 0xFFFu);
    return (uint16_t)((sign >> 16) | (shl1 > 0xFF000000u ? 0x7E00u : nonsign));
}
/* ggml-impl.h:396-415 */
float op_f16_to_f32(uint16_t h) {
    const uint32_t w = (uint32_t)h << 16, sign = w & 0x80000000u, two_w = w + w;
    const float norm = u2f((two_w >> 4) + (0xE0u << 23)) * u2f(0x07800000u);
    const float den = u2f((two_w >> 17) | (126u << 23)) - 0.5f;
    return u2f(sign | (two_w < (1u << 27) ? f2u(den) : f2u(norm)));
}
/* ggml-quants.c:621-626 */
int op_nearest_int(float f) {
    float v = f + 12582912.f;
    return (int)(f2u(v) & 0x007fffffu) - 0x00400000;
}
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }
static inline void put16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
static inline void put32(uint8_t *p, uint32_t v) { put16(p, (uint16_t)v); put16(p + 2, (uint16_t)(v >> 16)); }
#define EPS 1e-15f

/* ---- scale searches ------------------------------------------------------------------------------- */
/* ggml-quants.c:628-695, rmse_type 1; L gets codes offset by nmax */
float op_make_qx(int n, int nmax, const float *x, int8_t *L, const float *qw) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) { float ax = fabsf(x[i]); if (ax > amax) { amax = ax; max = x[i]; } }
    if (amax < EPS) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
    float iscale = -nmax / max, sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = clampi(op_nearest_int(iscale * x[i]), -nmax, nmax - 1);
        L[i] = (int8_t)(l + nmax);
        float w = qw ? qw[i] : x[i] * x[i];
        sumlx += w * x[i] * l; suml2 += w * l * l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.0f, best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (!is) continue;
        iscale = -(nmax + 0.1f * is) / max;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; ++i) {
            int l = clampi(op_nearest_int(iscale * x[i]), -nmax, nmax - 1);
            float w = qw ? qw[i] : x[i] * x[i];
            sumlx += w * x[i] * l; suml2 += w * l * l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) L[i] = (int8_t)(nmax + clampi(op_nearest_int(iscale * x[i]), -nmax, nmax - 1));
            scale = sumlx / suml2; best = scale * sumlx;
        }
    }
    return scale;
}

/* ggml-quants.c:697-754, do_rmse = true */
float op_make_q3(int n, int nmax, const float *x, int8_t *L) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) { float ax = fabsf(x[i]); if (ax > amax) { amax = ax; max = x[i]; } }
    if (amax < EPS) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
    float iscale = -nmax / max, sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = clampi(op_nearest_int(iscale * x[i]), -nmax, nmax - 1);
        L[i] = (int8_t)l;
        float w = x[i] * x[i];
        sumlx += w * x[i] * l; suml2 += w * l * l;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int changed = 0;
        for (int i = 0; i < n; ++i) {
            float w = x[i] * x[i];
            float slx = sumlx - w * x[i] * L[i];
            if (slx > 0) {
                float sl2 = suml2 - w * L[i] * L[i];
                int nl = clampi(op_nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
                if (nl != L[i]) {
                    slx += w * x[i] * nl; sl2 += w * nl * nl;
                    if (sl2 > 0 && slx * slx * suml2 > sumlx * sumlx * sl2) { L[i] = (int8_t)nl; sumlx = slx; suml2 = sl2; ++changed; }
                }
            }
        }
        if (!changed) break;
    }
    for (int i = 0; i < n; ++i) L[i] = (int8_t)(L[i] + nmax);
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

/* ggml-quants.c:799-878 (v3 = 0) and 993-1075 (v3 = 1) */
float op_make_qkx(int v3, int n, int nmax, const float *x, const float *wt, uint8_t *L, float *the_min,
                  float rmin, float rdelta, int nstep, int use_mad) {
    uint8_t Laux[64];
    float min = x[0], max = x[0], sum_w = wt[0], sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        sum_w += wt[i]; sum_x += wt[i] * x[i];
    }
    if (min > 0) min = 0;
    if (v3 ? max <= min : max == min) { memset(L, 0, n); *the_min = -min; return 0.f; }
    float iscale = nmax / (max - min), scale = 1 / iscale, best = 0;
    for (int i = 0; i < n; ++i) {
        int l = clampi(op_nearest_int(iscale * (x[i] - min)), 0, nmax);
        L[i] = (uint8_t)l;
        float diff = scale * L[i] + min - x[i];
        diff = use_mad ? fabsf(diff) : diff * diff;
        best += wt[i] * diff;
    }
    if (nstep < 1) { *the_min = -min; return scale; }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * is + nmax) / (max - min);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < n; ++i) {
            int l;
            if (v3) { float v = iscale * (x[i] - min); l = v > 0 ? op_nearest_int(v < nmax ? v : nmax) : 0; }
            else l = clampi(op_nearest_int(iscale * (x[i] - min)), 0, nmax);
            Laux[i] = (uint8_t)l;
            sum_l += wt[i] * l; sum_l2 += wt[i] * l * l; sum_xl += wt[i] * l * x[i];
        }
        float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float ts = (sum_w * sum_xl - sum_x * sum_l) / D, tm = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (tm > 0) { tm = 0; ts = sum_xl / sum_l2; }
            float err = 0;
            for (int i = 0; i < n; ++i) {
                float diff = ts * Laux[i] + tm - x[i];
                diff = use_mad ? fabsf(diff) : diff * diff;
                err += wt[i] * diff;
            }
            if (err < best) { memcpy(L, Laux, n); best = err; scale = ts; min = tm; }
        }
    }
    *the_min = -min;
    return scale;
}

/* ggml-quants.c:1077-1148 */
float op_make_qp(int n, int nmax, const float *x, uint8_t *L, const float *qw) {
    float max = 0;
    for (int i = 0; i < n; ++i) max = max > x[i] ? max : x[i];
    if (max < EPS) { memset(L, 0, n); return 0.f; }
    float iscale = nmax / max;
    for (int i = 0; i < n; ++i) L[i] = (uint8_t)op_nearest_int(iscale * x[i]);
    float scale = 1 / iscale, best = 0;
    for (int i = 0; i < n; ++i) { float d = x[i] - scale * L[i]; best += qw[i] * d * d; }
    for (int is = -4; is <= 4; ++is) {
        if (!is) continue;
        float isc = (0.1f * is + nmax) / max, sc = 1 / isc, mse = 0;
        for (int i = 0; i < n; ++i) {
            int l = op_nearest_int(isc * x[i]); if (l > nmax) l = nmax;
            float d = x[i] - sc * l; mse += qw[i] * d * d;
        }
        if (mse < best) { best = mse; iscale = isc; }
    }
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = op_nearest_int(iscale * x[i]); if (l > nmax) l = nmax;
        L[i] = (uint8_t)l;
        sumlx += qw[i] * x[i] * l; suml2 += qw[i] * l * l;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int changed = 0;
        for (int i = 0; i < n; ++i) {
            float w = qw[i], slx = sumlx - w * x[i] * L[i], sl2 = suml2 - w * L[i] * L[i];
            if (slx > 0 && sl2 > 0) {
                int nl = op_nearest_int(x[i] * sl2 / slx); if (nl > nmax) nl = nmax;
                if (nl != L[i]) {
                    slx += w * x[i] * nl; sl2 += w * nl * nl;
                    if (slx * slx * suml2 > sumlx * sumlx * sl2) { L[i] = (uint8_t)nl; sumlx = slx; suml2 = sl2; ++changed; }
                }
            }
        }
        if (!changed) break;
    }
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

/* ---- legacy blocks -------------------------------------------------------------------------------- */
static void pack_4bit(const uint8_t *L, uint8_t *qs) { for (int j = 0; j < 16; ++j) qs[j] = (uint8_t)(L[j] | (L[j + 16] << 4)); }
static uint32_t pack_5bit(const uint8_t *L, uint8_t *qs) {
    uint32_t qh = 0;
    for (int j = 0; j < 16; ++j) {
        qs[j] = (uint8_t)((L[j] & 0xF) | ((L[j + 16] & 0xF) << 4));
        qh |= (uint32_t)((L[j] & 0x10) >> 4) << j;
        qh |= (uint32_t)((L[j + 16] & 0x10) >> 4) << (j + 16);
    }
    return qh;
}
static float row_sigma2(const float *x, int64_t n) { float s = 0; for (int64_t j = 0; j < n; ++j) s += x[j] * x[j]; return s / n; }

/* ggml-quants.c:113-148, 2071-2097 */
static void row_q4_0(const float *x, uint8_t *y, int64_t n, const float *qw) {
    float sigma2 = qw ? row_sigma2(x, n) : 0;
    for (int64_t b = 0; b < n / 32; ++b, x += 32, y += 18) {
        uint8_t L[32];
        if (qw) {
            float w[32]; int8_t Ls[32];
            for (int j = 0; j < 32; ++j) w[j] = qw[32 * b + j] * sqrtf(sigma2 + x[j] * x[j]);
            put16(y, op_f32_to_f16(op_make_qx(32, 8, x, Ls, w)));
            for (int j = 0; j < 32; ++j) L[j] = (uint8_t)Ls[j];
        } else {
            float amax = 0, max = 0;
            for (int j = 0; j < 32; ++j) if (amax < fabsf(x[j])) { amax = fabsf(x[j]); max = x[j]; }
            float d = max / -8, id = d ? 1.0f / d : 0.0f;
            put16(y, op_f32_to_f16(d));
            for (int j = 0; j < 32; ++j) { int v = (int8_t)(x[j] * id + 8.5f); L[j] = (uint8_t)(v < 15 ? v : 15); }
        }
        pack_4bit(L, y + 2);
    }
}
/* ggml-quants.c:150-185, 2144-2172 */
static void row_q4_1(const float *x, uint8_t *y, int64_t n, const float *qw) {
    float sigma2 = qw ? row_sigma2(x, n) : 0;
    for (int64_t b = 0; b < n / 32; ++b, x += 32, y += 20) {
        uint8_t L[32];
        if (qw) {
            float w[32], mn;
            for (int j = 0; j < 32; ++j) w[j] = qw[32 * b + j] * sqrtf(sigma2 + x[j] * x[j]);
            float d = op_make_qkx(1, 32, 15, x, w, L, &mn, -0.9f, 0.05f, 36, 0);
            put16(y, op_f32_to_f16(d)); put16(y + 2, op_f32_to_f16(-mn));
        } else {
            float mn = 3.402823466e+38F, mx = -3.402823466e+38F;
            for (int j = 0; j < 32; ++j) { if (x[j] < mn) mn = x[j]; if (x[j] > mx) mx = x[j]; }
            float d = (mx - mn) / 15, id = d ? 1.0f / d : 0.0f;
            put16(y, op_f32_to_f16(d)); put16(y + 2, op_f32_to_f16(mn));
            for (int j = 0; j < 32; ++j) { int v = (int8_t)((x[j] - mn) * id + 0.5f); L[j] = (uint8_t)(v < 15 ? v : 15); }
        }
        pack_4bit(L, y + 4);
    }
}
/* ggml-quants.c:187-229, 2189-2226 */
static void row_q5_0(const float *x, uint8_t *y, int64_t n, const float *qw) {
    float sigma2 = qw ? row_sigma2(x, n) : 0;
    for (int64_t b = 0; b < n / 32; ++b, x += 32, y += 22) {
        uint8_t L[32];
        if (qw) {
            float w[32]; int8_t Ls[32];
            for (int j = 0; j < 32; ++j) w[j] = qw[32 * b + j] * sqrtf(sigma2 + x[j] * x[j]);
            put16(y, op_f32_to_f16(op_make_qx(32, 16, x, Ls, w)));
            for (int j = 0; j < 32; ++j) L[j] = (uint8_t)Ls[j];
        } else {
            float amax = 0, max = 0;
            for (int j = 0; j < 32; ++j) if (amax < fabsf(x[j])) { amax = fabsf(x[j]); max = x[j]; }
            float d = max / -16, id = d ? 1.0f / d : 0.0f;
            put16(y, op_f32_to_f16(d));
            for (int j = 0; j < 32; ++j) { int v = (int8_t)(x[j] * id + 16.5f); L[j] = (uint8_t)(v < 31 ? v : 31); }
        }
        put32(y + 2, pack_5bit(L, y + 6));
    }
}
/* ggml-quants.c:231-273, 2243-2279 */
static void row_q5_1(const float *x, uint8_t *y, int64_t n, const float *qw) {
    float sigma2 = qw ? row_sigma2(x, n) : 0;
    for (int64_t b = 0; b < n / 32; ++b, x += 32, y += 24) {
        uint8_t L[32];
        if (qw) {
            float w[32], mn;
            for (int j = 0; j < 32; ++j) w[j] = qw[32 * b + j] * sqrtf(sigma2 + x[j] * x[j]);
            float d = op_make_qkx(1, 32, 31, x, w, L, &mn, -0.9f, 0.05f, 36, 0);
            put16(y, op_f32_to_f16(d)); put16(y + 2, op_f32_to_f16(-mn));
        } else {
            float mn = 3.402823466e+38F, mx = -3.402823466e+38F;
            for (int j = 0; j < 32; ++j) { if (x[j] < mn) mn = x[j]; if (x[j] > mx) mx = x[j]; }
            float d = (mx - mn) / 31, id = d ? 1.0f / d : 0.0f;
            put16(y, op_f32_to_f16(d)); put16(y + 2, op_f32_to_f16(mn));
            for (int j = 0; j < 32; ++j) L[j] = (uint8_t)((x[j] - mn) * id + 0.5f);
        }
        put32(y + 4, pack_5bit(L, y + 8));
    }
}
/* ggml-quants.c:276-299 */
static void row_q8_0(const float *x, uint8_t *y, int64_t n) {
    for (int64_t b = 0; b < n / 32; ++b, x += 32, y += 34) {
        float amax = 0;
        for (int j = 0; j < 32; ++j) { float a = fabsf(x[j]); amax = amax > a ? amax : a; }
        float d = amax / 127, id = d ? 1.0f / d : 0.0f;
        put16(y, op_f32_to_f16(d));
        for (int j = 0; j < 32; ++j) y[2 + j] = (uint8_t)(int8_t)roundf(x[j] * id);
    }
}
/* ggml-quants.c:74-110 */
static void row_q2_0(const float *x, uint8_t *y, int64_t n) {
    for (int64_t b = 0; b < n / 64; ++b, x += 64, y += 18) {
        float amax = 0;
        for (int j = 0; j < 64; ++j) { float a = fabsf(x[j]); if (a > amax) amax = a; }
        float id = amax > 0.0f ? 1.0f / amax : 0.0f;
        put16(y, op_f32_to_f16(amax));
        memset(y + 2, 0, 16);
        for (int j = 0; j < 64; ++j) {
            int q = clampi((int)roundf(x[j] * id) + 1, 0, 3);
            y[2 + j / 4] |= (uint8_t)(q << ((j % 4) * 2));
        }
    }
}

/* ---- K-quants ------------------------------------------------------------------------------------- */
static void pack_2bit_planes(const uint8_t *L, uint8_t *qs) {
    for (int j = 0; j < 256; j += 128)
        for (int l = 0; l < 32; ++l) qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
}
static void k4_scales(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {       /* ggml-quants.c:880-887 */
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}
static float sb_sumsq(const float *x) { float s = 0; for (int j = 0; j < 256; ++j) s += x[j] * x[j]; return s; }

/* ggml-quants.c:891-959, 1150-1210.  block: scales[16] qs[64] d dmin */
static void row_q2_K(const float *x, uint8_t *y, int64_t n, const float *qw) {
    for (int64_t b = 0; b < n / 256; ++b, x += 256, y += 84) {
        uint8_t L[256], Ls[16], Lm[16], *sc = y;
        float mins[16], scales[16], w[16], sw[16];
        uint16_t dh, dmh;
        if (qw) {
            float sigma2 = sb_sumsq(x) / 256;
            for (int j = 0; j < 16; ++j) {
                for (int l = 0; l < 16; ++l) w[l] = qw[256 * b + 16 * j + l] * sqrtf(sigma2 + x[16 * j + l] * x[16 * j + l]);
                sw[j] = 0; for (int l = 0; l < 16; ++l) sw[j] += w[l];
                scales[j] = op_make_qkx(1, 16, 3, x + 16 * j, w, L + 16 * j, &mins[j], -0.9f, 0.05f, 36, 0);
            }
            dh = op_f32_to_f16(op_make_qp(16, 15, scales, Ls, sw));
            dmh = op_f32_to_f16(op_make_qp(16, 15, mins, Lm, sw));
            for (int j = 0; j < 16; ++j) sc[j] = (uint8_t)(Ls[j] | (Lm[j] << 4));
        } else {
            float max_scale = 0, max_min = 0;
            for (int j = 0; j < 16; ++j) {
                for (int l = 0; l < 16; ++l) w[l] = fabsf(x[16 * j + l]);
                scales[j] = op_make_qkx(0, 16, 3, x + 16 * j, w, L + 16 * j, &mins[j], -0.5f, 0.1f, 15, 1);
                if (scales[j] > max_scale) max_scale = scales[j];
                if (mins[j] > max_min) max_min = mins[j];
            }
            if (max_scale > 0) {
                float is = 15.f / max_scale;
                for (int j = 0; j < 16; ++j) sc[j] = (uint8_t)op_nearest_int(is * scales[j]);
                dh = op_f32_to_f16(max_scale / 15.f);
            } else { memset(sc, 0, 16); dh = op_f32_to_f16(0.f); }
            if (max_min > 0) {
                float is = 15.f / max_min;
                for (int j = 0; j < 16; ++j) sc[j] |= (uint8_t)(op_nearest_int(is * mins[j]) << 4);
                dmh = op_f32_to_f16(max_min / 15.f);
            } else dmh = op_f32_to_f16(0.f);
        }
        for (int j = 0; j < 16; ++j) {
            float d = op_f16_to_f32(dh) * (sc[j] & 0xF);
            if (!d) continue;
            float dm = op_f16_to_f32(dmh) * (sc[j] >> 4);
            for (int i = 0; i < 16; ++i) L[16 * j + i] = (uint8_t)clampi(op_nearest_int((x[16 * j + i] + dm) / d), 0, 3);
        }
        pack_2bit_planes(L, y + 16);
        put16(y + 80, dh); put16(y + 82, dmh);
    }
}

/* ggml-quants.c:1230-1304, 1356-1438.  block: hmask[32] qs[64] scales[12] d */
static void row_q3_K(const float *x, uint8_t *y, int64_t n, const float *qw) {
    for (int64_t b = 0; b < n / 256; ++b, x += 256, y += 110) {
        int8_t L[256], Ls[16];
        float scales[16], w[16], sw[16];
        uint8_t *hm = y, *qs = y + 32, *sc = y + 96;
        uint16_t dh;
        int pack = 1;            /* the matrix-free routine leaves the scale bytes zero when every sub-scale is zero */
        memset(sc, 0, 12);
        if (qw) {
            float sigma2 = 2 * sb_sumsq(x) / 256;
            for (int j = 0; j < 16; ++j) {
                for (int l = 0; l < 16; ++l) w[l] = qw[256 * b + 16 * j + l] * sqrtf(sigma2 + x[16 * j + l] * x[16 * j + l]);
                sw[j] = 0; for (int l = 0; l < 16; ++l) sw[j] += w[l];
                scales[j] = op_make_qx(16, 4, x + 16 * j, L + 16 * j, w);
            }
            dh = op_f32_to_f16(op_make_qx(16, 32, scales, Ls, sw));
        } else {
            float max_scale = 0, amax = 0;
            for (int j = 0; j < 16; ++j) {
                scales[j] = op_make_q3(16, 4, x + 16 * j, L + 16 * j);
                float a = fabsf(scales[j]);
                if (a > amax) { amax = a; max_scale = scales[j]; }
            }
            if (max_scale) {
                float is = -32.f / max_scale;
                for (int j = 0; j < 16; ++j) { int8_t l = (int8_t)op_nearest_int(is * scales[j]); Ls[j] = (int8_t)(clampi(l, -32, 31) + 32); }
                dh = op_f32_to_f16(1 / is);
            } else { pack = 0; dh = op_f32_to_f16(0.f); }
        }
        if (pack)
            for (int j = 0; j < 16; ++j) {
                int l = Ls[j];
                if (j < 8) sc[j] = (uint8_t)(l & 0xF); else sc[j - 8] |= (uint8_t)((l & 0xF) << 4);
                sc[j % 4 + 8] |= (uint8_t)((l >> 4) << (2 * (j / 4)));
            }
        for (int j = 0; j < 16; ++j) {
            int s = j < 8 ? sc[j] & 0xF : sc[j - 8] >> 4;
            s = (s | (((sc[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32;
            float d = op_f16_to_f32(dh) * s;
            if (!d) continue;
            for (int i = 0; i < 16; ++i) L[16 * j + i] = (int8_t)(clampi(op_nearest_int(x[16 * j + i] / d), -4, 3) + 4);
        }
        memset(hm, 0, 32);
        for (int j = 0; j < 256; ++j) if (L[j] > 3) { hm[j % 32] |= (uint8_t)(1 << (j / 32)); L[j] -= 4; }
        pack_2bit_planes((const uint8_t *)L, qs);
        put16(y + 108, dh);
    }
}

/* ggml-quants.c:1458-1528, 1554-1625 (bits 4) and 1645-1730, 1759-1850 (bits 5) */
static void row_q45_K(int bits, const float *x, uint8_t *y, int64_t n, const float *qw) {
    const int nmax = bits == 4 ? 15 : 31, bs = bits == 4 ? 144 : 176;
    for (int64_t b = 0; b < n / 256; ++b, x += 256, y += bs) {
        uint8_t L[256], Ls[8], Lm[8], *sc = y + 4;
        float mins[8], scales[8], w[32], sw[8];
        uint16_t dh, dmh;
        if (qw) {
            float sigma2 = 2 * sb_sumsq(x) / 256;
            for (int j = 0; j < 8; ++j) {
                for (int l = 0; l < 32; ++l) w[l] = qw[256 * b + 32 * j + l] * sqrtf(sigma2 + x[32 * j + l] * x[32 * j + l]);
                sw[j] = 0; for (int l = 0; l < 32; ++l) sw[j] += w[l];
                scales[j] = op_make_qkx(1, 32, nmax, x + 32 * j, w, L + 32 * j, &mins[j], -0.9f, 0.05f, 36, 0);
            }
            dh = op_f32_to_f16(op_make_qp(8, 63, scales, Ls, sw));
            dmh = op_f32_to_f16(op_make_qp(8, 63, mins, Lm, sw));
            if (bits == 5) for (int j = 0; j < 8; ++j) { if (Ls[j] > 63) Ls[j] = 63; if (Lm[j] > 63) Lm[j] = 63; }
        } else {
            float max_scale = 0, max_min = 0;
            for (int j = 0; j < 8; ++j) {
                float s2 = 0;
                for (int l = 0; l < 32; ++l) s2 += x[32 * j + l] * x[32 * j + l];
                float av = sqrtf(s2 / 32);
                for (int l = 0; l < 32; ++l) w[l] = av + fabsf(x[32 * j + l]);
                scales[j] = bits == 4 ? op_make_qkx(0, 32, 15, x + 32 * j, w, L + 32 * j, &mins[j], -1.f, 0.1f, 20, 0)
                                      : op_make_qkx(0, 32, 31, x + 32 * j, w, L + 32 * j, &mins[j], -0.5f, 0.1f, 15, 0);
                if (scales[j] > max_scale) max_scale = scales[j];
                if (mins[j] > max_min) max_min = mins[j];
            }
            float is = max_scale > 0 ? 63.f / max_scale : 0.f, im = max_min > 0 ? 63.f / max_min : 0.f;
            for (int j = 0; j < 8; ++j) {
                Ls[j] = (uint8_t)op_nearest_int(is * scales[j]); if (Ls[j] > 63) Ls[j] = 63;
                Lm[j] = (uint8_t)op_nearest_int(im * mins[j]); if (Lm[j] > 63) Lm[j] = 63;
            }
            dh = op_f32_to_f16(max_scale / 63.f); dmh = op_f32_to_f16(max_min / 63.f);
        }
        for (int j = 0; j < 4; ++j) { sc[j] = Ls[j]; sc[j + 4] = Lm[j]; }
        for (int j = 4; j < 8; ++j) {
            sc[j + 4] = (uint8_t)((Ls[j] & 0xF) | ((Lm[j] & 0xF) << 4));
            sc[j - 4] |= (uint8_t)((Ls[j] >> 4) << 6);
            sc[j] |= (uint8_t)((Lm[j] >> 4) << 6);
        }
        put16(y, dh); put16(y + 2, dmh);
        for (int j = 0; j < 8; ++j) {
            uint8_t s, m;
            k4_scales(j, sc, &s, &m);
            float d = op_f16_to_f32(dh) * s;
            if (!d) continue;
            float dm = op_f16_to_f32(dmh) * m;
            for (int i = 0; i < 32; ++i) L[32 * j + i] = (uint8_t)clampi(op_nearest_int((x[32 * j + i] + dm) / d), 0, nmax);
        }
        uint8_t *q = y + 16;
        if (bits == 5) {
            uint8_t *qh = y + 16; q = y + 48;
            memset(qh, 0, 32);
            for (int k = 0; k < 4; ++k)
                for (int j = 0; j < 32; ++j) {
                    if (L[64 * k + j] > 15) { L[64 * k + j] -= 16; qh[j] |= (uint8_t)(1 << (2 * k)); }
                    if (L[64 * k + j + 32] > 15) { L[64 * k + j + 32] -= 16; qh[j] |= (uint8_t)(2 << (2 * k)); }
                }
        }
        for (int k = 0; k < 4; ++k)
            for (int l = 0; l < 32; ++l) q[32 * k + l] = (uint8_t)(L[64 * k + l] | (L[64 * k + l + 32] << 4));
    }
}

/* ggml-quants.c:1870-1938, 1971-2053.  block: ql[128] qh[64] scales[16] d */
static void row_q6_K(const float *x, uint8_t *y, int64_t n, const float *qw) {
    for (int64_t b = 0; b < n / 256; ++b, x += 256, y += 210) {
        int8_t L[256], *sc = (int8_t *)(y + 192);
        float scales[16], max_scale = 0, max_abs = 0;
        for (int j = 0; j < 16; ++j) {
            scales[j] = op_make_qx(16, 32, x + 16 * j, L + 16 * j, qw ? qw + 256 * b + 16 * j : NULL);
            float a = fabsf(scales[j]);
            if (a > max_abs) { max_abs = a; max_scale = scales[j]; }
        }
        if (max_abs < EPS) { memset(y, 0, 210); continue; }
        float is = -128.f / max_scale;
        uint16_t dh = op_f32_to_f16(1 / is);
        for (int j = 0; j < 16; ++j) { int l = op_nearest_int(is * scales[j]); sc[j] = (int8_t)(l < 127 ? l : 127); }
        for (int j = 0; j < 16; ++j) {
            float d = op_f16_to_f32(dh) * sc[j];
            if (!d) continue;
            for (int i = 0; i < 16; ++i) L[16 * j + i] = (int8_t)(clampi(op_nearest_int(x[16 * j + i] / d), -32, 31) + 32);
        }
        uint8_t *ql = y, *qh = y + 128;
        for (int j = 0; j < 256; j += 128, ql += 64, qh += 32)
            for (int l = 0; l < 32; ++l) {
                ql[l] = (uint8_t)((L[j + l] & 0xF) | ((L[j + l + 64] & 0xF) << 4));
                ql[l + 32] = (uint8_t)((L[j + l + 32] & 0xF) | ((L[j + l + 96] & 0xF) << 4));
                qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
            }
        put16(y + 208, dh);
    }
}

/* ---- entry point: one row --------------------------------------------------------------------------- */
/* returns bytes written, 0 for a type this restatement does not cover */
size_t op_quantize_row(int type, const float *x, uint8_t *y, int64_t n, const float *qw) {
    switch (type) {
        case 2: row_q4_0(x, y, n, qw); return (size_t)(n / 32 * 18);
        case 3: row_q4_1(x, y, n, qw); return (size_t)(n / 32 * 20);
        case 6: row_q5_0(x, y, n, qw); return (size_t)(n / 32 * 22);
        case 7: row_q5_1(x, y, n, qw); return (size_t)(n / 32 * 24);
        case 8: row_q8_0(x, y, n); return (size_t)(n / 32 * 34);
        case 42: row_q2_0(x, y, n); return (size_t)(n / 64 * 18);
        case 10: row_q2_K(x, y, n, qw); return (size_t)(n / 256 * 84);
        case 11: row_q3_K(x, y, n, qw); return (size_t)(n / 256 * 110);
        case 12: row_q45_K(4, x, y, n, qw); return (size_t)(n / 256 * 144);
        case 13: row_q45_K(5, x, y, n, qw); return (size_t)(n / 256 * 176);
        case 14: row_q6_K(x, y, n, qw); return (size_t)(n / 256 * 210);
        default: return 0;
    }
}
