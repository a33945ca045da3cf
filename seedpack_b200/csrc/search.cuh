// Scale searches of the llama.cpp quantisers, one sub-block per thread, data in registers.
//
// Each routine reproduces, operation for operation, the fp32 expression trees and the loop-order
// tie rules of the C code (ggml-quants.c:628-695 make_qx_quants, 697-754 make_q3_quants, 799-878
// make_qkx2_quants, 993-1075 make_qkx3_quants, 1077-1148 make_qp_quants).  The candidate loops of
// make_qkx2/3 are inherently sequential (a winning candidate changes `min`, which feeds the next
// candidate), so the parallel axis is the sub-block: one thread owns one sub-block of N weights,
// with x[] and w[] held in registers through full unrolling, and the super-block level is stitched
// together with warp shuffles by the caller.
//
// Instead of keeping the running-best code array L[] (N registers) the searches remember the
// parameters that produced it and `*_codes` recomputes it on demand; the recomputation runs the same
// instructions on the same inputs, so it yields the same codes.
#pragma once
#include "common.cuh"

namespace sg {

#define SG_GROUP_MAX_EPS 1e-15f

SG_DEVINL int clampi(int v, int lo, int hi) { return max(lo, min(hi, v)); }

// ---- make_qx_quants, rmse_type == 1 (the only mode the quantisers on this path use) -------------
struct QxBest { float scale; float iscale; bool zero; };
// clamp(nearest_int(v), -nmax, nmax - 1) as a float, for |v| far below 2^22 (here |v| <= nmax + 1): the rounding add of
// nearest_int yields the integer's float directly
SG_DEVINL float qx_level(float v, float fn) { return fminf(fmaxf(fsub(fadd(v, 12582912.f), 12582912.f), -fn), fn - 1.f); }

template <int N, bool HAVE_W>
SG_DEVINL QxBest make_qx_quants(int nmax, const float (&x)[N], const float (&qw)[N]) {
    float mx = 0.f, amax = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; mx = x[i]; }
    }
    QxBest r;
    if (amax < SG_GROUP_MAX_EPS) { r.scale = 0.f; r.iscale = 0.f; r.zero = true; return r; }
    r.zero = false;
    const float fn = (float)nmax;
    float iscale = fdiv(-fn, mx);
    float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float w = HAVE_W ? qw[i] : fmul(x[i], x[i]);
        const float fl = qx_level(fmul(iscale, x[i]), fn);
        sumlx = fadd(sumlx, fmul(fmul(w, x[i]), fl));
        suml2 = fadd(suml2, fmul(fmul(w, fl), fl));
    }
    float scale = suml2 != 0.f ? fdiv(sumlx, suml2) : 0.0f;
    float best = fmul(scale, sumlx);
    r.iscale = iscale;
#pragma unroll 1
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = fdiv(-fadd(fn, fmul(0.1f, (float)is)), mx);
        sumlx = 0.f; suml2 = 0.f;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float w = HAVE_W ? qw[i] : fmul(x[i], x[i]);
            const float fl = qx_level(fmul(iscale, x[i]), fn);
            sumlx = fadd(sumlx, fmul(fmul(w, x[i]), fl));
            suml2 = fadd(suml2, fmul(fmul(w, fl), fl));
        }
        if (suml2 > 0.f && fmul(sumlx, sumlx) > fmul(best, suml2)) {
            r.iscale = iscale;
            scale = fdiv(sumlx, suml2);
            best = fmul(scale, sumlx);
        }
    }
    r.scale = scale;
    return r;
}
// code i of the winning candidate, already offset by nmax (0 .. 2*nmax-1)
SG_DEVINL int qx_code(const QxBest& b, int nmax, float xi) {
    if (b.zero) return 0;
    return nmax + clampi(nearest_int(fmul(b.iscale, xi)), -nmax, nmax - 1);
}

// ---- make_q3_quants(n, nmax, x, L, do_rmse = true) ------------------------------------------------
template <int N>
SG_DEVINL float make_q3_quants(int nmax, const float (&x)[N], int (&L)[N]) {
    float mx = 0.f, amax = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; mx = x[i]; }
    }
    if (amax < SG_GROUP_MAX_EPS) {
#pragma unroll
        for (int i = 0; i < N; ++i) L[i] = 0;
        return 0.f;
    }
    const float iscale = fdiv((float)(-nmax), mx);
    float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const int l = clampi(nearest_int(fmul(iscale, x[i])), -nmax, nmax - 1);
        L[i] = l;
        const float w = fmul(x[i], x[i]);
        const float fl = (float)l;
        sumlx = fadd(sumlx, fmul(fmul(w, x[i]), fl));
        suml2 = fadd(suml2, fmul(fmul(w, fl), fl));
    }
#pragma unroll 1
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float w = fmul(x[i], x[i]);
            const float fl = (float)L[i];
            float slx = fsub(sumlx, fmul(fmul(w, x[i]), fl));
            if (slx > 0.f) {
                float sl2 = fsub(suml2, fmul(fmul(w, fl), fl));
                int new_l = nearest_int(fdiv(fmul(x[i], sl2), slx));
                new_l = clampi(new_l, -nmax, nmax - 1);
                if (new_l != L[i]) {
                    const float fnl = (float)new_l;
                    slx = fadd(slx, fmul(fmul(w, x[i]), fnl));
                    sl2 = fadd(sl2, fmul(fmul(w, fnl), fnl));
                    if (sl2 > 0.f && fmul(fmul(slx, slx), suml2) > fmul(fmul(sumlx, sumlx), sl2)) {
                        L[i] = new_l; sumlx = slx; suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (!n_changed) break;
    }
#pragma unroll
    for (int i = 0; i < N; ++i) L[i] += nmax;
    return suml2 > 0.0f ? fdiv(sumlx, suml2) : 0.0f;
}

// ---- make_qkx2_quants / make_qkx3_quants ---------------------------------------------------------
// `kind` tells *_code which formula produced the winning codes: 0 all zero, 1 the initial
// round-and-clamp, 2 a candidate of the step loop.
struct QkxBest { float scale; float the_min; float iscale; float min_used; int kind; };

template <int N, bool V3>
SG_DEVINL int qkx_cand_code(float iscale, float mn, int nmax, float xi) {
    const float v = fmul(iscale, fsub(xi, mn));
    if (V3) return v > 0.f ? nearest_int(fminf(v, (float)nmax)) : 0;   // MIN(v, nmax): v if v < nmax
    return clampi(nearest_int(v), 0, nmax);
}

// the same code as a float.  V3: the value that goes into nearest_int lies in (0, nmax], where the rounding add of
// nearest_int yields the integer's float directly (v + 1.5 * 2^23 - 1.5 * 2^23), with no integer detour.
template <int N, bool V3>
SG_DEVINL float qkx_cand_level(float iscale, float mn, int nmax, float xi) {
    if (V3) {
        const float v = fmul(iscale, fsub(xi, mn));
        const float r = fsub(fadd(fminf(v, (float)nmax), 12582912.f), 12582912.f);
        return v > 0.f ? r : 0.f;
    }
    return (float)qkx_cand_code<N, V3>(iscale, mn, nmax, xi);
}

template <int N, bool V3>
SG_DEVINL QkxBest make_qkx_quants(int nmax, const float (&x)[N], const float (&wt)[N],
                                  float rmin, float rdelta, int nstep, bool use_mad) {
    float mn = x[0], mx = x[0];
    float sum_w = wt[0];
    float sum_x = fmul(sum_w, x[0]);
#pragma unroll
    for (int i = 1; i < N; ++i) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
        const float w = wt[i];
        sum_w = fadd(sum_w, w);
        sum_x = fadd(sum_x, fmul(w, x[i]));
    }
    if (mn > 0.f) mn = 0.f;
    QkxBest r;
    if (V3 ? (mx <= mn) : (mx == mn)) {
        r.scale = 0.f; r.the_min = -mn; r.iscale = 0.f; r.min_used = 0.f; r.kind = 0;
        return r;
    }
    const float fn = (float)nmax;
    float iscale = fdiv(fn, fsub(mx, mn));
    float scale = frcp(iscale);
    float best = 0.f;
    r.iscale = iscale; r.min_used = mn; r.kind = 1;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const int l = clampi(nearest_int(fmul(iscale, fsub(x[i], mn))), 0, nmax);
        float diff = fsub(fadd(fmul(scale, (float)l), mn), x[i]);
        diff = use_mad ? fabsf(diff) : fmul(diff, diff);
        best = fadd(best, fmul(wt[i], diff));
    }
    if (nstep >= 1) {
#pragma unroll 1
        for (int is = 0; is <= nstep; ++is) {
            iscale = fdiv(fadd(fadd(rmin, fmul(rdelta, (float)is)), fn), fsub(mx, mn));
            float sum_l = 0.f, sum_l2 = 0.f, sum_xl = 0.f;
            float lv[N];                       // the candidate's levels, kept for the error pass
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const float fl = lv[i] = qkx_cand_level<N, V3>(iscale, mn, nmax, x[i]);
                const float w = wt[i];
                sum_l = fadd(sum_l, fmul(w, fl));
                sum_l2 = fadd(sum_l2, fmul(fmul(w, fl), fl));
                sum_xl = fadd(sum_xl, fmul(fmul(w, fl), x[i]));
            }
            const float D = fsub(fmul(sum_w, sum_l2), fmul(sum_l, sum_l));
            if (D > 0.f) {
                float this_scale = fdiv(fsub(fmul(sum_w, sum_xl), fmul(sum_x, sum_l)), D);
                float this_min = fdiv(fsub(fmul(sum_l2, sum_x), fmul(sum_l, sum_xl)), D);
                if (this_min > 0.f) {
                    this_min = 0.f;
                    this_scale = fdiv(sum_xl, sum_l2);
                }
                float err = 0.f;
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    const float fl = lv[i];
                    float diff = fsub(fadd(fmul(this_scale, fl), this_min), x[i]);
                    diff = use_mad ? fabsf(diff) : fmul(diff, diff);
                    err = fadd(err, fmul(wt[i], diff));
                }
                if (err < best) {
                    r.iscale = iscale; r.min_used = mn; r.kind = 2;
                    best = err;
                    scale = this_scale;
                    mn = this_min;
                }
            }
        }
    }
    r.scale = scale;
    r.the_min = -mn;
    return r;
}
template <int N, bool V3>
SG_DEVINL int qkx_code(const QkxBest& b, int nmax, float xi) {
    if (b.kind == 0) return 0;
    if (b.kind == 1) return clampi(nearest_int(fmul(b.iscale, fsub(xi, b.min_used))), 0, nmax);
    return qkx_cand_code<N, V3>(b.iscale, b.min_used, nmax, xi);
}

// ---- make_qp_quants -------------------------------------------------------------------------------
template <int N>
SG_DEVINL float make_qp_quants(int nmax, const float (&x)[N], int (&L)[N], const float (&qw)[N]) {
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) mx = fmaxf(mx, x[i]);     // MAX(max, x[i])
    if (mx < SG_GROUP_MAX_EPS) {
#pragma unroll
        for (int i = 0; i < N; ++i) L[i] = 0;
        return 0.f;
    }
    const float fn = (float)nmax;
    float iscale = fdiv(fn, mx);
#pragma unroll
    for (int i = 0; i < N; ++i) L[i] = nearest_int(fmul(iscale, x[i])) & 0xff;   // stored in a uint8_t
    const float scale = frcp(iscale);
    float best_mse = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float diff = fsub(x[i], fmul(scale, (float)L[i]));
        best_mse = fadd(best_mse, fmul(fmul(qw[i], diff), diff));
    }
#pragma unroll 1
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        const float iscale_is = fdiv(fadd(fmul(0.1f, (float)is), fn), mx);
        const float scale_is = frcp(iscale_is);
        float mse = 0.f;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            int l = nearest_int(fmul(iscale_is, x[i]));
            l = min(nmax, l);
            const float diff = fsub(x[i], fmul(scale_is, (float)l));
            mse = fadd(mse, fmul(fmul(qw[i], diff), diff));
        }
        if (mse < best_mse) { best_mse = mse; iscale = iscale_is; }
    }
    float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        int l = nearest_int(fmul(iscale, x[i]));
        l = min(nmax, l);
        L[i] = l & 0xff;
        const float fl = (float)l;
        sumlx = fadd(sumlx, fmul(fmul(qw[i], x[i]), fl));
        suml2 = fadd(suml2, fmul(fmul(qw[i], fl), fl));
    }
#pragma unroll 1
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float w = qw[i];
            const float fl = (float)L[i];
            float slx = fsub(sumlx, fmul(fmul(w, x[i]), fl));
            float sl2 = fsub(suml2, fmul(fmul(w, fl), fl));
            if (slx > 0.f && sl2 > 0.f) {
                int new_l = nearest_int(fdiv(fmul(x[i], sl2), slx));
                new_l = min(nmax, new_l);
                if (new_l != L[i]) {
                    const float fnl = (float)new_l;
                    slx = fadd(slx, fmul(fmul(w, x[i]), fnl));
                    sl2 = fadd(sl2, fmul(fmul(w, fnl), fnl));
                    if (fmul(fmul(slx, slx), suml2) > fmul(fmul(sumlx, sumlx), sl2)) {
                        L[i] = new_l & 0xff; sumlx = slx; suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (!n_changed) break;
    }
    return suml2 > 0.0f ? fdiv(sumlx, suml2) : 0.0f;
}

}  // namespace sg
