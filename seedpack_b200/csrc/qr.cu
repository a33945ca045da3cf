// QR residual coder kernels: histogram, encode, decode of a batch of stored blocks against their predictions.
//
// Replaces qr_hist / qr_enc / qr_dec (seedpack/qr.py:674-807).  Format and symbol order are the reference's:
// per segment (seg_blocks(T) blocks, one rANS state) and per block, in decode order: the "equals its prediction"
// flag (context: previous block's flag), then for a differing block its scale fields and its codes.  The encoder
// walks the same symbols backwards.
//
// What is done differently: block equality comes from a separate memory-bound pass (sg_residual_blocks: one
// coalesced sweep over F and P, one flag byte per block) instead of a byte loop inside the serial walk, so the
// per-segment lanes only touch the few blocks that differ; the coder uses the reciprocal / register-window
// engine of rans.cuh; histogram counts of the flag symbols are accumulated per lane and added once.
#include "api_util.h"
#include "qr_model.cuh"
#include "rans.cuh"

namespace sg {
namespace qr {

struct Setup {
    SG g; TM m; int qk, bs, nf, sublen, hboff;
    const uchar* sbase;
};
SG_DEVINL Setup setup(int T, const uchar* seed, const TM* tm, const SG* sg, int s) {
    Setup u;
    u.g = sg[s]; u.m = tm[u.g.t];
    u.qk = qk_of(T); u.bs = bs_of(T); u.nf = nfield(T); u.sublen = sublen_of(T);
    u.sbase = seed + u.m.seed_off;
    u.hboff = u.m.seed_type == 98 ? HBOFF_COL : 8;
    return u;
}

// symbols of one field delta, in decode order, through `emit(tab, sym)`
template <class E> SG_DEVINL void field_symbols(int kd, int any, int tv, int dl, E&& emit) {
    if (kd < 2 && (dl < -127 || dl > 127)) { emit(fctx(kd, any), 128); emit(FESC_LO, tv & 255); emit(FESC_HI, tv >> 8); }
    else emit(fctx(kd, any), dl & 255);
}

// ---- histogram -----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64) k_qr_hist(int T, const uchar* __restrict__ F, const uchar* __restrict__ P,
                                                const uchar* __restrict__ ne, const uchar* __restrict__ seed,
                                                const TM* __restrict__ tm, const SG* __restrict__ sg, int nseg,
                                                unsigned* __restrict__ counts, int mv) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const Setup u = setup(T, seed, tm, sg, s);
    unsigned flagc[4] = {0, 0, 0, 0};                 // [prev * 2 + eq]
    int prev = 1;
    auto add = [&](int tab, int sym) { atomicAdd(counts + tab * 256 + sym, 1u); };
    for (long long b = u.g.b0; b < u.g.b0 + u.g.nb; ++b) {
        const int eq = !ne[b];
        ++flagc[prev * 2 + eq];
        prev = eq;
        if (eq) continue;
        const uchar* fb = F + b * u.bs; const uchar* pb = P + b * u.bs;
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, fb, tv); unpack_fields(T, pb, pv);
        int any = 0;
        for (int k = 0; k < u.nf; ++k) {
            const int dl = tv[k] - fpred(T, mv, pv, k, tv[0], u.nf > 1 ? tv[1] : 0);
            field_symbols(fkind(T, k), any, tv[k], dl, add);
            any |= dl != 0;
        }
        const long long gw0 = (b - u.m.blk0) * u.qk;
        const long long col0 = u.m.cols > 0 ? gw0 % u.m.cols : 0;
        int tsub = -1; float ta = 0.f, tc = 0.f;
        for (int w = 0; w < u.qk; ++w) {
            if (w / u.sublen != tsub) { tsub = w / u.sublen; wscale(T, tv, tsub, ta, tc); }
            float xv, hv; seed_val(u.m.seed_type, u.sbase, gw0 + w, xv, hv, u.m.cols);
            int r, sgn, ctx; predict_code(T, ta, tc, pb, w, xv, hv, u.hboff, r, sgn, ctx, mv, pos8(col0 + w, u.m.cols));
            add(ctx, (sgn * (get_code(T, fb, w) - r)) & 255);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) if (flagc[i]) atomicAdd(counts + (FLAG + (i >> 1)) * 256 + (i & 1), flagc[i]);
}

// ---- encode ----------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64) k_qr_enc(int T, const uchar* __restrict__ F, const uchar* __restrict__ P,
                                               const uchar* __restrict__ ne, const uchar* __restrict__ seed,
                                               const TM* __restrict__ tm, const SG* __restrict__ sg, int nseg,
                                               const RansSym* __restrict__ enc, uchar* __restrict__ out, size_t cap,
                                               unsigned* __restrict__ out_len, int mv) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const Setup u = setup(T, seed, tm, sg, s);
    uchar* slot = out + (size_t)s * cap;
    ByteWriterDown wr; wr.init(slot + cap);
    unsigned x = RANS_L;
    bool ovf = false;
    auto put = [&](int tab, int sym) {
        if (ovf) return;
        rans_put<12>(x, wr, enc[tab * 256 + sym]);
        if (wr.ptr() < slot + 64) ovf = true;
    };
    for (long long b = u.g.b0 + u.g.nb - 1; b >= u.g.b0; --b) {
        const int eq = !ne[b];
        const int prev = b > u.g.b0 ? !ne[b - 1] : 1;
        if (eq) { put(FLAG + prev, 1); continue; }
        const uchar* fb = F + b * u.bs; const uchar* pb = P + b * u.bs;
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, fb, tv); unpack_fields(T, pb, pv);
        const long long gw0 = (b - u.m.blk0) * u.qk;
        const long long col0 = u.m.cols > 0 ? gw0 % u.m.cols : 0;
        int tsub = -1; float ta = 0.f, tc = 0.f;
        for (int w = u.qk - 1; w >= 0; --w) {
            if (w / u.sublen != tsub) { tsub = w / u.sublen; wscale(T, tv, tsub, ta, tc); }
            float xv, hv; seed_val(u.m.seed_type, u.sbase, gw0 + w, xv, hv, u.m.cols);
            int r, sgn, ctx; predict_code(T, ta, tc, pb, w, xv, hv, u.hboff, r, sgn, ctx, mv, pos8(col0 + w, u.m.cols));
            put(ctx, (sgn * (get_code(T, fb, w) - r)) & 255);
        }
        {   // fields, last to first; `any` is what the decoder will have seen before field k
            int dl[MAXF], anyk[MAXF], any = 0;
            for (int k = 0; k < u.nf; ++k) {
                dl[k] = tv[k] - fpred(T, mv, pv, k, tv[0], u.nf > 1 ? tv[1] : 0);
                anyk[k] = any; any |= dl[k] != 0;
            }
            for (int k = u.nf - 1; k >= 0; --k) {
                const int kd = fkind(T, k);
                if (kd < 2 && (dl[k] < -127 || dl[k] > 127)) { put(FESC_HI, tv[k] >> 8); put(FESC_LO, tv[k] & 255); put(fctx(kd, anyk[k]), 128); }
                else put(fctx(kd, anyk[k]), dl[k] & 255);
            }
        }
        put(FLAG + prev, 0);
        if (ovf) break;
    }
    if (ovf) { out_len[s] = 0xffffffffu; return; }
    rans_flush(x, wr);
    wr.flush(slot);
    out_len[s] = (unsigned)(slot + cap - wr.ptr());
}

// ---- decode ----------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64) k_qr_dec(int T, const uchar* __restrict__ in, const unsigned long long* __restrict__ off,
                                               const uchar* __restrict__ P, const uchar* __restrict__ seed,
                                               const TM* __restrict__ tm, const SG* __restrict__ sg, int nseg,
                                               const RansSym* __restrict__ enc, const uchar* __restrict__ lut,
                                               uchar* __restrict__ F, int mv, int* __restrict__ status) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const Setup u = setup(T, seed, tm, sg, s);
    ByteReaderUp rd; rd.init(in + off[s], in + off[s + 1]);
    unsigned x = rans_init(rd);
    auto get = [&](int tab) -> int { return (int)rans_get<12>(x, rd, lut + ((size_t)tab << 12), enc + tab * 256); };
    int prev = 1;
    for (long long b = u.g.b0; b < u.g.b0 + u.g.nb; ++b) {
        uchar* fb = F + b * u.bs; const uchar* pb = P + b * u.bs;
        const int eq = get(FLAG + prev);
        prev = eq;
        if (eq) { for (int i = 0; i < u.bs; ++i) fb[i] = pb[i]; continue; }
        for (int i = 0; i < u.bs; ++i) fb[i] = 0;
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, pb, pv);
        int any = 0;
        for (int k = 0; k < u.nf; ++k) {
            const int kd = fkind(T, k);
            const int pr = fpred(T, mv, pv, k, k > 0 ? tv[0] : 0, k > 1 ? tv[1] : 0);
            const int sym = get(fctx(kd, any));
            int t;
            if (kd < 2 && sym == 128) { const int lo = get(FESC_LO), hi = get(FESC_HI); t = lo | (hi << 8); }
            else {
                t = pr + (int)(signed char)sym;
                if (kd < 2) t &= 0xffff;
                else if (T == 14) t = (int)(signed char)(t & 255);
            }
            tv[k] = t; any |= t != pr;
        }
        pack_fields(T, fb, tv);
        const long long gw0 = (b - u.m.blk0) * u.qk;
        const long long col0 = u.m.cols > 0 ? gw0 % u.m.cols : 0;
        int tsub = -1; float ta = 0.f, tc = 0.f;
        for (int w = 0; w < u.qk; ++w) {
            if (w / u.sublen != tsub) { tsub = w / u.sublen; wscale(T, tv, tsub, ta, tc); }
            float xv, hv; seed_val(u.m.seed_type, u.sbase, gw0 + w, xv, hv, u.m.cols);
            int r, sgn, ctx; predict_code(T, ta, tc, pb, w, xv, hv, u.hboff, r, sgn, ctx, mv, pos8(col0 + w, u.m.cols));
            const int v = get(ctx);
            int q = r + sgn * (int)(signed char)v;
            if (T == 8) q = (int)(signed char)(q & 255);
            put_code(T, fb, w, q);
        }
        if (rd.over) break;
    }
    if (rd.over || x != RANS_L || rd.p != rd.end) atomicOr(status, SG_ST_CORRUPT);
}

}  // namespace qr
}  // namespace sg

using namespace sg;
using namespace sg::qr;

static int qr_args(int T, const void* P, const void* seed, const void* tm, const void* sgp, int nseg, int mv) {
    if (!P || !seed || !tm || !sgp || nseg < 0 || (mv != 1 && mv != 2)) return SG_ERR_ARG;
    switch (T) { case 2: case 3: case 6: case 7: case 8: case 10: case 11: case 12: case 13: case 14: case 20: case 23: case 42: return SG_OK; }
    return SG_ERR_TYPE;      // the grid types (16 17 18 19 21 22 29) are coded by sg_qr_grid_* once available
}

extern "C" int sg_qr_hist(int device, void* stream, int T, const unsigned char* F, const unsigned char* P, const unsigned char* ne,
                          const unsigned char* seed, const void* tm, const void* sgp, int nseg, unsigned* counts, int mv) {
    int rc = qr_args(T, P, seed, tm, sgp, nseg, mv);
    if (rc != SG_OK) return rc;
    if (!F || !ne || !counts) return SG_ERR_ARG;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_qr_hist<<<(nseg + 63) / 64, 64, 0, (cudaStream_t)stream>>>(T, F, P, ne, seed, (const TM*)tm, (const SG*)sgp, nseg, counts, mv);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_encode(int device, void* stream, int T, const unsigned char* F, const unsigned char* P, const unsigned char* ne,
                            const unsigned char* seed, const void* tm, const void* sgp, int nseg, const void* enc_tab,
                            unsigned char* slots, size_t cap, unsigned* out_len, int mv) {
    int rc = qr_args(T, P, seed, tm, sgp, nseg, mv);
    if (rc != SG_OK) return rc;
    if (!F || !ne || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 128 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_qr_enc<<<(nseg + 63) / 64, 64, 0, (cudaStream_t)stream>>>(T, F, P, ne, seed, (const TM*)tm, (const SG*)sgp, nseg,
                                                                (const RansSym*)enc_tab, slots, cap, out_len, mv);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_decode(int device, void* stream, int T, const unsigned char* in, const unsigned long long* off,
                            const unsigned char* P, const unsigned char* seed, const void* tm, const void* sgp, int nseg,
                            const void* enc_tab, const unsigned char* lut, unsigned char* F, int mv) {
    int rc = qr_args(T, P, seed, tm, sgp, nseg, mv);
    if (rc != SG_OK) return rc;
    if (!in || !off || !enc_tab || !lut || !F) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_qr_dec<<<(nseg + 63) / 64, 64, 0, (cudaStream_t)stream>>>(T, in, off, P, seed, (const TM*)tm, (const SG*)sgp, nseg,
                                                                (const RansSym*)enc_tab, lut, F, mv, status_word(device));
    return cuda_ok(cudaGetLastError());
}
