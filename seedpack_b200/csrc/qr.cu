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

// ---- one coder for the three passes ---------------------------------------------------------------------------
struct Coder {
    int mode;                       // 0 histogram (symbols in decode order), 1 encode (symbols in reverse decode order),
                                    // 3 stage: like encode, but the (table, symbol) pairs are only written down
    unsigned* counts;
    unsigned* stage; int nstaged;
    const RansSym* enc;
    unsigned x; ByteWriterDown wr; uchar* slot; bool ovf;
    SG_DEVINL void put(int tab, int s) {
        if (mode == 0) { atomicAdd(counts + tab * 256 + s, 1u); return; }
        if (mode == 3) { stage[nstaged++] = (unsigned)(tab * 256 + s); return; }
        if (ovf) return;
        rans_put<12>(x, wr, enc[tab * 256 + s]);
        if (wr.ptr() < slot + 64) ovf = true;
    }
};

// ---- grid types: rank of the true lattice point among all points, by weighted distance to the seed -------------
// Per pair of weights a table in shared memory holds the weighted squared error of every pair of levels, so the
// distance of a lattice point is N/2 lookups (qr.py:496-515).  Laid out [entry][thread]: conflict-free.
constexpr int TOPK = 16;
constexpr int QR_TPB = 64;

template <int N, bool SGN>
SG_DEVINL void pair_tables(float* tab, const float* uu, const float* ww, float dl) {
    constexpr int B = N == 8 ? 2 : 3, L = 1 << B, E = L * L;
    for (int p = 0; p < N / 2; ++p)
        for (int e = 0; e < E; ++e) {
            const int la = e & (L - 1), lb = e >> B;
            const float qa = SGN ? (float)(2 * la + 1) : (float)(la - 1) + dl;
            const float qb = SGN ? (float)(2 * lb + 1) : (float)(lb - 1) + dl;
            const float ea = qa - uu[2 * p], eb = qb - uu[2 * p + 1];
            tab[(p * E + e) * QR_TPB + threadIdx.x] = ww[2 * p] * (ea * ea) + ww[2 * p + 1] * (eb * eb);
        }
}
template <int N> SG_DEVINL float point_dist(const float* tab, unsigned key) {
    constexpr int B = N == 8 ? 2 : 3, E = 1 << (2 * B);
    float d = 0.f;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) d = d + tab[(p * E + ((key >> (2 * B * p)) & (E - 1))) * QR_TPB + threadIdx.x];
    return isnan(d) ? __int_as_float(0x7f800000) : d;
}
// the two smallest distances and the rank of point t in the order (distance, index)        (encode / histogram)
// Keys are read two at a time (gs is even, gk 4-byte aligned); points before t count when they are at most as far as
// t, points from t on when they are strictly closer (t itself is not).
template <int N> SG_DEVINL void scan_rank(const float* tab, const uint16_t* __restrict__ gk, int gs, int t, float& d1, float& d2, int& rank) {
    const float inf = __int_as_float(0x7f800000);
    const float dt = point_dist<N>(tab, gk[t]);
    const unsigned* gk2 = reinterpret_cast<const unsigned*>(gk);
    d1 = inf; d2 = inf; rank = 0;
    auto two_smallest = [&](float d) { d2 = fminf(d2, fmaxf(d1, d)); d1 = fminf(d1, d); };
    for (int k = 0; k < gs / 2; ++k) {              // every lane runs the same trip count
        const unsigned kk = __ldg(gk2 + k);
        const float da = point_dist<N>(tab, kk & 0xffffu), db = point_dist<N>(tab, kk >> 16);
        two_smallest(da); two_smallest(db);
        rank += (2 * k < t ? da <= dt : da < dt) + (2 * k + 1 < t ? db <= dt : db < dt);
    }
}
// all symbols of one differing block of a grid type after its scale fields (qr.py:553-637), in the encoder's order.
// fb: stored block, tv: its unpacked fields.
template <int N, bool SGN>
SG_DEVINL void grid_block(Coder& c, int T, int mv, uchar* fb, const uchar* pb, const int* tv, const uint16_t* __restrict__ gk,
                          long long gw0, int st, const uchar* sbase, int cols, const float* im, float* tab) {
    constexpr int B = N == 8 ? 2 : 3, ng = 8 / N;
    const int gs = grid_size(T);
    const bool par = parity_type(T);
    float sx2 = 0.f;
    for (int i = 0; i < 256; ++i) { float xv, hv; seed_val(st, sbase, gw0 + i, xv, hv, cols); sx2 += xv * xv; }
    const float sigma2 = (T == 16 || T == 17) ? sx2 * (1.0f / 256.f) : 2.f * sx2 * (1.0f / 256.f);
    const long long col0 = cols > 0 ? gw0 % cols : 0;
    for (int ui = 0; ui < 32; ++ui) {
        const int u = 31 - ui;
        const int p4 = pos4(col0 + 8 * u, cols);
        const int rank0 = mv >= 2 ? GRANK2 + 4 * p4 : GRID_RANK;
        const int sign0 = mv >= 2 ? GSIGN2 + 16 * p4 : GRID_SIGN;
        float gu[8], gw[8], gs_, gdl;
        int pn[8];
        gscale(T, fb, tv, u, gs_, gdl);
        {
            float x[8], v[8];
            for (int i = 0; i < 8; ++i) {
                const long long gwi = gw0 + 8 * u + i;
                float hv; seed_val(st, sbase, gwi, x[i], hv, cols);
                float wi = sqrtf(sigma2 + x[i] * x[i]);
                if (im) wi = wi * im[gwi % cols];
                gw[i] = wi;
                pn[i] = x[i] < 0.f;
                v[i] = SGN ? fabsf(x[i]) : x[i];
            }
            if (SGN && par) {                  // an odd number of negatives: the least weighty one flips back
                int cnt = 0;
                for (int i = 0; i < 8; ++i) cnt += pn[i];
                if (cnt & 1) {
                    int imin = 0; float mn = gw[0] * x[0] * x[0];
                    for (int i = 1; i < 8; ++i) { const float a = gw[i] * x[i] * x[i]; if (a < mn) { mn = a; imin = i; } }
                    pn[imin] ^= 1; v[imin] = -v[imin];
                }
            }
            for (int i = 0; i < 8; ++i) gu[i] = v[i] / gs_;
        }
        int tg[2] = {0, 0};
        auto sign_ctx = [&](int j) {
            const int lev = (gk[tg[j / N]] >> (B * (j % N))) & ((1 << B) - 1);
            const float m4 = fabsf(gu[j]) * 4.f;
            return sign0 + (lev == 0) * 8 + (m4 < 7.f ? (int)m4 : 7);
        };
        for (int gg = 0; gg < ng; ++gg) tg[gg] = get_gidx(T, fb, u * ng + gg);
        if (SGN) for (int j = 7; j >= 0; --j) {
            if (par && j == 7) continue;
            c.put(sign_ctx(j), get_neg(T, fb, 8 * u + j) ^ pn[j]);
        }
        for (int gg = ng - 1; gg >= 0; --gg) {
            pair_tables<N, SGN>(tab, gu + gg * N, gw + gg * N, gdl);
            int rank; float d1, d2;
            scan_rank<N>(tab, gk, gs, tg[gg], d1, d2, rank);
            const int ctx = rank0 + gapctx(d1, d2);
            if (rank >= TOPK) { c.put(FESC_HI, tg[gg] >> 8); c.put(FESC_LO, tg[gg] & 255); c.put(ctx, TOPK); }
            else c.put(ctx, rank);
        }
        if (T == 29) c.put(GRID_SHIFT, get_shift(fb, u) ^ get_shift(pb, u));
        if (c.ovf) return;
    }
}
SG_DEVINL void grid_code(Coder& c, int T, int mv, uchar* fb, const uchar* pb, const int* tv, const uint16_t* gk, long long gw0, int st,
                         const uchar* sbase, int cols, const float* im, float* tab) {
    switch (T) {
        case 18: case 21: grid_block<4, true>(c, T, mv, fb, pb, tv, gk, gw0, st, sbase, cols, im, tab); return;
        case 19: case 29: grid_block<8, false>(c, T, mv, fb, pb, tv, gk, gw0, st, sbase, cols, im, tab); return;
        default: grid_block<8, true>(c, T, mv, fb, pb, tv, gk, gw0, st, sbase, cols, im, tab);
    }
}

// ---- the three passes -------------------------------------------------------------------------------------------
extern __shared__ float gtab[];          // grid types only: 64 (IQ3: 128) floats per thread

struct Args {
    int T, mv, nseg;
    const uchar *F, *P, *ne, *seed;
    const TM* tm; const SG* sg;
    const uint16_t* gk; const float* imx;
};

// scalar-code types: the codes of one differing block, forwards (histogram) or backwards (encode, stage)
SG_DEVINL void scalar_codes(Coder& c, int T, int mv, uchar* fb, const uchar* pb, const int* tv, const Setup& u, long long gw0) {
    const long long col0 = u.m.cols > 0 ? gw0 % u.m.cols : 0;
    const bool fwd = c.mode == 0;
    int tsub = -1; float ta = 0.f, tc = 0.f;
    for (int i = 0; i < u.qk; ++i) {
        const int w = fwd ? i : u.qk - 1 - i;
        if (w / u.sublen != tsub) { tsub = w / u.sublen; wscale(T, tv, tsub, ta, tc); }
        float xv, hv; seed_val(u.m.seed_type, u.sbase, gw0 + w, xv, hv, u.m.cols);
        int r, sgn, ctx; predict_code(T, ta, tc, pb, w, xv, hv, u.hboff, r, sgn, ctx, mv, pos8(col0 + w, u.m.cols));
        c.put(ctx, (sgn * (get_code(T, fb, w) - r)) & 255);
    }
}

__global__ void __launch_bounds__(QR_TPB) k_qr_hist(const Args a, unsigned* __restrict__ counts) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= a.nseg) return;
    const int T = a.T, mv = a.mv;
    const Setup u = setup(T, a.seed, a.tm, a.sg, s);
    const float* im = u.m.imx_off >= 0 ? a.imx + u.m.imx_off : nullptr;
    Coder c; c.mode = 0; c.counts = counts; c.ovf = false;
    unsigned flagc[4] = {0, 0, 0, 0};                 // [prev * 2 + eq], added once per lane
    int prev = 1;
    for (long long b = u.g.b0; b < u.g.b0 + u.g.nb; ++b) {
        const int eq = !a.ne[b];
        ++flagc[prev * 2 + eq];
        prev = eq;
        if (eq) continue;
        const uchar* fb = a.F + b * u.bs; const uchar* pb = a.P + b * u.bs;
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, fb, tv); unpack_fields(T, pb, pv);
        int any = 0;
        for (int k = 0; k < u.nf; ++k) {
            const int kd = fkind(T, k), dl = tv[k] - fpred(T, mv, pv, k, tv[0], u.nf > 1 ? tv[1] : 0);
            if (kd < 2 && (dl < -127 || dl > 127)) { c.put(fctx(kd, any), 128); c.put(FESC_LO, tv[k] & 255); c.put(FESC_HI, tv[k] >> 8); }
            else c.put(fctx(kd, any), dl & 255);
            any |= dl != 0;
        }
        const long long gw0 = (b - u.m.blk0) * u.qk;
        if (is_grid(T)) grid_code(c, T, mv, const_cast<uchar*>(fb), pb, tv, a.gk, gw0, u.m.seed_type, u.sbase, u.m.cols, im, gtab);
        else scalar_codes(c, T, mv, const_cast<uchar*>(fb), pb, tv, u, gw0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) if (flagc[i]) atomicAdd(counts + (FLAG + (i >> 1)) * 256 + (i & 1), flagc[i]);
}

__global__ void __launch_bounds__(QR_TPB) k_qr_enc(const Args a, const RansSym* __restrict__ enc, uchar* __restrict__ out, size_t cap,
                                                   unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= a.nseg) return;
    const int T = a.T, mv = a.mv;
    const Setup u = setup(T, a.seed, a.tm, a.sg, s);
    const float* im = u.m.imx_off >= 0 ? a.imx + u.m.imx_off : nullptr;
    Coder c; c.mode = 1; c.enc = enc; c.slot = out + (size_t)s * cap; c.wr.init(c.slot + cap); c.x = RANS_L; c.ovf = false;
    for (long long b = u.g.b0 + u.g.nb - 1; b >= u.g.b0 && !c.ovf; --b) {
        const int eq = !a.ne[b];
        const int prev = b > u.g.b0 ? !a.ne[b - 1] : 1;
        if (eq) { c.put(FLAG + prev, 1); continue; }
        const uchar* fb = a.F + b * u.bs; const uchar* pb = a.P + b * u.bs;
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, fb, tv); unpack_fields(T, pb, pv);
        const long long gw0 = (b - u.m.blk0) * u.qk;
        if (is_grid(T)) grid_code(c, T, mv, const_cast<uchar*>(fb), pb, tv, a.gk, gw0, u.m.seed_type, u.sbase, u.m.cols, im, gtab);
        else scalar_codes(c, T, mv, const_cast<uchar*>(fb), pb, tv, u, gw0);
        {   // fields, last to first; anyk = what the decoder will have seen before field k
            int dl[MAXF], anyk[MAXF], any = 0;
            for (int k = 0; k < u.nf; ++k) {
                dl[k] = tv[k] - fpred(T, mv, pv, k, tv[0], u.nf > 1 ? tv[1] : 0);
                anyk[k] = any; any |= dl[k] != 0;
            }
            for (int k = u.nf - 1; k >= 0; --k) {
                const int kd = fkind(T, k);
                if (kd < 2 && (dl[k] < -127 || dl[k] > 127)) { c.put(FESC_HI, tv[k] >> 8); c.put(FESC_LO, tv[k] & 255); c.put(fctx(kd, anyk[k]), 128); }
                else c.put(fctx(kd, anyk[k]), dl[k] & 255);
            }
        }
        c.put(FLAG + prev, 0);
    }
    if (c.ovf) { out_len[s] = 0xffffffffu; return; }
    rans_flush(c.x, c.wr);
    c.wr.flush(c.slot);
    out_len[s] = c.wr.bad ? LEN_NOFREQ : (unsigned)(c.slot + cap - c.wr.ptr());
}

// ---- decoder of the scalar-code types: a warp per segment ------------------------------------------------------------
// A segment is one rANS chain, so its symbols come out one after the other; but what a block's code symbols are coded
// WITH (context, predicted code, sign) depends only on the seed, the prediction and the block's scale fields, which
// are decoded first.  So the warp decodes flag and fields in lockstep (every lane runs the same chain on the same
// bytes, which costs what one lane would), then its lanes work out contexts and predictions of the block's weights
// side by side into shared memory, the chain runs over the staged contexts, and the lanes put the codes together.
// Table lookups for symbol 0 (by far the most frequent: cum = 0, freq from a small table in shared memory) stay off
// global memory.
constexpr int DW_WARPS = 4;
struct __align__(8) DecWarpSmem {
    unsigned fblk[56], pblk[56];            // the block being rebuilt / its prediction (block sizes <= 210 bytes)
    unsigned short ctx[256];
    short pred[256];
    signed char sgn[256];
    uchar sym[256];
};
// the decoder's state and byte source: bytes come through a 64-bit register refilled every 8 bytes, reads past the
// end give zeros and set `over`
struct WarpDec {
    unsigned x;
    unsigned long long buf; int nbuf;
    const uchar* p; const uchar* end; bool over;
    const RansSym* enc; const uchar* lut; const unsigned short* f0;
    SG_DEVINL void fill() {
        buf = 0;
        const long long left = end - p;
        if (left <= 0) { over = true; nbuf = 8; return; }
        const int n = left < 8 ? (int)left : 8;
        for (int i = 0; i < n; ++i) buf |= (unsigned long long)p[i] << (56 - 8 * i);
        p += n; nbuf = n;
    }
    SG_DEVINL unsigned byte() {
        if (nbuf == 0) fill();
        const unsigned b = (unsigned)(buf >> 56);
        buf <<= 8; --nbuf;
        return b;
    }
    SG_DEVINL void init(const uchar* b, const uchar* e) {
        p = b; end = e; over = false; nbuf = 0; buf = 0; x = 0;
        for (int i = 0; i < 4; ++i) x = (x << 8) | byte();
    }
    SG_DEVINL bool finished() const { return !over && x == RANS_L && p - nbuf == end; }
    SG_DEVINL int get(int tab) {
        const unsigned slot = x & 4095u, f = f0[tab];
        int s = 0;
        if (slot < f) x = f * (x >> 12) + slot;                  // symbol 0: cum = 0
        else {
            s = lut[((size_t)tab << 12) + slot];
            const unsigned fc = enc[tab * 256 + s].fc;
            x = (fc & 0xffffu) * (x >> 12) + slot - (fc >> 16);
        }
#pragma unroll 1
        for (int guard = 0; guard < 4 && x < RANS_L; ++guard) x = (x << 8) | byte();
        return s;
    }
};
SG_DEVINL void or_byte(unsigned* blk, int i, unsigned v) { atomicOr(blk + (i >> 2), (v & 255u) << (8 * (i & 3))); }
// put_code with the bits OR-ed into a zeroed block in shared memory, safe for lanes that share a byte
SG_DEVINL void put_code_shared(int T, unsigned* blk, int w, int q) {
    const CodeLoc L = code_loc(T, w);
    if (T == 8) { or_byte(blk, L.lo_byte, (unsigned)q); return; }
    if (L.hi_bits) {
        or_byte(blk, L.lo_byte, (unsigned)((q & ((1 << L.lo_bits) - 1)) << L.lo_shift));
        or_byte(blk, L.hi_byte, (unsigned)(((q >> L.lo_bits) & ((1 << L.hi_bits) - 1)) << L.hi_shift));
    } else if (L.lo_bits == 2) or_byte(blk, L.lo_byte, (unsigned)((q & 3) << L.lo_shift));
    else or_byte(blk, L.lo_byte, (unsigned)(q << L.lo_shift));
}

// W lanes per segment, 32 / W segments per warp.  A chain instruction issued by a warp advances 32 / W chains, so a
// small W wastes fewer issue slots on the lockstep parts, a large W spreads the per-weight work wider.  The warp's
// control flow is kept uniform (every segment of the warp is at its j-th block; segments whose block equals its
// prediction, or that have ended, sit the phases out), so the lane groups stay converged.
template <int W>
__global__ void __launch_bounds__(DW_WARPS * 32) k_qr_dec_warp(const Args a, const uchar* __restrict__ in, const unsigned long long* __restrict__ off,
                                                               const RansSym* __restrict__ enc, const uchar* __restrict__ lut,
                                                               uchar* __restrict__ F, int* __restrict__ status) {
    constexpr int SPW = 32 / W;
    __shared__ unsigned short f0[NTAB2];
    __shared__ DecWarpSmem wsm[DW_WARPS * SPW];
    for (int t = threadIdx.x; t < NTAB2; t += blockDim.x) f0[t] = (unsigned short)(enc[t * 256].fc & 0xffffu);
    __syncthreads();
    const int lane = threadIdx.x & 31, sub = lane % W, grp = (threadIdx.x >> 5) * SPW + lane / W;
    const int s = blockIdx.x * (DW_WARPS * SPW) + grp;
    const bool have = s < a.nseg;
    DecWarpSmem& m = wsm[grp];
    const int T = a.T, mv = a.mv;
    const Setup u = setup(T, a.seed, a.tm, a.sg, have ? s : a.nseg - 1);
    WarpDec c; c.enc = enc; c.lut = lut; c.f0 = f0;
    if (have) c.init(in + off[s], in + off[s + 1]);
    else { c.init(in, in); c.x = RANS_L; c.over = false; }
    uchar* fb = reinterpret_cast<uchar*>(m.fblk);
    const uchar* pbs = reinterpret_cast<const uchar*>(m.pblk);
    const int nb = have ? u.g.nb : 0;
    const int nbmax = (int)__reduce_max_sync(0xffffffffu, (unsigned)nb);
    int prev = 1;
    for (int j = 0; j < nbmax; ++j) {
        const bool live = j < nb && !c.over;
        const long long b = u.g.b0 + j;
        const uchar* pg = a.P + b * u.bs;
        uchar* fg = F + b * u.bs;
        int eq = 1;
        if (live) { eq = c.get(FLAG + prev); prev = eq; }
        if (live && eq) for (int i = sub; i < u.bs; i += W) fg[i] = pg[i];
        const bool code = live && !eq;
        if (!__any_sync(0xffffffffu, code)) continue;
        __syncwarp();
        if (code) {
            for (int i = sub; i < 56; i += W) m.fblk[i] = 0;
            for (int i = sub; i < u.bs; i += W) reinterpret_cast<uchar*>(m.pblk)[i] = pg[i];
        }
        __syncwarp();
        int tv[MAXF];
        if (code) {
            int pv[MAXF];
            unpack_fields(T, pbs, pv);
            int any = 0;
            for (int k = 0; k < u.nf; ++k) {
                const int kd = fkind(T, k);
                const int pr = fpred(T, mv, pv, k, k > 0 ? tv[0] : 0, k > 1 ? tv[1] : 0);
                const int sym = c.get(fctx(kd, any));
                int t;
                if (kd < 2 && sym == 128) { const int lo = c.get(FESC_LO), hi = c.get(FESC_HI); t = lo | (hi << 8); }
                else {
                    t = pr + (int)(signed char)sym;
                    if (kd < 2) t &= 0xffff;
                    else if (T == 14) t = (int)(signed char)(t & 255);
                }
                tv[k] = t; any |= t != pr;
            }
            if (sub == 0) pack_fields(T, fb, tv);
            // contexts and predictions of the block's weights, side by side
            const long long gw0 = (b - u.m.blk0) * u.qk;
            const long long col0 = u.m.cols > 0 ? gw0 % u.m.cols : 0;
            int tsub = -1; float ta = 0.f, tc = 0.f;
            for (int w = sub; w < u.qk; w += W) {
                if (w / u.sublen != tsub) { tsub = w / u.sublen; wscale(T, tv, tsub, ta, tc); }
                float xv, hv; seed_val(u.m.seed_type, u.sbase, gw0 + w, xv, hv, u.m.cols);
                int r, sgn, ctx; predict_code(T, ta, tc, pbs, w, xv, hv, u.hboff, r, sgn, ctx, mv, pos8(col0 + w, u.m.cols));
                m.ctx[w] = (unsigned short)ctx; m.pred[w] = (short)r; m.sgn[w] = (signed char)sgn;
            }
        }
        __syncwarp();
        if (code) {
#pragma unroll 1
            for (int w = 0; w < u.qk; w += 4) {          // four contexts per load, four symbols per store
                const uint2 cx = *reinterpret_cast<const uint2*>(m.ctx + w);
                unsigned sy = (unsigned)c.get((int)(cx.x & 0xffffu));
                sy |= (unsigned)c.get((int)(cx.x >> 16)) << 8;
                sy |= (unsigned)c.get((int)(cx.y & 0xffffu)) << 16;
                sy |= (unsigned)c.get((int)(cx.y >> 16)) << 24;
                if (sub == 0) *reinterpret_cast<unsigned*>(m.sym + w) = sy;
            }
        }
        __syncwarp();
        if (code) {
            for (int w = sub; w < u.qk; w += W) {
                int q = m.pred[w] + m.sgn[w] * (int)(signed char)m.sym[w];
                if (T == 8) q = (int)(signed char)(q & 255);
                put_code_shared(T, m.fblk, w, q);
            }
        }
        __syncwarp();
        if (code) for (int i = sub; i < u.bs; i += W) fg[i] = fb[i];
    }
    if (have && sub == 0 && !c.finished()) atomicOr(status, SG_ST_CORRUPT);
}

// ---- decoder of the lattice types: a warp per segment ------------------------------------------------------------------
// What makes these blocks expensive is the ordering of all 256 - 2048 lattice points by their weighted distance to the
// seed, once per group of 4 / 8 weights.  Here the 32 lanes of the warp share that: every lane measures the points
// lane, lane + 32, ... and keeps its own 16 closest in order; the warp's closest, second closest, ... come out of
// rounds of an arg-min over the lanes' list heads (only as many rounds as the decoded rank needs).  Everything that is
// one chain (flag, fields, ranks, signs) is decoded by all lanes in lockstep.
struct GridWarpSmem {
    unsigned fblk[28], pblk[28];            // block sizes <= 110 bytes
    float xs[256];                          // the block's seed values
    float tab[128];                         // pair tables of the group being ranked: [pair][levels]
    float dist[2048];                       // distance of every lattice point of the group being ranked
    float gu[256], gw[256];                 // per weight: seed value over the unit's scale (sign-folded), search weight
    unsigned char pn[32];                   // per unit of 8 weights: which seed values count as negative
};
template <int N> SG_DEVINL float point_dist_w(const float* tab, unsigned key) {
    constexpr int B = N == 8 ? 2 : 3, E = 1 << (2 * B);
    float d = 0.f;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) d = d + tab[p * E + ((key >> (2 * B * p)) & (E - 1))];
    return isnan(d) ? __int_as_float(0x7f800000) : d;
}
template <int N, bool SGN>
SG_DEVINL void grid_block_warp(WarpDec& c, GridWarpSmem& m, int lane, int T, int mv, const int* tv, const uint16_t* __restrict__ gk,
                               long long gw0, int cols, const float* im) {
    constexpr int B = N == 8 ? 2 : 3, ng = 8 / N, L = 1 << B, E = L * L;
    const float inf = __int_as_float(0x7f800000);
    uchar* fb = reinterpret_cast<uchar*>(m.fblk);
    const uchar* pb = reinterpret_cast<const uchar*>(m.pblk);
    const int gs = grid_size(T);
    const bool par = parity_type(T);
    float sx2 = 0.f;
    for (int i = 0; i < 256; ++i) { const float xv = m.xs[i]; sx2 += xv * xv; }
    const float sigma2 = (T == 16 || T == 17) ? sx2 * (1.0f / 256.f) : 2.f * sx2 * (1.0f / 256.f);
    const long long col0 = cols > 0 ? gw0 % cols : 0;
    // what a unit's ranking needs from the seed, one unit per lane: weights, sign folding with the parity repair, values
    // over the unit's scale (the scale does not depend on IQ1_M's shift bit, only the level offset does)
    {
        const int u = lane;
        float gs_, gdl0;
        gscale(T, fb, tv, u, gs_, gdl0);
        float x[8], v[8], wv[8];
        int pnb = 0;
        for (int i = 0; i < 8; ++i) {
            x[i] = m.xs[8 * u + i];
            float wi = sqrtf(sigma2 + x[i] * x[i]);
            if (im) wi = wi * im[(gw0 + 8 * u + i) % cols];
            wv[i] = wi;
            if (x[i] < 0.f) pnb |= 1 << i;
            v[i] = SGN ? fabsf(x[i]) : x[i];
        }
        if (SGN && par && (__popc(pnb) & 1)) {         // an odd number of negatives: the least weighty one flips back
            int imin = 0; float mn = wv[0] * x[0] * x[0];
            for (int i = 1; i < 8; ++i) { const float a = wv[i] * x[i] * x[i]; if (a < mn) { mn = a; imin = i; } }
            pnb ^= 1 << imin;
            for (int i = 0; i < 8; ++i) if (i == imin) v[i] = -v[i];
        }
        for (int i = 0; i < 8; ++i) { m.gu[8 * u + i] = v[i] / gs_; m.gw[8 * u + i] = wv[i]; }
        m.pn[u] = (unsigned char)pnb;
    }
    __syncwarp();
    for (int u = 0; u < 32; ++u) {
        const int p4 = pos4(col0 + 8 * u, cols);
        const int rank0 = mv >= 2 ? GRANK2 + 4 * p4 : GRID_RANK;
        const int sign0 = mv >= 2 ? GSIGN2 + 16 * p4 : GRID_SIGN;
        if (T == 29) { if (c.get(GRID_SHIFT) ^ get_shift(pb, u)) { if (lane == 0) put_shift(fb, u); } __syncwarp(); }
        float gu[8], gw[8], gs_, gdl;
        int pn[8];
        gscale(T, fb, tv, u, gs_, gdl);
        for (int i = 0; i < 8; ++i) { gu[i] = m.gu[8 * u + i]; gw[i] = m.gw[8 * u + i]; pn[i] = (m.pn[u] >> i) & 1; }
        int tg[2] = {0, 0};
        for (int gg = 0; gg < ng; ++gg) {
            // pair tables of this group, entries spread over the lanes
            __syncwarp();
            for (int e = lane; e < (N / 2) * E; e += 32) {
                const int p = e / E, ee = e % E, la = ee & (L - 1), lb = ee >> B;
                const float qa = SGN ? (float)(2 * la + 1) : (float)(la - 1) + gdl;
                const float qb = SGN ? (float)(2 * lb + 1) : (float)(lb - 1) + gdl;
                float ua = 0.f, ub = 0.f, wa = 0.f, wb = 0.f;
#pragma unroll
                for (int i = 0; i < N / 2; ++i) if (i == p) { ua = gu[gg * N + 2 * i]; ub = gu[gg * N + 2 * i + 1]; wa = gw[gg * N + 2 * i]; wb = gw[gg * N + 2 * i + 1]; }
                const float ea = qa - ua, eb = qb - ub;
                m.tab[e] = wa * (ea * ea) + wb * (eb * eb);
            }
            __syncwarp();
            // distances of all points; every lane remembers the closest of its own (points lane, lane + 32, ...)
            float md = inf; int mk = 0x7fffffff;
            for (int k = lane; k < gs; k += 32) {
                const float d = point_dist_w<N>(m.tab, __ldg(gk + k));
                m.dist[k] = d;
                if (d < md) { md = d; mk = k; }
            }
            // the warp's next closest point in the order (distance, index): arg-min over the lanes' closest; the winning
            // lane strikes its point out and looks for its next one.  Points at infinite distance never come up.
            auto next = [&](float& bd, int& bk) {
                bd = md; bk = mk;
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) {
                    const float od = __shfl_xor_sync(0xffffffffu, bd, sft);
                    const int ok = __shfl_xor_sync(0xffffffffu, bk, sft);
                    if (od < bd || (od == bd && ok < bk)) { bd = od; bk = ok; }
                }
                if (bk == mk && bk != 0x7fffffff) {
                    m.dist[mk] = inf;
                    md = inf; mk = 0x7fffffff;
                    for (int k = lane; k < gs; k += 32) { const float d = m.dist[k]; if (d < md) { md = d; mk = k; } }
                }
            };
            float d1, d2; int k1, k2;
            next(d1, k1); next(d2, k2);
            const int r = c.get(rank0 + gapctx(d1, d2));
            int t;
            if (r >= TOPK) { const int lo = c.get(FESC_LO), hi = c.get(FESC_HI); t = (lo | (hi << 8)) % gs; }
            else {
                // slot r of the ordered list; slots beyond the points at finite distance keep their own number
                t = r == 0 ? k1 : k2;
                for (int j = 2; j <= r; ++j) { float dj; next(dj, t); }
                if (t == 0x7fffffff) t = r;
            }
            if (lane == 0) put_gidx(T, fb, u * ng + gg, t);
            tg[gg] = t;
        }
        __syncwarp();
        if (SGN) for (int j = 0; j < 8; ++j) {
            if (par && j == 7) continue;
            const int lev = (gk[tg[j / N]] >> (B * (j % N))) & ((1 << B) - 1);
            const float m4 = fabsf(gu[j]) * 4.f;
            const int sctx = sign0 + (lev == 0) * 8 + (m4 < 7.f ? (int)m4 : 7);
            if (c.get(sctx) ^ pn[j]) { if (lane == 0) put_neg(T, fb, 8 * u + j); }
        }
        __syncwarp();
        if (c.over) return;
    }
}

__global__ void __launch_bounds__(DW_WARPS * 32) k_qr_dec_grid_warp(const Args a, const uchar* __restrict__ in, const unsigned long long* __restrict__ off,
                                                                    const RansSym* __restrict__ enc, const uchar* __restrict__ lut,
                                                                    uchar* __restrict__ F, int* __restrict__ status) {
    __shared__ unsigned short f0[NTAB2];
    __shared__ GridWarpSmem wsm[DW_WARPS];
    for (int t = threadIdx.x; t < NTAB2; t += blockDim.x) f0[t] = (unsigned short)(enc[t * 256].fc & 0xffffu);
    __syncthreads();
    const int lane = threadIdx.x & 31, s = blockIdx.x * DW_WARPS + (threadIdx.x >> 5);
    if (s >= a.nseg) return;
    GridWarpSmem& m = wsm[threadIdx.x >> 5];
    const int T = a.T, mv = a.mv;
    const Setup u = setup(T, a.seed, a.tm, a.sg, s);
    const float* im = u.m.imx_off >= 0 ? a.imx + u.m.imx_off : nullptr;
    WarpDec c; c.enc = enc; c.lut = lut; c.f0 = f0;
    c.init(in + off[s], in + off[s + 1]);
    uchar* fb = reinterpret_cast<uchar*>(m.fblk);
    const uchar* pbs = reinterpret_cast<const uchar*>(m.pblk);
    int prev = 1;
    for (long long b = u.g.b0; b < u.g.b0 + u.g.nb && !c.over; ++b) {
        const uchar* pg = a.P + b * u.bs;
        uchar* fg = F + b * u.bs;
        const int eq = c.get(FLAG + prev);
        prev = eq;
        if (eq) { for (int i = lane; i < u.bs; i += 32) fg[i] = pg[i]; continue; }
        const long long gw0 = (b - u.m.blk0) * u.qk;
        __syncwarp();
        if (lane < 28) m.fblk[lane] = 0;
        for (int i = lane; i < u.bs; i += 32) reinterpret_cast<uchar*>(m.pblk)[i] = pg[i];
        for (int i = lane; i < 256; i += 32) { float xv, hv; seed_val(u.m.seed_type, u.sbase, gw0 + i, xv, hv, u.m.cols); m.xs[i] = xv; }
        __syncwarp();
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, pbs, pv);
        int any = 0;
        for (int k = 0; k < u.nf; ++k) {
            const int kd = fkind(T, k);
            const int pr = fpred(T, mv, pv, k, k > 0 ? tv[0] : 0, k > 1 ? tv[1] : 0);
            const int sym = c.get(fctx(kd, any));
            int t;
            if (kd < 2 && sym == 128) { const int lo = c.get(FESC_LO), hi = c.get(FESC_HI); t = lo | (hi << 8); }
            else {
                t = pr + (int)(signed char)sym;
                if (kd < 2) t &= 0xffff;
            }
            tv[k] = t; any |= t != pr;
        }
        if (lane == 0) pack_fields(T, fb, tv);
        __syncwarp();
        switch (T) {
            case 18: case 21: grid_block_warp<4, true>(c, m, lane, T, mv, tv, a.gk, gw0, u.m.cols, im); break;
            case 19: case 29: grid_block_warp<8, false>(c, m, lane, T, mv, tv, a.gk, gw0, u.m.cols, im); break;
            default: grid_block_warp<8, true>(c, m, lane, T, mv, tv, a.gk, gw0, u.m.cols, im);
        }
        __syncwarp();
        for (int i = lane; i < u.bs; i += 32) fg[i] = fb[i];
    }
    if (lane == 0 && !c.finished()) atomicOr(status, SG_ST_CORRUPT);
}

// ---- encoding in two steps ---------------------------------------------------------------------------------------
// The model (fields, predictions, contexts, lattice ranks) of a block does not depend on the coder's state, only the
// rANS walk does.  So one lane per BLOCK first writes the block's (table, symbol) pairs down in the order the encoder
// consumes them; the histogram is a count over those pairs, and the coder proper is one lane per segment walking
// staged pairs.  The model runs once instead of twice, on seg_blocks(T) times as many lanes.
// Staging: cnt[b] pairs of block b at stage[b * capb ...], a pair is table * 256 + symbol.
__global__ void __launch_bounds__(QR_TPB) k_qr_stage(const Args a, int segb, unsigned* __restrict__ stage, unsigned short* __restrict__ cnt,
                                                     int capb) {
    const long long lane = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int s = (int)(lane / segb), j = (int)(lane % segb);
    if (s >= a.nseg) return;
    const int T = a.T, mv = a.mv;
    const Setup u = setup(T, a.seed, a.tm, a.sg, s);
    if (j >= u.g.nb) return;
    const long long b = u.g.b0 + j;
    const float* im = u.m.imx_off >= 0 ? a.imx + u.m.imx_off : nullptr;
    Coder c; c.mode = 3; c.stage = stage + (size_t)b * capb; c.nstaged = 0; c.ovf = false;
    const int eq = !a.ne[b];
    const int prev = j > 0 ? !a.ne[b - 1] : 1;
    if (eq) c.put(FLAG + prev, 1);
    else {
        const uchar* fb = a.F + b * u.bs; const uchar* pb = a.P + b * u.bs;
        int tv[MAXF], pv[MAXF];
        unpack_fields(T, fb, tv); unpack_fields(T, pb, pv);
        const long long gw0 = (b - u.m.blk0) * u.qk;
        if (is_grid(T)) grid_code(c, T, mv, const_cast<uchar*>(fb), pb, tv, a.gk, gw0, u.m.seed_type, u.sbase, u.m.cols, im, gtab);
        else scalar_codes(c, T, mv, const_cast<uchar*>(fb), pb, tv, u, gw0);
        int dl[MAXF], anyk[MAXF], any = 0;
        for (int k = 0; k < u.nf; ++k) {
            dl[k] = tv[k] - fpred(T, mv, pv, k, tv[0], u.nf > 1 ? tv[1] : 0);
            anyk[k] = any; any |= dl[k] != 0;
        }
        for (int k = u.nf - 1; k >= 0; --k) {
            const int kd = fkind(T, k);
            if (kd < 2 && (dl[k] < -127 || dl[k] > 127)) { c.put(FESC_HI, tv[k] >> 8); c.put(FESC_LO, tv[k] & 255); c.put(fctx(kd, anyk[k]), 128); }
            else c.put(fctx(kd, anyk[k]), dl[k] & 255);
        }
        c.put(FLAG + prev, 0);
    }
    cnt[b] = (unsigned short)c.nstaged;
}

// counts over the staged pairs, equal pairs of a warp added once.  A warp takes 32 blocks at a time: blocks with a
// single pair (equal to their prediction: just the flag) are counted one per lane, the others one after the other
// by the whole warp.
__global__ void __launch_bounds__(256) k_qr_stage_hist(long long nblocks, const unsigned* __restrict__ stage, const unsigned short* __restrict__ cnt,
                                                        int capb, unsigned* __restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    auto add = [&](unsigned e, bool live) {
        const unsigned peers = __match_any_sync(0xffffffffu, live ? e : 0xffffffffu);
        if (live && lane == __ffs(peers) - 1) atomicAdd(counts + e, (unsigned)__popc(peers));
    };
    for (long long b0 = warp * 32; b0 < nblocks; b0 += nwarps * 32) {
        const long long b = b0 + lane;
        const int n = b < nblocks ? cnt[b] : 0;
        add(n == 1 ? stage[(size_t)b * capb] : 0u, n == 1);
        unsigned many = __ballot_sync(0xffffffffu, n > 1);
        while (many) {
            const int src = __ffs(many) - 1;
            many &= many - 1;
            const int nn = __shfl_sync(0xffffffffu, n, src);
            const unsigned* p = stage + (size_t)(b0 + src) * capb;
            for (int i0 = 0; i0 < nn; i0 += 32) add(i0 + lane < nn ? p[i0 + lane] : 0u, i0 + lane < nn);
        }
    }
}

// the coder proper: one lane per segment, blocks last to first, each block's staged pairs in order
__global__ void __launch_bounds__(QR_TPB) k_qr_stage_code(const SG* __restrict__ sg, int nseg, const unsigned* __restrict__ stage,
                                                           const unsigned short* __restrict__ cnt, int capb, const RansSym* __restrict__ enc,
                                                           uchar* __restrict__ out, size_t cap, unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const SG g = sg[s];
    uchar* slot = out + (size_t)s * cap;
    ByteWriterDown wr; wr.init(slot + cap);
    unsigned x = RANS_L;
    bool ovf = false;
    for (long long b = g.b0 + g.nb - 1; b >= g.b0 && !ovf; --b) {
        const int n = cnt[b];
        const unsigned* p = stage + (size_t)b * capb;
        int i = 0;
        for (; i + 4 <= n; i += 4) {            // table entries do not depend on the coder state: four loads in flight
            const uint4 e4 = *reinterpret_cast<const uint4*>(p + i);
            const RansSym s0 = enc[e4.x], s1 = enc[e4.y], s2 = enc[e4.z], s3 = enc[e4.w];
            rans_put<12>(x, wr, s0); rans_put<12>(x, wr, s1); rans_put<12>(x, wr, s2); rans_put<12>(x, wr, s3);
            if (wr.ptr() < slot + 64) { ovf = true; break; }
        }
        for (; i < n && !ovf; ++i) {
            rans_put<12>(x, wr, enc[p[i]]);
            if (wr.ptr() < slot + 64) ovf = true;
        }
    }
    if (ovf) { out_len[s] = 0xffffffffu; return; }
    rans_flush(x, wr);
    wr.flush(slot);
    out_len[s] = wr.bad ? LEN_NOFREQ : (unsigned)(slot + cap - wr.ptr());
}

}  // namespace qr
}  // namespace sg

using namespace sg;
using namespace sg::qr;

static size_t grid_smem(int T) {
    switch (T) { case 18: case 21: return (size_t)QR_TPB * 4 * 128; case 16: case 17: case 19: case 22: case 29: return (size_t)QR_TPB * 4 * 64; }
    return 0;
}
static int grid_table_index(int T) {
    switch (T) { case 16: return 0; case 17: return 1; case 19: case 29: return 2; case 22: return 3; case 18: return 4; case 21: return 5; }
    return -1;
}
namespace sg { const uint16_t* device_grid_keys(int device, int which); }      // tables.cu

static int qr_args(int device, Args& a, int T, const void* F, const void* P, const void* ne, const void* seed, const void* tm,
                   const void* sgp, int nseg, const float* imx, int mv) {
    if (!P || !seed || !tm || !sgp || nseg < 0 || (mv != 1 && mv != 2)) return SG_ERR_ARG;
    int qk, bs;
    if (sg_type_info(T, &qk, &bs) != SG_OK) return SG_ERR_TYPE;
    a.T = T; a.mv = mv; a.nseg = nseg;
    a.F = (const uchar*)F; a.P = (const uchar*)P; a.ne = (const uchar*)ne; a.seed = (const uchar*)seed;
    a.tm = (const TM*)tm; a.sg = (const SG*)sgp; a.imx = imx; a.gk = nullptr;
    const int gi = grid_table_index(T);
    if (gi >= 0) {
        a.gk = device_grid_keys(device, gi);
        if (!a.gk) return SG_ERR_TABLES;
    }
    return SG_OK;
}

extern "C" int sg_qr_hist(int device, void* stream, int T, const unsigned char* F, const unsigned char* P, const unsigned char* ne,
                          const unsigned char* seed, const void* tm, const void* sgp, int nseg, const float* imx, unsigned* counts, int mv) {
    Args a;
    int rc = qr_args(device, a, T, F, P, ne, seed, tm, sgp, nseg, imx, mv);
    if (rc != SG_OK) return rc;
    if (!F || !ne || !counts) return SG_ERR_ARG;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_qr_hist<<<(nseg + QR_TPB - 1) / QR_TPB, QR_TPB, grid_smem(T), (cudaStream_t)stream>>>(a, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_encode(int device, void* stream, int T, const unsigned char* F, const unsigned char* P, const unsigned char* ne,
                            const unsigned char* seed, const void* tm, const void* sgp, int nseg, const float* imx, const void* enc_tab,
                            unsigned char* slots, size_t cap, unsigned* out_len, int mv) {
    Args a;
    int rc = qr_args(device, a, T, F, P, ne, seed, tm, sgp, nseg, imx, mv);
    if (rc != SG_OK) return rc;
    if (!F || !ne || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 128 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_qr_enc<<<(nseg + QR_TPB - 1) / QR_TPB, QR_TPB, grid_smem(T), (cudaStream_t)stream>>>(a, (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_decode(int device, void* stream, int T, const unsigned char* in, const unsigned long long* off,
                            const unsigned char* P, const unsigned char* seed, const void* tm, const void* sgp, int nseg, const float* imx,
                            const void* enc_tab, const unsigned char* lut, unsigned char* F, int mv) {
    Args a;
    int rc = qr_args(device, a, T, nullptr, P, nullptr, seed, tm, sgp, nseg, imx, mv);
    if (rc != SG_OK) return rc;
    if (!in || !off || !enc_tab || !lut || !F) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    if (qr::is_grid(T))
        k_qr_dec_grid_warp<<<(nseg + DW_WARPS - 1) / DW_WARPS, DW_WARPS * 32, 0, (cudaStream_t)stream>>>(a, in, off, (const RansSym*)enc_tab, lut, F,
                                                                                                      status_word(device));
    else
    {
        constexpr int W = 8, per_cta = DW_WARPS * (32 / W);
        k_qr_dec_warp<W><<<(nseg + per_cta - 1) / per_cta, DW_WARPS * 32, 0, (cudaStream_t)stream>>>(a, in, off, (const RansSym*)enc_tab, lut, F,
                                                                                                  status_word(device));
    }
    return cuda_ok(cudaGetLastError());
}

// pairs one block can produce: flag + fields (an escaped field takes three) + codes, or for a lattice type per unit of
// 8 weights the ranks (an escaped rank takes three), 8 signs and a shift bit; rounded up to a multiple of 4
static int stage_capb(int T) {
    int qk, bs;
    if (sg_type_info(T, &qk, &bs) != SG_OK) return 0;
    const int nf = qr::nfield(T);
    const int n = 1 + 3 * nf + (qr::is_grid(T) ? 32 * (2 * 3 + 8 + 1) : qk);
    return (n + 3) / 4 * 4;
}
static size_t stage_cnt_bytes(long long nblocks) { return ((size_t)nblocks * 2 + 255) / 256 * 256; }

extern "C" size_t sg_qr_stage_bytes(int T, long long nblocks) {
    const int capb = stage_capb(T);
    if (!capb || nblocks < 0) return 0;
    return stage_cnt_bytes(nblocks) + (size_t)nblocks * capb * 4;
}

extern "C" int sg_qr_stage(int device, void* stream, int T, const unsigned char* F, const unsigned char* P, const unsigned char* ne,
                           const unsigned char* seed, const void* tm, const void* sgp, int nseg, const float* imx, int mv,
                           long long nblocks, void* stage, size_t stage_bytes) {
    Args a;
    int rc = qr_args(device, a, T, F, P, ne, seed, tm, sgp, nseg, imx, mv);
    if (rc != SG_OK) return rc;
    if (!F || !ne || !stage || nblocks < 0) return SG_ERR_ARG;
    if ((uintptr_t)stage % 16) return SG_ERR_ALIGN;
    if (stage_bytes < sg_qr_stage_bytes(T, nblocks)) return SG_ERR_SCRATCH;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    const int segb = 16384 / qr::qk_of(T) > 16 ? 16384 / qr::qk_of(T) : 16, capb = stage_capb(T);      // seg_blocks, qr.py:952-954
    const long long lanes = (long long)nseg * segb;
    k_qr_stage<<<(unsigned)((lanes + QR_TPB - 1) / QR_TPB), QR_TPB, grid_smem(T), (cudaStream_t)stream>>>(
        a, segb, (unsigned*)((uchar*)stage + stage_cnt_bytes(nblocks)), (unsigned short*)stage, capb);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_stage_hist(int device, void* stream, int T, long long nblocks, const void* stage, unsigned* counts) {
    const int capb = stage_capb(T);
    if (!capb) return SG_ERR_TYPE;
    if (!stage || !counts || nblocks < 0) return SG_ERR_ARG;
    if (nblocks == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long want = (nblocks + 255) / 256;
    k_qr_stage_hist<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), 256, 0, (cudaStream_t)stream>>>(
        nblocks, (const unsigned*)((const uchar*)stage + stage_cnt_bytes(nblocks)), (const unsigned short*)stage, capb, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_qr_stage_encode(int device, void* stream, int T, long long nblocks, const void* stage, const void* sgp, int nseg,
                                  const void* enc_tab, unsigned char* slots, size_t cap, unsigned* out_len) {
    const int capb = stage_capb(T);
    if (!capb) return SG_ERR_TYPE;
    if (!stage || !sgp || !enc_tab || !slots || !out_len || nseg < 0 || nblocks < 0) return SG_ERR_ARG;
    if (cap < 128 || cap % 16 || (uintptr_t)slots % 16 || (uintptr_t)stage % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_qr_stage_code<<<(nseg + QR_TPB - 1) / QR_TPB, QR_TPB, 0, (cudaStream_t)stream>>>(
        (const SG*)sgp, nseg, (const unsigned*)((const uchar*)stage + stage_cnt_bytes(nblocks)), (const unsigned short*)stage, capb,
        (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}
