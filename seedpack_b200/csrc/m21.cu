// M21: Q8_0 GGUFs that no base predicts (the "seed" of a repository without its BF16 model).  Kernels of the
// reference's GPU2 / GPU3 codecs (seedpack/gpu2.py:100-262 hist_a / enc_a / dec_a / hist_b / enc_b / dec_b,
// seedpack/gpu3.py:90-232 predict / predict_multi / hist_c / enc_c / dec_c), rANS at 12 probability bits (rans.cuh).
//
// A Q8_0 block = fp16 scale + 32 int8 codes.  Three phases share the blocks (34 bytes each, tensors back to back):
//   A  per block: scale high byte | previous block's high byte (and the column block's class), scale low byte | high
//      byte, position of the largest magnitude (its rank among the column block's usual positions), the code there;
//      segments of `sega` blocks
//   B  the other 31 codes: magnitude | bin of the expected magnitude (column factor, row mean and block scale), sign |
//      bin and column class; segments of `segb` blocks
//   C  rows of selected tensors predicted from similar rows decoded earlier: code minus prediction | the same bin
//      shifted by the row's class; segments of a few rows, ordered wave by wave
// skip[b]: bit 0 = the block is not coded at all (a duplicate row), bit 1 = phase C codes its 31 codes, bit 2 = phase C
// codes position and largest code too.  Records: Meta { int32 first, nblocks, nb_row, grp, colbase, rowbase, off, qset }
// per tensor (gpu2.py:56).  Tables are addressed by raw id; counts / enc_tab / lut cover the id space of the phase's call.
#include "api_util.h"
#include "common.cuh"
#include "rans.cuh"

namespace sg {
namespace m21 {

struct Meta { int first, nblocks, nb_row, grp, colbase, rowbase, off, qset; };

// ByteWriterDown that knows where its slot begins: the reference sizes these slots for typical data (68 bytes a block)
// and does not look; here a window that would land below the slot is not stored and the segment reports an overflow
struct SlotWriter {
    uint8_t* base; unsigned long long lo, hi; int pos; unsigned bad; uint8_t* lim; bool over;
    SG_DEVINL void init(uint8_t* end, uint8_t* slot_begin) { base = end - 16; lo = hi = 0; pos = 16; bad = 0; lim = slot_begin; over = false; }
    SG_DEVINL void put(unsigned b) {
        --pos;
        if (pos >= 8) hi |= (unsigned long long)b << (8 * (pos - 8));
        else          lo |= (unsigned long long)b << (8 * pos);
        if (pos == 0) {
            if (base >= lim) *reinterpret_cast<ulonglong2*>(base) = make_ulonglong2(lo, hi); else over = true;
            base -= 16; lo = hi = 0; pos = 16;
        }
    }
    SG_DEVINL uint8_t* ptr() const { return base + pos; }
    // the partial window; -> the segment's length, or the overflow mark
    SG_DEVINL unsigned finish(uint8_t* end) {
        if (over || ptr() < lim) return LEN_OVERFLOW;
        if (pos < 16) {
            if (base >= lim) *reinterpret_cast<ulonglong2*>(base) = make_ulonglong2(lo, hi);
            else for (int k = pos; k < 16; ++k) base[k] = (uint8_t)((k >= 8 ? hi >> (8 * (k - 8)) : lo >> (8 * k)) & 0xff);
        }
        return bad ? LEN_NOFREQ : (unsigned)(end - ptr());
    }
};

// compile-time switches of the reference's module, passed at run time
struct Opt { int sign, rank, hicf, preda; };

SG_DEVINL int tensor_of(const Meta* __restrict__ M, int ntens, int b) {           // the last tensor that starts at or before block b
    int lo = 0, hi = ntens - 1;
    while (lo < hi) { const int m = (lo + hi + 1) >> 1; if (M[m].first <= b) lo = m; else hi = m - 1; }
    return lo;
}
SG_DEVINL int magnitude_bin(int cf, int sh) {
    const int u = (cf * 128 + sh) >> 7;
    return u < 0 ? 0 : (u > 63 ? 63 : u);
}
SG_DEVINL int clamp63(int v) { return v < 0 ? 0 : (v > 63 ? 63 : v); }

// ---- phase A ---------------------------------------------------------------------------------------------------------
// (column classes, spreads and column-block factors come from the archive's side information: 16 of each by format, masked
// to that range where they select a table)
struct SideA { const unsigned char* bcf; const unsigned char* spread; const unsigned char* perm; const unsigned char* rankof; const unsigned char* scls; };
struct TabA {
    int lo, pos, mx, per_group;
    SG_DEVINL explicit TabA(const Opt& o) { lo = 256 * (o.hicf ? 16 : 1); pos = lo + 256; mx = pos + 16; per_group = mx + 16; }
};
// the block's four (table, symbol) pairs in decode order; n = 2 when position and largest code belong to phase C
SG_DEVINL int symbols_a(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos, const unsigned char* __restrict__ skip,
                        const Meta& m, const SideA& sd, const Opt& o, const TabA& ta, int b, int prev, unsigned* out) {
    const unsigned char* blk = blocks + (size_t)b * 34;
    const int inrow = (b - m.first) % m.nb_row;
    const int cb = m.colbase / 32 + inrow, c0 = m.colbase + inrow * 32, base = m.grp * ta.per_group;
    const int hi = blk[1], p = pos[b];
    out[0] = (unsigned)(base + prev + (o.hicf ? 256 * (sd.bcf[cb] & 15) : 0)) << 8 | (unsigned)hi;
    out[1] = (unsigned)(base + ta.lo + hi) << 8 | blk[0];
    if (skip[b] & 4) return 2;
    out[2] = o.rank ? (unsigned)(base + ta.pos + (sd.spread[cb] & 15)) << 8 | sd.rankof[cb * 32 + p] : (unsigned)(base + ta.pos) << 8 | (unsigned)p;
    out[3] = (unsigned)(base + ta.mx + (o.sign ? (sd.scls[c0 + p] & 15) : 0)) << 8 | blk[2 + p];
    return 4;
}

__global__ void __launch_bounds__(64) k_hist_a(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                               const unsigned char* __restrict__ skip, const Meta* __restrict__ M, int ntens, int nblocks,
                                               SideA sd, Opt o, int seg, unsigned* __restrict__ counts) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long b0 = (long long)s * seg;
    if (b0 >= nblocks) return;
    const int b1 = (int)min(b0 + seg, (long long)nblocks);
    const TabA ta(o);
    int t = tensor_of(M, ntens, (int)b0);
    unsigned sy[4];
    for (int b = (int)b0; b < b1; ++b) {
        while (t + 1 < ntens && b >= M[t + 1].first) ++t;
        if (skip[b] & 1) continue;
        const int inrow = (b - M[t].first) % M[t].nb_row;
        const int prev = (inrow == 0 || b == (int)b0) ? 0 : blocks[(size_t)(b - 1) * 34 + 1];
        const int n = symbols_a(blocks, pos, skip, M[t], sd, o, ta, b, prev, sy);
        for (int i = 0; i < n; ++i) atomicAdd(counts + sy[i], 1u);
    }
}

__global__ void __launch_bounds__(64) k_enc_a(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                              const unsigned char* __restrict__ skip, const Meta* __restrict__ M, int ntens, int nblocks,
                                              SideA sd, Opt o, int seg, const RansSym* __restrict__ enc, unsigned char* __restrict__ out, size_t cap,
                                              unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long b0 = (long long)s * seg;
    if (b0 >= nblocks) return;
    const int b1 = (int)min(b0 + seg, (long long)nblocks);
    const TabA ta(o);
    unsigned char* slot = out + (size_t)s * cap;
    SlotWriter wr; wr.init(slot + cap, slot);
    unsigned x = RANS_L;
    int t = tensor_of(M, ntens, b1 - 1);
    unsigned sy[4];
    for (int b = b1 - 1; b >= (int)b0; --b) {
        while (b < M[t].first) --t;
        if (skip[b] & 1) continue;
        const int inrow = (b - M[t].first) % M[t].nb_row;
        const int prev = (inrow == 0 || b == (int)b0) ? 0 : blocks[(size_t)(b - 1) * 34 + 1];
        const int n = symbols_a(blocks, pos, skip, M[t], sd, o, ta, b, prev, sy);
        for (int i = n - 1; i >= 0; --i) rans_put<12>(x, wr, enc[sy[i]]);
    }
    rans_flush(x, wr);
    out_len[s] = wr.finish(slot + cap);
}

__global__ void __launch_bounds__(64) k_dec_a(const unsigned char* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                              const unsigned long long* __restrict__ in_end, const unsigned char* __restrict__ skip,
                                              const Meta* __restrict__ M, int ntens, int nblocks, SideA sd, Opt o, int seg,
                                              const RansSym* __restrict__ enc, const unsigned char* __restrict__ lut, unsigned char* __restrict__ blocks,
                                              unsigned char* __restrict__ pos, int* __restrict__ status) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long b0 = (long long)s * seg;
    if (b0 >= nblocks) return;
    const int b1 = (int)min(b0 + seg, (long long)nblocks);
    const TabA ta(o);
    ByteReaderUp rd; rd.init(in + in_off[s], in + in_end[s]);
    unsigned x = rans_init(rd);
    auto get = [&](int tab) { return (int)rans_get<12>(x, rd, lut + ((size_t)tab << 12), enc + (size_t)tab * 256); };
    int t = tensor_of(M, ntens, (int)b0), prev = 0;
    for (int b = (int)b0; b < b1 && !rd.over; ++b) {
        while (t + 1 < ntens && b >= M[t + 1].first) ++t;
        if (skip[b] & 1) continue;
        const Meta m = M[t];
        unsigned char* blk = blocks + (size_t)b * 34;
        const int inrow = (b - m.first) % m.nb_row;
        const int cb = m.colbase / 32 + inrow, c0 = m.colbase + inrow * 32, base = m.grp * ta.per_group;
        if (inrow == 0 || b == (int)b0) prev = 0;
        const int hi = get(base + prev + (o.hicf ? 256 * (sd.bcf[cb] & 15) : 0));
        const int lo = get(base + ta.lo + hi);
        blk[0] = (unsigned char)lo; blk[1] = (unsigned char)hi; prev = hi;
        if (!(skip[b] & 4)) {
            int p;
            if (o.rank) p = sd.perm[cb * 32 + (get(base + ta.pos + (sd.spread[cb] & 15)) & 31)];
            else p = get(base + ta.pos);
            p &= 31;
            const int mx = get(base + ta.mx + (o.sign ? (sd.scls[c0 + p] & 15) : 0));
            blk[2 + p] = (unsigned char)mx; pos[b] = (unsigned char)p;
        }
    }
    if (rd.over || x != RANS_L || rd.p != rd.end) atomicOr(status, SG_ST_CORRUPT);
}

// ---- phase B ---------------------------------------------------------------------------------------------------------
struct SideB { const short* cfi; const unsigned char* scls; const int* row_m; };
SG_DEVINL int tables_b(const Opt& o) { return 64 + (o.sign ? 1024 : 0); }
SG_DEVINL int shift_b(const unsigned char* blk, const Meta& m, const SideB& sd, int b) {
    const int rm = sd.row_m[m.rowbase + (b - m.first) / m.nb_row];
    return rm - (blk[0] | (blk[1] << 8)) - m.off;
}

__global__ void __launch_bounds__(64) k_hist_b(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                               const unsigned char* __restrict__ skip, const Meta* __restrict__ M, int ntens, int nblocks,
                                               SideB sd, int qbase, int G, Opt o, int seg, unsigned* __restrict__ counts) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long b0 = (long long)s * seg;
    if (b0 >= nblocks) return;
    const int b1 = (int)min(b0 + seg, (long long)nblocks), tq = tables_b(o);
    int t = tensor_of(M, ntens, (int)b0);
    for (int b = (int)b0; b < b1; ++b) {
        while (t + 1 < ntens && b >= M[t + 1].first) ++t;
        if (skip[b]) continue;
        const unsigned char* blk = blocks + (size_t)b * 34;
        const Meta m = M[t];
        const int c0 = m.colbase + ((b - m.first) % m.nb_row) * 32, sh = shift_b(blk, m, sd, b), p = pos[b];
        const int qb = qbase + (G + t) * tq;                         // one histogram per tensor: the host merges them into table sets
        for (int j = 0; j < 32; ++j) {
            if (j == p) continue;
            const int c = c0 + j, pb = magnitude_bin(sd.cfi[c], sh), v = (signed char)blk[2 + j];
            if (o.sign) {
                const int mag = v < 0 ? -v : v;
                atomicAdd(counts + (size_t)(qb + pb) * 256 + mag, 1u);
                if (mag) atomicAdd(counts + (size_t)(qb + 64 + pb * 16 + (sd.scls[c] & 15)) * 256 + (v < 0), 1u);
            } else atomicAdd(counts + (size_t)(qb + pb) * 256 + (v + 128), 1u);
        }
    }
}

__global__ void __launch_bounds__(64) k_enc_b(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                              const unsigned char* __restrict__ skip, const Meta* __restrict__ M, int ntens, int nblocks,
                                              SideB sd, int qbase, Opt o, int seg, const RansSym* __restrict__ enc, unsigned char* __restrict__ out,
                                              size_t cap, unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long b0 = (long long)s * seg;
    if (b0 >= nblocks) return;
    const int b1 = (int)min(b0 + seg, (long long)nblocks), tq = tables_b(o);
    unsigned char* slot = out + (size_t)s * cap;
    SlotWriter wr; wr.init(slot + cap, slot);
    unsigned x = RANS_L;
    int t = tensor_of(M, ntens, b1 - 1);
    for (int b = b1 - 1; b >= (int)b0; --b) {
        while (b < M[t].first) --t;
        if (skip[b]) continue;
        const unsigned char* blk = blocks + (size_t)b * 34;
        const Meta m = M[t];
        const int c0 = m.colbase + ((b - m.first) % m.nb_row) * 32, sh = shift_b(blk, m, sd, b), p = pos[b];
        const int qb = qbase + m.qset * tq;
        for (int j = 31; j >= 0; --j) {
            if (j == p) continue;
            const int c = c0 + j, pb = magnitude_bin(sd.cfi[c], sh), v = (signed char)blk[2 + j];
            if (o.sign) {
                const int mag = v < 0 ? -v : v;
                if (mag) rans_put<12>(x, wr, enc[(size_t)(qb + 64 + pb * 16 + (sd.scls[c] & 15)) * 256 + (v < 0)]);
                rans_put<12>(x, wr, enc[(size_t)(qb + pb) * 256 + mag]);
            } else rans_put<12>(x, wr, enc[(size_t)(qb + pb) * 256 + (v + 128)]);
        }
    }
    rans_flush(x, wr);
    out_len[s] = wr.finish(slot + cap);
}

__global__ void __launch_bounds__(64) k_dec_b(const unsigned char* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                              const unsigned long long* __restrict__ in_end, const unsigned char* __restrict__ skip,
                                              const Meta* __restrict__ M, int ntens, int nblocks, SideB sd, int qbase, Opt o, int seg,
                                              const RansSym* __restrict__ enc, const unsigned char* __restrict__ lut, unsigned char* __restrict__ blocks,
                                              const unsigned char* __restrict__ pos, int* __restrict__ status) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long b0 = (long long)s * seg;
    if (b0 >= nblocks) return;
    const int b1 = (int)min(b0 + seg, (long long)nblocks), tq = tables_b(o);
    ByteReaderUp rd; rd.init(in + in_off[s], in + in_end[s]);
    unsigned x = rans_init(rd);
    auto get = [&](int tab) { return (int)rans_get<12>(x, rd, lut + ((size_t)tab << 12), enc + (size_t)tab * 256); };
    int t = tensor_of(M, ntens, (int)b0);
    for (int b = (int)b0; b < b1 && !rd.over; ++b) {
        while (t + 1 < ntens && b >= M[t + 1].first) ++t;
        if (skip[b]) continue;
        unsigned char* blk = blocks + (size_t)b * 34;
        const Meta m = M[t];
        const int c0 = m.colbase + ((b - m.first) % m.nb_row) * 32, sh = shift_b(blk, m, sd, b), p = pos[b];
        const int qb = qbase + m.qset * tq;
        for (int j = 0; j < 32; ++j) {
            if (j == p) continue;
            const int c = c0 + j, pb = magnitude_bin(sd.cfi[c], sh);
            int v;
            if (o.sign) {
                const int mag = get(qb + pb);
                const int neg = mag ? get(qb + 64 + pb * 16 + (sd.scls[c] & 15)) : 0;
                v = neg ? -mag : mag;
            } else v = get(qb + pb) - 128;
            blk[2 + j] = (unsigned char)(v & 0xff);
        }
    }
    if (rd.over || x != RANS_L || rd.p != rd.end) atomicOr(status, SG_ST_CORRUPT);
}

// ---- phase C ---------------------------------------------------------------------------------------------------------
// one weight of a predicted row: mean + sum over the row's parents of coefficient * (parent's weight - mean), every
// operation an explicit IEEE one in this order, then divided by the block's scale and rounded (gpu3.py:74-93)
SG_DEVINL signed char predict_one(const unsigned char* __restrict__ blocks, int first, int nbr, int r, int j, const int* __restrict__ par,
                                  const float* __restrict__ coef, int K, const float* __restrict__ mu) {
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) {
        const int p = par[(size_t)r * K + k];
        if (p < 0) continue;
        const unsigned char* pb = blocks + ((size_t)first + (size_t)p * nbr + j / 32) * 34;
        const float w = __fmul_rn((float)(signed char)pb[2 + j % 32], f16_to_f32((uint16_t)(pb[0] | (pb[1] << 8))));
        acc = __fadd_rn(acc, __fmul_rn(coef[(size_t)r * K + k], __fsub_rn(w, mu[j])));
    }
    const float m = __fadd_rn(acc, mu[j]);
    const unsigned char* tb = blocks + ((size_t)first + (size_t)r * nbr + j / 32) * 34;
    const float d = f16_to_f32((uint16_t)(tb[0] | (tb[1] << 8)));
    int v = 0;
    if (d > 0.0f) v = (int)fmaxf(-127.0f, fminf(127.0f, rintf(__fdiv_rn(m, d))));
    return (signed char)v;
}

__global__ void __launch_bounds__(256) k_predict(const unsigned char* __restrict__ blocks, int first, int nbr, int C, const int* __restrict__ rows,
                                                 int nrw, const int* __restrict__ par, const float* __restrict__ coef, int K,
                                                 const float* __restrict__ mu, signed char* __restrict__ pint) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)nrw * C) return;
    const int r = rows[idx / C], j = (int)(idx % C);
    pint[(size_t)r * C + j] = predict_one(blocks, first, nbr, r, j, par, coef, K, mu);
}

// the rows of one wave of every predicted tensor at once (decoder): entry e = row ent_row[e] of slot ent_slot[e]
__global__ void __launch_bounds__(256) k_predict_multi(const unsigned char* __restrict__ blocks, const int* __restrict__ ent_slot,
                                                       const int* __restrict__ ent_row, int nent, int CMAX, const int* __restrict__ s_first,
                                                       const int* __restrict__ s_nbr, const long long* __restrict__ s_rbase,
                                                       const long long* __restrict__ s_pbase, const int* __restrict__ s_mubase,
                                                       const int* __restrict__ par, const float* __restrict__ coef, int K,
                                                       const float* __restrict__ mu, signed char* __restrict__ pint) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)nent * CMAX) return;
    const int e = (int)(idx / CMAX), j = (int)(idx % CMAX), s = ent_slot[e], r = ent_row[e];
    const int nbr = s_nbr[s], C = nbr * 32;
    if (j >= C) return;
    pint[s_pbase[s] + (size_t)r * C + j] = predict_one(blocks, s_first[s], nbr, r, j, par + s_rbase[s] * K, coef + s_rbase[s] * K, K, mu + s_mubase[s]);
}

struct SegC { const int* t; const int* r0; const int* nr; const int* slot; };
struct SideC { const short* cfi; const int* row_m; const signed char* fbin; const long long* rbase; const signed char* pint; const long long* pbase; };
SG_DEVINL int tables_c(const Opt& o) { return 64 + (o.preda ? 24 : 0); }
// rank of position p among the block's |prediction| values (descending, ties by index), and back
SG_DEVINL int rank_of(const signed char* pr, int p) {
    const int ap = abs((int)pr[p]);
    int r = 0;
    for (int k = 0; k < 32; ++k) { const int a = abs((int)pr[k]); r += (a > ap) || (a == ap && k < p); }
    return r;
}
SG_DEVINL int pos_of_rank(const signed char* pr, int rk) {
    for (int j = 0; j < 32; ++j) if (rank_of(pr, j) == rk) return j;
    return 0;
}
SG_DEVINL int rank_ctx(const signed char* pr) {
    int m = 0;
    for (int k = 0; k < 32; ++k) m = max(m, abs((int)pr[k]));
    return min(m / 16, 7);
}
SG_DEVINL int mx_ctx(const signed char* pr, int p) { const int v = pr[p]; return (v < 0) * 8 + min(abs(v) / 16, 7); }

__global__ void __launch_bounds__(64) k_hist_c(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                               const unsigned char* __restrict__ skip, const Meta* __restrict__ M, SegC sg, int nseg, SideC sd, Opt o,
                                               unsigned* __restrict__ counts) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const int t = sg.t[s], slot = sg.slot[s], nbr = M[t].nb_row, C = nbr * 32, tb = slot * tables_c(o);
    const signed char* fb = sd.fbin + sd.rbase[slot];
    const signed char* pi = sd.pint + sd.pbase[slot];
    for (int r = sg.r0[s]; r < sg.r0[s] + sg.nr[s]; ++r)
        for (int kk = 0; kk < nbr; ++kk) {
            const size_t b = (size_t)M[t].first + (size_t)r * nbr + kk;
            if (skip[b] & 1) continue;
            const unsigned char* blk = blocks + b * 34;
            const int sh = sd.row_m[M[t].rowbase + r] - (blk[0] | (blk[1] << 8)) - M[t].off, p = pos[b];
            const signed char* pr = pi + (size_t)r * C + kk * 32;
            if (o.preda) {
                atomicAdd(counts + (size_t)(tb + 64 + rank_ctx(pr)) * 256 + rank_of(pr, p), 1u);
                atomicAdd(counts + (size_t)(tb + 72 + mx_ctx(pr, p)) * 256 + blk[2 + p], 1u);
            }
            for (int j = 0; j < 32; ++j) {
                if (j == p) continue;
                const int ctx = clamp63(magnitude_bin(sd.cfi[M[t].colbase + kk * 32 + j], sh) + fb[r]);
                atomicAdd(counts + (size_t)(tb + ctx) * 256 + (((signed char)blk[2 + j] - pr[j]) & 255), 1u);
            }
        }
}

__global__ void __launch_bounds__(64) k_enc_c(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                              const unsigned char* __restrict__ skip, const Meta* __restrict__ M, SegC sg, int nseg, SideC sd, Opt o,
                                              const RansSym* __restrict__ enc, unsigned char* __restrict__ out, size_t cap, unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const int t = sg.t[s], slot = sg.slot[s], nbr = M[t].nb_row, C = nbr * 32, tb = slot * tables_c(o);
    const signed char* fb = sd.fbin + sd.rbase[slot];
    const signed char* pi = sd.pint + sd.pbase[slot];
    unsigned char* sl = out + (size_t)s * cap;
    SlotWriter wr; wr.init(sl + cap, sl);
    unsigned x = RANS_L;
    for (int r = sg.r0[s] + sg.nr[s] - 1; r >= sg.r0[s]; --r)
        for (int kk = nbr - 1; kk >= 0; --kk) {
            const size_t b = (size_t)M[t].first + (size_t)r * nbr + kk;
            if (skip[b] & 1) continue;
            const unsigned char* blk = blocks + b * 34;
            const int sh = sd.row_m[M[t].rowbase + r] - (blk[0] | (blk[1] << 8)) - M[t].off, p = pos[b];
            const signed char* pr = pi + (size_t)r * C + kk * 32;
            for (int j = 31; j >= 0; --j) {
                if (j == p) continue;
                const int ctx = clamp63(magnitude_bin(sd.cfi[M[t].colbase + kk * 32 + j], sh) + fb[r]);
                rans_put<12>(x, wr, enc[(size_t)(tb + ctx) * 256 + (((signed char)blk[2 + j] - pr[j]) & 255)]);
            }
            if (o.preda) {
                rans_put<12>(x, wr, enc[(size_t)(tb + 72 + mx_ctx(pr, p)) * 256 + blk[2 + p]]);
                rans_put<12>(x, wr, enc[(size_t)(tb + 64 + rank_ctx(pr)) * 256 + rank_of(pr, p)]);
            }
        }
    rans_flush(x, wr);
    out_len[s] = wr.finish(sl + cap);
}

// Phase C decoder: ONE segment per CTA.  A wave of the format has a few hundred segments at most and waves decode one
// after another, so the launch is as long as one segment's chain; what shortens it is taking the loads off the chain:
//   * the slot's tables go to shared memory in the compact form of rans.cuh (256 coarse entries + the symbols' freq | cum
//     words, 1.25 KiB a table), built here by the whole CTA from the encoder entries, so that a symbol costs two or three
//     shared-memory reads instead of two dependent global ones;
//   * the 32 lanes of warp 0 fetch a block's predictions and contexts side by side (and rank the predictions, where the
//     largest code's position is coded by rank) and hand them to lane 0, which runs the chain; all lanes store the codes.
constexpr int DEC_C_THREADS = 128;
static inline size_t dec_c_smem(int ntab) { return (size_t)ntab * RANS_COMPACT + 96; }

__global__ void __launch_bounds__(DEC_C_THREADS) k_dec_c(const unsigned char* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                                         const unsigned long long* __restrict__ in_end, int seg0, unsigned char* __restrict__ pos,
                                                         const unsigned char* __restrict__ skip, const Meta* __restrict__ M, SegC sg, int nseg, SideC sd,
                                                         Opt o, const RansSym* __restrict__ enc, unsigned char* __restrict__ blocks,
                                                         int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char sm[];
    const int s = seg0 + blockIdx.x;
    if (s >= nseg) return;
    const int t = sg.t[s], slot = sg.slot[s], ntab = tables_c(o), tb = slot * ntab;
    unsigned char* ct = sm;
    unsigned char* st_ctx = sm + (size_t)ntab * RANS_COMPACT;       // 32 contexts, 32 predictions, 32 decoded codes
    unsigned char* st_pr = st_ctx + 32;
    unsigned char* st_out = st_ctx + 64;
    for (int i = threadIdx.x; i < ntab * 64; i += blockDim.x)
        reinterpret_cast<unsigned*>(ct + (size_t)(i >> 6) * RANS_COMPACT)[i & 63] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < ntab * 256; i += blockDim.x) {
        const int tt = i >> 8, sy = i & 255;
        const unsigned fc = enc[(size_t)(tb + tt) * 256 + sy].fc, f = fc & 0xffffu, cu = fc >> 16;
        unsigned char* c = ct + (size_t)tt * RANS_COMPACT;
        reinterpret_cast<unsigned*>(c + 256)[sy] = fc;
        if (f) for (unsigned bk = (cu + 15) >> 4; bk < 256 && (bk << 4) < cu + f; ++bk) c[bk] = (unsigned char)sy;   // buckets that begin in the range
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    const unsigned FULL = 0xffffffffu;
    const int lane = threadIdx.x;
    const Meta mt = M[t];
    const int nbr = mt.nb_row, C = nbr * 32;
    const signed char* fb = sd.fbin + sd.rbase[slot];
    const signed char* pi = sd.pint + sd.pbase[slot];
    ByteReaderUp rd;
    unsigned x = RANS_L;
    if (lane == 0) { rd.init(in + in_off[s], in + in_end[s]); x = rans_init(rd); }
    else rd.init(in, in);
    bool stop = false;
    for (int r = sg.r0[s]; r < sg.r0[s] + sg.nr[s] && !stop; ++r) {
        const int fbr = fb[r], rm = sd.row_m[mt.rowbase + r];
        for (int kk = 0; kk < nbr && !stop; ++kk) {
            const size_t b = (size_t)mt.first + (size_t)r * nbr + kk;
            if (skip[b] & 1) continue;
            unsigned char* blk = blocks + b * 34;
            const int sh = rm - (blk[0] | (blk[1] << 8)) - mt.off;
            const int prj = pi[(size_t)r * C + kk * 32 + lane];
            st_ctx[lane] = (unsigned char)clamp63(magnitude_bin(sd.cfi[mt.colbase + kk * 32 + lane], sh) + fbr);
            st_pr[lane] = (unsigned char)prj;
            int p;
            if (o.preda) {
                const int ap = abs(prj);
                int rk = 0, mx = ap;                    // rank of this position among the |predictions|: descending, ties by index
                for (int k = 0; k < 32; ++k) {
                    const int a = __shfl_sync(FULL, ap, k);
                    rk += (a > ap) || (a == ap && k < lane);
                    mx = max(mx, a);
                }
                int sym = 0;
                if (lane == 0) sym = (int)rans_get_compact<12>(x, rd, ct + (size_t)(64 + min(mx / 16, 7)) * RANS_COMPACT);
                sym = __shfl_sync(FULL, sym, 0);
                const unsigned hit = __ballot_sync(FULL, rk == sym);
                p = hit ? __ffs(hit) - 1 : 0;
                const int vp = __shfl_sync(FULL, prj, p);
                int val = 0;
                if (lane == 0) val = (int)rans_get_compact<12>(x, rd, ct + (size_t)(72 + (vp < 0) * 8 + min(abs(vp) / 16, 7)) * RANS_COMPACT);
                val = __shfl_sync(FULL, val, 0);
                if (lane == p) blk[2 + p] = (unsigned char)val;
                if (lane == 0) pos[b] = (unsigned char)p;
            } else p = pos[b];
            __syncwarp();
            if (lane == 0) {
                const uint4 c0 = reinterpret_cast<const uint4*>(st_ctx)[0], c1 = reinterpret_cast<const uint4*>(st_ctx)[1];
                const uint4 p0 = reinterpret_cast<const uint4*>(st_pr)[0], p1 = reinterpret_cast<const uint4*>(st_pr)[1];
                const unsigned cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const unsigned pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                unsigned ow[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (j == p) continue;
                    const unsigned cx = (cw[j >> 2] >> (8 * (j & 3))) & 0xffu;
                    const int pv = (int)(signed char)((pw[j >> 2] >> (8 * (j & 3))) & 0xffu);
                    const unsigned sy = rans_get_compact<12>(x, rd, ct + (size_t)cx * RANS_COMPACT);
                    ow[j >> 2] |= ((unsigned)(pv + (int)sy) & 255u) << (8 * (j & 3));
                }
                reinterpret_cast<uint4*>(st_out)[0] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                reinterpret_cast<uint4*>(st_out)[1] = make_uint4(ow[4], ow[5], ow[6], ow[7]);
            }
            __syncwarp();
            if (lane != p) blk[2 + lane] = st_out[lane];
            stop = __shfl_sync(FULL, (int)rd.over, 0) != 0;
        }
    }
    if (lane == 0 && (rd.over || x != RANS_L || rd.p != rd.end)) atomicOr(status, SG_ST_CORRUPT);
}

static unsigned grid_of(long long n, int per) { return (unsigned)((n + per - 1) / per); }

}  // namespace m21
}  // namespace sg

using namespace sg;
using m21::Meta;
using m21::Opt;

static int common_ab(const void* blocks, const void* pos, const void* skip, const void* meta, int ntens, int nblocks, int seg) {
    if (!blocks || !pos || !skip || !meta || ntens <= 0 || nblocks < 0 || seg <= 0) return SG_ERR_ARG;
    return SG_OK;
}
static Opt opt_of(int flags) { Opt o; o.sign = flags & 1; o.rank = (flags >> 1) & 1; o.hicf = (flags >> 2) & 1; o.preda = (flags >> 3) & 1; return o; }

extern "C" int sg_m21_hist_a(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const unsigned char* skip,
                             const void* meta, int ntens, int nblocks, const unsigned char* bcf, const unsigned char* spread,
                             const unsigned char* perm, const unsigned char* rankof, const unsigned char* scls, int flags, int seg, unsigned* counts) {
    int rc = common_ab(blocks, pos, skip, meta, ntens, nblocks, seg);
    if (rc != SG_OK || !counts) return SG_ERR_ARG;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SideA sd = {bcf, spread, perm, rankof, scls};
    const long long nseg = ((long long)nblocks + seg - 1) / seg;
    m21::k_hist_a<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(blocks, pos, skip, (const Meta*)meta, ntens, nblocks, sd, opt_of(flags), seg, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_encode_a(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const unsigned char* skip,
                               const void* meta, int ntens, int nblocks, const unsigned char* bcf, const unsigned char* spread,
                               const unsigned char* perm, const unsigned char* rankof, const unsigned char* scls, int flags, int seg,
                               const void* enc_tab, unsigned char* slots, size_t cap, unsigned* out_len) {
    int rc = common_ab(blocks, pos, skip, meta, ntens, nblocks, seg);
    if (rc != SG_OK || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 16 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SideA sd = {bcf, spread, perm, rankof, scls};
    const long long nseg = ((long long)nblocks + seg - 1) / seg;
    m21::k_enc_a<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(blocks, pos, skip, (const Meta*)meta, ntens, nblocks, sd, opt_of(flags), seg,
                                                                         (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_decode_a(int device, void* stream, const unsigned char* in, const unsigned long long* in_off, const unsigned long long* in_end,
                               const unsigned char* skip, const void* meta, int ntens, int nblocks, const unsigned char* bcf,
                               const unsigned char* spread, const unsigned char* perm, const unsigned char* rankof, const unsigned char* scls,
                               int flags, int seg, const void* enc_tab, const unsigned char* lut, unsigned char* blocks, unsigned char* pos) {
    int rc = common_ab(blocks, pos, skip, meta, ntens, nblocks, seg);
    if (rc != SG_OK || !in || !in_off || !in_end || !enc_tab || !lut) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SideA sd = {bcf, spread, perm, rankof, scls};
    const long long nseg = ((long long)nblocks + seg - 1) / seg;
    m21::k_dec_a<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(in, in_off, in_end, skip, (const Meta*)meta, ntens, nblocks, sd, opt_of(flags), seg,
                                                                         (const RansSym*)enc_tab, lut, blocks, pos, status_word(device));
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_hist_b(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const unsigned char* skip,
                             const void* meta, int ntens, int nblocks, const short* cfi, const unsigned char* scls, const int* row_m, int qbase,
                             int G, int flags, int seg, unsigned* counts) {
    int rc = common_ab(blocks, pos, skip, meta, ntens, nblocks, seg);
    if (rc != SG_OK || !cfi || !row_m || !counts) return SG_ERR_ARG;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SideB sd = {cfi, scls, row_m};
    const long long nseg = ((long long)nblocks + seg - 1) / seg;
    m21::k_hist_b<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(blocks, pos, skip, (const Meta*)meta, ntens, nblocks, sd, qbase, G, opt_of(flags), seg, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_encode_b(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const unsigned char* skip,
                               const void* meta, int ntens, int nblocks, const short* cfi, const unsigned char* scls, const int* row_m, int qbase,
                               int flags, int seg, const void* enc_tab, unsigned char* slots, size_t cap, unsigned* out_len) {
    int rc = common_ab(blocks, pos, skip, meta, ntens, nblocks, seg);
    if (rc != SG_OK || !cfi || !row_m || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 16 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SideB sd = {cfi, scls, row_m};
    const long long nseg = ((long long)nblocks + seg - 1) / seg;
    m21::k_enc_b<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(blocks, pos, skip, (const Meta*)meta, ntens, nblocks, sd, qbase, opt_of(flags), seg,
                                                                         (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_decode_b(int device, void* stream, const unsigned char* in, const unsigned long long* in_off, const unsigned long long* in_end,
                               const unsigned char* skip, const void* meta, int ntens, int nblocks, const short* cfi, const unsigned char* scls,
                               const int* row_m, int qbase, int flags, int seg, const void* enc_tab, const unsigned char* lut, unsigned char* blocks,
                               const unsigned char* pos) {
    int rc = common_ab(blocks, pos, skip, meta, ntens, nblocks, seg);
    if (rc != SG_OK || !in || !in_off || !in_end || !cfi || !row_m || !enc_tab || !lut) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SideB sd = {cfi, scls, row_m};
    const long long nseg = ((long long)nblocks + seg - 1) / seg;
    m21::k_dec_b<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(in, in_off, in_end, skip, (const Meta*)meta, ntens, nblocks, sd, qbase, opt_of(flags), seg,
                                                                         (const RansSym*)enc_tab, lut, blocks, pos, status_word(device));
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_predict(int device, void* stream, const unsigned char* blocks, int first, int nbr, int C, const int* rows, int nrw,
                              const int* par, const float* coef, int K, const float* mu, signed char* pint) {
    if (!blocks || !rows || !par || !coef || !mu || !pint || nbr <= 0 || C != nbr * 32 || nrw < 0 || K < 0) return SG_ERR_ARG;
    if (nrw == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    m21::k_predict<<<m21::grid_of((long long)nrw * C, 256), 256, 0, (cudaStream_t)stream>>>(blocks, first, nbr, C, rows, nrw, par, coef, K, mu, pint);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_predict_multi(int device, void* stream, const unsigned char* blocks, const int* ent_slot, const int* ent_row, int nent, int CMAX,
                                    const int* s_first, const int* s_nbr, const long long* s_rbase, const long long* s_pbase, const int* s_mubase,
                                    const int* par, const float* coef, int K, const float* mu, signed char* pint) {
    if (!blocks || !ent_slot || !ent_row || !s_first || !s_nbr || !s_rbase || !s_pbase || !s_mubase || !par || !coef || !mu || !pint ||
        nent < 0 || CMAX <= 0 || K < 0) return SG_ERR_ARG;
    if (nent == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    m21::k_predict_multi<<<m21::grid_of((long long)nent * CMAX, 256), 256, 0, (cudaStream_t)stream>>>(blocks, ent_slot, ent_row, nent, CMAX, s_first, s_nbr,
                                                                                                     s_rbase, s_pbase, s_mubase, par, coef, K, mu, pint);
    return cuda_ok(cudaGetLastError());
}

static int common_c(const void* blocks, const void* pos, const void* skip, const void* meta, const int* seg_t, const int* seg_r0, const int* seg_nr,
                    const int* seg_slot, int nseg, const short* cfi, const int* row_m, const signed char* fbin, const long long* rbase,
                    const signed char* pint, const long long* pbase) {
    if (!blocks || !pos || !skip || !meta || !seg_t || !seg_r0 || !seg_nr || !seg_slot || nseg < 0 || !cfi || !row_m || !fbin || !rbase || !pint || !pbase)
        return SG_ERR_ARG;
    return SG_OK;
}

extern "C" int sg_m21_hist_c(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const unsigned char* skip, const void* meta,
                             const int* seg_t, const int* seg_r0, const int* seg_nr, const int* seg_slot, int nseg, const short* cfi, const int* row_m,
                             const signed char* fbin, const long long* rbase, const signed char* pint, const long long* pbase, int flags, unsigned* counts) {
    int rc = common_c(blocks, pos, skip, meta, seg_t, seg_r0, seg_nr, seg_slot, nseg, cfi, row_m, fbin, rbase, pint, pbase);
    if (rc != SG_OK || !counts) return SG_ERR_ARG;
    if (nseg == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SegC sg = {seg_t, seg_r0, seg_nr, seg_slot};
    const m21::SideC sd = {cfi, row_m, fbin, rbase, pint, pbase};
    m21::k_hist_c<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(blocks, pos, skip, (const Meta*)meta, sg, nseg, sd, opt_of(flags), counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_encode_c(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const unsigned char* skip, const void* meta,
                               const int* seg_t, const int* seg_r0, const int* seg_nr, const int* seg_slot, int nseg, const short* cfi, const int* row_m,
                               const signed char* fbin, const long long* rbase, const signed char* pint, const long long* pbase, int flags,
                               const void* enc_tab, unsigned char* slots, size_t cap, unsigned* out_len) {
    int rc = common_c(blocks, pos, skip, meta, seg_t, seg_r0, seg_nr, seg_slot, nseg, cfi, row_m, fbin, rbase, pint, pbase);
    if (rc != SG_OK || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 16 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SegC sg = {seg_t, seg_r0, seg_nr, seg_slot};
    const m21::SideC sd = {cfi, row_m, fbin, rbase, pint, pbase};
    m21::k_enc_c<<<m21::grid_of(nseg, 64), 64, 0, (cudaStream_t)stream>>>(blocks, pos, skip, (const Meta*)meta, sg, nseg, sd, opt_of(flags),
                                                                         (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m21_decode_c(int device, void* stream, const unsigned char* in, const unsigned long long* in_off, const unsigned long long* in_end,
                               int seg0, unsigned char* pos, const unsigned char* skip, const void* meta, const int* seg_t, const int* seg_r0,
                               const int* seg_nr, const int* seg_slot, int nseg, const short* cfi, const int* row_m, const signed char* fbin,
                               const long long* rbase, const signed char* pint, const long long* pbase, int flags, const void* enc_tab,
                               const unsigned char* lut, unsigned char* blocks) {
    int rc = common_c(blocks, pos, skip, meta, seg_t, seg_r0, seg_nr, seg_slot, nseg, cfi, row_m, fbin, rbase, pint, pbase);
    (void)lut;                                   // the kernel builds its own compact tables from the encoder entries
    if (rc != SG_OK || !in || !in_off || !in_end || !enc_tab || seg0 < 0) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nseg <= seg0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const m21::SegC sg = {seg_t, seg_r0, seg_nr, seg_slot};
    const m21::SideC sd = {cfi, row_m, fbin, rbase, pint, pbase};
    const size_t smem = m21::dec_c_smem(64 + ((flags & 8) ? 24 : 0));
    if ((rc = cuda_ok(cudaFuncSetAttribute(m21::k_dec_c, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem))) != SG_OK) return rc;
    m21::k_dec_c<<<(unsigned)(nseg - seg0), m21::DEC_C_THREADS, smem, (cudaStream_t)stream>>>(in, in_off, in_end, seg0, pos, skip, (const Meta*)meta, sg,
                                                                                             nseg, sd, opt_of(flags), (const RansSym*)enc_tab, blocks,
                                                                                             status_word(device));
    return cuda_ok(cudaGetLastError());
}
