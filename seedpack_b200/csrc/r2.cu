// R2: the BF16 base-model codec (context-modelled rANS over exponent, mantissa and sign of every weight) and the
// order-fixed float64 statistics that define its contexts.
//
// Replaces v2_hist / v2_enc / v2_dec / row_hash (seedpack/bf16v2.py:63-155) and the statistics pass `_stats`
// (seedpack/bf16v2.py:225-244) with its detmath kernels (seedpack/detmath.py:67-106).  Format: 15 probability bits,
// segments of 16384 weights, three symbols per weight in decode order exponent, mantissa, sign; contexts
//   exponent: clamp(rfi[row] + cfi[col] + 256, 0, 511)          (predicted log2 sigma in 1/8 octave)
//   mantissa: 512 + clamp(8 * exponent - pred - 952, 0, 127)
//   sign:     640 + scl[col]                                       (column bias class)
// plus the tensor's role offset (656 tables per role).
#include "api_util.h"
#include "detmath.cuh"
#include "rans.cuh"

namespace sg {
namespace r2 {

constexpr int PB = 15;
constexpr int TPB = 64;

struct TB { long long doff; int rowlen, rowbase, colbase, tab, rmap, pad; };       // bf16v2.py:158
struct SG { int t, n; long long i0; };                                             // bf16v2.py:159

SG_DEVINL int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

struct Ctx {
    const short* rfi; const short* cfi; const signed char* scl; const int* rowmap;
};

// position of a lane inside its tensor: compact row rc (after duplicate-row removal), column j, original row
struct Cursor {
    TB T; int rc, j, orow; const unsigned short* w;
    SG_DEVINL void seek(const unsigned char* dev, const TB& t, long long i, const int* rowmap) {
        T = t; rc = (int)(i / T.rowlen); j = (int)(i % T.rowlen);
        orow = T.rmap >= 0 ? rowmap[T.rmap + rc] : rc;
        w = reinterpret_cast<const unsigned short*>(dev + T.doff) + (size_t)orow * T.rowlen;
    }
    SG_DEVINL void row(const unsigned char* dev, const int* rowmap) {
        orow = T.rmap >= 0 ? rowmap[T.rmap + rc] : rc;
        w = reinterpret_cast<const unsigned short*>(dev + T.doff) + (size_t)orow * T.rowlen;
    }
};

SG_DEVINL void contexts(const Ctx& c, const TB& T, int orow, int j, int& pred, int& pe, int& sc) {
    pred = c.rfi[T.rowbase + orow] + c.cfi[T.colbase + j];
    pe = clampi(pred + 256, 0, 511);
    sc = clampi(c.scl[T.colbase + j], 0, 15);         // (0..15 by construction, bf16v2.py:243; a damaged side part must not index past the tables)
}
SG_DEVINL int mctx(int ex, int pred) { return clampi(8 * ex - pred - 1016 + 64, 0, 127); }

// warp-aggregated histogram add: lanes hitting the same counter make one atomic
SG_DEVINL void hadd(unsigned* counts, unsigned key) {
    const unsigned m = __match_any_sync(__activemask(), key);
    if ((threadIdx.x & 31) == (unsigned)(__ffs(m) - 1)) atomicAdd(counts + key, (unsigned)__popc(m));
}

// counts do not depend on the order of the weights: a warp per segment, lanes on consecutive weights (coalesced reads).
// Exponent and sign symbols repeat inside a warp and are added once per distinct value; mantissa symbols are spread
// over 128 x 128 counters per role, which a CTA collects in shared memory (64 KB) and adds to global memory at its end;
// so are the exponent symbols inside a window of 128 contexts x 64 exponents around the CTA's first weight (weights
// of one tensor keep to a few octaves; what falls outside the window goes to global memory directly).
constexpr int R2H_WARPS = 8, R2H_SEGS = 8;         // segments per warp
__global__ void __launch_bounds__(R2H_WARPS * 32) k_r2_hist(const unsigned char* __restrict__ dev, const TB* __restrict__ tb,
                                                            const SG* __restrict__ sg, int nseg, Ctx c, unsigned* __restrict__ counts) {
    extern __shared__ unsigned mhist[];            // [128 contexts][128 symbols] of the role of the CTA's first segment
    unsigned* ehist = mhist + 128 * 128;           // [128 contexts from pe0][64 exponents from ex0] of the same role
    __shared__ int win[2];
    for (int i = threadIdx.x; i < 128 * 128 + 128 * 64; i += blockDim.x) mhist[i] = 0;
    const int lane = threadIdx.x & 31;
    const int first = blockIdx.x * (R2H_WARPS * R2H_SEGS);
    const int cta_tab = first < nseg ? tb[sg[first].t].tab : -1;
    if (threadIdx.x == 0 && first < nseg) {
        const SG g = sg[first];
        const TB T = tb[g.t];
        const int rc = (int)(g.i0 / T.rowlen), j = (int)(g.i0 % T.rowlen);
        const int orow = T.rmap >= 0 ? c.rowmap[T.rmap + rc] : rc;
        const unsigned u = reinterpret_cast<const unsigned short*>(dev + T.doff)[(size_t)orow * T.rowlen + j];
        int pred, pe, sc; contexts(c, T, orow, j, pred, pe, sc);
        win[0] = pe - 64; win[1] = (int)((u >> 7) & 255) - 40;      // weights mostly lie below the typical magnitude
    }
    __syncthreads();
    const int pe0 = win[0], ex0 = win[1];
    for (int q = 0; q < R2H_SEGS; ++q) {
        const int s = first + (threadIdx.x >> 5) * R2H_SEGS + q;
        if (s >= nseg) break;
        const SG g = sg[s];
        const TB T = tb[g.t];
        const bool local = T.tab == cta_tab;
        // this lane's weight: compact row rc, column j; 32 weights further every turn (no division inside the loop)
        int rc = (int)((g.i0 + lane) / T.rowlen), j = (int)((g.i0 + lane) % T.rowlen), orow = -1, have_rc = -1;
        const unsigned short* base = reinterpret_cast<const unsigned short*>(dev + T.doff);
        for (int k0 = 0; k0 < g.n; k0 += 32) {
            const int k = k0 + lane;
            const bool live = k < g.n;
            unsigned e0 = 0xffffffffu, e2 = 0xffffffffu;
            if (live) {
                if (rc != have_rc) { orow = T.rmap >= 0 ? c.rowmap[T.rmap + rc] : rc; have_rc = rc; }
                const unsigned u = base[(size_t)orow * T.rowlen + j];
                const int ex = (u >> 7) & 255, man = u & 127, sgn = u >> 15;
                int pred, pe, sc; contexts(c, T, orow, j, pred, pe, sc);
                if (local && (unsigned)(pe - pe0) < 128u && (unsigned)(ex - ex0) < 64u) atomicAdd(ehist + (pe - pe0) * 64 + (ex - ex0), 1u);
                else e0 = (unsigned)(T.tab + pe) * 256 + ex;
                e2 = (unsigned)(T.tab + 640 + sc) * 256 + sgn;
                const int mc = mctx(ex, pred);
                if (local) atomicAdd(mhist + mc * 128 + man, 1u);
                else atomicAdd(counts + (size_t)(T.tab + 512 + mc) * 256 + man, 1u);
                j += 32;
                while (j >= T.rowlen) { j -= T.rowlen; ++rc; }
            }
            if (__any_sync(0xffffffffu, e0 != 0xffffffffu)) {
                const unsigned m0 = __match_any_sync(0xffffffffu, e0);
                if (e0 != 0xffffffffu && lane == __ffs(m0) - 1) atomicAdd(counts + e0, (unsigned)__popc(m0));
            }
            const unsigned m2 = __match_any_sync(0xffffffffu, e2);
            if (live && lane == __ffs(m2) - 1) atomicAdd(counts + e2, (unsigned)__popc(m2));
        }
    }
    __syncthreads();
    if (cta_tab >= 0)
        for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) {
            const unsigned v = mhist[i];
            if (v) atomicAdd(counts + (size_t)(cta_tab + 512 + (i >> 7)) * 256 + (i & 127), v);
        }
    if (cta_tab >= 0)
        for (int i = threadIdx.x; i < 128 * 64; i += blockDim.x) {
            const unsigned v = ehist[i];
            const int pe = pe0 + (i >> 6), ex = ex0 + (i & 63);
            if (v) atomicAdd(counts + (size_t)(cta_tab + pe) * 256 + ex, v);
        }
}

// Encoder: a few lanes per segment, like the decoder below.  The table entries of a weight's three symbols depend on the
// data only, not on the coder state: for every 32 weights (taken from the segment's end backwards) the lanes look
// them up side by side into shared memory, and lane 0 runs the chain over the 96 staged entries.  Four lanes per segment:
// the chain is what a warp spends its issue slots on, and a warp instruction of the chain then serves eight segments.
constexpr int EG = 4, EB = 32, ESEG = 32, EW = EB / EG;          // lanes per segment, weights per batch, segments per CTA, weights per lane
__global__ void __launch_bounds__(EG * ESEG) k_r2_enc(const unsigned char* __restrict__ dev, const TB* __restrict__ tb, const SG* __restrict__ sg,
                                                      int nseg, Ctx c, const RansSym* __restrict__ enc, unsigned char* __restrict__ out, size_t cap,
                                                      unsigned* __restrict__ out_len) {
    // per weight of the batch: sign, mantissa, exponent entries (coding order); a row is padded by one entry so that the
    // chain lanes of a warp's segments, which read the same weight of their rows together, hit different banks
    __shared__ RansSym s_e[ESEG][EB * 3 + 1];
    const int grp = threadIdx.x / EG, gl = threadIdx.x % EG;
    const int s = blockIdx.x * ESEG + grp;
    const bool live = s < nseg;
    SG g; g.t = 0; g.n = 0; g.i0 = 0;
    if (live) g = sg[s];
    const TB T = tb[g.t];
    int nmax = g.n;
    for (int o = 16; o; o >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, o));
    unsigned char* slot = out + (size_t)(live ? s : 0) * cap;
    ByteWriterDown wr; wr.init(slot + cap);
    unsigned x = RANS_L;
    bool full = false;
    const unsigned short* base = reinterpret_cast<const unsigned short*>(dev + T.doff);
    // batches of 32 weights, the last one first; this lane's first weight of the batch: compact row rc, column j
    const int nb_max = (nmax + EB - 1) / EB;
    int rc = 0, j = 0;
    {
        const long long i = g.i0 + (long long)(nb_max - 1) * EB + EW * gl;
        if (live) { rc = (int)(i / T.rowlen); j = (int)(i % T.rowlen); }
    }
    for (int b = nb_max - 1; b >= 0; --b) {
        const int k0 = b * EB;
        {
            int r = rc, col = j, have = -1, orow = 0;
#pragma unroll
            for (int v = 0; v < EW; ++v) {
                const int k = k0 + EW * gl + v;
                if (live && k < g.n) {
                    if (r != have) { orow = T.rmap >= 0 ? c.rowmap[T.rmap + r] : r; have = r; }
                    const unsigned u = base[(size_t)orow * T.rowlen + col];
                    const int ex = (u >> 7) & 255, man = u & 127, sgn = u >> 15;
                    int pred, pe, sc; contexts(c, T, orow, col, pred, pe, sc);
                    s_e[grp][3 * (EW * gl + v)] = enc[(size_t)(T.tab + 640 + sc) * 256 + sgn];
                    s_e[grp][3 * (EW * gl + v) + 1] = enc[(size_t)(T.tab + 512 + mctx(ex, pred)) * 256 + man];
                    s_e[grp][3 * (EW * gl + v) + 2] = enc[(size_t)(T.tab + pe) * 256 + ex];
                    if (++col == T.rowlen) { col = 0; ++r; }
                }
            }
        }
        __syncwarp();
        if (live && gl == 0 && !full && k0 < g.n) {
            const int n = min(EB, g.n - k0);
            for (int w = n - 1; w >= 0; --w) {
                rans_put<PB>(x, wr, s_e[grp][3 * w]);
                rans_put<PB>(x, wr, s_e[grp][3 * w + 1]);
                rans_put<PB>(x, wr, s_e[grp][3 * w + 2]);
                if ((w & 3) == 0 && wr.ptr() < slot + 64) { full = true; break; }
            }
        }
        __syncwarp();
        j -= EB;
        if (live) while (j < 0) { j += T.rowlen; --rc; }
    }
    if (live && gl == 0) {
        if (full) out_len[s] = LEN_OVERFLOW;
        else {
            rans_flush(x, wr);
            wr.flush(slot);
            out_len[s] = wr.bad ? LEN_NOFREQ : (unsigned)(slot + cap - wr.ptr());
        }
    }
}

// Decoder: a segment is one rANS chain by format, but what a weight's symbols are decoded WITH - the exponent's and the
// sign's tables, the prediction the mantissa's table is picked by - depends on its row and column only.  Four lanes
// share a segment: for every 32 weights they look the contexts up side by side (eight weights each) into shared memory,
// lane 0 then runs the chain over the staged contexts - three table walks per weight and nothing else - and all four
// store the 32 decoded weights.  Eight segments per warp decode in lockstep.
constexpr int DG = 4, DB = 32, DSEG = 32, DW = DB / DG;          // lanes per segment, weights per batch, segments per CTA, weights per lane
__global__ void __launch_bounds__(DG * DSEG) k_r2_dec(const unsigned char* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                                      const unsigned long long* __restrict__ in_end, unsigned char* __restrict__ dev,
                                                      const TB* __restrict__ tb, const SG* __restrict__ sg, int nseg, Ctx c,
                                                      const RansSym* __restrict__ enc, const unsigned char* __restrict__ lut, int* __restrict__ status) {
    // rows padded: the chain lanes of a warp's segments touch the same weight of their rows together
    __shared__ int s_t0[DSEG][DB + 1], s_pred[DSEG][DB + 1], s_t2[DSEG][DB + 1];
    __shared__ unsigned short s_out[DSEG][DB + 2];
    const int grp = threadIdx.x / DG, gl = threadIdx.x % DG;
    const int s = blockIdx.x * DSEG + grp;
    const bool live = s < nseg;
    SG g; g.t = 0; g.n = 0; g.i0 = 0;
    if (live) g = sg[s];
    const TB T = tb[g.t];
    int nmax = g.n;
    for (int o = 16; o; o >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, o));
    ByteReaderUp rd; rd.over = false; rd.p = rd.end = nullptr;
    unsigned x = RANS_L;
    if (live && gl == 0) { rd.init(in + in_off[s], in + in_end[s]); x = rans_init(rd); }
    unsigned short* base = reinterpret_cast<unsigned short*>(dev + T.doff);
    // this lane's first weight of the batch: compact row rc, column j; 32 weights further every batch
    int rc = 0, j = 0;
    if (live) { const long long i = g.i0 + DW * gl; rc = (int)(i / T.rowlen); j = (int)(i % T.rowlen); }
    bool bad = false;
    for (int k0 = 0; k0 < nmax; k0 += DB) {
        size_t at[DW];
        {
            int r = rc, col = j, have = -1, orow = 0;
#pragma unroll
            for (int v = 0; v < DW; ++v) {
                const int k = k0 + DW * gl + v;
                at[v] = 0;
                if (live && k < g.n) {
                    if (r != have) { orow = T.rmap >= 0 ? c.rowmap[T.rmap + r] : r; have = r; }
                    int pred, pe, sc; contexts(c, T, orow, col, pred, pe, sc);
                    s_t0[grp][DW * gl + v] = T.tab + pe; s_pred[grp][DW * gl + v] = pred; s_t2[grp][DW * gl + v] = T.tab + 640 + sc;
                    at[v] = (size_t)orow * T.rowlen + col;
                    if (++col == T.rowlen) { col = 0; ++r; }
                }
            }
        }
        __syncwarp();
        if (live && gl == 0 && !bad) {
            const int n = min(DB, g.n - k0);
#pragma unroll 2
            for (int w = 0; w < n; ++w) {
                const int t0 = s_t0[grp][w], pred = s_pred[grp][w], t2 = s_t2[grp][w];
                const int ex = (int)rans_get_compact<PB>(x, rd, lut + (size_t)t0 * RANS_COMPACT);
                const int t1 = T.tab + 512 + mctx(ex, pred);
                const int man = (int)rans_get_compact<PB>(x, rd, lut + (size_t)t1 * RANS_COMPACT);
                const int sgn = (int)rans_get_bit<PB>(x, rd, lut + (size_t)t2 * RANS_COMPACT);
                s_out[grp][w] = (unsigned short)((sgn << 15) | (ex << 7) | man);
            }
            bad = rd.over;
        }
        __syncwarp();
#pragma unroll
        for (int v = 0; v < DW; ++v) {
            const int k = k0 + DW * gl + v;
            if (live && k < g.n) base[at[v]] = s_out[grp][DW * gl + v];
        }
        j += DB;
        if (live) while (j >= T.rowlen) { j -= T.rowlen; ++rc; }
    }
    if (live && gl == 0 && (bad || rd.over || x != RANS_L || rd.p != rd.end)) atomicOr(status, SG_ST_CORRUPT);
}

// 64-bit row fingerprints for duplicate-row detection (bf16v2.py:148-155): an order-dependent integer recurrence, one
// lane per row
__global__ void __launch_bounds__(128) k_row_hash(const unsigned short* __restrict__ w, int nrows, int rowlen, unsigned long long* __restrict__ h) {
    // the recurrence runs along a row, one lane per row; the rows' data comes in through shared memory in tiles of
    // 128 rows x 64 weights loaded with the lanes along the row (coalesced), read back with a 33-word row pitch
    __shared__ unsigned tile[128][33];
    const int r0 = blockIdx.x * 128, r = r0 + threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long a = 1469598103934665603ull;
    if ((rowlen & 63) || (reinterpret_cast<uintptr_t>(w) & 3)) {           // odd shapes: straight from global memory
        if (r < nrows) {
            const unsigned short* p = w + (size_t)r * rowlen;
            for (int j = 0; j < rowlen; ++j) { a ^= p[j]; a *= 1099511628211ull; a ^= a >> 29; }
            h[r] = a;
        }
        return;
    }
    for (int c0 = 0; c0 < rowlen; c0 += 64) {
        __syncthreads();
        for (int rr = warp; rr < 128; rr += 4)
            tile[rr][lane] = r0 + rr < nrows ? reinterpret_cast<const unsigned*>(w + (size_t)(r0 + rr) * rowlen + c0)[lane] : 0u;
        __syncthreads();
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
            const unsigned v = tile[threadIdx.x][i];
            a ^= v & 0xffffu; a *= 1099511628211ull; a ^= a >> 29;
            a ^= v >> 16;     a *= 1099511628211ull; a ^= a >> 29;
        }
    }
    if (r < nrows) h[r] = a;
}

// duplicate rows copied from their source rows after decoding (bf16v2.py:475-480): pairs = (dup row, source row)
__global__ void __launch_bounds__(256) k_copy_rows(unsigned short* __restrict__ w, int rowlen, const long long* __restrict__ pairs, int npairs) {
    const int p = blockIdx.x;
    if (p >= npairs) return;
    unsigned short* d = w + (size_t)pairs[2 * p] * rowlen;
    const unsigned short* s = w + (size_t)pairs[2 * p + 1] * rowlen;
    for (int j = threadIdx.x; j < rowlen; j += blockDim.x) d[j] = s[j];
}

// ---- statistics ----------------------------------------------------------------------------------------------------
// rfi[r] = rint(8 log2 rms(row r)), and rfa[r] = (float) 2^(log2 rms) used to normalise the row in the column pass.
// One warp per row; the float64 sum of squares runs in column order (lane 0 extends the chain over staged squares).
__global__ void __launch_bounds__(128) k_r2_rowstat(const unsigned short* __restrict__ w, int nrows, int rowlen, short* __restrict__ rfi,
                                                    float* __restrict__ rfa) {
    __shared__ double sq[4][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + warp;
    if (r >= nrows) return;
    const unsigned short* p = w + (size_t)r * rowlen;
    double s = 0.0;
    for (int c0 = 0; c0 < rowlen; c0 += 256) {
        const int n = min(256, rowlen - c0);
        for (int i = lane; i < n; i += 32) { const double v = (double)__uint_as_float((unsigned)p[c0 + i] << 16); sq[warp][i] = v * v; }
        __syncwarp();
        if (lane == 0) for (int i = 0; i < n; ++i) s = s + sq[warp][i];
        __syncwarp();
    }
    if (lane == 0) {
        const double rf = dm::log2v(sqrt(s / (double)rowlen) + 1e-30);
        rfa[r] = (float)dm::exp2v(rf);
        rfi[r] = (short)fmin(fmax(rint(rf * 8.0), -32768.0), 32767.0);
    }
}
// per (row chunk, column): float64 sums of v^2 and v over the chunk's rows in row order, v = weight / rfa[row] in float32.
// The sums are one dependent chain per column by format; what does not depend on the chain (load, the IEEE division,
// the conversion) is done by all 256 threads of a CTA for a tile of 64 rows x 32 columns into shared memory, and the
// first warp then extends its 32 columns' chains over the tile while the other warps fetch the next one.
__global__ void __launch_bounds__(256) k_r2_colpart(const unsigned short* __restrict__ w, int nrows, int rowlen, int step,
                                                    const float* __restrict__ rfa, double* __restrict__ part) {
    constexpr int TR = 64, TC = 32;
    __shared__ float tile[2][TR][TC + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * TC + lane;
    const int q = blockIdx.y;
    const int r0 = q * step, r1 = min(nrows, r0 + step);
    const bool live = c < rowlen;
    double s2 = 0.0, s1 = 0.0;
    int buf = 0;
    for (int t0 = r0; t0 < r1; t0 += TR, buf ^= 1) {
#pragma unroll
        for (int j = 0; j < TR / 8; ++j) {
            const int r = t0 + warp + 8 * j;
            float f = 0.0f;
            if (live && r < r1) f = __fdiv_rn(__uint_as_float((unsigned)w[(size_t)r * rowlen + c] << 16), rfa[r]);
            tile[buf][warp + 8 * j][lane] = f;
        }
        __syncthreads();
        if (warp == 0) {
            const int n = min(TR, r1 - t0);
            for (int i = 0; i < n; ++i) {
                const double v = (double)tile[buf][i][lane];
                s2 = s2 + v * v;
                s1 = s1 + v;
            }
        }
    }
    if (warp == 0 && live) {
        part[((size_t)q * rowlen + c) * 2] = s2;
        part[((size_t)q * rowlen + c) * 2 + 1] = s1;
    }
}
__global__ void __launch_bounds__(256) k_r2_colfinal(const double* __restrict__ part, int nchunks, int nrows, int rowlen,
                                                     short* __restrict__ cfi, signed char* __restrict__ scl) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= rowlen) return;
    double s2 = 0.0, s1 = 0.0;
    for (int q = 0; q < nchunks; ++q) { s2 = s2 + part[((size_t)q * rowlen + c) * 2]; s1 = s1 + part[((size_t)q * rowlen + c) * 2 + 1]; }
    const double cf = dm::log2v(sqrt(s2 / (double)nrows) + 1e-30);
    const double ci = fmin(fmax(rint(cf * 8.0), -32768.0), 32767.0);
    cfi[c] = (short)ci;
    const double bias = (s1 / (double)nrows) / dm::exp2v((double)(short)ci / 8.0);
    scl[c] = (signed char)fmin(fmax(floor(bias * 16.0) + 8.0, 0.0), 15.0);
}

// ---- generic detmath entry points (seedpack/detmath.py:67-106) --------------------------------------------------------
__global__ void k_dm_log2(const double* x, long long n, double* y) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = dm::log2v(x[i]);
}
__global__ void k_dm_exp2(const double* x, long long n, double* y) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = dm::exp2v(x[i]);
}
__global__ void k_dm_rows(const float* x, long long nr, long long nc, int sq, double* out) {
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nr) return;
    const float* p = x + r * nc;
    double s = 0.0;
    if (sq) for (long long j = 0; j < nc; ++j) { const double v = p[j]; s = s + v * v; }
    else for (long long j = 0; j < nc; ++j) s = s + (double)p[j];
    out[r] = s;
}
__global__ void k_dm_cols(const float* x, long long nr, long long nc, int sq, const unsigned char* mask, double* out) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nc) return;
    double s = 0.0;
    for (long long r = 0; r < nr; ++r) {
        if (mask && !mask[r]) continue;
        const double v = x[r * nc + c];
        s = s + (sq ? v * v : v);
    }
    out[c] = s;
}

}  // namespace r2
}  // namespace sg

using namespace sg;
using namespace sg::r2;

static int r2_common(const void* dev, const void* tb, const void* sgp, int nseg, const void* rfi, const void* cfi, const void* scl) {
    if (!dev || !tb || !sgp || !rfi || !cfi || !scl || nseg < 0) return SG_ERR_ARG;
    return SG_OK;
}

extern "C" int sg_r2_hist(int device, void* stream, const unsigned char* dev, const void* tb, const void* sgp, int nseg, const short* rfi,
                          const short* cfi, const signed char* scl, const int* rowmap, unsigned* counts) {
    int rc = r2_common(dev, tb, sgp, nseg, rfi, cfi, scl);
    if (rc != SG_OK || !counts) return rc != SG_OK ? rc : SG_ERR_ARG;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    Ctx c = {rfi, cfi, scl, rowmap};
    {
        rc = cuda_ok(cudaFuncSetAttribute(k_r2_hist, cudaFuncAttributeMaxDynamicSharedMemorySize, (128 * 128 + 128 * 64) * 4));
        if (rc != SG_OK) return rc;
        const int per_cta = R2H_WARPS * R2H_SEGS;
        k_r2_hist<<<(nseg + per_cta - 1) / per_cta, R2H_WARPS * 32, (128 * 128 + 128 * 64) * 4, (cudaStream_t)stream>>>(dev, (const TB*)tb, (const SG*)sgp,
                                                                                                           nseg, c, counts);
    }
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_r2_encode(int device, void* stream, const unsigned char* dev, const void* tb, const void* sgp, int nseg, const short* rfi,
                            const short* cfi, const signed char* scl, const int* rowmap, const void* enc_tab, unsigned char* slots,
                            size_t cap, unsigned* out_len) {
    int rc = r2_common(dev, tb, sgp, nseg, rfi, cfi, scl);
    if (rc != SG_OK) return rc;
    if (!enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 128 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    Ctx c = {rfi, cfi, scl, rowmap};
    k_r2_enc<<<(nseg + ESEG - 1) / ESEG, EG * ESEG, 0, (cudaStream_t)stream>>>(dev, (const TB*)tb, (const SG*)sgp, nseg, c, (const RansSym*)enc_tab,
                                                                       slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_r2_decode(int device, void* stream, const unsigned char* in, const unsigned long long* in_off,
                            const unsigned long long* in_end, unsigned char* dev, const void* tb, const void* sgp, int nseg, const short* rfi,
                            const short* cfi, const signed char* scl, const int* rowmap, const void* enc_tab, const unsigned char* lut) {
    int rc = r2_common(dev, tb, sgp, nseg, rfi, cfi, scl);
    if (rc != SG_OK) return rc;
    if (!in || !in_off || !in_end || !enc_tab || !lut) return SG_ERR_ARG;
    if ((uintptr_t)in % 16 || (uintptr_t)lut % 8) return SG_ERR_ALIGN;           // (the sign tables' two words are one 8-byte load)
    if (nseg == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    Ctx c = {rfi, cfi, scl, rowmap};
    k_r2_dec<<<(nseg + DSEG - 1) / DSEG, DG * DSEG, 0, (cudaStream_t)stream>>>(in, in_off, in_end, dev, (const TB*)tb, (const SG*)sgp, nseg, c,
                                                                       (const RansSym*)enc_tab, lut, status_word(device));
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_row_hash(int device, void* stream, const void* w, int nrows, int rowlen, unsigned long long* h) {
    if (!w || !h || nrows < 0 || rowlen <= 0) return SG_ERR_ARG;
    if (nrows == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_row_hash<<<(nrows + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const unsigned short*)w, nrows, rowlen, h);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_copy_rows(int device, void* stream, void* w, int rowlen, const long long* pairs, int npairs) {
    if (!w || !pairs || npairs < 0 || rowlen <= 0) return SG_ERR_ARG;
    if (npairs == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_copy_rows<<<npairs, 256, 0, (cudaStream_t)stream>>>((unsigned short*)w, rowlen, pairs, npairs);
    return cuda_ok(cudaGetLastError());
}

static int r2_step(int rowlen) { const int s = (16 << 20) / rowlen; return s < 1 ? 1 : s; }

extern "C" size_t sg_r2_stats_scratch_bytes(int nrows, int rowlen) {
    if (nrows <= 0 || rowlen <= 0) return 0;
    const int step = r2_step(rowlen), nchunks = (nrows + step - 1) / step;
    return ((size_t)nrows * 4 + 255) / 256 * 256 + (size_t)nchunks * rowlen * 16;
}

extern "C" int sg_r2_stats(int device, void* stream, const void* w, int nrows, int rowlen, short* rfi, short* cfi, signed char* scl,
                           void* scratch, size_t scratch_bytes) {
    if (!w || !rfi || !cfi || !scl || nrows <= 0 || rowlen <= 0) return SG_ERR_ARG;
    if (!scratch || scratch_bytes < sg_r2_stats_scratch_bytes(nrows, rowlen) || (uintptr_t)scratch % 16) return SG_ERR_SCRATCH;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int step = r2_step(rowlen), nchunks = (nrows + step - 1) / step;
    if (nchunks > 65535) return SG_ERR_LIMIT;
    float* rfa = (float*)scratch;
    double* part = (double*)((unsigned char*)scratch + ((size_t)nrows * 4 + 255) / 256 * 256);
    k_r2_rowstat<<<(nrows + 3) / 4, 128, 0, st>>>((const unsigned short*)w, nrows, rowlen, rfi, rfa);
    k_r2_colpart<<<dim3((rowlen + 31) / 32, nchunks), 256, 0, st>>>((const unsigned short*)w, nrows, rowlen, step, rfa, part);
    k_r2_colfinal<<<(rowlen + 255) / 256, 256, 0, st>>>(part, nchunks, nrows, rowlen, cfi, scl);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_dm_log2(int device, void* stream, const double* x, long long n, double* y) {
    if (n < 0 || (n && (!x || !y))) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_dm_log2<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, y);
    return cuda_ok(cudaGetLastError());
}
extern "C" int sg_dm_exp2(int device, void* stream, const double* x, long long n, double* y) {
    if (n < 0 || (n && (!x || !y))) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_dm_exp2<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, y);
    return cuda_ok(cudaGetLastError());
}
extern "C" int sg_dm_rows(int device, void* stream, const float* x, long long nr, long long nc, int square, double* out) {
    if (nr < 0 || nc < 0 || (nr && (!x || !out))) return SG_ERR_ARG;
    if (nr == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_dm_rows<<<(unsigned)((nr + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, nr, nc, square, out);
    return cuda_ok(cudaGetLastError());
}
extern "C" int sg_dm_cols(int device, void* stream, const float* x, long long nr, long long nc, int square, const unsigned char* mask,
                          double* out) {
    if (nr < 0 || nc < 0 || (nc && (!x || !out))) return SG_ERR_ARG;
    if (nc == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_dm_cols<<<(unsigned)((nc + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, nr, nc, square, mask, out);
    return cuda_ok(cudaGetLastError());
}
