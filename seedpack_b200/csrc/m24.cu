// M24: the earlier BF16 base codec (`--method m28` archives), kernels bf_hist / bf_enc / bf_dec of the reference
// (seedpack/gpu_bf16.py:63-137).  Same coder as R2 (rans.cuh) at 12 probability bits; per-tensor tables; contexts from
// quarter-octave side information:
//   pred4   = rfi[row] + cfi[col]
//   exponent table  = tab + clamp((pred4 + 108) >> 1, 0, 127)
//   mantissa table  = tab + 128 + clamp(exponent - ((pred4 + 508) >> 2) + 8, 0, 15)
//   sign table      = tab + 144 + scl[col]
// symbols per weight in decode order exponent, mantissa, sign; segments of up to 16384 weights inside one tensor, one
// rANS state each.  Records: TB { int64 off; int32 rowlen, rowbase, colbase, tab } per tensor, SG { int32 t, n; int64 i0 }
// per segment (gpu_bf16.py:283-284).  Tables are addressed by their raw id: counts / enc_tab / lut cover ntensors * 160.
#include "api_util.h"
#include "rans.cuh"

namespace sg {
namespace m24 {

struct TB { long long off; int rowlen, rowbase, colbase, tab; };
struct SG { int t, n; long long i0; };
struct Side { const short* rfi; const short* cfi; const signed char* scl; };

SG_DEVINL int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
SG_DEVINL int exp_table(int pred4) { return clampi((pred4 + 108) >> 1, 0, 127); }
SG_DEVINL int man_table(int ex, int pred4) { return 128 + clampi(ex - ((pred4 + 508) >> 2) + 8, 0, 15); }

// counts are order-free: a warp per segment, lanes on consecutive weights
__global__ void __launch_bounds__(256) k_hist(const unsigned char* __restrict__ file, const TB* __restrict__ tb, const SG* __restrict__ sg, int nseg,
                                              Side sd, unsigned* __restrict__ counts) {
    const int s = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= nseg) return;
    const SG g = sg[s];
    const TB T = tb[g.t];
    const unsigned short* w = reinterpret_cast<const unsigned short*>(file + T.off) + g.i0;
    for (int k = lane; k < g.n; k += 32) {
        const long long i = g.i0 + k;
        const int r = (int)(i / T.rowlen), j = (int)(i % T.rowlen);
        const unsigned u = w[k];
        const int ex = (u >> 7) & 255, man = u & 127, sgn = u >> 15;
        const int pred4 = sd.rfi[T.rowbase + r] + sd.cfi[T.colbase + j];
        atomicAdd(counts + (size_t)(T.tab + exp_table(pred4)) * 256 + ex, 1u);
        atomicAdd(counts + (size_t)(T.tab + man_table(ex, pred4)) * 256 + man, 1u);
        atomicAdd(counts + (size_t)(T.tab + 144 + sd.scl[T.colbase + j]) * 256 + sgn, 1u);
    }
}

__global__ void __launch_bounds__(64) k_enc(const unsigned char* __restrict__ file, const TB* __restrict__ tb, const SG* __restrict__ sg, int nseg,
                                            Side sd, const RansSym* __restrict__ enc, unsigned char* __restrict__ out, size_t cap,
                                            unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const SG g = sg[s];
    const TB T = tb[g.t];
    const unsigned short* w = reinterpret_cast<const unsigned short*>(file + T.off) + g.i0;
    const long long last = g.i0 + g.n - 1;
    int r = (int)(last / T.rowlen), j = (int)(last % T.rowlen);
    int rf = sd.rfi[T.rowbase + r];
    unsigned char* slot = out + (size_t)s * cap;
    ByteWriterDown wr; wr.init(slot + cap);
    unsigned x = RANS_L;
    for (int k = g.n - 1; k >= 0; --k) {
        const unsigned u = w[k];
        const int ex = (u >> 7) & 255, man = u & 127, sgn = u >> 15;
        const int pred4 = rf + sd.cfi[T.colbase + j];
        const RansSym e2 = enc[(size_t)(T.tab + 144 + sd.scl[T.colbase + j]) * 256 + sgn];
        const RansSym e1 = enc[(size_t)(T.tab + man_table(ex, pred4)) * 256 + man];
        const RansSym e0 = enc[(size_t)(T.tab + exp_table(pred4)) * 256 + ex];
        rans_put<12>(x, wr, e2); rans_put<12>(x, wr, e1); rans_put<12>(x, wr, e0);
        if (wr.ptr() < slot + 64) { out_len[s] = LEN_OVERFLOW; return; }
        if (--j < 0) { j = T.rowlen - 1; --r; if (k > 0) rf = sd.rfi[T.rowbase + r]; }
    }
    rans_flush(x, wr);
    wr.flush(slot);
    out_len[s] = wr.bad ? LEN_NOFREQ : (unsigned)(slot + cap - wr.ptr());
}

__global__ void __launch_bounds__(64) k_dec(const unsigned char* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                            const unsigned long long* __restrict__ in_end, unsigned char* __restrict__ file,
                                            const TB* __restrict__ tb, const SG* __restrict__ sg, int nseg, Side sd,
                                            const RansSym* __restrict__ enc, const unsigned char* __restrict__ lut, int* __restrict__ status) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const SG g = sg[s];
    const TB T = tb[g.t];
    unsigned short* w = reinterpret_cast<unsigned short*>(file + T.off) + g.i0;
    int r = (int)(g.i0 / T.rowlen), j = (int)(g.i0 % T.rowlen);
    int rf = sd.rfi[T.rowbase + r];
    ByteReaderUp rd; rd.init(in + in_off[s], in + in_end[s]);
    unsigned x = rans_init(rd);
    for (int k = 0; k < g.n; ++k) {
        const int pred4 = rf + sd.cfi[T.colbase + j];
        const int t0 = T.tab + exp_table(pred4);
        const int ex = (int)rans_get<12>(x, rd, lut + ((size_t)t0 << 12), enc + (size_t)t0 * 256);
        const int t1 = T.tab + man_table(ex, pred4);
        const int man = (int)rans_get<12>(x, rd, lut + ((size_t)t1 << 12), enc + (size_t)t1 * 256);
        const int t2 = T.tab + 144 + sd.scl[T.colbase + j];
        const int sgn = (int)rans_get<12>(x, rd, lut + ((size_t)t2 << 12), enc + (size_t)t2 * 256);
        w[k] = (unsigned short)((sgn << 15) | (ex << 7) | man);
        if (rd.over) break;
        if (++j == T.rowlen) { j = 0; ++r; if (k + 1 < g.n) rf = sd.rfi[T.rowbase + r]; }
    }
    if (rd.over || x != RANS_L || rd.p != rd.end) atomicOr(status, SG_ST_CORRUPT);
}

}  // namespace m24
}  // namespace sg

using namespace sg;

static int m24_args(const void* file, const void* tb, const void* sgp, int nseg, const void* rfi, const void* cfi, const void* scl) {
    return (!file || !tb || !sgp || !rfi || !cfi || !scl || nseg < 0) ? SG_ERR_ARG : SG_OK;
}

extern "C" int sg_m24_hist(int device, void* stream, const unsigned char* file, const void* tb, const void* sgp, int nseg, const short* rfi,
                           const short* cfi, const signed char* scl, unsigned* counts) {
    int rc = m24_args(file, tb, sgp, nseg, rfi, cfi, scl);
    if (rc != SG_OK || !counts) return SG_ERR_ARG;
    if (nseg == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    m24::k_hist<<<(unsigned)((nseg + 7) / 8), 256, 0, (cudaStream_t)stream>>>(file, (const m24::TB*)tb, (const m24::SG*)sgp, nseg,
                                                                           m24::Side{rfi, cfi, scl}, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m24_encode(int device, void* stream, const unsigned char* file, const void* tb, const void* sgp, int nseg, const short* rfi,
                             const short* cfi, const signed char* scl, const void* enc_tab, unsigned char* slots, size_t cap, unsigned* out_len) {
    int rc = m24_args(file, tb, sgp, nseg, rfi, cfi, scl);
    if (rc != SG_OK || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 128 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    m24::k_enc<<<(unsigned)((nseg + 63) / 64), 64, 0, (cudaStream_t)stream>>>(file, (const m24::TB*)tb, (const m24::SG*)sgp, nseg,
                                                                           m24::Side{rfi, cfi, scl}, (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m24_decode(int device, void* stream, const unsigned char* in, const unsigned long long* in_off, const unsigned long long* in_end,
                             unsigned char* file, const void* tb, const void* sgp, int nseg, const short* rfi, const short* cfi,
                             const signed char* scl, const void* enc_tab, const unsigned char* lut) {
    int rc = m24_args(file, tb, sgp, nseg, rfi, cfi, scl);
    if (rc != SG_OK || !in || !in_off || !in_end || !enc_tab || !lut) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nseg == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    m24::k_dec<<<(unsigned)((nseg + 63) / 64), 64, 0, (cudaStream_t)stream>>>(in, in_off, in_end, file, (const m24::TB*)tb, (const m24::SG*)sgp, nseg,
                                                                           m24::Side{rfi, cfi, scl}, (const RansSym*)enc_tab, lut, status_word(device));
    return cuda_ok(cudaGetLastError());
}
