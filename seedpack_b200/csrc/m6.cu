// M6: the first GPU codec of the reference - Q8_0 files coded without a base (seedpack/gpu_codec.py:73-159, kernels
// hist / encode / decode).  Blocks are cut into segments of 512, one rANS state per segment (rans.cuh, 12 probability
// bits).  A block's 35 symbols in decode order and their tables (770 per tensor group):
//   scale high byte   table grp*770 + previous block's high byte (0 at a row start and at a segment start)
//   scale low byte    table grp*770 + 256 + high byte
//   position of the largest magnitude        table grp*770 + 512
//   the weight there                          table grp*770 + 513
//   the other 31 weights                      table grp*770 + 514 + 16 * bucket(scale) + column class
// bucket(scale) = clamp(((fp16 bits - tensor median) >> 8) + 8, 0, 15).  Records: Meta { int32 first, nblocks, nb_row,
// grp, colbase, med } per tensor; tfirst[t] = first block of tensor t; colmap = one class byte per column.
#include "api_util.h"
#include "rans.cuh"

namespace sg {
namespace m6 {

constexpr int SEG = 512, TPG = 770, T_LO = 256, T_POS = 512, T_MX = 513, T_QS = 514, NCOL = 16, NSB = 16;
struct Meta { int first, nblocks, nb_row, grp, colbase, med; };

SG_DEVINL int tensor_of(const int* __restrict__ tfirst, int ntens, int b) {      // the last tensor that starts at or before block b
    int lo = 0, hi = ntens - 1;
    while (lo < hi) { const int m = (lo + hi + 1) >> 1; if (tfirst[m] <= b) lo = m; else hi = m - 1; }
    return lo;
}
SG_DEVINL int bucket(int lo, int hi, int med) {
    const int v = (((lo | (hi << 8)) - med) >> 8) + NSB / 2;
    return v < 0 ? 0 : (v > NSB - 1 ? NSB - 1 : v);
}

// the 35 (table, symbol) pairs of block b in decode order, packed table << 8 | symbol
SG_DEVINL void block_symbols(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos, const Meta& M,
                             const unsigned char* __restrict__ colmap, int b, int b0, unsigned* out) {
    const unsigned char* blk = blocks + (size_t)b * 34;
    const int inrow = (b - M.first) % M.nb_row, base = M.grp * TPG;
    const int prev = (inrow == 0 || b == b0) ? 0 : blocks[(size_t)(b - 1) * 34 + 1];
    const int lo = blk[0], hi = blk[1], p = pos[b];
    out[0] = (unsigned)(base + prev) << 8 | (unsigned)hi;
    out[1] = (unsigned)(base + T_LO + hi) << 8 | (unsigned)lo;
    out[2] = (unsigned)(base + T_POS) << 8 | (unsigned)p;
    out[3] = (unsigned)(base + T_MX) << 8 | blk[2 + p];
    const int qb = base + T_QS + bucket(lo, hi, M.med) * NCOL;
    const unsigned char* cm = colmap + M.colbase + inrow * 32;
    int n = 4;
    for (int j = 0; j < 32; ++j) if (j != p) out[n++] = (unsigned)(qb + cm[j]) << 8 | blk[2 + j];
}

__global__ void __launch_bounds__(128) k_hist(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                              const Meta* __restrict__ M, const int* __restrict__ tfirst, int ntens,
                                              const unsigned char* __restrict__ colmap, int nblocks, unsigned* __restrict__ counts) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x, b0 = s * SEG;
    if (b0 >= nblocks) return;
    const int b1 = min(b0 + SEG, nblocks);
    int t = tensor_of(tfirst, ntens, b0);
    unsigned sy[35];
    for (int b = b0; b < b1; ++b) {
        if (t + 1 < ntens && b >= tfirst[t + 1]) ++t;
        block_symbols(blocks, pos, M[t], colmap, b, b0, sy);
        for (int i = 0; i < 35; ++i) atomicAdd(counts + sy[i], 1u);               // table * 256 + symbol
    }
}

__global__ void __launch_bounds__(128) k_enc(const unsigned char* __restrict__ blocks, const unsigned char* __restrict__ pos,
                                             const Meta* __restrict__ M, const int* __restrict__ tfirst, int ntens,
                                             const unsigned char* __restrict__ colmap, int nblocks, const RansSym* __restrict__ enc,
                                             unsigned char* __restrict__ out, size_t cap, unsigned* __restrict__ out_len) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x, b0 = s * SEG;
    if (b0 >= nblocks) return;
    const int b1 = min(b0 + SEG, nblocks);
    unsigned char* slot = out + (size_t)s * cap;
    ByteWriterDown wr; wr.init(slot + cap);
    unsigned x = RANS_L;
    int t = tensor_of(tfirst, ntens, b1 - 1);
    unsigned sy[35];
    for (int b = b1 - 1; b >= b0; --b) {
        while (b < M[t].first) --t;
        block_symbols(blocks, pos, M[t], colmap, b, b0, sy);
        for (int i = 34; i >= 0; --i) rans_put<12>(x, wr, enc[sy[i]]);
        if (wr.ptr() < slot + 96) { out_len[s] = LEN_OVERFLOW; return; }         // a block writes at most 70 bytes
    }
    rans_flush(x, wr);
    wr.flush(slot);
    out_len[s] = wr.bad ? LEN_NOFREQ : (unsigned)(slot + cap - wr.ptr());
}

__global__ void __launch_bounds__(128) k_dec(const unsigned char* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                             const unsigned long long* __restrict__ in_end, const Meta* __restrict__ M,
                                             const int* __restrict__ tfirst, int ntens, const unsigned char* __restrict__ colmap, int nblocks,
                                             const RansSym* __restrict__ enc, const unsigned char* __restrict__ lut,
                                             unsigned char* __restrict__ blocks, int* __restrict__ status) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x, b0 = s * SEG;
    if (b0 >= nblocks) return;
    const int b1 = min(b0 + SEG, nblocks);
    ByteReaderUp rd; rd.init(in + in_off[s], in + in_end[s]);
    unsigned x = rans_init(rd);
    auto get = [&](int tab) { return (int)rans_get<12>(x, rd, lut + ((size_t)tab << 12), enc + (size_t)tab * 256); };
    int t = tensor_of(tfirst, ntens, b0), prev = 0;
    for (int b = b0; b < b1 && !rd.over; ++b) {
        if (t + 1 < ntens && b >= tfirst[t + 1]) ++t;
        const Meta m = M[t];
        unsigned char* blk = blocks + (size_t)b * 34;
        const int inrow = (b - m.first) % m.nb_row, base = m.grp * TPG;
        if (inrow == 0 || b == b0) prev = 0;
        const int hi = get(base + prev), lo = get(base + T_LO + hi), p = get(base + T_POS) & 31, mx = get(base + T_MX);
        blk[0] = (unsigned char)lo; blk[1] = (unsigned char)hi; blk[2 + p] = (unsigned char)mx; prev = hi;
        const int qb = base + T_QS + bucket(lo, hi, m.med) * NCOL;
        const unsigned char* cm = colmap + m.colbase + inrow * 32;
        for (int j = 0; j < 32; ++j) if (j != p) blk[2 + j] = (unsigned char)get(qb + cm[j]);
    }
    if (rd.over || x != RANS_L || rd.p != rd.end) atomicOr(status, SG_ST_CORRUPT);
}

}  // namespace m6
}  // namespace sg

using namespace sg;

static int m6_args(const void* blocks, const void* pos, const void* M, const void* tfirst, int ntens, const void* colmap, int nblocks) {
    return (!blocks || !pos || !M || !tfirst || !colmap || ntens <= 0 || nblocks < 0) ? SG_ERR_ARG : SG_OK;
}

extern "C" int sg_m6_hist(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const void* meta, const int* tfirst,
                          int ntens, const unsigned char* colmap, int nblocks, unsigned* counts) {
    int rc = m6_args(blocks, pos, meta, tfirst, ntens, colmap, nblocks);
    if (rc != SG_OK || !counts) return SG_ERR_ARG;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const int nseg = (nblocks + m6::SEG - 1) / m6::SEG;
    m6::k_hist<<<(nseg + 127) / 128, 128, 0, (cudaStream_t)stream>>>(blocks, pos, (const m6::Meta*)meta, tfirst, ntens, colmap, nblocks, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m6_encode(int device, void* stream, const unsigned char* blocks, const unsigned char* pos, const void* meta, const int* tfirst,
                            int ntens, const unsigned char* colmap, int nblocks, const void* enc_tab, unsigned char* slots, size_t cap,
                            unsigned* out_len) {
    int rc = m6_args(blocks, pos, meta, tfirst, ntens, colmap, nblocks);
    if (rc != SG_OK || !enc_tab || !slots || !out_len) return SG_ERR_ARG;
    if (cap < 256 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const int nseg = (nblocks + m6::SEG - 1) / m6::SEG;
    m6::k_enc<<<(nseg + 127) / 128, 128, 0, (cudaStream_t)stream>>>(blocks, pos, (const m6::Meta*)meta, tfirst, ntens, colmap, nblocks,
                                                                 (const RansSym*)enc_tab, slots, cap, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_m6_decode(int device, void* stream, const unsigned char* in, const unsigned long long* in_off, const unsigned long long* in_end,
                            const void* meta, const int* tfirst, int ntens, const unsigned char* colmap, int nblocks, const void* enc_tab,
                            const unsigned char* lut, unsigned char* blocks) {
    int rc = m6_args(blocks, in, meta, tfirst, ntens, colmap, nblocks);
    if (rc != SG_OK || !in_off || !in_end || !enc_tab || !lut) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    if ((rc = use_device(device)) != SG_OK) return rc;
    const int nseg = (nblocks + m6::SEG - 1) / m6::SEG;
    m6::k_dec<<<(nseg + 127) / 128, 128, 0, (cudaStream_t)stream>>>(in, in_off, in_end, (const m6::Meta*)meta, tfirst, ntens, colmap, nblocks,
                                                                 (const RansSym*)enc_tab, lut, blocks, status_word(device));
    return cuda_ok(cudaGetLastError());
}
