// Segment-parallel rANS over a plain symbol stream with per-block context tables (the residual-codec
// microbenchmark, and the engine the QR and BF16 coders share): histogram, table preparation, encode,
// prefix-sum + gather of the per-segment slots, decode.
//
// Stream model: `nsym` byte symbols cut into blocks of `block_len` symbols (a quantised block's codes);
// block b is coded with context table block_tab[b]; segments of `seg_len` symbols (a multiple of block_len
// and of 16) are independent rANS streams, one lane each.  Arithmetic and byte order follow the
// reference's coder (seedpack/qr.py:651-663, seedpack/rans.py:54-105 with PROB_BITS = PB).
#include "api_util.h"
#include "rans.cuh"

namespace sg {

// ---- tables: frequencies -> encoder entries (+ decoder LUT) ---------------------------------------------
// Replaces cum_of (seedpack/gpu2.py:483-486) and build_lut (seedpack/qr.py:889-895).  One CTA per table.
__global__ void __launch_bounds__(256) k_rans_tables(const uint16_t* __restrict__ freq, int pb, RansSym* __restrict__ enc,
                                                     uint8_t* __restrict__ lut, int* __restrict__ status) {
    __shared__ unsigned cum[257];
    const int t = blockIdx.x, s = threadIdx.x;
    const unsigned f = freq[t * 256 + s];
    // inclusive scan of 256 frequencies
    __shared__ unsigned warp_tot[8];
    unsigned v = f;
    for (int o = 1; o < 32; o <<= 1) { const unsigned n = __shfl_up_sync(0xffffffffu, v, o); if ((s & 31) >= o) v += n; }
    if ((s & 31) == 31) warp_tot[s >> 5] = v;
    __syncthreads();
    unsigned base = 0;
    for (int w = 0; w < (s >> 5); ++w) base += warp_tot[w];
    const unsigned incl = v + base;
    cum[s + 1] = incl;
    if (s == 0) cum[0] = 0;
    __syncthreads();
    const bool whole = cum[256] == (1u << pb);                                             // a used table must sum to 2^PB
    if (s == 255 && incl != 0 && !whole) atomicOr(status, SG_ST_CORRUPT);
    const unsigned c = incl - f;
    RansSym e;
    e.fc = f | (c << 16);
    if (f >= 2) {
        const unsigned sh = rans_shift(f);
        e.rcp = (unsigned)((((unsigned long long)1 << (sh + 31)) + f - 1) / f);
    } else e.rcp = 0xffffffffu;
    enc[t * 256 + s] = e;
    if (lut && whole) {               // any other row would write outside its 2^PB slots: its LUT is left alone
        if (pb == 15) {               // compact: one entry per 128 slots (the decoder scans on from it), then the symbols' words
            uint8_t* l = lut + (size_t)t * RANS_COMPACT;
            for (unsigned b = (c + 127) >> 7; (b << 7) < incl; ++b) l[b] = (uint8_t)s;
            reinterpret_cast<unsigned*>(l + 256)[s] = e.fc;
        } else {
            uint8_t* l = lut + ((size_t)t << pb);
            for (unsigned i = c; i < incl; ++i) l[i] = (uint8_t)s;
        }
    }
}

// ---- histogram -------------------------------------------------------------------------------------------
// One lane per block.  Zero symbols (the bulk of a residual stream) are counted in registers and added once
// per warp and table; the others go out individually.
__global__ void __launch_bounds__(256) k_rans_hist(const uint8_t* __restrict__ sym, const uint16_t* __restrict__ block_tab,
                                                   int block_len, long long nblocks, unsigned* __restrict__ counts) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = b < nblocks;
    unsigned tab = 0xffffffffu, zeros = 0;
    if (live) {
        tab = block_tab[b];
        const uint4* p = reinterpret_cast<const uint4*>(sym + b * block_len);
        for (int i = 0; i < block_len / 16; ++i) {
            const uint4 v = __ldg(p + i);
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned s = (w[k] >> (8 * j)) & 0xff;
                    if (s == 0) ++zeros; else atomicAdd(counts + tab * 256 + s, 1u);
                }
            }
        }
    }
    const unsigned peers = __match_any_sync(0xffffffffu, tab);
    const unsigned total = __reduce_add_sync(peers, zeros);
    if (live && (threadIdx.x & 31) == (unsigned)(__ffs(peers) - 1) && total) atomicAdd(counts + tab * 256, total);
}

// ---- encode ----------------------------------------------------------------------------------------------
template <int PB>
__global__ void __launch_bounds__(64) k_rans_encode(const uint8_t* __restrict__ sym, const uint16_t* __restrict__ block_tab,
                                                    int block_len, long long nsym, int seg_len, const RansSym* __restrict__ enc,
                                                    uint8_t* __restrict__ out, size_t cap, unsigned* __restrict__ out_len, int nseg) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const long long s0 = (long long)s * seg_len;
    const long long n = min((long long)seg_len, nsym - s0);            // multiple of 16
    uint8_t* slot = out + (size_t)s * cap;
    ByteWriterDown w;
    w.init(slot + cap);
    unsigned x = RANS_L;
    const RansSym* tab = nullptr;
    RansSym e0 = {0, 0};
    long long cur_block = -1;
    // The lanes of a warp sit in different segments, hence different tables: a table look-up by all lanes touches 32
    // cache lines, and with one per symbol the kernel is bound by the L1's line rate, not by its chains.  Most residual
    // symbols are 0: the current table's entry for 0 is kept in registers, and only the lanes with another symbol load.
    for (long long i = n - 16; i >= 0; i -= 16) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(sym + s0 + i));
        const unsigned wv[4] = {v.x, v.y, v.z, v.w};
        const long long blk = (s0 + i) / block_len;                     // 16 | block_len: one table per 16 symbols
        if (blk != cur_block) { cur_block = blk; tab = enc + (size_t)block_tab[blk] * 256; e0 = tab[0]; }
#pragma unroll
        for (int k = 3; k >= 0; --k) {
#pragma unroll
            for (int j = 3; j >= 0; --j) {
                const unsigned sy = (wv[k] >> (8 * j)) & 0xff;
                RansSym e = e0;
                if (sy) e = tab[sy];
                rans_put<PB>(x, w, e);
            }
        }
        if (w.ptr() < slot + 64) { out_len[s] = 0xffffffffu; return; }   // 16 symbols write at most 32 bytes
    }
    rans_flush(x, w);
    w.flush(slot);
    out_len[s] = w.bad ? LEN_NOFREQ : (unsigned)(slot + cap - w.ptr());
}

// ---- scan + gather ---------------------------------------------------------------------------------------
// Replaces cumsum + gather (seedpack/qr.py:1054-1056, 880-887).  k_scan: exclusive prefix sum of the
// segment lengths by one CTA (segments number in the thousands to hundreds of thousands);
// k_gather: one warp per segment copies its bytes to its place.
__global__ void __launch_bounds__(1024) k_scan_lens(const unsigned* __restrict__ len, int nseg, unsigned long long* __restrict__ off,
                                                    int* __restrict__ status) {
    __shared__ unsigned long long wsum[32];
    __shared__ unsigned long long carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < nseg; base += 1024) {
        const int i = base + threadIdx.x;
        unsigned l = i < nseg ? len[i] : 0;
        if (l == LEN_OVERFLOW) { atomicOr(status, SG_ST_OVERFLOW); l = 0; }
        else if (l == LEN_NOFREQ) { atomicOr(status, SG_ST_CORRUPT); l = 0; }
        unsigned long long v = l;
        for (int o = 1; o < 32; o <<= 1) { const unsigned long long n = __shfl_up_sync(0xffffffffu, v, o); if ((threadIdx.x & 31) >= o) v += n; }
        if ((threadIdx.x & 31) == 31) wsum[threadIdx.x >> 5] = v;
        __syncthreads();
        unsigned long long pre = carry;
        for (int w = 0; w < (threadIdx.x >> 5); ++w) pre += wsum[w];
        if (i < nseg) off[i] = pre + v - l;
        __syncthreads();
        if (threadIdx.x == 1023) carry = pre + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) off[nseg] = carry;
}

__global__ void __launch_bounds__(256) k_gather(const uint8_t* __restrict__ src, size_t cap, const unsigned* __restrict__ len,
                                                const unsigned long long* __restrict__ off, int nseg, uint8_t* __restrict__ dst,
                                                unsigned long long dst_cap) {
    const int s = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= nseg) return;
    const unsigned l = len[s];
    if (l >= LEN_NOFREQ || off[s] + l > dst_cap) return;
    const uint8_t* a = src + (size_t)(s + 1) * cap - l;
    uint8_t* d = dst + off[s];
    for (unsigned i = lane; i < l; i += 32) d[i] = a[i];
}

// ---- decode ----------------------------------------------------------------------------------------------
template <int PB>
__global__ void __launch_bounds__(64) k_rans_decode(const uint8_t* __restrict__ in, const unsigned long long* __restrict__ off,
                                                    const uint16_t* __restrict__ block_tab, int block_len, long long nsym, int seg_len,
                                                    const RansSym* __restrict__ enc, const uint8_t* __restrict__ lut,
                                                    uint8_t* __restrict__ sym, int nseg, int* __restrict__ status) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const long long s0 = (long long)s * seg_len;
    const long long n = min((long long)seg_len, nsym - s0);
    ByteReaderUp r;
    r.init(in + off[s], in + off[s + 1]);
    unsigned x = rans_init(r);
    const RansSym* tab = nullptr;
    const uint8_t* l = nullptr;
    long long cur_block = -1;
    for (long long i = 0; i < n; i += 16) {
        const long long blk = (s0 + i) / block_len;
        if (blk != cur_block) { cur_block = blk; const unsigned t = block_tab[blk]; tab = enc + (size_t)t * 256; l = lut + ((size_t)t << PB); }
        unsigned wv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) word |= rans_get<PB>(x, r, l, tab) << (8 * j);
            wv[k] = word;
        }
        *reinterpret_cast<uint4*>(sym + s0 + i) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        if (r.over) { atomicOr(status, SG_ST_CORRUPT); return; }
    }
    if (x != RANS_L || r.p != r.end) atomicOr(status, SG_ST_CORRUPT);     // a well-formed segment ends in the initial state
}

// The same decoder with the tables it needs in shared memory.  A residual stream is mostly the symbol 0, whose slots are
// [0, freq(0)) of every table: for those the step is x = freq(0) (x >> PB) + slot with freq(0) from a small array in
// shared memory.  The other slots of a table - [freq(0), 2^PB), few when zeros dominate - get one 4-byte entry each,
// symbol | (freq - 1) << 8 | (slot - cum) << 20, also in shared memory as far as they fit (tables in id order; the rest
// keep the two dependent global loads lut[slot] -> enc[symbol]).  Every CTA builds the entries from enc / lut itself
// (a few per cent of its decoding time): the caller passes no further buffer.  One CTA of 512 lanes per SM.
constexpr unsigned NOFIT = 0xffffffffu;
template <int PB>
__global__ void __launch_bounds__(512, 1) k_rans_decode_sm(const uint8_t* __restrict__ in, const unsigned long long* __restrict__ off,
                                                           const uint16_t* __restrict__ block_tab, int block_len, long long nsym, int seg_len,
                                                           const RansSym* __restrict__ enc, const uint8_t* __restrict__ lut,
                                                           uint8_t* __restrict__ sym, int nseg, int ntab, unsigned cap, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned smem[];
    unsigned* base = smem;                                   // [ntab] first entry of the table, NOFIT if not staged
    unsigned* ent = smem + ntab;                             // [cap]
    unsigned short* f0 = reinterpret_cast<unsigned short*>(ent + cap);     // [ntab] freq(0)
    constexpr unsigned SLOTS = 1u << PB;
    for (int t = threadIdx.x; t < ntab; t += blockDim.x) {
        const unsigned first = enc[(size_t)t * 256].fc & 0xffffu, last = enc[(size_t)t * 256 + 255].fc;
        const bool used = (last >> 16) + (last & 0xffffu) == SLOTS;
        f0[t] = (unsigned short)(used ? first : 0);
        base[t] = used ? SLOTS - first : 0;                  // for now: the number of entries the table needs
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned run = 0;
        for (int t = 0; t < ntab; ++t) {
            const unsigned n = base[t];
            if (n == 0 && f0[t] == 0) { base[t] = NOFIT; continue; }           // an unused table
            if (run + n <= cap) { base[t] = run; run += n; } else base[t] = NOFIT;
        }
    }
    __syncthreads();
    for (int t = threadIdx.x >> 5; t < ntab; t += blockDim.x >> 5) {
        const unsigned b = base[t];
        if (b == NOFIT) continue;
        const unsigned f = f0[t];
        for (unsigned slot = f + (threadIdx.x & 31); slot < SLOTS; slot += 32) {
            const unsigned s = lut[((size_t)t << PB) + slot];
            const unsigned fc = enc[(size_t)t * 256 + s].fc;
            ent[b + slot - f] = s | (((fc & 0xffffu) - 1u) << 8) | ((slot - (fc >> 16)) << 20);
        }
    }
    __syncthreads();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= nseg) return;
    const long long s0 = (long long)s * seg_len;
    const long long n = min((long long)seg_len, nsym - s0);
    ByteReaderUp r;
    r.init(in + off[s], in + off[s + 1]);
    unsigned x = rans_init(r);
    unsigned tf0 = 0, tb = NOFIT, tid = 0;
    long long cur_block = -1;
    for (long long i = 0; i < n; i += 16) {
        const long long blk = (s0 + i) / block_len;
        if (blk != cur_block) { cur_block = blk; tid = block_tab[blk]; tf0 = f0[tid]; tb = base[tid]; }
        unsigned wv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned slot = x & (SLOTS - 1);
                unsigned sy = 0;
                if (slot < tf0) x = tf0 * (x >> PB) + slot;
                else if (tb != NOFIT) {
                    const unsigned e = ent[tb + slot - tf0];
                    sy = e & 0xffu;
                    x = (((e >> 8) & 0xfffu) + 1u) * (x >> PB) + (e >> 20);
                } else {
                    sy = lut[((size_t)tid << PB) + slot];
                    const unsigned fc = enc[(size_t)tid * 256 + sy].fc;
                    x = (fc & 0xffffu) * (x >> PB) + slot - (fc >> 16);
                }
                if (x < RANS_L) { x = (x << 8) | r.get(); if (x < RANS_L) x = (x << 8) | r.get(); }
                word |= sy << (8 * j);
            }
            wv[k] = word;
        }
        *reinterpret_cast<uint4*>(sym + s0 + i) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        if (r.over) { atomicOr(status, SG_ST_CORRUPT); return; }
    }
    if (x != RANS_L || r.p != r.end) atomicOr(status, SG_ST_CORRUPT);     // a well-formed segment ends in the initial state
}

}  // namespace sg

using namespace sg;

static int stream_args_ok(const void* sym, const void* block_tab, int block_len, long long nsym, int seg_len) {
    if (!sym || !block_tab || nsym < 0) return SG_ERR_ARG;
    if (block_len <= 0 || block_len % 16 || seg_len <= 0 || seg_len % block_len || nsym % block_len) return SG_ERR_SHAPE;
    if ((uintptr_t)sym % 16 || (uintptr_t)block_tab % 2) return SG_ERR_ALIGN;
    return SG_OK;
}

extern "C" int sg_rans_hist(int device, void* stream, const unsigned char* sym, const unsigned short* block_tab, int block_len,
                            long long nsym, unsigned* counts) {
    if (!counts) return SG_ERR_ARG;
    int rc = stream_args_ok(sym, block_tab, block_len, nsym, block_len);
    if (rc != SG_OK) return rc;
    if (nsym == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long nblocks = nsym / block_len, grid = (nblocks + 255) / 256;
    if (grid > 0x7fffffffLL) return SG_ERR_LIMIT;
    k_rans_hist<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(sym, block_tab, block_len, nblocks, counts);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_rans_tables(int device, void* stream, const unsigned short* freq, int ntab, int pb, void* enc_tab, unsigned char* lut) {
    if (!freq || !enc_tab || ntab < 0 || (pb != 12 && pb != 14 && pb != 15)) return SG_ERR_ARG;
    if ((uintptr_t)enc_tab % 8) return SG_ERR_ALIGN;
    if (ntab == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    k_rans_tables<<<ntab, 256, 0, (cudaStream_t)stream>>>(freq, pb, (RansSym*)enc_tab, lut, status_word(device));
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_rans_encode(int device, void* stream, const unsigned char* sym, const unsigned short* block_tab, int block_len,
                              long long nsym, int seg_len, int pb, const void* enc_tab, unsigned char* slots, size_t cap,
                              unsigned* out_len) {
    if (!enc_tab || !slots || !out_len || pb != 12) return SG_ERR_ARG;
    int rc = stream_args_ok(sym, block_tab, block_len, nsym, seg_len);
    if (rc != SG_OK) return rc;
    if (cap < 128 || cap % 16 || (uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nsym == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long nseg = (nsym + seg_len - 1) / seg_len;
    if (nseg > 0x7fffffffLL) return SG_ERR_LIMIT;
    k_rans_encode<12><<<(unsigned)((nseg + 63) / 64), 64, 0, (cudaStream_t)stream>>>(sym, block_tab, block_len, nsym, seg_len,
                                                                                     (const RansSym*)enc_tab, slots, cap, out_len, (int)nseg);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_scan_gather(int device, void* stream, const unsigned char* slots, size_t cap, const unsigned* out_len, int nseg,
                              unsigned char* dst, unsigned long long dst_cap, unsigned long long* off) {
    if (!slots || !out_len || !off || nseg < 0 || (!dst && dst_cap)) return SG_ERR_ARG;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    k_scan_lens<<<1, 1024, 0, st>>>(out_len, nseg, off, status_word(device));
    rc = cuda_ok(cudaGetLastError());
    if (rc != SG_OK || nseg == 0 || !dst) return rc;
    k_gather<<<(nseg + 7) / 8, 256, 0, st>>>(slots, cap, out_len, off, nseg, dst, dst_cap);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_rans_decode(int device, void* stream, const unsigned char* in, const unsigned long long* off,
                              const unsigned short* block_tab, int block_len, long long nsym, int seg_len, int pb,
                              const void* enc_tab, const unsigned char* lut, int ntab, unsigned char* sym_out) {
    if (!in || !off || !enc_tab || !lut || pb != 12 || ntab < 0) return SG_ERR_ARG;
    int rc = stream_args_ok(sym_out, block_tab, block_len, nsym, seg_len);
    if (rc != SG_OK) return rc;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nsym == 0) return SG_OK;
    rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long nseg = (nsym + seg_len - 1) / seg_len;
    if (nseg > 0x7fffffffLL) return SG_ERR_LIMIT;
    cudaStream_t st = (cudaStream_t)stream;
    // tables staged in shared memory when their number is given and small enough to leave room for entries
    const size_t smem_max = 200 * 1024;
    if (ntab > 0 && (size_t)ntab * 6 + 8192 <= smem_max) {
        const unsigned cap = (unsigned)((smem_max - (size_t)ntab * 6 - 16) / 4);
        const size_t smem = (size_t)ntab * 4 + (size_t)cap * 4 + (size_t)ntab * 2 + 16;
        static bool configured[64] = {false};
        if (device < 64 && !configured[device]) {
            rc = cuda_ok(cudaFuncSetAttribute(k_rans_decode_sm<12>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max + 1024));
            if (rc != SG_OK) return rc;
            configured[device] = true;
        }
        k_rans_decode_sm<12><<<(unsigned)((nseg + 511) / 512), 512, smem, st>>>(in, off, block_tab, block_len, nsym, seg_len,
                                                                            (const RansSym*)enc_tab, lut, sym_out, (int)nseg, ntab, cap,
                                                                            status_word(device));
        return cuda_ok(cudaGetLastError());
    }
    k_rans_decode<12><<<(unsigned)((nseg + 63) / 64), 64, 0, st>>>(in, off, block_tab, block_len, nsym, seg_len,
                                                                  (const RansSym*)enc_tab, lut, sym_out, (int)nseg, status_word(device));
    return cuda_ok(cudaGetLastError());
}
