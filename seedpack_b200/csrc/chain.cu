// The scalar coder of the reference's first codec generations (seedpack/rans.py:54-105): ONE rANS state per stream, 14
// probability bits, a context (table number) per symbol handed in by the caller.  M22, the BF16 codec without a base
// (seedpack/bf16codec.py:35-103), codes three such streams per tensor (exponents, mantissas, signs).  A stream is one
// dependent chain by format, so a stream is one lane here; a launch takes any number of streams (one lane each) that
// share their tables.  Bytes and symbols equal rans.py's (tests/test_m22_gpu.py).
#include "api_util.h"
#include "rans.cuh"

namespace sg {

template <class C>
__global__ void __launch_bounds__(32) k_chain_enc(const uint8_t* __restrict__ sym, const C* __restrict__ ctx,
                                                  const unsigned long long* __restrict__ sym_off, int nchain, int ntab,
                                                  const RansSym* __restrict__ enc, uint8_t* __restrict__ slots,
                                                  const unsigned long long* __restrict__ slot_off, unsigned long long* __restrict__ out_len) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nchain) return;
    uint8_t* slot = slots + slot_off[c];
    uint8_t* end = slots + slot_off[c + 1];
    ByteWriterDown wr; wr.init(end);
    unsigned x = RANS_L;
    const long long a = (long long)sym_off[c], z = (long long)sym_off[c + 1];
    for (long long i = z - 1; i >= a; --i) {
        const unsigned t = (unsigned)ctx[i];
        if (t >= (unsigned)ntab) { out_len[c] = LEN_NOFREQ; return; }
        rans_put<14>(x, wr, enc[(size_t)t * 256 + sym[i]]);
        if (wr.ptr() < slot + 32) { out_len[c] = LEN_OVERFLOW; return; }
    }
    rans_flush(x, wr);
    wr.flush(slot);
    out_len[c] = wr.bad ? (unsigned long long)LEN_NOFREQ : (unsigned long long)(end - wr.ptr());
}

template <class C>
__global__ void __launch_bounds__(32) k_chain_dec(const uint8_t* __restrict__ in, const unsigned long long* __restrict__ in_off,
                                                  const unsigned long long* __restrict__ in_end, const C* __restrict__ ctx,
                                                  const unsigned long long* __restrict__ sym_off, int nchain, int ntab,
                                                  const RansSym* __restrict__ enc, const uint8_t* __restrict__ lut,
                                                  uint8_t* __restrict__ sym, unsigned long long* __restrict__ used, int* __restrict__ status) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nchain) return;
    ByteReaderUp rd; rd.init(in + in_off[c], in + in_end[c]);
    unsigned x = rans_init(rd);
    const long long a = (long long)sym_off[c], z = (long long)sym_off[c + 1];
    for (long long i = a; i < z; ++i) {
        const unsigned t = (unsigned)ctx[i];
        if (t >= (unsigned)ntab || rd.over) { atomicOr(status, SG_ST_CORRUPT); return; }
        sym[i] = (uint8_t)rans_get<14>(x, rd, lut + ((size_t)t << 14), enc + (size_t)t * 256);
    }
    if (rd.over) atomicOr(status, SG_ST_CORRUPT);
    if (used) used[c] = (unsigned long long)(rd.p - (in + in_off[c]));           // rans.py's decode returns the bytes it read
}

}  // namespace sg

using namespace sg;

extern "C" int sg_rans_chain_encode(int device, void* stream, const unsigned char* sym, const void* ctx, int ctx_bytes,
                                    const unsigned long long* sym_off, int nchain, int ntab, const void* enc_tab, unsigned char* slots,
                                    const unsigned long long* slot_off, unsigned long long* out_len) {
    if (!sym || !ctx || !sym_off || !enc_tab || !slots || !slot_off || !out_len || nchain < 0 || ntab <= 0) return SG_ERR_ARG;
    if (ctx_bytes != 1 && ctx_bytes != 2 && ctx_bytes != 4) return SG_ERR_ARG;
    if ((uintptr_t)slots % 16) return SG_ERR_ALIGN;
    if (nchain == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned g = (unsigned)((nchain + 31) / 32);
    const RansSym* e = (const RansSym*)enc_tab;
    if (ctx_bytes == 1) k_chain_enc<uint8_t><<<g, 32, 0, st>>>(sym, (const uint8_t*)ctx, sym_off, nchain, ntab, e, slots, slot_off, out_len);
    else if (ctx_bytes == 2) k_chain_enc<uint16_t><<<g, 32, 0, st>>>(sym, (const uint16_t*)ctx, sym_off, nchain, ntab, e, slots, slot_off, out_len);
    else k_chain_enc<uint32_t><<<g, 32, 0, st>>>(sym, (const uint32_t*)ctx, sym_off, nchain, ntab, e, slots, slot_off, out_len);
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_rans_chain_decode(int device, void* stream, const unsigned char* in, const unsigned long long* in_off,
                                    const unsigned long long* in_end, const void* ctx, int ctx_bytes, const unsigned long long* sym_off,
                                    int nchain, int ntab, const void* enc_tab, const unsigned char* lut, unsigned char* sym_out,
                                    unsigned long long* used) {
    if (!in || !in_off || !in_end || !ctx || !sym_off || !enc_tab || !lut || !sym_out || nchain < 0 || ntab <= 0) return SG_ERR_ARG;
    if (ctx_bytes != 1 && ctx_bytes != 2 && ctx_bytes != 4) return SG_ERR_ARG;
    if ((uintptr_t)in % 16) return SG_ERR_ALIGN;
    if (nchain == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned g = (unsigned)((nchain + 31) / 32);
    const RansSym* e = (const RansSym*)enc_tab;
    int* sw = status_word(device);
    if (ctx_bytes == 1) k_chain_dec<uint8_t><<<g, 32, 0, st>>>(in, in_off, in_end, (const uint8_t*)ctx, sym_off, nchain, ntab, e, lut, sym_out, used, sw);
    else if (ctx_bytes == 2) k_chain_dec<uint16_t><<<g, 32, 0, st>>>(in, in_off, in_end, (const uint16_t*)ctx, sym_off, nchain, ntab, e, lut, sym_out, used, sw);
    else k_chain_dec<uint32_t><<<g, 32, 0, st>>>(in, in_off, in_end, (const uint32_t*)ctx, sym_off, nchain, ntab, e, lut, sym_out, used, sw);
    return cuda_ok(cudaGetLastError());
}
