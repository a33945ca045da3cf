// Per-block residual of the stored quantised tensor against its prediction, on the device.
//
// Replaces the host NumPy helpers of the reference (seedpack/repo3.py:456-510): _xor_async / _xor_chunk
// (residual = file ^ prediction, "is anything left"), _diff_async (do they differ at all), _count_diff
// (bytes that differ - the score that picks a quantiser variant) and _xor3 (a ^ b ^ c and its non-zero
// byte count), plus the block-equality test the QR coder uses (same(), seedpack/qr.py:114-117).
// Keeping this on the GPU removes the device-to-host copy of every prediction that the reference needs
// before it can compare.
//
// Memory-bound: 16-byte loads and stores, a grid of a few CTAs per SM striding over the buffer, one
// atomic per CTA for the counters.
#include "api_util.h"

namespace sg {

__device__ __forceinline__ unsigned nz_bytes(unsigned v) {
    // number of non-zero bytes in a 32-bit word
    unsigned t = v | (v >> 4);
    t |= t >> 2;
    t |= t >> 1;
    return __popc(t & 0x01010101u);
}

template <bool HAVE_C, bool WRITE>
// `out` may be the same buffer as `a` (r ^= p in place): neither is declared restrict, and a kernel that writes reads
// `a` with ordinary loads, not through the read-only path
__global__ void __launch_bounds__(256) k_residual(const uint8_t* a, const uint8_t* __restrict__ b,
                                                  const uint8_t* __restrict__ c, uint8_t* out, size_t nbytes,
                                                  unsigned long long* __restrict__ counts, bool vec) {
    unsigned long long local = 0;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    size_t done = 0;
    if (vec) {
        const size_t nv = nbytes / 16;
        const uint4* av = reinterpret_cast<const uint4*>(a);
        const uint4* bv = reinterpret_cast<const uint4*>(b);
        const uint4* cv = reinterpret_cast<const uint4*>(c);
        uint4* ov = reinterpret_cast<uint4*>(out);
        for (size_t i = tid; i < nv; i += nth) {
            uint4 x = WRITE ? av[i] : __ldg(av + i);
            if (b) { const uint4 y = __ldg(bv + i); x.x ^= y.x; x.y ^= y.y; x.z ^= y.z; x.w ^= y.w; }
            if (HAVE_C) { const uint4 z = __ldg(cv + i); x.x ^= z.x; x.y ^= z.y; x.z ^= z.z; x.w ^= z.w; }
            if (WRITE) ov[i] = x;
            local += nz_bytes(x.x) + nz_bytes(x.y) + nz_bytes(x.z) + nz_bytes(x.w);
        }
        done = nv * 16;
    }
    for (size_t i = done + tid; i < nbytes; i += nth) {
        uint8_t x = a[i];
        if (b) x ^= b[i];
        if (HAVE_C) x ^= c[i];
        if (WRITE) out[i] = x;
        local += x != 0;
    }
    // CTA reduction, one atomic
    for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    __shared__ unsigned long long part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long s = 0;
        for (int i = 0; i < 8; ++i) s += part[i];
        if (s) atomicAdd(counts, s);
    }
}

// one thread per block of `bs` bytes (even): does the stored block equal the predicted one
__global__ void __launch_bounds__(256) k_block_ne(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, int bs,
                                                  long long nblocks, uint8_t* __restrict__ ne, unsigned long long* __restrict__ counts) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned differ = 0;
    if (i < nblocks) {
        const uint16_t* pa = reinterpret_cast<const uint16_t*>(a + (size_t)i * bs);
        const uint16_t* pb = reinterpret_cast<const uint16_t*>(b + (size_t)i * bs);
        unsigned acc = 0;
        for (int k = 0; k < bs / 2; ++k) acc |= (unsigned)(pa[k] ^ pb[k]);
        differ = acc != 0;
        if (ne) ne[i] = (uint8_t)differ;
    }
    const unsigned m = __ballot_sync(0xffffffffu, differ);
    __shared__ unsigned part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = __popc(m);
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned s = 0;
        for (int k = 0; k < 8; ++k) s += part[k];
        if (s) atomicAdd(counts, (unsigned long long)s);
    }
}

}  // namespace sg

using namespace sg;

extern "C" int sg_residual_xor(int device, void* stream, const void* a, const void* b, const void* c, void* out, size_t nbytes,
                               unsigned long long* d_nonzero) {
    if (!a || !d_nonzero || (c && !b)) return SG_ERR_ARG;
    if (nbytes == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = ((uintptr_t)a % 16 == 0) && (!b || (uintptr_t)b % 16 == 0) && (!c || (uintptr_t)c % 16 == 0) &&
                     (!out || (uintptr_t)out % 16 == 0);
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const size_t work = (nbytes / 16 + 255) / 256 + 1;
    const unsigned grid = (unsigned)(work < (size_t)sms * 8 ? work : (size_t)sms * 8);
    const uint8_t *pa = (const uint8_t*)a, *pb = (const uint8_t*)b, *pc = (const uint8_t*)c;
    uint8_t* po = (uint8_t*)out;
    if (c) {
        if (out) k_residual<true, true><<<grid, 256, 0, st>>>(pa, pb, pc, po, nbytes, d_nonzero, vec);
        else     k_residual<true, false><<<grid, 256, 0, st>>>(pa, pb, pc, po, nbytes, d_nonzero, vec);
    } else {
        if (out) k_residual<false, true><<<grid, 256, 0, st>>>(pa, pb, pc, po, nbytes, d_nonzero, vec);
        else     k_residual<false, false><<<grid, 256, 0, st>>>(pa, pb, pc, po, nbytes, d_nonzero, vec);
    }
    return cuda_ok(cudaGetLastError());
}

extern "C" int sg_residual_blocks(int device, void* stream, const void* file, const void* pred, int block_bytes, long long nblocks,
                                  unsigned char* ne_flags, unsigned long long* d_differ) {
    if (!file || !pred || !d_differ || block_bytes <= 0 || (block_bytes & 1) || nblocks < 0) return SG_ERR_ARG;
    if (((uintptr_t)file | (uintptr_t)pred) & 1) return SG_ERR_ALIGN;
    if (nblocks == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    const long long grid = (nblocks + 255) / 256;
    if (grid > 0x7fffffffLL) return SG_ERR_LIMIT;
    k_block_ne<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)file, (const uint8_t*)pred, block_bytes, nblocks,
                                                                ne_flags, d_differ);
    return cuda_ok(cudaGetLastError());
}
