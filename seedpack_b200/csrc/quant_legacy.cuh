// Legacy block formats: Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 and Q2_0 (32 or 64 weights per block).
//
// Without an importance matrix these are the *_ref routines (ggml-quants.c:74-299): one pass for the
// block extremum, one for the codes - memory-bound work.  With an importance matrix Q4_0/Q5_0 run
// make_qx_quants and Q4_1/Q5_1 run make_qkx3_quants per block (ggml-quants.c:2071-2279) with weights
// qw[j] * sqrt(sigma2 + x[j]^2), where sigma2 is the mean square of the WHOLE ROW - a strictly
// in-order fp32 sum over n_per_row terms, computed by k_row_meansq into a per-row scratch float
// before the block kernel runs.
//
// Mapping: one thread per block, 8 (Q2_0: 4) neighbouring lanes per 256-weight slab of a row.
#pragma once
#include "quant_k.cuh"

namespace sg {

// ---- row-wide mean square, in index order -------------------------------------------------------
// One warp per row.  The warp stages 256 weights at a time: every lane squares its 8 weights into
// shared memory, then lane 0 extends the single fp32 chain over the 256 squares in index order.
template <int DT>
__global__ void __launch_bounds__(128) k_row_meansq(const __grid_constant__ Job job, long long nrows_total) {
    __shared__ float sq[4][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 4 + warp;
    if (row >= nrows_total) return;
    int ti = 0;
    for (int i = 1; i < job.ntens; ++i) if (row >= job.t[i].row0) ti = i;
    const Tensor& t = job.t[ti];
    const long long x0 = t.xoff + (row - t.row0) * t.npr;
    float sum = 0.f;
    for (int c = 0; c < t.npr; c += 256) {
        const int n = min(256, t.npr - c);           // multiple of 32
        if (lane * 8 < n) {
            float v[8];
            Src<DT>::load8(job.x, x0 + c + lane * 8, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) sq[warp][lane * 8 + i] = fmul(v[i], v[i]);
        }
        __syncwarp();
        if (lane == 0) {
            for (int i = 0; i < n; i += 4) {
                const float4 q = *reinterpret_cast<const float4*>(&sq[warp][i]);
                sum = fadd(sum, q.x); sum = fadd(sum, q.y); sum = fadd(sum, q.z); sum = fadd(sum, q.w);
            }
        }
        __syncwarp();
    }
    if (lane == 0) job.rowstat[row] = fdiv(sum, (float)t.npr);      // sum_x2 / n_per_row
}

// ---- *_ref -----------------------------------------------------------------------------------------
SG_DEVINL int trunc_i8(float v) { return (int)(int8_t)(int)v; }      // (int8_t)(float) as x86 does it

template <int TYPE> struct LegacyRef;

template <> struct LegacyRef<SG_Q4_0> {
    static constexpr int QK = 32, BS = 18;
    static SG_DEVINL void block(const float (&x)[32], uint8_t* y) {
        float amax = 0.f, mx = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) if (amax < fabsf(x[j])) { amax = fabsf(x[j]); mx = x[j]; }
        const float d = fmul(mx, -0.125f);                 // max / -8
        const float id = d != 0.f ? frcp(d) : 0.0f;
        st2(y, f32_to_f16(d));
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            uint32_t w = 0;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int a = min(15, trunc_i8(fadd(fmul(x[j + k], id), 8.5f)));
                const int b = min(15, trunc_i8(fadd(fmul(x[16 + j + k], id), 8.5f)));
                w |= (uint32_t)(((a & 0xff) | (b << 4)) & 0xff) << (8 * k);
            }
            st2(y + 2 + j, w);
        }
    }
};
template <> struct LegacyRef<SG_Q4_1> {
    static constexpr int QK = 32, BS = 20;
    static SG_DEVINL void block(const float (&x)[32], uint8_t* y) {
        float mn = 3.402823466e+38F, mx = -3.402823466e+38F;
#pragma unroll
        for (int j = 0; j < 32; ++j) { if (x[j] < mn) mn = x[j]; if (x[j] > mx) mx = x[j]; }
        const float d = fdiv(fsub(mx, mn), c_div[DIV_15]);
        const float id = d != 0.f ? frcp(d) : 0.0f;
        st4(y, (uint32_t)f32_to_f16(d) | ((uint32_t)f32_to_f16(mn) << 16));
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            uint32_t w = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int a = min(15, trunc_i8(fadd(fmul(fsub(x[j + k], mn), id), 0.5f)));
                const int b = min(15, trunc_i8(fadd(fmul(fsub(x[16 + j + k], mn), id), 0.5f)));
                w |= (uint32_t)(((a & 0xff) | (b << 4)) & 0xff) << (8 * k);
            }
            st4(y + 4 + j, w);
        }
    }
};
template <> struct LegacyRef<SG_Q5_0> {
    static constexpr int QK = 32, BS = 22;
    static SG_DEVINL void block(const float (&x)[32], uint8_t* y) {
        float amax = 0.f, mx = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) if (amax < fabsf(x[j])) { amax = fabsf(x[j]); mx = x[j]; }
        const float d = fmul(mx, -0.0625f);                // max / -16
        const float id = d != 0.f ? frcp(d) : 0.0f;
        st2(y, f32_to_f16(d));
        uint32_t qh = 0;
        uint32_t qs[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t a = (uint32_t)min(31, trunc_i8(fadd(fmul(x[j], id), 16.5f))) & 0xff;
            const uint32_t b = (uint32_t)min(31, trunc_i8(fadd(fmul(x[16 + j], id), 16.5f))) & 0xff;
            qs[j >> 2] |= ((a & 0x0F) | ((b & 0x0F) << 4)) << (8 * (j & 3));
            qh |= ((a & 0x10u) >> 4) << j;
            qh |= ((b & 0x10u) >> 4) << (j + 16);
        }
        st4_a2(y + 2, qh);
#pragma unroll
        for (int m = 0; m < 4; ++m) st4_a2(y + 6 + 4 * m, qs[m]);
    }
};
template <> struct LegacyRef<SG_Q5_1> {
    static constexpr int QK = 32, BS = 24;
    static SG_DEVINL void block(const float (&x)[32], uint8_t* y) {
        float mn = 3.402823466e+38F, mx = -3.402823466e+38F;
#pragma unroll
        for (int j = 0; j < 32; ++j) { if (x[j] < mn) mn = x[j]; if (x[j] > mx) mx = x[j]; }
        const float d = fdiv(fsub(mx, mn), c_div[DIV_31]);
        const float id = d != 0.f ? frcp(d) : 0.0f;
        uint32_t qh = 0;
        uint32_t qs[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t a = (uint32_t)(int)fadd(fmul(fsub(x[j], mn), id), 0.5f) & 0xff;        // (uint8_t)(x0 + 0.5f)
            const uint32_t b = (uint32_t)(int)fadd(fmul(fsub(x[16 + j], mn), id), 0.5f) & 0xff;
            qs[j >> 2] |= ((a & 0x0F) | ((b & 0x0F) << 4)) << (8 * (j & 3));
            qh |= ((a & 0x10u) >> 4) << j;
            qh |= ((b & 0x10u) >> 4) << (j + 16);
        }
        st4(y, (uint32_t)f32_to_f16(d) | ((uint32_t)f32_to_f16(mn) << 16));
        st4(y + 4, qh);
#pragma unroll
        for (int m = 0; m < 4; ++m) st4(y + 8 + 4 * m, qs[m]);
    }
};
// (int)roundf(v) for |v| < 2^22 in five instructions: v + copysign(0.5, v) is exact except at |v| = 0.5 - 2^-25, where it
// rounds up to 1; that value, like everything below 0.5, rounds to 0.  NaN gives 0 (roundf's conversion gives INT_MIN on
// the reference's host, whose low byte is 0 too - only the low byte is used below).
SG_DEVINL int round_away_small(float v) {
    const int q = __float2int_rz(fadd(v, copysignf(0.5f, v)));
    return fabsf(v) < 0.5f ? 0 : q;
}
template <> struct LegacyRef<SG_Q8_0> {
    static constexpr int QK = 32, BS = 34;
    static SG_DEVINL void block(const float (&x)[32], uint8_t* y) {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
        const float d = fdiv(amax, c_div[DIV_127]);
        const float id = d != 0.f ? frcp(d) : 0.0f;
        st2(y, f32_to_f16(d));
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const int a = round_away_small(fmul(x[j], id)), b = round_away_small(fmul(x[j + 1], id));
            st2(y + 2 + j, (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8));
        }
    }
};
template <> struct LegacyRef<SG_Q2_0> {
    static constexpr int QK = 64, BS = 18;
    static SG_DEVINL void block(const float (&x)[64], uint8_t* y) {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) { const float a = fabsf(x[j]); if (a > amax) amax = a; }
        const float d = amax;
        const float id = d > 0.0f ? frcp(d) : 0.0f;
        st2(y, f32_to_f16(d));
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
            uint32_t w = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int q = clampi((int)roundf(fmul(x[j + k], id)) + 1, 0, 3);
                w |= (uint32_t)q << (2 * k);
            }
            st2(y + 2 + (j >> 2), w);
        }
    }
};

template <int TYPE> struct LegacyRefSlab {
    using R = LegacyRef<TYPE>;
    static constexpr int SLAB = 256, SUB = R::QK, LANES = 256 / R::QK, QK = R::QK, BS = R::BS;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid) {
        if (!valid || sub * SUB >= sl.n) return;
        float x[SUB];
        load_vals<DT, SUB>(job.x, sl.x + sub * SUB, x);
        R::block(x, job.y + out_offset<256, QK, BS>(sl, sub));
    }
};

// Memory-bound launch shape for the matrix-free legacy types: 128 blocks per CTA.  Each thread builds its block
// in shared memory; when the CTA's 128 blocks are one contiguous, 16-byte aligned run of the output (the usual
// case: full slabs of one tensor) the CTA then streams 128 * BS bytes out with 16-byte stores.  Blocks of
// 18..34 bytes written straight from the threads would cost up to 17 two-byte stores each.
template <int TYPE, int DT>
__global__ void __launch_bounds__(128) k_quant_legacy_ref(const __grid_constant__ Job job) {
    using R = LegacyRef<TYPE>;
    constexpr int QK = R::QK, BS = R::BS, LANES = 256 / QK;
    __shared__ __align__(16) uint8_t stage[128 * BS];
    __shared__ long long s_first;
    __shared__ int s_ok;
    const long long g = (long long)blockIdx.x * 128 + threadIdx.x;
    const long long s = g / LANES;
    const int sub = (int)(g - s * LANES);
    const bool valid = s < job.nslabs;
    bool live = false;
    long long yoff = 0;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (valid) {
        const Slab sl = locate<256>(job, s);
        live = sub * QK < sl.n;
        if (live) {
            yoff = out_offset<256, QK, BS>(sl, sub);
            float x[QK];
            load_vals<DT, QK>(job.x, sl.x + sub * QK, x);
            R::block(x, stage + threadIdx.x * BS);
        }
    }
    if (threadIdx.x == 0) s_first = yoff;
    __syncthreads();
    // contiguous run?  every thread's block must sit at first + tid * BS, and the run must start 16-byte aligned
    const bool mine = live && yoff == s_first + (long long)threadIdx.x * BS && ((s_first + (long long)(uintptr_t)job.y) & 15) == 0;
    if (!mine) s_ok = 0;
    __syncthreads();
    if (s_ok) {
        uint4* dst = reinterpret_cast<uint4*>(job.y + s_first);
        const uint4* src = reinterpret_cast<const uint4*>(stage);
        for (int i = threadIdx.x; i < 128 * BS / 16; i += 128) dst[i] = src[i];
    } else if (live) {
        uint8_t* y = job.y + yoff;
        const uint16_t* src = reinterpret_cast<const uint16_t*>(stage + threadIdx.x * BS);
        for (int i = 0; i < BS / 2; ++i) reinterpret_cast<uint16_t*>(y)[i] = src[i];
    }
}

// ---- importance-matrix paths -----------------------------------------------------------------------
template <int TYPE> struct LegacyImx {
    static constexpr int SLAB = 256, SUB = 32, LANES = 8, QK = 32;
    static constexpr int BS = TYPE == SG_Q4_0 ? 18 : TYPE == SG_Q4_1 ? 20 : TYPE == SG_Q5_0 ? 22 : 24;
    static constexpr bool HASMIN = TYPE == SG_Q4_1 || TYPE == SG_Q5_1;
    static constexpr bool FIVE = TYPE == SG_Q5_0 || TYPE == SG_Q5_1;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid) {
        if (!valid || sub * 32 >= sl.n) return;
        float x[32], wt[32];
        load_vals<DT, 32>(job.x, sl.x + sub * 32, x);
        load_f32<32>(job.w, sl.w + sub * 32, wt);
        const float sigma2 = job.rowstat[sl.grow];
#pragma unroll
        for (int j = 0; j < 32; ++j) wt[j] = fmul(wt[j], fsqrt(fadd(sigma2, fmul(x[j], x[j]))));
        uint8_t* y = job.y + out_offset<256, 32, BS>(sl, sub);
        uint32_t qs[4] = {0, 0, 0, 0};
        uint32_t qh = 0;
        uint32_t head;
        if (HASMIN) {
            const QkxBest b = make_qkx_quants<32, true>(FIVE ? 31 : 15, x, wt, -0.9f, 0.05f, 36, false);
            // m = -min where min = the_min returned (ggml-quants.c:2167): the_min = -min_internal
            head = (uint32_t)f32_to_f16(b.scale) | ((uint32_t)f32_to_f16(-b.the_min) << 16);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t a = (uint32_t)qkx_code<32, true>(b, FIVE ? 31 : 15, x[j]);
                const uint32_t c = (uint32_t)qkx_code<32, true>(b, FIVE ? 31 : 15, x[j + 16]);
                qs[j >> 2] |= ((a & 0x0F) | ((c & 0x0F) << 4)) << (8 * (j & 3));
                qh |= ((a & 0x10u) >> 4) << j;
                qh |= ((c & 0x10u) >> 4) << (j + 16);
            }
        } else {
            const QxBest b = make_qx_quants<32, true>(FIVE ? 16 : 8, x, wt);
            head = f32_to_f16(b.scale);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t a = (uint32_t)qx_code(b, FIVE ? 16 : 8, x[j]);
                const uint32_t c = (uint32_t)qx_code(b, FIVE ? 16 : 8, x[j + 16]);
                qs[j >> 2] |= ((a & 0x0F) | ((c & 0x0F) << 4)) << (8 * (j & 3));
                qh |= ((a & 0x10u) >> 4) << j;
                qh |= ((c & 0x10u) >> 4) << (j + 16);
            }
        }
        if (TYPE == SG_Q4_0) {
            st2(y, head);
#pragma unroll
            for (int m = 0; m < 4; ++m) st4_a2(y + 2 + 4 * m, qs[m]);
        } else if (TYPE == SG_Q4_1) {
            st4(y, head);
#pragma unroll
            for (int m = 0; m < 4; ++m) st4(y + 4 + 4 * m, qs[m]);
        } else if (TYPE == SG_Q5_0) {
            st2(y, head); st4_a2(y + 2, qh);
#pragma unroll
            for (int m = 0; m < 4; ++m) st4_a2(y + 6 + 4 * m, qs[m]);
        } else {
            st4(y, head); st4(y + 4, qh);
#pragma unroll
            for (int m = 0; m < 4; ++m) st4(y + 8 + 4 * m, qs[m]);
        }
    }
};

}  // namespace sg
