// IQ quantisers: IQ4_NL / IQ4_XS (non-uniform 16-level codebook), the lattice types IQ2_XXS, IQ2_XS,
// IQ2_S, IQ3_XXS, IQ3_S (grid + neighbour-list search) and the ternary IQ1_S / IQ1_M (sorted
// two-boundary split search).
//
// Mapping: one thread per block of 32 or 16 weights, the 8 or 16 threads of a super-block are
// neighbouring lanes of a warp; super-block quantities (in-order sum of squares, maximum scale, the
// packed scale nibbles) travel by warp shuffle.  Per-thread block data that is indexed dynamically
// (sign-folded values, weights, sort order) lives in shared memory laid out [element][thread], so
// a warp's accesses hit 32 different banks.
//
// Reference arithmetic: ggml-quants.c:4938-5047 (IQ4), 3271-3651 (IQ2_XXS/XS), 5114-5281 (IQ2_S),
// 3915-4351 (IQ3_XXS/S), 4444-4671 (IQ1_S), 4693-4916 (IQ1_M); the IQ1_M variant 1 is the direct-sum
// split search of the pre-f95b0d9539 llama.cpp sources.
#pragma once
#include <type_traits>

#include "api_util.h"
#include "quant_k.cuh"

namespace sg {

// ---- device-resident tables ----------------------------------------------------------------------
struct GridTable {
    const void* grid;            // uint64 (IQ2 family, 8 int8 per point) or uint32 (IQ3 family, 4 int8)
    const int* map;              // >= 0: grid index, < 0: -(offset into neighbours) - 1
    const uint16_t* neighbours;  // [count, indices...] lists
    const uint16_t* keys;        // per point: its levels packed as a map index (2 bits x 8 or 3 bits x 4)
    const uint16_t* nbkeys;      // the neighbour lists with keys in place of point indices, padded by 64 entries
    int nb_size, map_size;       // entries of neighbours / map
};
// index: 0 IQ2_XXS (256), 1 IQ2_XS (512), 2 IQ1_S/IQ1_M (2048), 3 IQ2_S (1024), 4 IQ3_XXS (256), 5 IQ3_S (512)
struct IqTables { GridTable t[6]; };

static __constant__ int8_t c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};


// ==================================================================================================
// IQ4_NL / IQ4_XS
// best_index_int8(16, kvalues_iq4nl, x), ggml-quants.c:28-37.  The search of the C code ends with val[ml] <= x < val[ml + 1]
// (its two early returns fall out of the same formula with ml clamped to 14), so ml is the largest index whose level
// is <= x: four halving steps over the 16-entry table in shared memory (16 distinct banks: a warp's lookups never
// conflict).  Returns the index, *q = its level.
SG_DEVINL int best_index_iq4(float x, const float* __restrict__ kv, float* q) {
    int ml = x >= kv[8] ? 8 : 0;
    ml += x >= kv[ml + 4] ? 4 : 0;
    ml += x >= kv[ml + 2] ? 2 : 0;
    ml += x >= kv[ml + 1] ? 1 : 0;
    if (ml > 14 || x != x) ml = 14;                        // NaN: every `x < val` test of the search fails
    const float a = kv[ml], b = kv[ml + 1];
    const bool lower = fsub(x, a) < fsub(b, x);
    *q = lower ? a : b;
    return lower ? ml : ml + 1;
}

template <bool XS> struct IQ4 {
    static constexpr int SLAB = 256, SUB = 32, LANES = 8, QK = XS ? 256 : 32, BS = XS ? 136 : 18;
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid, const float* __restrict__ kv) {
        const bool live = valid && sub * 32 < sl.n;
        float x[32], wt[32];
        if (live || XS) load_vals<DT, 32>(job.x, sl.x + sub * 32, x);
        else {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = 0.f;
        }
        float sigma2;
        if (XS) {
            sigma2 = ordered_sumsq<32, 8>(x, sub);
            sigma2 = fmul(sigma2, 2.f / 256);
        } else {
            sigma2 = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) sigma2 = fadd(sigma2, fmul(x[j], x[j]));
            sigma2 = fmul(sigma2, 2.f / 32);
        }
        if (IMX) {
            if (live || XS) load_f32<32>(job.w, sl.w + sub * 32, wt);
#pragma unroll
            for (int j = 0; j < 32; ++j) wt[j] = fmul(wt[j], fsqrt(fadd(sigma2, fmul(x[j], x[j]))));
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) wt[j] = fmul(x[j], x[j]);
        }
        float amax = 0.f, mx = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) { const float ax = fabsf(x[j]); if (ax > amax) { amax = ax; mx = x[j]; } }
        float d = 0.f;
        const float v0 = kv[0];                       // -127, read at run time: the division below must stay a division
        if (!(amax < SG_GROUP_MAX_EPS)) {
            d = fdiv(-mx, v0);                        // ntry > 0: -max / values[0]
            float id = frcp(d);
            float sumqx = 0.f, sumq2 = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float q;
                best_index_iq4(fmul(id, x[j]), kv, &q);
                sumqx = fadd(sumqx, fmul(fmul(wt[j], q), x[j]));
                sumq2 = fadd(sumq2, fmul(fmul(wt[j], q), q));
            }
            d = sumq2 > 0.f ? fdiv(sumqx, sumq2) : 0.f;
            float best = fmul(d, sumqx);
#pragma unroll 1
            for (int itry = -7; itry <= 7; ++itry) {
                id = fdiv((float)(itry - 127), mx);
                sumqx = 0.f; sumq2 = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float q;
                    best_index_iq4(fmul(id, x[j]), kv, &q);
                    sumqx = fadd(sumqx, fmul(fmul(wt[j], q), x[j]));
                    sumq2 = fadd(sumq2, fmul(fmul(wt[j], q), q));
                }
                if (sumq2 > 0.f && fmul(sumqx, sumqx) > fmul(best, sumq2)) { d = fdiv(sumqx, sumq2); best = fmul(d, sumqx); }
            }
        }
        // d is scales[ib]
        float idl;
        uint16_t dh;
        int l6 = 0;
        if (XS) {
            float scales[8];
            gather<8>(d, scales);
            float max_scale = 0.f, amax_scale = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float a = fabsf(scales[j]); if (a > amax_scale) { amax_scale = a; max_scale = scales[j]; } }
            const float dd = fmul(-max_scale, 1.0f / 32);
            dh = f32_to_f16(dd);
            const float id = dd != 0.f ? frcp(dd) : 0.f;
            int l = clampi(nearest_int(fmul(id, d)), -32, 31);
            const float dl = fmul(dd, (float)l);
            idl = dl != 0.f ? frcp(dl) : 0.f;
            l6 = l + 32;
        } else {
            dh = f32_to_f16(d);
            idl = d != 0.f ? frcp(d) : 0.f;
        }
        uint32_t qs[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float qa, qb;
            const uint32_t a = (uint32_t)best_index_iq4(fmul(idl, x[j]), kv, &qa);
            const uint32_t b = (uint32_t)best_index_iq4(fmul(idl, x[j + 16]), kv, &qb);
            qs[j >> 2] |= (a | (b << 4)) << (8 * (j & 3));
        }
        if (XS) {
            // block_iq4_xs: d, scales_h (u16), scales_l[4], qs[128]
            unsigned l6s[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) l6s[j] = (unsigned)gshfl<8>(l6, j);
            if (!valid) return;
            uint8_t* y = job.y + out_offset<256, 256, 136>(sl, 0);
            if (sub == 0) {
                uint32_t sh = 0, slw = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    sh |= (l6s[j] >> 4) << (2 * j);
                    slw |= (l6s[j] & 0xf) << (4 * j);
                }
                st4(y, (uint32_t)dh | ((sh & 0xffff) << 16));
                st4(y + 4, slw);
            }
            uint8_t* p = y + 8 + 16 * sub;
            st4(p, qs[0]); st4(p + 4, qs[1]); st4(p + 8, qs[2]); st4(p + 12, qs[3]);
        } else {
            if (!live) return;
            uint8_t* y = job.y + out_offset<256, 32, 18>(sl, sub);
            st2(y, dh);
#pragma unroll
            for (int m = 0; m < 4; ++m) st4_a2(y + 2 + 4 * m, qs[m]);
        }
    }
};

// ==================================================================================================
// Lattice types.  Values that are indexed dynamically live in shared memory as [element][thread]; TPB is the
// CTA size of the kernel that owns the storage.
template <int BLK, int TPB, int NTERM> struct IqSmem {
    float xval[BLK][TPB];         // sign-folded values
    float waux[BLK][TPB];         // sqrt(weight): the weights of the neighbour search
    float term[NTERM][TPB];       // three-level lattices: the list walker's distance terms, [4 * weight + level]
};

// codes of up to 8 groups, 16 bits per group (the group's map index u)
struct Codes {
    unsigned long long a, b;
    SG_DEVINL Codes() : a(0), b(0) {}
    SG_DEVINL unsigned get(int k) const { return (unsigned)((k < 4 ? a : b) >> (16 * (k & 3))) & 0xffffu; }
    SG_DEVINL void set(int k, unsigned u) {
        const int sh = 16 * (k & 3);
        if (k < 4) a = (a & ~(0xffffull << sh)) | ((unsigned long long)u << sh);
        else       b = (b & ~(0xffffull << sh)) | ((unsigned long long)u << sh);
    }
};

// TYPE-specific constants of the five lattice quantisers
template <int TYPE> struct Lat;
template <> struct Lat<SG_IQ2_XXS> { static constexpr int BLK = 32, G = 8, CB = 2, KMAXQ = 3, TAB = 0, BS = 66, IS0 = -6, IS1 = 6; static constexpr bool PARITY = true; };
template <> struct Lat<SG_IQ2_XS>  { static constexpr int BLK = 16, G = 8, CB = 2, KMAXQ = 3, TAB = 1, BS = 74, IS0 = -9, IS1 = 9; static constexpr bool PARITY = true; };
template <> struct Lat<SG_IQ2_S>   { static constexpr int BLK = 16, G = 8, CB = 2, KMAXQ = 3, TAB = 3, BS = 82, IS0 = -9, IS1 = 9; static constexpr bool PARITY = false; };
template <> struct Lat<SG_IQ3_XXS> { static constexpr int BLK = 32, G = 4, CB = 3, KMAXQ = 8, TAB = 4, BS = 98, IS0 = -15, IS1 = 15; static constexpr bool PARITY = true; };
template <> struct Lat<SG_IQ3_S>   { static constexpr int BLK = 32, G = 4, CB = 3, KMAXQ = 8, TAB = 5, BS = 110, IS0 = -9, IS1 = 9; static constexpr bool PARITY = false; };

// what a search reads: tuple -> point index or list, and the lists themselves (keys in place of point indices).
// MapT is int (tables in global memory) or int16_t (the IQ3 tables copied into shared memory; their offsets fit).
template <class MapT> struct TabView {
    const MapT* map;
    const uint16_t* nbk;
    unsigned key0;               // levels of point 0: what a search that found nothing falls back to
};

// Work queue of a CTA.  Neighbour lists run from one entry to a few hundred, so a warp whose lanes each walked the
// list of their own block would wait for its longest list.  Instead every thread registers the groups of its block
// that fell off the lattice, the queue is ordered by list length (a counting sort over length classes, longest
// first), and the CTA's threads then take queue entries side by side: the lanes of a warp walk lists of equal
// length, whichever blocks they belong to.  Results go back through u[][].
constexpr int ilog2_ce(int v) { return v <= 1 ? 0 : 1 + ilog2_ce((v + 1) / 2); }     // bits that hold 0 .. v-1
template <int TPB, int NS, int R> struct WorkQueue {
    static constexpr int RANK_BITS = ilog2_ce(TPB * NS), CLS_BITS = 16 - RANK_BITS;
    static constexpr int NCLS = CLS_BITS >= 5 ? 32 : (1 << CLS_BITS);
    uint16_t u[NS][TPB];          // codes of every block's groups, one slot per (candidate scale, group)
    uint16_t rank[NS][TPB];       // class << RANK_BITS | position inside the class; 0xffff = nothing to search
    uint16_t item[NS * TPB];      // the ordered queue: thread * NS + slot
    float scale[R][TPB];          // the candidate scales each block is searched at
    uint8_t flag[TPB];            // per block, for the kernel's use
    int count[32], base[32], total;

    // every lane of the warp calls this once per slot k; off: the group needs a search of a list of n entries,
    // lists of up to 2^cshift entries more or less count as equally long
    SG_DEVINL void put(int k, unsigned codes, bool off, int n, int cshift) {
        const int tid = threadIdx.x, lane = tid & 31;
        u[k][tid] = (uint16_t)codes;
        int cls = -1;
        if (off) { cls = (n + (1 << cshift) - 1) >> cshift; cls = cls > NCLS - 2 ? NCLS - 2 : cls; }
        const unsigned peers = __match_any_sync(SG_FULL, cls);
        unsigned r = 0xffffu;
        if (off) {
            const int leader = __ffs(peers) - 1;
            int b = 0;
            if (lane == leader) b = atomicAdd(&count[cls], __popc(peers));
            b = __shfl_sync(peers, b, leader);
            r = (unsigned)cls << RANK_BITS | (unsigned)(b + __popc(peers & ((1u << lane) - 1)));
        }
        rank[k][tid] = (uint16_t)r;
    }
    // all threads of the CTA, after their puts into slots 0 .. ns-1: orders the queue, returns its length
    SG_DEVINL int sort(int ns) {
        const int tid = threadIdx.x;
        __syncthreads();
        if (tid == 0) {
            int acc = 0;
            for (int c = NCLS - 1; c >= 0; --c) { base[c] = acc; acc += count[c]; count[c] = 0; }
            total = acc;
        }
        __syncthreads();
#pragma unroll 1
        for (int k = 0; k < ns; ++k) {
            const unsigned r = rank[k][tid];
            if (r != 0xffffu) item[base[r >> RANK_BITS] + (int)(r & ((1u << RANK_BITS) - 1))] = (uint16_t)(tid * NS + k);
        }
        __syncthreads();
        return total;
    }
};

// exact float of a small non-negative integer without the conversion pipe: 0x4b000000 is 8388608.0f
SG_DEVINL float small_to_float(unsigned v) { return fsub(__int_as_float(0x4b000000u | v), 8388608.f); }

// iq3_find_best_neighbour (ggml-quants.c:3915-3937) over a list of keys in shared memory, for the group of 4 weights
// of thread column t2 that starts at element e0.  Four entries at a time (independent distance chains, each added
// up in index order), compared in list order so that the first strictly smaller distance wins as in the C loop.
// Reads up to three entries past the list's end, which the padding of the key lists allows.
template <int BLK, int TPB, int NTERM>
SG_DEVINL unsigned search_list4(const uint16_t* nbk, int list, float scale, int e0, const IqSmem<BLK, TPB, NTERM>& sm, int t2, unsigned key0, int* status) {
    const uint16_t* nb = nbk + list;
    const int n = nb[0];
    float xv[4], wv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { xv[i] = sm.xval[e0 + i][t2]; wv[i] = sm.waux[e0 + i][t2]; }
    float best = 3.402823466e+38F;
    unsigned bu = 0xffffffffu;
#pragma unroll 1
    for (int j = 0; j < n; j += 4) {
        unsigned key[4];
        float d[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) key[q] = nb[1 + j + q];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float d2 = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float lv = small_to_float(2 * ((key[q] >> (3 * i)) & 7u) + 1);
                const float diff = fsub(fmul(scale, lv), xv[i]);
                d2 = fadd(d2, fmul(fmul(wv[i], diff), diff));
            }
            d[q] = d2;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (j + q < n && d[q] < best) { best = d[q]; bu = key[q]; }
    }
    if (bu == 0xffffffffu) { atomicOr(status, SG_ST_OFFGRID); bu = key0; }
    return bu;
}

// iq2_find_best_neighbour (ggml-quants.c:3271-3293) and iq1_find_best_neighbour2 (4444-4499) over a list of keys in
// global memory, for 8 weights with three levels each.  xs / ws: the group's values and weights, [8][TPB], column
// t2; sq[c]: scale times the value of level c.  The 24 possible terms w * (sq[c] - x)^2 go into the calling
// thread's own column of `term` first; a distance is then 8 looked-up terms added in index order.
template <int TPB>
SG_DEVINL unsigned search_list8(const uint16_t* __restrict__ nbk, int list, const float (&sq)[3], const float (*xs)[TPB], const float (*ws)[TPB],
                                int t2, float (*term)[TPB], unsigned key0, int* status) {
    const int tid = threadIdx.x;
    const uint16_t* nb = nbk + list;
    const int n = __ldg(nb);
    unsigned key[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) key[q] = __ldg(nb + 1 + q);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x = xs[i][t2], w = ws[i][t2];
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            const float d = fsub(sq[c], x);
            term[4 * i + c][tid] = fmul(fmul(w, d), d);
        }
    }
    float best = 3.402823466e+38F;
    unsigned bu = 0xffffffffu;
#pragma unroll 1
    for (int j = 0; j < n; j += 4) {
        float d[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float d2 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) d2 = fadd(d2, term[4 * i + (int)((key[q] >> (2 * i)) & 3u)][tid]);
            d[q] = d2;
        }
        unsigned nk[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) nk[q] = __ldg(nb + 5 + j + q);          // the padding covers the overrun
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (j + q < n && d[q] < best) { best = d[q]; bu = key[q]; }
#pragma unroll
        for (int q = 0; q < 4; ++q) key[q] = nk[q];
    }
    if (bu == 0xffffffffu) { atomicOr(status, SG_ST_OFFGRID); bu = key0; }
    return bu;
}

// sumqx / sumq2 over the block in index order with q = 2*L + 1
template <int BLK, int G, int CB, class SM>
SG_DEVINL void block_sums(const Codes& c, const float (&wgt)[BLK], const SM& sm, int tid, float& sumqx, float& sumq2) {
    sumqx = 0.f; sumq2 = 0.f;
#pragma unroll
    for (int k = 0; k < BLK / G; ++k) {
        const unsigned u = c.get(k);
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const float q = small_to_float(2 * ((u >> (CB * i)) & ((1u << CB) - 1)) + 1);
            const float w = wgt[k * G + i];
            sumqx = fadd(sumqx, fmul(fmul(w, sm.xval[k * G + i][tid]), q));
            sumq2 = fadd(sumq2, fmul(fmul(w, q), q));
        }
    }
}

template <int TYPE> struct Lattice {
    using P = Lat<TYPE>;
    static constexpr int SLAB = 256, SUB = P::BLK, LANES = 256 / P::BLK, QK = 256, BS = P::BS;
    static constexpr int BLK = P::BLK, G = P::G, CB = P::CB, NG = BLK / G, KMAXQ = P::KMAXQ;
    static constexpr int TYPE_ID = TYPE, TAB = P::TAB;
    static constexpr bool SMEM_TABLES = G == 4;      // IQ3: map 4096 entries, lists < 29 K entries
    static constexpr int TPB = SMEM_TABLES ? 512 : 256, NTERM = G == 8 ? 32 : 1;
    using MapT = typename std::conditional<SMEM_TABLES, int16_t, int>::type;
    using View = TabView<MapT>;
    using SM = IqSmem<BLK, TPB, NTERM>;
    static constexpr int R = 8 / NG;                 // candidate scales searched per pass over the queue (8 slots a block)
    using Q = WorkQueue<TPB, 8, R>;

    // nr candidate scales for every block of the CTA.  cand(r, id, sc, want) describes candidate r of a block: all
    // its groups are rounded with inverse scale id and looked up; those that fell off the lattice and are wanted
    // (`want`, one bit per group) are searched through the CTA's queue at scale sc; each thread then reads its
    // block's codes back into aux[r].  on: bit r * NG + k is set where group k of candidate r was on the lattice.
    template <class F>
    static SG_DEVINL void queue_round(const View& T, SM& sm, Q& q, int nr, F cand, Codes (&aux)[R], unsigned& on, int* status) {
        const int tid = threadIdx.x;
        on = 0;
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            float id, sc;
            unsigned want;
            cand(r, id, sc, want);
            q.scale[r][tid] = sc;
#pragma unroll 1
            for (int k = 0; k < NG; ++k) {
                unsigned u = 0;
#pragma unroll
                for (int i = 0; i < G; ++i) {
                    const int l = nearest_int(fmul(0.5f, fsub(fmul(id, sm.xval[G * k + i][tid]), 1.f)));
                    u |= (unsigned)clampi(l, 0, KMAXQ - 1) << (CB * i);
                }
                const int gi = T.map[u];
                if (gi >= 0) on |= 1u << (r * NG + k);
                const bool off = ((want >> k) & 1) && gi < 0;
                q.put(r * NG + k, u, off, off ? (int)T.nbk[-gi - 1] : 0, G == 4 ? 2 : 3);
            }
        }
        const int total = q.sort(nr * NG);
#pragma unroll 1
        // the queue runs from long lists to short ones: threads take it back and forth (0 .. TPB-1, TPB-1 .. 0, ...), so
        // that no warp collects the longest entry of every turn
        for (int p0 = 0, turn = 0; p0 < total; p0 += TPB, ++turn) {
            const int p = p0 + ((turn & 1) ? TPB - 1 - tid : tid);
            if (p >= total) continue;
            const unsigned it = q.item[p];
            const int t2 = (int)(it >> 3), slot = (int)(it & 7), k = slot % NG;
            const int list = -(int)T.map[q.u[slot][t2]] - 1;
            const float s1 = q.scale[slot / NG][t2];
            unsigned res;
            if constexpr (G == 4) res = search_list4(T.nbk, list, s1, G * k, sm, t2, T.key0, status);
            else {
                const float sq[3] = {s1, fmul(s1, 3.f), fmul(s1, 5.f)};
                res = search_list8<TPB>(T.nbk, list, sq, &sm.xval[G * k], &sm.waux[G * k], t2, sm.term, T.key0, status);
            }
            q.u[slot][t2] = (uint16_t)res;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int k = 0; k < NG; ++k) aux[r].set(k, q.u[r * NG + k][tid]);
    }

    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid, const View& T, SM& sm, Q& q) {
        const int tid = threadIdx.x;
        float wgt[BLK];
        float scale = 0.f;                 // scales[ib]
        Codes L;
        unsigned signs[4] = {0, 0, 0, 0};  // block_signs[k], per group of 8 weights
        bool wrote = false;                // did this block reach the code-emitting tail (else its bytes stay zero)
        {
            float x[BLK];
            load_vals<DT, BLK>(job.x, sl.x + sub * BLK, x);
            const float sumx2 = ordered_sumsq<BLK, LANES>(x, sub);
            const float sigma2 = TYPE == SG_IQ2_XXS || TYPE == SG_IQ2_XS ? fmul(sumx2, 1.0f / 256)
                                                                         : fmul(fmul(2.f, sumx2), 1.0f / 256);
            float qw[BLK];
            if (IMX) load_f32<BLK>(job.w, sl.w + sub * BLK, qw);
#pragma unroll
            for (int i = 0; i < BLK; ++i) {
                float w;
                if (IMX) w = fmul(qw[i], fsqrt(fadd(sigma2, fmul(x[i], x[i]))));
                else if (TYPE == SG_IQ2_S) w = fadd(fmul(0.25f, sigma2), fmul(x[i], x[i]));
                else w = fmul(x[i], x[i]);
                wgt[i] = w;
                sm.waux[i][tid] = fsqrt(w);
            }
            // sign folding (ggml-quants.c:3341-3362): groups of 8; with PARITY an odd number of flips is repaired
            // by un-flipping the weight with the smallest w*x*x (first minimum)
#pragma unroll
            for (int k = 0; k < BLK / 8; ++k) {
                int nflip = 0;
                unsigned s = 0;
                float xv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float v = x[8 * k + i];
                    if (v >= 0.f) xv[i] = v;
                    else { xv[i] = -v; ++nflip; s |= 1u << i; }
                }
                if (P::PARITY) {
                    if (nflip & 1) {
                        int imin = 0;
                        float mn = fmul(fmul(wgt[8 * k], x[8 * k]), x[8 * k]);
#pragma unroll
                        for (int i = 1; i < 8; ++i) {
                            const float ax = fmul(fmul(wgt[8 * k + i], x[8 * k + i]), x[8 * k + i]);
                            if (ax < mn) { mn = ax; imin = i; }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) if (i == imin) xv[i] = -xv[i];
                        s ^= 1u << imin;
                    }
                    s &= 127;
                }
                signs[k] = s;
#pragma unroll
                for (int i = 0; i < 8; ++i) sm.xval[8 * k + i][tid] = xv[i];
            }
        }
        float mx = sm.xval[0][tid];
#pragma unroll
        for (int i = 1; i < BLK; ++i) mx = fmaxf(mx, sm.xval[i][tid]);
        const float eps = TYPE == SG_IQ3_XXS ? 1e-8f : TYPE == SG_IQ2_S ? 1e-8f : SG_GROUP_MAX_EPS;
        const bool dead = TYPE == SG_IQ3_S ? !(mx != 0.f) : (mx < eps);
        const float c2k1 = (float)(2 * KMAXQ - 1);
        // Every thread runs the candidate loop, because the neighbour searches inside it go through the CTA's queue;
        // `act` marks the threads whose block is really being searched.
        bool act = !dead;
        float best = 0.f;
        float rng = 1.f;                     // denominator of the candidate inverse scales
        unsigned ongrid = TYPE == SG_IQ3_S ? 0u : 0xffu;
        if (act) {
            if (TYPE == SG_IQ2_XXS) {
                float xv[32], wv[32];
                int Lq[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) { xv[i] = sm.xval[i][tid]; wv[i] = wgt[i]; }
                scale = make_qp_quants<32>(KMAXQ + 1, xv, Lq, wv);
                rng = fmul(scale, (float)KMAXQ);       // eff_max
                if (rng <= 0.f) act = false;
            } else {
                rng = mx;
                scale = fdiv(mx, TYPE == SG_IQ2_XS || TYPE == SG_IQ2_S ? c_div[DIV_5] : c_div[DIV_15]);
            }
        }
        {
            const float step = (TYPE == SG_IQ3_XXS || TYPE == SG_IQ3_S) ? 0.2f : 0.1f;
            constexpr unsigned ALL = (1u << NG) - 1;
#pragma unroll 1
            for (int is0 = P::IS0; is0 <= P::IS1; is0 += R) {
                const int nr = P::IS1 - is0 + 1 < R ? P::IS1 - is0 + 1 : R;
                Codes aux[R];
                unsigned on;
                queue_round(T, sm, q, nr, [&](int r, float& id, float& sc, unsigned& want) {
                    id = fdiv(fadd(c2k1, fmul((float)(is0 + r), step)), rng);
                    sc = frcp(id);
                    want = act ? ALL : 0u;
                }, aux, on, job.status);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r >= nr) break;
                    float sumqx, sumq2;
                    block_sums<BLK, G, CB>(aux[r], wgt, sm, tid, sumqx, sumq2);
                    if (act && sumq2 > 0.f && fmul(sumqx, sumqx) > fmul(best, sumq2)) {
                        scale = fdiv(sumqx, sumq2); best = fmul(scale, sumqx);
                        L = aux[r]; ongrid = (on >> (r * NG)) & ALL;
                    }
                }
            }
            // second pass at the winning scale
            bool refit;
            if (TYPE == SG_IQ2_XXS) refit = act && scale > 0.f;
            else {
                refit = act && (ongrid & ALL) != ALL && scale > 0.f;
            }
            if (__syncthreads_or(refit)) {
                unsigned want0 = 0;
                if (refit) want0 = (TYPE == SG_IQ2_XS || TYPE == SG_IQ2_S || TYPE == SG_IQ3_XXS) ? ~ongrid & ALL : ALL;
                Codes aux[R];
                unsigned on;
                const float win = scale;
                queue_round(T, sm, q, 1, [&](int, float& id, float& sc, unsigned& want) { id = frcp(win); sc = win; want = want0; }, aux, on, job.status);
#pragma unroll
                for (int k = 0; k < NG; ++k) if ((want0 >> k) & 1) L.set(k, aux[0].get(k));     // on the grid the codes ARE the grid point
                if (refit) {
                    float sumqx, sumq2;
                    block_sums<BLK, G, CB>(L, wgt, sm, tid, sumqx, sumq2);
                    if (sumq2 > 0.f) scale = fdiv(sumqx, sumq2);
                }
            }
            if (act) {
                if (scale < 0.f) {
                    scale = -scale;
                    if (P::PARITY) {
#pragma unroll
                        for (int k = 0; k < (TYPE == SG_IQ2_XS ? 2 : 4); ++k) signs[k] = (~signs[k]) & 127;
                    } else {
#pragma unroll
                        for (int k = 0; k < BLK / 8; ++k) signs[k] = (~signs[k]) & 0xff;
                    }
                }
                wrote = true;
            }
        }
        if (!wrote) scale = 0.f;
        // grid indices of the final codes
        unsigned gidx[NG];
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            int gi = wrote ? (int)T.map[L.get(k)] : 0;
            if (gi < 0) { atomicOr(job.status, SG_ST_OFFGRID); gi = 0; }
            gidx[k] = (unsigned)gi;
        }
        // super-block scale
        float scales[LANES];
        gather<LANES>(scale, scales);
        float max_scale = 0.f;
#pragma unroll
        for (int j = 0; j < LANES; ++j) max_scale = fmaxf(max_scale, scales[j]);
        const bool nz = max_scale != 0.f;
        const float d = fdiv(max_scale, c_div[DIV_31]);
        const float fudge = TYPE == SG_IQ3_XXS ? 1.0125f : TYPE == SG_IQ3_S ? 1.033f : TYPE == SG_IQ2_S ? 0.9875f : 1.0f;
        const uint16_t dh = nz ? f32_to_f16(fudge == 1.0f ? d : fmul(d, fudge)) : f32_to_f16(0.f);
        int l4 = 0;
        if (nz) l4 = clampi(nearest_int(fmul(0.5f, fsub(fmul(frcp(d), scale), 1.f))), 0, 15);
        const unsigned l4n = (unsigned)__shfl_xor_sync(SG_FULL, l4, 1);     // partner's nibble
        unsigned qh_bits = 0;                 // this block's contribution to the shared high-bit bytes
        if (TYPE == SG_IQ2_S) qh_bits = (gidx[0] >> 8) | ((gidx[1] >> 8) << 2);       // 4 bits
        const unsigned qh_n = (unsigned)__shfl_xor_sync(SG_FULL, (int)qh_bits, 1);
        // IQ3_S advances its qs / signs cursors only for blocks that were coded (ggml-quants.c:4241-4243 `continue`
        // skips `qs += bs4; signs += bs8` at 4327-4329), so coded blocks are packed towards the front and the
        // tail stays zero; qh keeps absolute positions.
        int slot = sub;
        if (TYPE == SG_IQ3_S) {
            const unsigned lanebase = (threadIdx.x & 31) & ~7u;
            const unsigned m = (__ballot_sync(SG_FULL, wrote) >> lanebase) & 0xffu;
            const unsigned below = (1u << sub) - 1;
            slot = wrote ? __popc(m & below) : __popc(m) + __popc(~m & below);
        }
        if (!valid) return;
        uint8_t* y = job.y + out_offset<256, 256, BS>(sl, 0);
        if (sub == 0) st2(y, dh);
        if (TYPE == SG_IQ2_XXS) {
            uint32_t w0 = 0, w1 = 0;
            if (nz && wrote) {
                w0 = gidx[0] | (gidx[1] << 8) | (gidx[2] << 16) | (gidx[3] << 24);
                w1 = signs[0] | (signs[1] << 7) | (signs[2] << 14) | (signs[3] << 21);
            }
            if (nz) w1 |= (uint32_t)l4 << 28;
            st4_a2(y + 2 + 8 * sub, w0); st4_a2(y + 6 + 8 * sub, w1);
        } else if (TYPE == SG_IQ2_XS) {
            uint32_t w0 = 0;
            if (nz && wrote) w0 = (gidx[0] | (signs[0] << 9)) | ((gidx[1] | (signs[1] << 9)) << 16);
            st4_a2(y + 2 + 4 * sub, w0);
            if (!(sub & 1)) y[66 + (sub >> 1)] = (uint8_t)(nz ? (l4 | (l4n << 4)) : 0);
        } else if (TYPE == SG_IQ2_S) {
            // block_iq2_s: d, qs[64] (32 grid bytes + 32 sign bytes), qh[8], scales[8]
            st2(y + 2 + 2 * sub, wrote ? ((gidx[0] & 255) | ((gidx[1] & 255) << 8)) : 0);
            st2(y + 34 + 2 * sub, wrote ? (signs[0] | (signs[1] << 8)) : 0);
            if (!(sub & 1)) {
                y[66 + (sub >> 1)] = (uint8_t)((wrote ? qh_bits : 0) | (qh_n << 4));
                y[74 + (sub >> 1)] = (uint8_t)(nz ? (l4 | (l4n << 4)) : 0);
            }
        } else if (TYPE == SG_IQ3_XXS) {
            // block_iq3_xxs: d, qs[64 grid bytes + 8 x u32 scales_and_signs]
            uint32_t w0 = 0, w1 = 0, ss = 0;
            if (nz && wrote) {
                w0 = gidx[0] | (gidx[1] << 8) | (gidx[2] << 16) | (gidx[3] << 24);
                w1 = gidx[4] | (gidx[5] << 8) | (gidx[6] << 16) | (gidx[7] << 24);
                ss = signs[0] | (signs[1] << 7) | (signs[2] << 14) | (signs[3] << 21);
            }
            if (nz) ss |= (uint32_t)l4 << 28;
            st4_a2(y + 2 + 8 * sub, w0); st4_a2(y + 6 + 8 * sub, w1);
            st4_a2(y + 66 + 4 * sub, ss);
        } else {   // IQ3_S: d, qs[64], qh[8], signs[32], scales[4]
            uint32_t w0 = 0, w1 = 0, sg = 0, qh = 0;
            if (wrote) {
                w0 = (gidx[0] & 255) | ((gidx[1] & 255) << 8) | ((gidx[2] & 255) << 16) | ((gidx[3] & 255) << 24);
                w1 = (gidx[4] & 255) | ((gidx[5] & 255) << 8) | ((gidx[6] & 255) << 16) | ((gidx[7] & 255) << 24);
                sg = signs[0] | (signs[1] << 8) | (signs[2] << 16) | (signs[3] << 24);
#pragma unroll
                for (int k = 0; k < 8; ++k) qh |= (gidx[k] >> 8) << k;
            }
            st4_a2(y + 2 + 8 * slot, w0); st4_a2(y + 6 + 8 * slot, w1);
            y[66 + sub] = (uint8_t)qh;
            st4_a2(y + 74 + 4 * slot, sg);
            if (!(sub & 1)) y[106 + (sub >> 1)] = (uint8_t)(nz ? (l4 | (l4n << 4)) : 0);
        }
    }
};

// ==================================================================================================
// IQ1_S / IQ1_M
template <int BLK, int NPS, int TPB> struct Iq1Smem {
    float xb[BLK][TPB];
    float wgt[BLK][TPB];
    float pa[NPS][TPB];           // prefix sums of weight * x in sorted order; later the list walker's 32 distance terms
    float pb[NPS][TPB];           // prefix sums of weight
    uint8_t idx[BLK][TPB];        // sorted position -> element
    uint8_t L[BLK][TPB];          // ternary codes 0,1,2
};

// stable insertion sort of (value, index) by value (seedpack/gpuquant.py:70-80 replaces qsort with exactly this)
template <int BLK, class SM> SG_DEVINL void sort_block(SM& sm, int tid) {
#pragma unroll 1
    for (int j = 0; j < BLK; ++j) sm.idx[j][tid] = (uint8_t)j;
#pragma unroll 1
    for (int i = 1; i < BLK; ++i) {
        const int ti = sm.idx[i][tid];
        const float tv = sm.xb[ti][tid];
        int j = i;
        while (j > 0) {
            const int pj = sm.idx[j - 1][tid];
            if (!(sm.xb[pj][tid] > tv)) break;
            sm.idx[j][tid] = (uint8_t)pj;
            --j;
        }
        sm.idx[j][tid] = (uint8_t)ti;
    }
}

template <bool M, int VARIANT> struct IQ1 {
    static constexpr int BLK = M ? 16 : 32, NPS = M ? 34 : 33;
    static constexpr int SLAB = 256, SUB = BLK, LANES = 256 / BLK, QK = 256, BS = M ? 56 : 50;
    static constexpr int TPB = M ? 448 : 320, NG = BLK / 8;         // CTA size: what the shared memory allows
    static constexpr bool SMEM_TABLES = false;
    static constexpr int TAB = 2;
    using SM = Iq1Smem<BLK, NPS, TPB>;
    using Q = WorkQueue<TPB, NG, 1>;
    using View = TabView<int>;

    // The grid snap (iq1_find_best_neighbour2) goes through the CTA's sorted queue like the lattice types' searches:
    // its lists have 91 entries on average and up to 205.
    template <int DT, bool IMX>
    static SG_DEVINL void run(const Job& job, const Slab& sl, int sub, bool valid, const View& T, SM& sm, Q& q) {
        const int tid = threadIdx.x;
        const float x_p[3] = {-1 + 0.125f, 0.125f, 1 + 0.125f};
        const float x_m[3] = {-1 - 0.125f, -0.125f, 1 - 0.125f};
        float sigma2, mx;
        {
            float x[BLK];
            load_vals<DT, BLK>(job.x, sl.x + sub * BLK, x);
            const float sumx2 = ordered_sumsq<BLK, LANES>(x, sub);
            sigma2 = fmul(fmul(2.f, sumx2), 1.0f / 256);
            float qw[BLK];
            if (IMX) load_f32<BLK>(job.w, sl.w + sub * BLK, qw);
            mx = fabsf(x[0]);
#pragma unroll
            for (int i = 0; i < BLK; ++i) {
                sm.xb[i][tid] = x[i];
                sm.wgt[i][tid] = IMX ? fmul(qw[i], fsqrt(fadd(sigma2, fmul(x[i], x[i])))) : fmul(x[i], x[i]);
                if (i) mx = fmaxf(mx, fabsf(x[i]));
            }
        }
        float scale = 0.f;
        int shift = M ? 0 : 1;             // shifts[ib]: IQ1_S +1 / -1, IQ1_M best_k 0..3
        unsigned index[BLK / 8];
#pragma unroll
        for (int k = 0; k < BLK / 8; ++k) index[k] = 0;
        bool wrote = false, found = false;
        int best_k = M ? -1 : 0;
        if (!(mx < (M ? 1e-7f : 1e-12f))) {
            sort_block<BLK>(sm, tid);
            float best_score = -3.402823466e+38F;
            scale = mx;
            int besti1 = -1, besti2 = -1;
            if (!M) {
                sm.pa[0][tid] = 0.f; sm.pb[0][tid] = 0.f;
                {
                    float a = 0.f, b = 0.f;
#pragma unroll 1
                    for (int j = 0; j < BLK; ++j) {
                        const int i = sm.idx[j][tid];
                        const float w = sm.wgt[i][tid];
                        a = fadd(a, fmul(w, sm.xb[i][tid]));
                        b = fadd(b, w);
                        sm.pa[j + 1][tid] = a; sm.pb[j + 1][tid] = b;
                    }
                }
                const float sx0 = sm.pa[0][tid], sw0 = sm.pb[0][tid], sxn = sm.pa[BLK][tid], swn = sm.pb[BLK][tid];
#pragma unroll 1
                for (int i1 = 0; i1 <= BLK; ++i1) {
                    const float sx1 = sm.pa[i1][tid], sw1 = sm.pb[i1][tid];
                    const float ax = fsub(sx1, sx0), aw = fsub(sw1, sw0);
#pragma unroll 4
                    for (int i2 = i1; i2 <= BLK; ++i2) {
                        const float sx2 = sm.pa[i2][tid], sw2 = sm.pb[i2][tid];
                        const float bx = fsub(sx2, sx1), cx = fsub(sxn, sx2);
                        const float bw = fsub(sw2, sw1), cw = fsub(swn, sw2);
                        float sumqx = fadd(fadd(fmul(ax, x_p[0]), fmul(bx, x_p[1])), fmul(cx, x_p[2]));
                        float sumq2 = fadd(fadd(fmul(fmul(aw, x_p[0]), x_p[0]), fmul(fmul(bw, x_p[1]), x_p[1])), fmul(fmul(cw, x_p[2]), x_p[2]));
                        if (sumq2 > 0.f && fmul(sumqx, sumqx) > fmul(best_score, sumq2)) {
                            scale = fdiv(sumqx, sumq2); best_score = fmul(scale, sumqx);
                            besti1 = i1; besti2 = i2; best_k = 1;
                        }
                        sumqx = fadd(fadd(fmul(ax, x_m[0]), fmul(bx, x_m[1])), fmul(cx, x_m[2]));
                        sumq2 = fadd(fadd(fmul(fmul(aw, x_m[0]), x_m[0]), fmul(fmul(bw, x_m[1]), x_m[1])), fmul(fmul(cw, x_m[2]), x_m[2]));
                        if (sumq2 > 0.f && fmul(sumqx, sumqx) > fmul(best_score, sumq2)) {
                            scale = fdiv(sumqx, sumq2); best_score = fmul(scale, sumqx);
                            besti1 = i1; besti2 = i2; best_k = -1;
                        }
                    }
                }
            } else if (VARIANT == 0) {
                // per-half prefix sums: pa[h*17 + j], pb[h*17 + j]   (ggml-quants.c:4777-4822)
                sm.pa[0][tid] = 0.f; sm.pa[17][tid] = 0.f; sm.pb[0][tid] = 0.f; sm.pb[17][tid] = 0.f;
#pragma unroll 1
                for (int j = 0; j < 16; ++j) {
                    const int i = sm.idx[j][tid];
                    const int h = i < 8 ? 0 : 1;
                    const float w = sm.wgt[i][tid];
                    sm.pa[h * 17 + j + 1][tid] = fadd(sm.pa[h * 17 + j][tid], fmul(w, sm.xb[i][tid]));
                    sm.pa[(1 - h) * 17 + j + 1][tid] = sm.pa[(1 - h) * 17 + j][tid];
                    sm.pb[h * 17 + j + 1][tid] = fadd(sm.pb[h * 17 + j][tid], w);
                    sm.pb[(1 - h) * 17 + j + 1][tid] = sm.pb[(1 - h) * 17 + j][tid];
                }
                const float txs0 = sm.pa[16][tid], txs1 = sm.pa[33][tid], tws0 = sm.pb[16][tid], tws1 = sm.pb[33][tid];
                const float p2 = x_p[2], m2 = x_m[2];
                const float cp1 = fsub(fmul(x_p[0], x_p[0]), fmul(x_p[1], x_p[1]));
                const float cp2 = fsub(fmul(x_p[1], x_p[1]), fmul(x_p[2], x_p[2]));
                const float cm1 = fsub(fmul(x_m[0], x_m[0]), fmul(x_m[1], x_m[1]));
                const float cm2 = fsub(fmul(x_m[1], x_m[1]), fmul(x_m[2], x_m[2]));
                const float tp0 = fmul(txs0, p2), tp1 = fmul(txs1, p2), tm0 = fmul(txs0, m2), tm1 = fmul(txs1, m2);
                const float wp0 = fmul(fmul(tws0, p2), p2), wp1 = fmul(fmul(tws1, p2), p2);
                const float wm0 = fmul(fmul(tws0, m2), m2), wm1 = fmul(fmul(tws1, m2), m2);
#pragma unroll 1
                for (int i1 = 0; i1 <= 16; ++i1) {
                    const float x10 = sm.pa[i1][tid], x11 = sm.pa[17 + i1][tid];
                    const float w10 = sm.pb[i1][tid], w11 = sm.pb[17 + i1][tid];
#pragma unroll 4
                    for (int i2 = i1; i2 <= 16; ++i2) {
                        const float x20 = sm.pa[i2][tid], x21 = sm.pa[17 + i2][tid];
                        const float w20 = sm.pb[i2][tid], w21 = sm.pb[17 + i2][tid];
                        const float s0 = fadd(x10, x20), s1 = fadd(x11, x21);
                        const float qx_p0 = fsub(tp0, s0), qx_m0 = fsub(tm0, s0), qx_p1 = fsub(tp1, s1), qx_m1 = fsub(tm1, s1);
                        const float q2_p0 = fadd(fadd(wp0, fmul(w10, cp1)), fmul(w20, cp2));
                        const float q2_m0 = fadd(fadd(wm0, fmul(w10, cm1)), fmul(w20, cm2));
                        const float q2_p1 = fadd(fadd(wp1, fmul(w11, cp1)), fmul(w21, cp2));
                        const float q2_m1 = fadd(fadd(wm1, fmul(w11, cm1)), fmul(w21, cm2));
                        const float sqx[4] = {fadd(qx_p0, qx_p1), fadd(qx_p0, qx_m1), fadd(qx_m0, qx_p1), fadd(qx_m0, qx_m1)};
                        const float sq2[4] = {fadd(q2_p0, q2_p1), fadd(q2_p0, q2_m1), fadd(q2_m0, q2_p1), fadd(q2_m0, q2_m1)};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (sq2[k] > 0.f && fmul(sqx[k], sqx[k]) > fmul(best_score, sq2[k])) {
                                scale = fdiv(sqx[k], sq2[k]); best_score = fmul(scale, sqx[k]);
                                besti1 = i1; besti2 = i2; best_k = k;
                            }
                        }
                    }
                }
            } else {
                // direct sums per split, three ranges of the sorted order (pre-f95b0d9539 llama.cpp)
#pragma unroll 1
                for (int i1 = 0; i1 <= 16; ++i1) {
#pragma unroll 1
                    for (int i2 = i1; i2 <= 16; ++i2) {
                        float sqx[4] = {0.f, 0.f, 0.f, 0.f}, sq2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                        for (int j = 0; j < 16; ++j) {
                            const int i = sm.idx[j][tid];
                            const int g = j < i1 ? 0 : j < i2 ? 1 : 2;
                            const float xp = g == 0 ? x_p[0] : g == 1 ? x_p[1] : x_p[2];
                            const float xm = g == 0 ? x_m[0] : g == 1 ? x_m[1] : x_m[2];
                            const float w = sm.wgt[i][tid], xv = sm.xb[i][tid];
                            const float pqx = fmul(fmul(w, xp), xv), mqx = fmul(fmul(w, xm), xv);
                            const float pq2 = fmul(fmul(w, xp), xp), mq2 = fmul(fmul(w, xm), xm);
                            const bool first = i < 8;
                            // k: 0 = (+,+), 1 = (+,-), 2 = (-,+), 3 = (-,-): first sign for the first half of the block
                            sqx[0] = fadd(sqx[0], pqx);                 sq2[0] = fadd(sq2[0], pq2);
                            sqx[1] = fadd(sqx[1], first ? pqx : mqx);   sq2[1] = fadd(sq2[1], first ? pq2 : mq2);
                            sqx[2] = fadd(sqx[2], first ? mqx : pqx);   sq2[2] = fadd(sq2[2], first ? mq2 : pq2);
                            sqx[3] = fadd(sqx[3], mqx);                 sq2[3] = fadd(sq2[3], mq2);
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (sq2[k] > 0.f && fmul(sqx[k], sqx[k]) > fmul(best_score, sq2[k])) {
                                scale = fdiv(sqx[k], sq2[k]); best_score = fmul(scale, sqx[k]);
                                besti1 = i1; besti2 = i2; best_k = k;
                            }
                        }
                    }
                }
            }
            found = besti1 >= 0 && besti2 >= 0 && (M ? best_k >= 0 : best_k != 0);
            if (found) {
#pragma unroll 1
                for (int j = 0; j < BLK; ++j) sm.L[sm.idx[j][tid]][tid] = (uint8_t)(j < besti1 ? 0 : j < besti2 ? 1 : 2);
                if (scale < 0.f) {
#pragma unroll 1
                    for (int j = 0; j < BLK; ++j) sm.L[j][tid] = (uint8_t)(2 - sm.L[j][tid]);
                    scale = -scale;
                    best_k = M ? 3 - best_k : -best_k;
                }
            } else {
                scale = 0.f;
            }
        }
        // grid snap of every group of 8 through the queue
        unsigned plusmask = 0;
#pragma unroll
        for (int k = 0; k < NG; ++k)
            if (M ? (k == 0 ? best_k < 2 : (best_k % 2 == 0)) : best_k == 1) plusmask |= 1u << k;
        q.scale[0][tid] = scale;
        q.flag[tid] = (uint8_t)plusmask;
        bool all_on_grid = true;
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            unsigned u = 0;
            if (found) {
#pragma unroll
                for (int j = 0; j < 8; ++j) u |= (unsigned)sm.L[8 * k + j][tid] << (2 * j);
            }
            const int gi = found ? T.map[u] : 0;
            const bool off = gi < 0;
            if (off) all_on_grid = false;
            q.put(k, u, off, off ? (int)T.nbk[-gi - 1] : 0, 3);
        }
        {
            const int total = q.sort(NG);
            float (*term)[TPB] = sm.pa;               // the prefix sums are dead by now
#pragma unroll 1
            for (int p0 = 0, turn = 0; p0 < total; p0 += TPB, ++turn) {
                const int p = p0 + ((turn & 1) ? TPB - 1 - tid : tid);
                if (p >= total) continue;
                const unsigned it = q.item[p];
                const int t2 = (int)(it / NG), k = (int)(it % NG);
                const int list = -T.map[q.u[k][t2]] - 1;
                const float s1 = q.scale[0][t2];
                const bool plus = (q.flag[t2] >> k) & 1;
                const float sq[3] = {fmul(s1, plus ? x_p[0] : x_m[0]), fmul(s1, plus ? x_p[1] : x_m[1]), fmul(s1, plus ? x_p[2] : x_m[2])};
                q.u[k][t2] = (uint16_t)search_list8<TPB>(T.nbk, list, sq, &sm.xb[8 * k], &sm.wgt[8 * k], t2, term, T.key0, job.status);
            }
            __syncthreads();
        }
        unsigned ukey[NG];                  // levels of the chosen grid points, 2 bits a weight
#pragma unroll
        for (int k = 0; k < NG; ++k) ukey[k] = T.key0;      // bytes that stay zero name grid point 0
        if (found) {
#pragma unroll
            for (int k = 0; k < NG; ++k) {
                ukey[k] = q.u[k][tid];
                int gi = T.map[ukey[k]];
                if (gi < 0) { atomicOr(job.status, SG_ST_OFFGRID); gi = 0; ukey[k] = T.key0; }
                index[k] = (unsigned)gi;
            }
            if (!all_on_grid) {
                float sumqx = 0.f, sumq2 = 0.f;
#pragma unroll
                for (int k = 0; k < NG; ++k) {
                    const bool plus = (plusmask >> k) & 1;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const unsigned c = (ukey[k] >> (2 * j)) & 3u;
                        const float qv = plus ? (c == 0 ? x_p[0] : c == 1 ? x_p[1] : x_p[2]) : (c == 0 ? x_m[0] : c == 1 ? x_m[1] : x_m[2]);
                        const float w = sm.wgt[8 * k + j][tid];
                        sumqx = fadd(sumqx, fmul(fmul(w, qv), sm.xb[8 * k + j][tid]));
                        sumq2 = fadd(sumq2, fmul(fmul(w, qv), qv));
                    }
                }
                if (sumqx > 0.f && sumq2 > 0.f) scale = fdiv(sumqx, sumq2);
            }
            shift = best_k;
            wrote = true;
        }
        if (!wrote) { scale = 0.f; shift = M ? 0 : 1; }
        float scales[LANES];
        gather<LANES>(scale, scales);
        float max_scale = 0.f;
#pragma unroll
        for (int j = 0; j < LANES; ++j) max_scale = fmaxf(max_scale, scales[j]);
        const bool nz = max_scale != 0.f;
        float d = fdiv(max_scale, c_div[DIV_15]);
        const float id = frcp(d);
        int l3 = 0;
        if (nz) l3 = clampi(nearest_int(fmul(0.5f, fsub(fmul(id, scale), 1.f))), 0, 7);
        uint8_t* y = job.y + out_offset<256, 256, BS>(sl, 0);
        if (!M) {
            // block_iq1_s: d, qs[32], qh[8] (u16)
            unsigned h = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) h |= (index[k] >> 8) << (3 * k);
            if (nz) h |= (unsigned)(l3 | (shift == -1 ? 8 : 0)) << 12;
            if (!valid) return;
            if (sub == 0) st2(y, nz ? f32_to_f16(fmul(d, 1.125f)) : f32_to_f16(0.f));
            st4_a2(y + 2 + 4 * sub, (index[0] & 255) | ((index[1] & 255) << 8) | ((index[2] & 255) << 16) | ((index[3] & 255) << 24));
            st2(y + 34 + 2 * sub, h);
        } else {
            // final pass over the super-block in block order (ggml-quants.c:4884-4909): an in-order chain, handed
            // from lane to lane
            float sumqx_f = 0.f, sumq2_f = 0.f;
#pragma unroll 1
            for (int stage = 0; stage < 16; ++stage) {
                float a = sumqx_f, b = sumq2_f;
                if (sub == stage && nz) {
                    const float ql = (float)(2 * l3 + 1);
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const bool plus = k == 0 ? shift < 2 : (shift % 2 == 0);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const unsigned c = (ukey[k] >> (2 * j)) & 3u;
                            const float xx = plus ? (c == 0 ? x_p[0] : c == 1 ? x_p[1] : x_p[2]) : (c == 0 ? x_m[0] : c == 1 ? x_m[1] : x_m[2]);
                            const float q = fmul(xx, ql);
                            const float w = sm.wgt[8 * k + j][tid];
                            a = fadd(a, fmul(fmul(w, q), sm.xb[8 * k + j][tid]));
                            b = fadd(b, fmul(fmul(w, q), q));
                        }
                    }
                }
                sumqx_f = gshfl<16>(a, stage);
                sumq2_f = gshfl<16>(b, stage);
            }
            if (sumq2_f > 0.f) d = fdiv(sumqx_f, sumq2_f);
            const unsigned s16 = f32_to_f16(fmul(d, 1.1125f));
            // scales: four u16, each 4 x 3-bit block scales + one nibble of the fp16 super-scale
            unsigned l3s[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) l3s[k] = (unsigned)gshfl<16>(l3, (sub & ~3) + k);
            const unsigned masks = shift == 0 ? 0x00u : shift == 1 ? 0x80u : shift == 2 ? 0x08u : 0x88u;
            if (!valid) return;
            st2(y + 2 * sub, (index[0] & 255) | ((index[1] & 255) << 8));
            y[32 + sub] = (uint8_t)((index[0] >> 8) | ((index[1] >> 8) << 4) | (nz ? masks : 0u));
            if ((sub & 3) == 0) {
                unsigned v = 0;
                if (nz) {
                    v = l3s[0] | (l3s[1] << 3) | (l3s[2] << 6) | (l3s[3] << 9);
                    const int q = sub >> 2;
                    v |= ((s16 >> (4 * q)) & 0xf) << 12;
                }
                st2(y + 48 + 2 * (sub >> 2), v);
            }
        }
    }
};

// ---- launch ------------------------------------------------------------------------------------------
const IqTables* device_tables(int device);     // tables.cu; null until sg_tables_install ran on the device

// Lattice and ternary kernels: CTAs of T::TPB threads, one block of 16 / 32 weights per thread, walking over tiles
// of T::TPB blocks.  The IQ3 tables are small, so each CTA copies them into shared memory first; the IQ2 tables stay in global
// memory (they are L2-resident).
template <class T> struct LatSmem {
    typename T::SM v;
    typename T::Q q;
    int16_t map[T::SMEM_TABLES ? 4096 : 1];
    uint16_t nbk[1];              // SMEM_TABLES: nb_size + 64 entries follow
};
template <class T, int DT, bool IMX>
__global__ void __launch_bounds__(T::TPB, T::TPB == 256 ? 2 : 1) k_quant_lat(const __grid_constant__ Job job, const __grid_constant__ GridTable tab, long long ntiles) {
    extern __shared__ __align__(16) unsigned char raw[];
    LatSmem<T>& sm = *reinterpret_cast<LatSmem<T>*>(raw);
    constexpr int TPB = T::TPB, LANES = T::LANES;
    typename T::View view;
    view.key0 = __ldg(tab.keys);
    if constexpr (T::SMEM_TABLES) {
        for (int i = threadIdx.x; i < 4096; i += TPB) sm.map[i] = (int16_t)__ldg(tab.map + i);
        for (int i = threadIdx.x; i < tab.nb_size + 64; i += TPB) sm.nbk[i] = __ldg(tab.nbkeys + i);
        view.map = sm.map; view.nbk = sm.nbk;
    } else {
        view.map = tab.map; view.nbk = tab.nbkeys;
    }
    if (threadIdx.x < 32) sm.q.count[threadIdx.x] = 0;
    __syncthreads();
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long g = tile * TPB + threadIdx.x;
        long long s = g / LANES;
        const int sub = (int)(g - s * LANES);
        const bool valid = s < job.nslabs;
        if (!valid) s = job.nslabs - 1;
        const Slab sl = locate<T::SLAB>(job, s);
        T::template run<DT, IMX>(job, sl, sub, valid, view, sm.v, sm.q);
    }
}

template <class T, int DT, bool IMX>
__global__ void __launch_bounds__(128) k_quant_iq4(const __grid_constant__ Job job) {
    constexpr int LANES = T::LANES;
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long s = g / LANES;
    const int sub = (int)(g - s * LANES);
    const bool valid = s < job.nslabs;
    if (!valid) s = job.nslabs - 1;
    __shared__ float kv[16];
    if (threadIdx.x < 16) kv[threadIdx.x] = (float)c_iq4nl[threadIdx.x];
    __syncthreads();
    const Slab sl = locate<T::SLAB>(job, s);
    T::template run<DT, IMX>(job, sl, sub, valid, kv);
}

template <class T, bool IMX>
static int launch_lat(const Job& job, int dt, cudaStream_t st, const IqTables& tabs) {
    const GridTable& tab = tabs.t[T::TAB];
    const long long threads = job.nslabs * T::LANES;
    if (threads == 0) return SG_OK;
    size_t smem = sizeof(LatSmem<T>);
    if (T::SMEM_TABLES) {
        if (tab.map_size != 4096 || tab.nb_size > 32767) return SG_ERR_TABLES;
        smem += (size_t)(tab.nb_size + 64) * sizeof(uint16_t);
    }
    const long long ntiles = (threads + T::TPB - 1) / T::TPB;
    int dev = 0, sms = 0;
    int rc = cuda_ok(cudaGetDevice(&dev));
    if (rc == SG_OK) rc = cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (rc != SG_OK) return rc;
    auto go = [&](auto kern) -> int {
        int r = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int per_sm = 0;
        if (r == SG_OK) r = cuda_ok(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, T::TPB, smem));
        if (r != SG_OK) return r;
        if (per_sm < 1) return SG_ERR_LIMIT;
        const long long resident = (long long)sms * per_sm;
        kern<<<(unsigned)(ntiles < resident ? ntiles : resident), T::TPB, smem, st>>>(job, tab, ntiles);
        return SG_OK;
    };
    switch (dt) {
        case SG_DT_BF16: rc = go(k_quant_lat<T, SG_DT_BF16, IMX>); break;
        case SG_DT_F16:  rc = go(k_quant_lat<T, SG_DT_F16, IMX>); break;
        case SG_DT_F32:  rc = go(k_quant_lat<T, SG_DT_F32, IMX>); break;
        default: return SG_ERR_ARG;
    }
    if (rc != SG_OK) return rc;
    return cuda_ok(cudaGetLastError());
}
template <class T, bool IMX>
static int launch_iq4(const Job& job, int dt, cudaStream_t st) {
    const long long threads = job.nslabs * T::LANES;
    const unsigned grid = (unsigned)((threads + 127) / 128);
    if (grid == 0) return SG_OK;
    switch (dt) {
        case SG_DT_BF16: k_quant_iq4<T, SG_DT_BF16, IMX><<<grid, 128, 0, st>>>(job); break;
        case SG_DT_F16:  k_quant_iq4<T, SG_DT_F16, IMX><<<grid, 128, 0, st>>>(job); break;
        case SG_DT_F32:  k_quant_iq4<T, SG_DT_F32, IMX><<<grid, 128, 0, st>>>(job); break;
        default: return SG_ERR_ARG;
    }
    return cuda_ok(cudaGetLastError());
}

static int dispatch_iq(int type, int variant, bool imx, int device, const Job& job, int dt, cudaStream_t st) {
    if (type == SG_IQ4_NL) return imx ? launch_iq4<IQ4<false>, true>(job, dt, st) : launch_iq4<IQ4<false>, false>(job, dt, st);
    if (type == SG_IQ4_XS) return imx ? launch_iq4<IQ4<true>, true>(job, dt, st) : launch_iq4<IQ4<true>, false>(job, dt, st);
    const IqTables* tp = device_tables(device);
    if (!tp) return SG_ERR_TABLES;
    const IqTables& tabs = *tp;
    switch (type) {
        case SG_IQ2_XXS: return imx ? launch_lat<Lattice<SG_IQ2_XXS>, true>(job, dt, st, tabs) : SG_ERR_IMATRIX;
        case SG_IQ2_XS:  return imx ? launch_lat<Lattice<SG_IQ2_XS>, true>(job, dt, st, tabs) : SG_ERR_IMATRIX;
        case SG_IQ2_S:   return imx ? launch_lat<Lattice<SG_IQ2_S>, true>(job, dt, st, tabs) : launch_lat<Lattice<SG_IQ2_S>, false>(job, dt, st, tabs);
        case SG_IQ3_XXS: return imx ? launch_lat<Lattice<SG_IQ3_XXS>, true>(job, dt, st, tabs) : launch_lat<Lattice<SG_IQ3_XXS>, false>(job, dt, st, tabs);
        case SG_IQ3_S:   return imx ? launch_lat<Lattice<SG_IQ3_S>, true>(job, dt, st, tabs) : launch_lat<Lattice<SG_IQ3_S>, false>(job, dt, st, tabs);
        case SG_IQ1_S:   return imx ? launch_lat<IQ1<false, 0>, true>(job, dt, st, tabs) : SG_ERR_IMATRIX;
        case SG_IQ1_M:
            if (variant == 1) return imx ? launch_lat<IQ1<true, 1>, true>(job, dt, st, tabs) : launch_lat<IQ1<true, 1>, false>(job, dt, st, tabs);
            return imx ? launch_lat<IQ1<true, 0>, true>(job, dt, st, tabs) : launch_lat<IQ1<true, 0>, false>(job, dt, st, tabs);
        default: return SG_ERR_TYPE;
    }
}

}  // namespace sg
