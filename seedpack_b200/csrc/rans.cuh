// Byte-renormalising rANS coder core, one 32-bit state per segment, one segment per lane.
//
// The bitstream is fixed by the reference (seedpack/qr.py:651-663 PUT / GET, seedpack/bf16v2.py:84-137,
// seedpack/rans.py:54-105): state in [2^23, 2^31), static per-context tables with frequencies summing to
// 2^PB, the encoder walks its symbols backwards writing bytes downwards from the end of a private slot and
// finishes with the 4 state bytes, so that a segment's stream reads forwards as state (big endian)
// followed by the renormalisation bytes in decode order.
//
// What differs from the reference is only how a lane gets there:
//   * x / f and x % f use a per-(table, symbol) 32-bit reciprocal (exact for x < 2^31, which the
//     renormalisation guarantees) instead of integer division;
//   * bytes move through a 16-byte register window per lane, so that global memory only sees aligned
//     16-byte loads and stores.
#pragma once
#include "common.cuh"

namespace sg {

constexpr unsigned RANS_L = 1u << 23;
constexpr unsigned LEN_OVERFLOW = 0xffffffffu;     // out_len of a segment whose slot was too small (retry with more)
constexpr unsigned LEN_NOFREQ   = 0xfffffffeu;     // out_len of a segment that met a symbol its table gives no frequency

// encoder entry for one (table, symbol): rcp = ceil(2^(31+s) / freq) with s = ceil(log2 freq); fc = freq | cum << 16
struct __align__(8) RansSym { unsigned rcp, fc; };

SG_DEVINL unsigned rans_shift(unsigned freq) { return freq < 2 ? 0u : 32u - __clz(freq - 1); }

// quotient x / freq for x < 2^31, 1 <= freq <= 2^15
SG_DEVINL unsigned rans_div(unsigned x, unsigned freq, unsigned rcp) {
    if (freq < 2) return x;
    const unsigned s = rans_shift(freq);            // >= 1
    return __umulhi(x, rcp) >> (s - 1);
}

// ---- downward byte writer ----------------------------------------------------------------------------
// Writes bytes at decreasing addresses ending at `end` (16-byte aligned).  Holds the 16-byte window that
// contains the next byte; full windows are stored with one 16-byte store.
struct ByteWriterDown {
    uint8_t* base;                 // address of the current window
    unsigned long long lo, hi;     // window contents (byte k of the window at bits 8k of lo / hi)
    int pos;                       // bytes still free in the window: next byte goes to index pos - 1
    unsigned bad;                  // set when a symbol with frequency 0 was coded (tables not made from these symbols)
    SG_DEVINL void init(uint8_t* end) { base = end - 16; lo = hi = 0; pos = 16; bad = 0; }
    SG_DEVINL void put(unsigned b) {
        --pos;
        if (pos >= 8) hi |= (unsigned long long)b << (8 * (pos - 8));
        else          lo |= (unsigned long long)b << (8 * pos);
        if (pos == 0) {
            *reinterpret_cast<ulonglong2*>(base) = make_ulonglong2(lo, hi);
            base -= 16; lo = hi = 0; pos = 16;
        }
    }
    // bytes written so far end at this address (the lowest written byte)
    SG_DEVINL uint8_t* ptr() const { return base + pos; }
    // store the partial window; the bytes below ptr() inside it are zero filler in the lane's private slot
    SG_DEVINL void flush(uint8_t* slot_begin) {
        if (pos < 16 && base >= slot_begin) *reinterpret_cast<ulonglong2*>(base) = make_ulonglong2(lo, hi);
        else if (pos < 16) {       // window straddles the slot start: byte stores for the part inside the slot
            for (int k = pos; k < 16; ++k)
                base[k] = (uint8_t)((k >= 8 ? hi >> (8 * (k - 8)) : lo >> (8 * k)) & 0xff);
        }
    }
};

// ---- forward byte reader -----------------------------------------------------------------------------
// Reads bytes at increasing addresses from [p, end) through aligned 16-byte loads; reads past `end` return 0
// and set `over`.
struct ByteReaderUp {
    const uint8_t* win;            // aligned address of the loaded window
    unsigned long long lo, hi;     // the window
    unsigned long long nlo, nhi;   // the window after it, fetched when this one was entered (its latency is off the chain)
    const uint8_t* p;
    const uint8_t* end;
    bool over;
    SG_DEVINL void fetch_next() {
        if (win + 16 < end) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(win + 16);
            nlo = v.x; nhi = v.y;
        }
    }
    SG_DEVINL void init(const uint8_t* begin, const uint8_t* e) {
        p = begin; end = e; over = false;
        win = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(begin) & ~(uintptr_t)15);
        lo = hi = nlo = nhi = 0;
        if (begin < e) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(win);
            lo = v.x; hi = v.y;
            fetch_next();
        }
    }
    SG_DEVINL unsigned get() {
        if (p >= end) { over = true; return 0; }
        const int k = (int)(p - win);
        const unsigned b = (unsigned)((k >= 8 ? hi >> (8 * (k - 8)) : lo >> (8 * k)) & 0xff);
        ++p;
        if (k == 15) { win += 16; lo = nlo; hi = nhi; fetch_next(); }
        return b;
    }
};

// ---- coder steps -------------------------------------------------------------------------------------
template <int PB, class W>
SG_DEVINL void rans_put(unsigned& x, W& w, const RansSym e) {
    const unsigned f = e.fc & 0xffffu, c = e.fc >> 16;
    const unsigned xm = ((RANS_L >> PB) << 8) * f;
    // x < 2^31 and xm >= 2^(31 - PB) for f >= 1: at most two bytes leave per symbol (PB <= 15).  Written as two steps,
    // not a loop: a zero frequency (xm = 0) would never end it; such a symbol marks the segment instead.
    w.bad |= (unsigned)(f == 0);
    if (x >= xm) { w.put(x & 0xff); x >>= 8; if (x >= xm) { w.put(x & 0xff); x >>= 8; } }
    const unsigned q = rans_div(x, f, e.rcp);
    x = (q << PB) + (x - q * f) + c;
}
template <class W> SG_DEVINL void rans_flush(unsigned x, W& w) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { w.put(x & 0xff); x >>= 8; }
}
template <class R> SG_DEVINL unsigned rans_init(R& r) {
    unsigned x = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) x = (x << 8) | r.get();
    return x;
}
// decode one symbol of table `t`: lut = symbol per slot, tab = encoder entries of the same table (freq, cum)
template <int PB, class R>
SG_DEVINL unsigned rans_get(unsigned& x, R& r, const uint8_t* __restrict__ lut, const RansSym* __restrict__ tab) {
    const unsigned slot = x & ((1u << PB) - 1);
    const unsigned s = lut[slot];
    const unsigned fc = tab[s].fc;
    x = (fc & 0xffffu) * (x >> PB) + slot - (fc >> 16);
#pragma unroll 1
    for (int guard = 0; guard < 4 && x < RANS_L; ++guard) x = (x << 8) | r.get();
    return s;
}

// The same through a compact table (RANS_COMPACT bytes per context: 256 coarse entries, one per 2^(PB - 8) slots = the
// symbol whose range holds the bucket's first slot, then the 256 symbols' freq | cum << 16 words) and a walk over the
// words from the coarse entry: 1.25 KiB per context instead of 2^PB + 2 KiB.
constexpr int RANS_COMPACT = 256 + 256 * 4;
template <int PB, class R>
SG_DEVINL unsigned rans_get_compact(unsigned& x, R& r, const uint8_t* __restrict__ ct) {
    const unsigned* __restrict__ words = reinterpret_cast<const unsigned*>(ct + 256);
    const unsigned slot = x & ((1u << PB) - 1);
    unsigned s = ct[slot >> (PB - 8)];
    unsigned fc = words[s];
#pragma unroll 1
    while (slot >= (fc >> 16) + (fc & 0xffffu) && s < 255u) fc = words[++s];
    x = (fc & 0xffffu) * (x >> PB) + slot - (fc >> 16);
#pragma unroll 1
    for (int guard = 0; guard < 4 && x < RANS_L; ++guard) x = (x << 8) | r.get();
    return s;
}
// a table of two symbols (a sign): both words in one 8-byte load, no coarse entry
template <int PB, class R>
SG_DEVINL unsigned rans_get_bit(unsigned& x, R& r, const uint8_t* __restrict__ ct) {
    const unsigned slot = x & ((1u << PB) - 1);
    const uint2 e = *reinterpret_cast<const uint2*>(ct + 256);
    const unsigned s = slot >= (e.x & 0xffffu) ? 1u : 0u;
    const unsigned fc = s ? e.y : e.x;
    x = (fc & 0xffffu) * (x >> PB) + slot - (fc >> 16);
#pragma unroll 1
    for (int guard = 0; guard < 4 && x < RANS_L; ++guard) x = (x << 8) | r.get();
    return s;
}

}  // namespace sg
