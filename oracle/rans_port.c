/* TEST INFRASTRUCTURE - plain-C restatement of the reference's rANS coder over a symbol stream (CPU checker).
 *
 * Follows seedpack/rans.py:54-105 (_encode / _decode) with PROB_BITS = pb, applied per segment as the
 * reference's GPU coders do (seedpack/qr.py:651-663 PUT / GET: identical arithmetic, pb = 12): state 32 bit,
 * RANS_L = 2^23, x_max = ((RANS_L >> pb) << 8) * f, byte renormalisation, the encoder runs backwards and the
 * segment's bytes are state (big endian) + renormalisation bytes in decode order.  True integer division. */
#include <string.h>

#include "oracle_port.h"

#define RL (1u << 23)

/* encode all segments; out receives the streams back to back, off[0..nseg] their offsets; returns total bytes
 * (or (size_t)-1 if out_cap is too small) */
size_t op_rans_encode(const uint8_t *sym, const uint16_t *block_tab, int block_len, int64_t nsym, int seg_len, int pb,
                      const uint16_t *freq, uint8_t *out, size_t out_cap, uint64_t *off, uint8_t *tmp, size_t tmp_cap) {
    int64_t nseg = (nsym + seg_len - 1) / seg_len;
    size_t total = 0;
    for (int64_t s = 0; s < nseg; ++s) {
        int64_t s0 = s * seg_len, n = nsym - s0 < seg_len ? nsym - s0 : seg_len;
        size_t pos = tmp_cap;
        uint32_t x = RL;
        for (int64_t i = n - 1; i >= 0; --i) {
            const uint16_t *f = freq + (size_t)block_tab[(s0 + i) / block_len] * 256;
            uint32_t sy = sym[s0 + i], fr = f[sy], cum = 0;
            for (uint32_t k = 0; k < sy; ++k) cum += f[k];
            uint32_t xmax = ((RL >> pb) << 8) * fr;
            while (x >= xmax) { if (!pos) return (size_t)-1; tmp[--pos] = (uint8_t)(x & 0xff); x >>= 8; }
            x = ((x / fr) << pb) + (x % fr) + cum;
        }
        for (int i = 0; i < 4; ++i) { if (!pos) return (size_t)-1; tmp[--pos] = (uint8_t)(x & 0xff); x >>= 8; }
        off[s] = total;
        if (total + (tmp_cap - pos) > out_cap) return (size_t)-1;
        memcpy(out + total, tmp + pos, tmp_cap - pos);
        total += tmp_cap - pos;
    }
    off[nseg] = total;
    return total;
}

/* decode; returns 0 on success, 1 if a segment read past its end or did not finish in the initial state */
int op_rans_decode(const uint8_t *in, const uint64_t *off, const uint16_t *block_tab, int block_len, int64_t nsym, int seg_len,
                   int pb, const uint16_t *freq, uint8_t *sym) {
    int64_t nseg = (nsym + seg_len - 1) / seg_len;
    const uint32_t mask = (1u << pb) - 1;
    for (int64_t s = 0; s < nseg; ++s) {
        int64_t s0 = s * seg_len, n = nsym - s0 < seg_len ? nsym - s0 : seg_len;
        const uint8_t *p = in + off[s], *end = in + off[s + 1];
        uint32_t x = 0;
        for (int i = 0; i < 4; ++i) { if (p >= end) return 1; x = (x << 8) | *p++; }
        for (int64_t i = 0; i < n; ++i) {
            const uint16_t *f = freq + (size_t)block_tab[(s0 + i) / block_len] * 256;
            uint32_t slot = x & mask, cum = 0, sy = 0;
            while (cum + f[sy] <= slot) { cum += f[sy]; ++sy; }
            sym[s0 + i] = (uint8_t)sy;
            x = f[sy] * (x >> pb) + slot - cum;
            while (x < RL) { if (p >= end) return 1; x = (x << 8) | *p++; }
        }
        if (x != RL || p != end) return 1;
    }
    return 0;
}
