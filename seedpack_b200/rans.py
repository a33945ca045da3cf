"""Segment-parallel rANS codec over a symbol stream with per-block context tables - host side.

Mirrors the framing of the reference's QR batches (seedpack/qr.py:1007-1090): histogram on the device, table
normalisation on the host (`normalize`, copied from seedpack/qr.py:904-923 - fifteen lines of host NumPy whose every
tie-break decides archive bytes; with the reference bound through seedpack_b200.refbind its own copy runs), encode into per-segment slots with the doubling retry of seedpack/qr.py:1043-1053, prefix sum +
gather, and the inverse.  All coding runs in libseedgrow.so; there is no CPU coder here.
"""
import ctypes

import numpy as np
import torch

from . import _lib

PB = 12
SEG = 16384          # symbols per segment (seedpack/qr.py:952-954: max(16, 16384 // QK) blocks)


def normalize(counts, scale=1 << PB):
    """counts (T, 256) int -> (uint16 freqs of the used rows, used row ids): every row sums to `scale`, every
    seen symbol keeps at least 1; the rounding deficit / surplus goes to the largest entry (first maximum).
    Copied from the reference (seedpack/qr.py:904-923) with NumPy arrays in and out: the format is defined by it."""
    c = np.asarray(counts).astype(np.int64).reshape(-1, 256)
    tot = c.sum(1)
    used = np.flatnonzero(tot)
    f = np.zeros((len(used), 256), np.int64)
    for k, r in enumerate(used):
        row = c[r]
        fr = np.where(row > 0, np.maximum(1, row * scale // tot[r]), 0)
        diff = scale - int(fr.sum())
        while diff != 0:
            j = int(np.argmax(fr))
            step = diff if diff > 0 else -min(-diff, int(fr[j]) - 1)
            if step == 0:
                j = int(np.flatnonzero(fr > 1)[0]); step = -1
            fr[j] += step; diff -= step
        f[k] = fr
    return f.astype(np.uint16), used.astype(np.int32)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


class RansCodec:
    """encode / decode a uint8 symbol stream on one GPU"""

    def __init__(self, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.lib = _lib.lib()

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def status(self):
        bits = ctypes.c_int(0)
        _lib.check(self.lib.sg_status_fetch(self.device.index, self._stream(), ctypes.byref(bits)), "sg_status_fetch")
        return bits.value

    def hist(self, sym, block_tab, block_len, ntab):
        counts = torch.zeros(ntab * 256, dtype=torch.int32, device=self.device)
        with _lib.timed("rans_hist"):
            _lib.check(self.lib.sg_rans_hist(self.device.index, self._stream(), _p(sym), _p(block_tab), block_len, sym.numel(), _p(counts)),
                       "sg_rans_hist")
        return counts

    def tables(self, freq_full, lut=True):
        """freq_full: (ntab, 256) uint16 on the host (unused rows zero) -> (enc_tab, lut) device tensors"""
        ntab = freq_full.shape[0]
        f = torch.from_numpy(np.ascontiguousarray(freq_full, np.uint16).view(np.int16)).to(self.device)
        enc = torch.empty(ntab * 256 * 2, dtype=torch.int32, device=self.device)
        l = torch.empty(ntab << PB, dtype=torch.uint8, device=self.device) if lut else None
        _lib.check(self.lib.sg_rans_tables(self.device.index, self._stream(), _p(f), ntab, PB, _p(enc), _p(l)), "sg_rans_tables")
        return enc, l

    def encode_with(self, sym, block_tab, block_len, enc, seg_len=SEG, cap=None):
        """-> (stream uint8 device tensor padded to 16, segment offsets uint64-as-int64 device tensor [nseg + 1])"""
        n = sym.numel()
        nseg = (n + seg_len - 1) // seg_len
        cap = cap or (seg_len // 4 + 256)
        for _ in range(6):
            slots = torch.empty(nseg * cap, dtype=torch.uint8, device=self.device)
            lens = torch.empty(nseg, dtype=torch.int32, device=self.device)
            with _lib.timed("rans_encode"):
                _lib.check(self.lib.sg_rans_encode(self.device.index, self._stream(), _p(sym), _p(block_tab), block_len, n, seg_len, PB,
                                                   _p(enc), _p(slots), cap, _p(lens)), "sg_rans_encode")
            off = torch.empty(nseg + 1, dtype=torch.int64, device=self.device)
            with _lib.timed("scan_gather"):
                _lib.check(self.lib.sg_scan_gather(self.device.index, self._stream(), _p(slots), cap, _p(lens), nseg, None, 0, _p(off)),
                           "sg_scan_gather")
            bits = self.status()
            if bits & 4:
                raise ValueError("rANS encoder: a coded symbol has frequency 0 in its table")
            if bits & 2:                          # a slot overflowed: retry with twice the room (seedpack/qr.py:1043-1053)
                cap *= 2
                continue
            total = int(off[-1].item())
            dst = torch.zeros((total + 15) // 16 * 16 + 16, dtype=torch.uint8, device=self.device)
            with _lib.timed("scan_gather"):
                _lib.check(self.lib.sg_scan_gather(self.device.index, self._stream(), _p(slots), cap, _p(lens), nseg, _p(dst), total, _p(off)),
                           "sg_scan_gather")
            return dst, off, total
        raise RuntimeError("rANS slots overflowed after 6 doublings")

    def encode(self, sym, block_tab, block_len, ntab, seg_len=SEG):
        """full pipeline -> dict(stream, off, total, freq (used rows), used, lens)"""
        counts = self.hist(sym, block_tab, block_len, ntab).cpu().numpy().reshape(ntab, 256)
        freq, used = normalize(counts)
        full = np.zeros((ntab, 256), np.uint16)
        full[used] = freq
        enc, _ = self.tables(full, lut=False)
        stream, off, total = self.encode_with(sym, block_tab, block_len, enc, seg_len)
        return {"stream": stream, "off": off, "total": total, "freq": freq, "used": used, "ntab": ntab}

    def decode(self, stream, off, block_tab, block_len, nsym, freq, used, ntab, seg_len=SEG):
        full = np.zeros((ntab, 256), np.uint16)
        full[used] = freq
        enc, lut = self.tables(full, lut=True)
        out = torch.empty(nsym, dtype=torch.uint8, device=self.device)
        with _lib.timed("rans_decode"):
            _lib.check(self.lib.sg_rans_decode(self.device.index, self._stream(), _p(stream), _p(off), _p(block_tab), block_len, nsym,
                                               seg_len, PB, _p(enc), _p(lut), ntab, _p(out)), "sg_rans_decode")
        return out
