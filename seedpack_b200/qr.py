"""QR: quantiser-aware residual coding of a stored quantised tensor against its regrown prediction - host side.

Mirror of the reference's `qr.encode` / `qr.decode` (seedpack/qr.py:1007-1090) over the seedgrow C ABI, with the
same argument meanings and the same bytes out: segment layout (`seg_blocks`, `_layout`, qr.py:952-968), batch
split (`batches`, 971-980), table normalisation (rans.normalize = qr.py:904-923), table storage
(`store_tables` / `load_tables`, seedpack/gpu2.py:489-500), the pack framing (seedpack/codecs_gguf.py:33-56) and
the slot-doubling retry (qr.py:1043-1053).  Arrays are torch CUDA tensors (or host numpy / bytes, uploaded here).
"""
import ctypes
import struct

import numpy as np
import torch

from . import _lib, zstd
from .rans import PB, normalize

SELF_TYPES = {2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 20, 23, 42}
GRID_TYPES = {16, 17, 18, 19, 21, 22, 29}
QR_TYPES = SELF_TYPES | GRID_TYPES
BS = {2: 18, 3: 20, 6: 22, 7: 24, 8: 34, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210, 20: 18, 23: 136, 42: 18,
      16: 66, 17: 74, 18: 98, 19: 50, 21: 110, 22: 82, 29: 56}
QK = {t: (32 if t in (2, 3, 6, 7, 8, 20) else 64 if t == 42 else 256) for t in QR_TYPES}
NSB_MAX = 20
NTAB2 = NSB_MAX + 64 + 2 + 208
MODEL = 2
BATCH = 384 << 20
TM_DT = np.dtype([("blk0", "<i8"), ("seed_off", "<i8"), ("seed_type", "<i4"), ("cols", "<i4"), ("imx_off", "<i8")])
SG_DT = np.dtype([("t", "<i4"), ("nb", "<i4"), ("b0", "<i8")])


# ---- framing shared with the archive layer -----------------------------------------------------------------------
def pack(chunks):
    out = [struct.pack("<I", len(chunks))]
    for name, data in chunks.items():
        nb = name.encode()
        out += [struct.pack("<H", len(nb)), nb, struct.pack("<Q", len(data)), bytes(data)]
    return b"".join(out)


def unpack(buf):
    (n,), pos, chunks = struct.unpack_from("<I", buf), 4, {}
    for _ in range(n):
        (ln,) = struct.unpack_from("<H", buf, pos); pos += 2
        name = bytes(buf[pos:pos + ln]).decode(); pos += ln
        (dl,) = struct.unpack_from("<Q", buf, pos); pos += 8
        chunks[name] = buf[pos:pos + dl]; pos += dl
    return chunks


def store_tables(freq, used):
    u = np.asarray(used).astype(np.int64)
    du = np.diff(u, prepend=0).astype(np.uint32)
    return zstd.compress(struct.pack("<I", len(u)) + du.tobytes() + np.ascontiguousarray(freq, np.uint16).tobytes(), 19)


def load_tables(buf, pb=PB, ntab=None):
    """the `t` part of a batch -> (freq uint16 [n][256], used table ids).  A part whose rows do not each sum to 2^pb, or
    whose ids are not increasing and below `ntab`, is rejected here, before any kernel sees it"""
    raw = zstd.decompress(bytes(buf), max_output_size=1 << 30)
    if len(raw) < 4:
        raise ValueError("coder tables: truncated part")
    (n,) = struct.unpack_from("<I", raw)
    if len(raw) != 4 + 4 * n + 512 * n:
        raise ValueError("coder tables: the part's length does not match its table count")
    du = np.frombuffer(raw, np.uint32, n, 4).astype(np.int64)
    used = np.cumsum(du)
    freq = np.frombuffer(raw, np.uint16, n * 256, 4 + 4 * n).reshape(n, 256)
    if n and ((du[1:] <= 0).any() or (ntab is not None and used[-1] >= ntab)):
        raise ValueError("coder tables: table ids out of order or out of range")
    if n and (freq.sum(1, dtype=np.int64) != (1 << pb)).any():
        raise ValueError("coder tables: a row of frequencies does not sum to 2^PB")
    return freq, used


LEN_OVERFLOW, LEN_NOFREQ = 0xffffffff, 0xfffffffe       # sentinels in a coder launch's segment lengths


def check_lens(lens):
    """raise if a segment met a symbol to which its table gives no frequency (tables made from other symbols)"""
    if (np.asarray(lens) == LEN_NOFREQ).any():
        raise ValueError("rANS encoder: a coded symbol has frequency 0 in its table")


def check_tables(freq, used, counts):
    """every (table, symbol) that occurs in `counts` [ntab][256] must have a frequency >= 1 in (freq, used)"""
    c = np.asarray(counts).reshape(-1, 256)
    full = np.zeros(c.shape, np.uint16)
    full[np.asarray(used)] = freq
    if ((c > 0) & (full == 0)).any():
        raise ValueError("rANS encoder: the tables give no frequency to a symbol that occurs")


def seg_blocks(T):
    """blocks per rANS segment: about 16 K symbols"""
    return max(16, 16384 // QK[T])


def _layout(T, nblocks):
    """tensors' block counts -> (TM rows without the seed fields, SG array, total blocks); copied from the reference
    (seedpack/qr.py:957-968): the segmentation is part of the format"""
    sb = seg_blocks(T)
    tm = np.zeros(len(nblocks), TM_DT)
    segs, b0 = [], 0
    for i, nb in enumerate(nblocks):
        tm[i]["blk0"] = b0
        for o in range(0, nb, sb):
            segs.append((i, min(sb, nb - o), b0 + o))
        b0 += nb
    sg = np.array(segs, SG_DT) if segs else np.zeros(0, SG_DT)
    return tm, sg, b0


def batches(T, sizes):
    """tensor indices split into coding batches of about BATCH bytes (same split on both sides); copied from the
    reference (seedpack/qr.py:971-980): the split is part of the format"""
    out, cur, n = [], [], 0
    for i, s in enumerate(sizes):
        if cur and n + s > BATCH:
            out.append(cur); cur, n = [], 0
        cur.append(i); n += s
    if cur:
        out.append(cur)
    return out


# ---- records: checked on the host before anything is launched -----------------------------------------------------------
SEED_ITEM = {30: 2, 1: 2, 0: 4, 99: 8}          # bytes per weight of the seed types the kernels read: BF16, F16, F32, (x, h) pairs
COLRMS = 98                                      # no seed: one float32 per column (seedpack/qr.py:899)


def check_records(T, nblocks, seed_offs, seed_types, cols, imx_offs, seed_bytes, imx_floats):
    """every offset a kernel will add to the seed or importance buffer stays inside it, every seed type is one the
    kernels know.  Raises ValueError; nothing has been launched at that point.  (The reference trusts its caller:
    seedpack/qr.py:1014-1019.)"""
    for i, nb in enumerate(nblocks):
        st, off, c, io = int(seed_types[i]), int(seed_offs[i]), int(cols[i]), int(imx_offs[i])
        nw = nb * QK[T]
        if c < 0 or (c and (c % QK[T] or nw % c)):
            raise ValueError(f"tensor {i}: {c} weights per row do not divide its {nw} weights into rows of whole blocks")
        if st in SEED_ITEM:
            item = SEED_ITEM[st]
            if off < 0 or off % min(item, 4) or off + nw * item > seed_bytes:
                raise ValueError(f"tensor {i}: seed bytes {off}..{off + nw * item} (type {st}) are outside the seed buffer of {seed_bytes}")
        elif st in SELF_TYPES:                            # a sibling quant as the seed: that type's blocks
            need = nw // QK[st] * BS[st]
            if nw % QK[st] or off < 0 or off % 2 or off + need > seed_bytes:
                raise ValueError(f"tensor {i}: seed blocks {off}..{off + need} (quant type {st}) are outside the seed buffer of {seed_bytes}")
        elif st == COLRMS:
            if c <= 0 or off < 0 or off % 4 or off + 4 * c > seed_bytes:
                raise ValueError(f"tensor {i}: column statistics {off}..{off + 4 * c} are outside the seed buffer of {seed_bytes}")
        else:
            raise ValueError(f"tensor {i}: seed type {st} is not one the coder reads (BF16 30, F16 1, F32 0, 98, 99, scalar-code quants)")
        if io >= 0 and (c <= 0 or io + c > imx_floats):
            raise ValueError(f"tensor {i}: importance values {io}..{io + c} are outside the {imx_floats} given")
        if io < -1:
            raise ValueError(f"tensor {i}: importance offset {io}")


# ---- device plumbing ---------------------------------------------------------------------------------------------------
def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _dev_u8(a, device):
    if isinstance(a, torch.Tensor):
        return a.to(device).view(torch.uint8).reshape(-1)
    _lib.count_h2d(len(a) if not isinstance(a, np.ndarray) else a.nbytes)
    return torch.from_numpy(np.frombuffer(memoryview(a), np.uint8).copy() if not isinstance(a, np.ndarray) else np.ascontiguousarray(a).view(np.uint8).reshape(-1)).to(device)


def _gather(arrs, device):
    parts = [_dev_u8(a, device) for a in arrs]
    return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts)


class QRCodec:
    def __init__(self, device=None, staged=True):
        """staged: run the model once with one lane per block and code from the staged (table, symbol) pairs
        (sg_qr_stage*); False: the single-pass kernels, one lane per segment, as the reference has them"""
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.lib = _lib.lib()
        self.staged = staged

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _status(self):
        bits = ctypes.c_int(0)
        _lib.check(self.lib.sg_status_fetch(self.device.index, self._stream(), ctypes.byref(bits)), "sg_status_fetch")
        return bits.value

    def _imx(self, T, imx_dev):
        if T in GRID_TYPES:
            from . import tables
            tables.install(self.device.index)
        if imx_dev is None:
            return None
        if isinstance(imx_dev, torch.Tensor):
            return imx_dev.to(self.device, torch.float32).contiguous().reshape(-1)
        return torch.from_numpy(np.ascontiguousarray(imx_dev, np.float32).reshape(-1)).to(self.device)

    def _records(self, T, nbs, seed_offs, seed_types, cols, imx_offs, seed_bytes, imx_floats):
        check_records(T, nbs, seed_offs, seed_types, cols, imx_offs, seed_bytes, imx_floats)
        tm, sg, nb = _layout(T, nbs)
        tm["seed_off"], tm["seed_type"], tm["cols"], tm["imx_off"] = seed_offs, seed_types, cols, imx_offs
        tm_d = torch.from_numpy(tm.view(np.uint8).copy()).to(self.device)
        sg_d = torch.from_numpy(sg.view(np.uint8).copy()).to(self.device)
        return tm_d, sg_d, len(sg), nb

    def _tables(self, freq, used, lut):
        full = np.zeros((NTAB2, 256), np.uint16)
        full[np.asarray(used)] = freq
        f = torch.from_numpy(full.view(np.int16)).to(self.device)
        enc = torch.empty(NTAB2 * 256 * 2, dtype=torch.int32, device=self.device)
        l = torch.empty(NTAB2 << PB, dtype=torch.uint8, device=self.device) if lut else None
        _lib.check(self.lib.sg_rans_tables(self.device.index, self._stream(), _p(f), NTAB2, PB, _p(enc), _p(l)), "sg_rans_tables")
        return enc, l

    # ---- encoding, in the three steps a sharded run needs ------------------------------------------------------------
    # A batch's segments are independent once its tables are fixed, and its tables are the normalised SUM of the
    # segments' symbol counts.  So: hist() models this rank's segments and counts their symbols; the counts of all
    # ranks are added (seedpack_b200.shard.sum_counts) and normalised on every rank alike; code() codes this rank's
    # segments with those tables; the ranks' lengths and bytes, joined in segment order (shard.gather_segments), go
    # into finish().  encode() is the three steps over all segments on one GPU.
    def hist(self, T, items, seed_dev, imx_dev=None, mv=None, segs=None):
        """model the segments [s0, s1) of the batch (default: all) -> (state for code(), counts [294, 256] int64).
        Only the blocks of those segments are brought to the device."""
        if T not in QR_TYPES:
            raise ValueError(f"ggml type {T} has no QR model")
        mv = MODEL if mv is None else mv
        imx = self._imx(T, imx_dev)
        bs, d, st = BS[T], self.device.index, self._stream()
        nbs = [len(it[0]) // bs for it in items]
        for k, it in enumerate(items):
            if len(it[0]) % bs or len(it[0]) != len(it[1]):
                raise ValueError(f"tensor {k}: file and prediction must be the same whole number of {bs}-byte blocks")
        seed = _dev_u8(seed_dev, self.device)
        seed_offs, seed_types = [it[2] for it in items], [it[3] for it in items]
        cols = [it[4] if len(it) > 4 else 0 for it in items]
        imx_offs = [it[5] if len(it) > 5 else -1 for it in items]
        check_records(T, nbs, seed_offs, seed_types, cols, imx_offs, seed.numel(), 0 if imx is None else imx.numel())
        tm, sg, nb_all = _layout(T, nbs)
        tm["seed_off"], tm["seed_type"], tm["cols"], tm["imx_off"] = seed_offs, seed_types, cols, imx_offs
        s0, s1 = (0, len(sg)) if segs is None else segs
        if not 0 <= s0 <= s1 <= len(sg):
            raise ValueError(f"segments {s0}..{s1} of a batch of {len(sg)}")
        sg = sg[s0:s1].copy()
        nseg = len(sg)
        # this share's blocks are one contiguous range [B0, B1) of the batch: records are rebased to it
        B0 = int(sg["b0"][0]) if nseg else 0
        B1 = int(sg["b0"][-1] + sg["nb"][-1]) if nseg else 0
        nb = B1 - B0
        sg["b0"] -= B0
        tm = tm.copy()
        tm["blk0"] -= B0
        fparts, pparts = [], []
        for k, it in enumerate(items):
            a = max(B0, int(tm["blk0"][k]) + B0) - (int(tm["blk0"][k]) + B0)        # first block of tensor k in the range
            z = min(B1, int(tm["blk0"][k]) + B0 + nbs[k]) - (int(tm["blk0"][k]) + B0)
            if z > a:
                fparts.append(it[0][a * bs:z * bs]); pparts.append(it[1][a * bs:z * bs])
        F = _gather(fparts, self.device) if fparts else torch.empty(0, dtype=torch.uint8, device=self.device)
        P = _gather(pparts, self.device) if pparts else torch.empty(0, dtype=torch.uint8, device=self.device)
        tm_d = torch.from_numpy(tm.view(np.uint8).copy()).to(self.device)
        sg_d = torch.from_numpy(sg.view(np.uint8).copy()).to(self.device) if nseg else torch.zeros(16, dtype=torch.uint8, device=self.device)
        ne = torch.empty(max(nb, 1), dtype=torch.uint8, device=self.device)
        ndiff = torch.zeros(1, dtype=torch.int64, device=self.device)
        counts = torch.zeros(NTAB2 * 256, dtype=torch.int32, device=self.device)
        stage = None
        if nseg:
            with _lib.timed("residual_blocks"):
                _lib.check(self.lib.sg_residual_blocks(d, st, _p(F), _p(P), bs, nb, _p(ne), _p(ndiff)), "sg_residual_blocks")
            if self.staged:            # the model once, one lane per block; histogram and coder work on the staged pairs
                nstage = self.lib.sg_qr_stage_bytes(T, nb)
                stage = torch.empty(max(nstage, 16), dtype=torch.uint8, device=self.device)
                with _lib.timed("qr_stage"):
                    _lib.check(self.lib.sg_qr_stage(d, st, T, _p(F), _p(P), _p(ne), _p(seed), _p(tm_d), _p(sg_d), nseg, _p(imx), mv, nb, _p(stage),
                                                    nstage), "sg_qr_stage")
                with _lib.timed("qr_stage_hist"):
                    _lib.check(self.lib.sg_qr_stage_hist(d, st, T, nb, _p(stage), _p(counts)), "sg_qr_stage_hist")
            else:
                with _lib.timed("qr_hist"):
                    _lib.check(self.lib.sg_qr_hist(d, st, T, _p(F), _p(P), _p(ne), _p(seed), _p(tm_d), _p(sg_d), nseg, _p(imx), _p(counts), mv),
                               "sg_qr_hist")
        state = dict(T=T, mv=mv, F=F, P=P, seed=seed, imx=imx, tm_d=tm_d, sg_d=sg_d, nseg=nseg, nb=nb, ne=ne, stage=stage)
        _lib.count_d2h(NTAB2 * 1024)
        return state, counts.cpu().numpy().view(np.uint32).astype(np.int64).reshape(NTAB2, 256)

    def code(self, state, freq, used):
        """code the segments hist() modelled with the tables (freq, used) -> (their lengths uint32, their bytes)"""
        T, mv, nseg, nb = state["T"], state["mv"], state["nseg"], state["nb"]
        if not nseg:
            return np.zeros(0, np.uint32), b""
        d, st = self.device.index, self._stream()
        F, P, seed, imx, tm_d, sg_d, ne, stage = (state[k] for k in ("F", "P", "seed", "imx", "tm_d", "sg_d", "ne", "stage"))
        enc, _ = self._tables(freq, used, lut=False)
        cap = seg_blocks(T) * (3 * BS[T] if T in GRID_TYPES else (QK[T] + NSB_MAX) * 2) + 1024
        cap = (cap + 15) // 16 * 16
        for _ in range(3):
            slots = torch.empty(nseg * cap, dtype=torch.uint8, device=self.device)
            lens = torch.zeros(nseg, dtype=torch.int32, device=self.device)
            if self.staged:
                with _lib.timed("qr_stage_encode"):
                    _lib.check(self.lib.sg_qr_stage_encode(d, st, T, nb, _p(stage), _p(sg_d), nseg, _p(enc), _p(slots), cap, _p(lens)),
                               "sg_qr_stage_encode")
            else:
                with _lib.timed("qr_encode"):
                    _lib.check(self.lib.sg_qr_encode(d, st, T, _p(F), _p(P), _p(ne), _p(seed), _p(tm_d), _p(sg_d), nseg, _p(imx), _p(enc),
                                                     _p(slots), cap, _p(lens), mv), "sg_qr_encode")
            # the segments' lengths are read on the host (they are part of the batch anyway): sentinels are seen there,
            # not through the device status word, which other threads' calls share
            lens_h = lens.cpu().numpy().view(np.uint32)
            check_lens(lens_h)
            if not (lens_h == LEN_OVERFLOW).any():
                break
            cap *= 2
        else:
            raise RuntimeError("QR segment overflow")
        total = int(lens_h.sum(dtype=np.uint64))
        off = torch.empty(nseg + 1, dtype=torch.int64, device=self.device)
        dst = torch.empty(total + 32, dtype=torch.uint8, device=self.device)
        with _lib.timed("scan_gather"):
            _lib.check(self.lib.sg_scan_gather(d, st, _p(slots), cap, _p(lens), nseg, _p(dst), total, _p(off)), "sg_scan_gather")
        stream = dst[:total].cpu().numpy().tobytes()
        _lib.count_d2h(total + 4 * nseg)
        return lens_h.astype(np.uint32), stream

    @staticmethod
    def finish(freq, used, lens, stream, mv=MODEL):
        """the batch as the archive holds it (seedpack/qr.py:1058-1061): tables, segment lengths, streams, model byte"""
        out = {"t": store_tables(freq, used), "l": zstd.compress(np.asarray(lens, np.uint32).tobytes(), 19), "s": bytes(stream)}
        if mv != 1:
            out["v"] = bytes([mv])
        return pack(out)

    def encode(self, T, items, seed_dev, imx_dev=None, mv=None):
        """items: [(file tensor bytes, predicted bytes, seed byte offset, seed type[, weights per row, imatrix
        offset])] of one batch, all of ggml type T -> bytes of the coded batch (seedpack/qr.py:1007-1061)"""
        state, counts = self.hist(T, items, seed_dev, imx_dev, mv)
        freq, used = normalize(counts)
        lens, stream = self.code(state, freq, used)
        return self.finish(freq, used, lens, stream, state["mv"])

    def decode(self, T, buf, items, seed_dev, imx_dev=None):
        """items: [(predicted bytes, seed byte offset, seed type[, weights per row, imatrix offset])] -> device uint8
        tensor of the batch's tensors back to back (seedpack/qr.py:1064-1090)"""
        if T not in QR_TYPES:
            raise ValueError(f"ggml type {T} has no QR model")
        imx = self._imx(T, imx_dev)
        ch = unpack(buf)
        mv = ch["v"][0] if "v" in ch else 1
        bs, d, st = BS[T], self.device.index, self._stream()
        nbs = [len(it[0]) // bs for it in items]
        seed = _dev_u8(seed_dev, self.device)
        tm_d, sg_d, nseg, nb = self._records(T, nbs, [it[1] for it in items], [it[2] for it in items],
                                             [it[3] if len(it) > 3 else 0 for it in items],
                                             [it[4] if len(it) > 4 else -1 for it in items], seed.numel(),
                                             0 if imx is None else imx.numel())
        P = _gather([it[0] for it in items], self.device)
        freq, used = load_tables(ch["t"], PB, NTAB2)
        enc, lut = self._tables(freq, used, lut=True)
        lens = np.frombuffer(zstd.decompress(bytes(ch["l"]), max_output_size=1 << 30), np.uint32).astype(np.uint64)
        offs = np.zeros(nseg + 1, np.uint64); offs[1:] = np.cumsum(lens)
        s = np.frombuffer(ch["s"], np.uint8)
        if int(offs[-1]) != len(s):
            raise ValueError("QR batch: segment lengths do not add up to the stream length")
        sd = torch.zeros((len(s) + 31) // 16 * 16, dtype=torch.uint8, device=self.device)
        sd[:len(s)] = torch.from_numpy(s.copy()).to(self.device)
        _lib.count_h2d(len(s) + 8 * nseg)
        F = torch.empty(nb * bs, dtype=torch.uint8, device=self.device)
        off_d = torch.from_numpy(offs.view(np.int64)).to(self.device)
        with _lib.timed("qr_decode"):
            _lib.check(self.lib.sg_qr_decode(d, st, T, _p(sd), _p(off_d), _p(P), _p(seed), _p(tm_d), _p(sg_d), nseg, _p(imx), _p(enc), _p(lut), _p(F),
                                             mv), "sg_qr_decode")
        if self._status() & 4:
            raise ValueError("QR batch: corrupt stream")
        return F
