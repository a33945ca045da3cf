"""R2: the BF16 base-model codec - host side.  Mirror of the reference's `BF16v2` and `R2Tensors`
(seedpack/bf16v2.py:174-617) over the seedgrow C ABI: the same layout / group / plan logic, side information,
role-shared tables normalised like `normalize_gpu` (seedpack/gpu2.py:460-480), duplicate-row removal, and the same
bytes in the parts `meta`, `side`, `tables`, `lens`, `stream`.

Outside this module's scope: parsing the GGUF file into the layout (the caller passes the layout the reference
stores in `meta`: {"size", "t": [[offset, nbytes, rowlen, "bf16"]...], "role": [...], "nroles"}) and the `rest` part
(header bytes around the tensors, coded on the host with xz) - both are host-side pieces of the archive layer.
"""
import ctypes
import json
import re

import numpy as np
import torch

from . import _lib, zstd
from .qr import load_tables, store_tables

PB = 15
SEG = 16384
K = 8
NE, NM, NS = 512, 128, 16
TPT = NE + NM + NS
TB_DT = np.dtype([("doff", "<i8"), ("rowlen", "<i4"), ("rowbase", "<i4"), ("colbase", "<i4"), ("tab", "<i4"), ("rmap", "<i4"), ("pad", "<i4")])
SG_DT = np.dtype([("t", "<i4"), ("n", "<i4"), ("i0", "<i8")])


def role(name):
    return re.sub(r"blk\.\d+\.", "", name)


def layout_of(tensors, size):
    """tensors: [(name, offset, nbytes, rowlen)] of the file's 2-D BF16 tensors -> the layout dict (bf16v2.py:182-189)"""
    ts = sorted(tensors, key=lambda t: t[1])
    roles = []
    for t in ts:
        if role(t[0]) not in roles:
            roles.append(role(t[0]))
    return {"size": size, "t": [[t[1], t[2], t[3], "bf16"] for t in ts], "role": [roles.index(role(t[0])) for t in ts],
            "nroles": len(roles)}


def normalize_gpu(counts, scale=1 << PB):
    """counts (T, 256) -> (uint16 freqs of the used rows, used row ids); every seen symbol >= 1, rows sum to `scale`.
    Restates seedpack/gpu2.py:460-480 in NumPy with stable sorts (the reference's array back ends sort stably)."""
    counts = np.asarray(counts).astype(np.int64).reshape(-1, 256)
    tot = counts.sum(1)
    used = np.flatnonzero(tot)
    c = counts[used]
    t = tot[used][:, None]
    f = np.where(c > 0, np.maximum(1, (c * scale + t // 2) // t), 0)
    rows = np.arange(len(used))
    for _ in range(64):
        diff = scale - f.sum(1)
        if not (diff != 0).any():
            break
        am = np.argmax(f, 1)
        f[rows, am] += np.maximum(diff, 0)
        need = np.maximum(-diff, 0)
        rank = np.argsort(np.argsort(-f, axis=1, kind="stable"), axis=1, kind="stable")
        f = f - ((rank < need[:, None]) & (f > 1)).astype(np.int64)
    assert (f.sum(1) == scale).all() and ((c > 0) <= (f > 0)).all()
    return f.astype(np.uint16), used.astype(np.int32)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _dev(a, device):
    a = np.ascontiguousarray(a)
    view = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32, np.dtype(np.uint64): np.int64}.get(a.dtype)
    return torch.from_numpy(a.view(view) if view else a).to(device)


class BF16v2:
    def __init__(self, group_bytes=400 << 20, dedup=True, device=None):
        self.group_bytes, self.dedup = group_bytes, dedup
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.lib = _lib.lib()

    # ---- layout helpers (bf16v2.py:193-222) ----------------------------------------------------------------------------
    def _groups(self, layout):
        gs, cur, cb = [], [], 0
        for i, (off, nb, rl, _) in enumerate(layout["t"]):
            if cur and cb + nb > self.group_bytes:
                gs.append(cur); cur, cb = [], 0
            cur.append(i); cb += nb
        if cur:
            gs.append(cur)
        return gs

    @staticmethod
    def _bases(layout):
        rb, cb, rowbase, colbase = [], [], 0, 0
        for off, nb, rl, _ in layout["t"]:
            rb.append(rowbase); cb.append(colbase)
            rowbase += nb // 2 // rl; colbase += rl
        return rb, cb, rowbase, colbase

    def _plan(self, layout, grp, nrows_c, rmap_off):
        rb, cb, _, _ = self._bases(layout)
        tb = np.zeros(len(grp), TB_DT); segs = []
        a = layout["t"][grp[0]][0]
        for k, i in enumerate(grp):
            off, nb, rl, _ = layout["t"][i]
            tb[k] = (off - a, rl, rb[i], cb[i], layout["role"][i] * TPT, rmap_off.get(i, -1), 0)
            n = nrows_c[i] * rl
            for i0 in range(0, n, SEG):
                segs.append((k, min(SEG, n - i0), i0))
        return tb, np.array(segs, SG_DT) if segs else np.zeros(0, SG_DT)

    # ---- device steps ----------------------------------------------------------------------------------------------------
    def _st(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _status(self):
        bits = ctypes.c_int(0)
        _lib.check(self.lib.sg_status_fetch(self.device.index, self._st(), ctypes.byref(bits)), "sg_status_fetch")
        return bits.value

    def _stats(self, d, rl):
        """side information of one tensor (device uint8 slice): rfi (rows), cfi, scl (columns)  (bf16v2.py:225-244)"""
        nr = d.numel() // 2 // rl
        rfi = torch.empty(nr, dtype=torch.int16, device=self.device)
        cfi = torch.empty(rl, dtype=torch.int16, device=self.device)
        scl = torch.empty(rl, dtype=torch.int8, device=self.device)
        need = self.lib.sg_r2_stats_scratch_bytes(nr, rl)
        scratch = torch.empty(need + 16, dtype=torch.uint8, device=self.device)
        with _lib.timed("r2_stats"):
            _lib.check(self.lib.sg_r2_stats(self.device.index, self._st(), _p(d), nr, rl, _p(rfi), _p(cfi), _p(scl), _p(scratch), need),
                       "sg_r2_stats")
        return rfi, cfi, scl

    def _dups(self, d, rl, host):
        """exact duplicate rows -> (rows kept (sorted), [(dup row, source row)])  (bf16v2.py:246-271)"""
        nr = d.numel() // 2 // rl
        h = torch.empty(nr, dtype=torch.int64, device=self.device)
        with _lib.timed("row_hash"):
            _lib.check(self.lib.sg_row_hash(self.device.index, self._st(), _p(d), nr, rl, _p(h)), "sg_row_hash")
        h = h.cpu().numpy().view(np.uint64)
        order = np.argsort(h, kind="stable")
        hs = h[order]
        same = np.flatnonzero(hs[1:] == hs[:-1])
        if len(same) == 0:
            return None, []
        hu = host.reshape(-1, rl)
        pairs, isdup, first = [], np.zeros(nr, bool), {}
        for k in np.unique(np.concatenate([same, same + 1])):
            r = int(order[k]); key = int(hs[k])
            cands = first.setdefault(key, [])
            src = next((c for c in cands if np.array_equal(hu[c], hu[r])), None)
            if src is None:
                cands.append(r)
            else:
                pairs.append((r, src)); isdup[r] = True
        if not pairs:
            return None, []
        return np.flatnonzero(~isdup).astype(np.int32), sorted(pairs)

    def _tables(self, freq, used, ntab, lut):
        full = np.zeros((ntab, 256), np.uint16)
        full[np.asarray(used)] = freq
        f = _dev(full, self.device)
        enc = torch.empty(ntab * 256 * 2, dtype=torch.int32, device=self.device)
        l = torch.empty(ntab << PB, dtype=torch.uint8, device=self.device) if lut else None
        _lib.check(self.lib.sg_rans_tables(self.device.index, self._st(), _p(f), ntab, PB, _p(enc), _p(l)), "sg_rans_tables")
        return enc, l

    # ---- compression ---------------------------------------------------------------------------------------------------
    def compress_parts(self, data, layout):
        """data: the file's bytes (bytes / uint8 array), layout: see module docstring -> dict of the coded parts
        meta, side, tables, lens, stream (bf16v2.py:276-291 without `rest`)"""
        host = np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else data
        groups = self._groups(layout)
        rb, cb, nrow, ncol = self._bases(layout)
        d, st = self.device.index, self._st()
        rfi = torch.zeros(max(nrow, 1), dtype=torch.int16, device=self.device)
        cfi = torch.zeros(max(ncol, 1), dtype=torch.int16, device=self.device)
        scl = torch.zeros(max(ncol, 1), dtype=torch.int8, device=self.device)
        ntab = layout["nroles"] * TPT
        counts = torch.zeros(ntab * 256, dtype=torch.int32, device=self.device)
        nrows_c, dup_pairs, plans, rmap_all, nrm = {}, {}, {}, [], 0
        span = lambda grp: (layout["t"][grp[0]][0], layout["t"][grp[-1]][0] + layout["t"][grp[-1]][1])
        devs = {}
        for gi, grp in enumerate(groups):
            a, b = span(grp)
            hb = host[a:b]
            dev = torch.from_numpy(np.ascontiguousarray(hb)).to(self.device)
            rmap_off, mine = {}, []
            for i in grp:
                off, nb, rl, _ = layout["t"][i]
                dt = dev[off - a:off - a + nb]
                r_, c_, s_ = self._stats(dt, rl)
                rfi[rb[i]:rb[i] + r_.numel()] = r_; cfi[cb[i]:cb[i] + rl] = c_; scl[cb[i]:cb[i] + rl] = s_
                keep, pairs = self._dups(dt, rl, hb[off - a:off - a + nb].view(np.uint16)) if self.dedup else (None, [])
                nrows_c[i] = nb // 2 // rl if keep is None else len(keep)
                if keep is not None:
                    rmap_off[i] = nrm; nrm += len(keep); rmap_all.append(keep); mine.append(keep)
                    dup_pairs[i] = pairs
            plans[gi] = self._plan(layout, grp, nrows_c, rmap_off)
            tb, sg = plans[gi]
            if mine:
                tb = tb.copy(); m = tb["rmap"] >= 0; tb["rmap"][m] -= min(rmap_off.values())
                rm = _dev(np.concatenate(mine), self.device)
            else:
                rm = torch.zeros(1, dtype=torch.int32, device=self.device)
            tb_d, sg_d = _dev(tb.view(np.uint8), self.device), _dev(sg.view(np.uint8), self.device)
            with _lib.timed("r2_hist"):
                _lib.check(self.lib.sg_r2_hist(d, st, _p(dev), _p(tb_d), _p(sg_d), len(sg), _p(rfi), _p(cfi), _p(scl), _p(rm), _p(counts)),
                           "sg_r2_hist")
            devs[gi] = dev
        rowmap = _dev(np.concatenate(rmap_all), self.device) if rmap_all else torch.zeros(1, dtype=torch.int32, device=self.device)
        freq, used = normalize_gpu(counts.cpu().numpy().view(np.uint32).reshape(ntab, 256), 1 << PB)
        enc, _ = self._tables(freq, used, ntab, lut=False)
        cap = SEG * 2 + 1024
        streams, lens_all = [], []
        for gi, grp in enumerate(groups):
            tb, sg = plans[gi]
            nseg = len(sg)
            tb_d, sg_d = _dev(tb.view(np.uint8), self.device), _dev(sg.view(np.uint8), self.device)
            slots = torch.empty(max(nseg, 1) * cap, dtype=torch.uint8, device=self.device)
            lens = torch.zeros(max(nseg, 1), dtype=torch.int32, device=self.device)
            with _lib.timed("r2_encode"):
                _lib.check(self.lib.sg_r2_encode(d, st, _p(devs[gi]), _p(tb_d), _p(sg_d), nseg, _p(rfi), _p(cfi), _p(scl), _p(rowmap), _p(enc),
                                                 _p(slots), cap, _p(lens)), "sg_r2_encode")
            off = torch.empty(nseg + 1, dtype=torch.int64, device=self.device)
            with _lib.timed("scan_gather"):
                _lib.check(self.lib.sg_scan_gather(d, st, _p(slots), cap, _p(lens), nseg, None, 0, _p(off)), "sg_scan_gather")
            bits = self._status()
            if bits & 4:
                raise ValueError("rANS encoder: a coded symbol has frequency 0 in its table")
            if bits & 2:
                raise RuntimeError("rANS segment overflow")
            total = int(off[-1].item())
            dst = torch.empty(total + 32, dtype=torch.uint8, device=self.device)
            with _lib.timed("scan_gather"):
                _lib.check(self.lib.sg_scan_gather(d, st, _p(slots), cap, _p(lens), nseg, _p(dst), total, _p(off)), "sg_scan_gather")
            streams.append(dst[:total].cpu().numpy().tobytes())
            lens_all.append(lens[:nseg].cpu().numpy().view(np.uint32))
            devs[gi] = None
        dups = [[i, r, s] for i, ps in dup_pairs.items() for r, s in ps]
        meta = dict(layout=layout, dups=dups, nrows_c=[nrows_c[i] for i in range(len(layout["t"]))])
        side = (rfi[:nrow].cpu().numpy().tobytes() + cfi[:ncol].cpu().numpy().tobytes() + scl[:ncol].cpu().numpy().tobytes())
        return {"meta": zstd.compress(json.dumps(meta).encode(), 19), "side": zstd.compress(side, 19), "tables": store_tables(freq, used),
                "lens": zstd.compress(np.concatenate(lens_all).astype(np.uint32).tobytes() if lens_all else b"", 19),
                "stream": b"".join(streams)}


class R2Tensors:
    """random access to an R2-coded file: any of its 2-D BF16 tensors decoded on the GPU alone
    (seedpack/bf16v2.py:489-597).  parts: dict with meta, side, tables, lens, stream."""

    def __init__(self, parts, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.lib = _lib.lib()
        meta = json.loads(zstd.decompress(bytes(parts["meta"]), 1 << 30))
        self.layout = layout = meta["layout"]
        t = layout["t"]
        self.rb, self.cb, nrow, ncol = BF16v2._bases(layout)
        side = zstd.decompress(bytes(parts["side"]), 1 << 32)
        self.rfi = _dev(np.frombuffer(side, np.int16, nrow, 0).copy(), self.device)
        self.cfi = _dev(np.frombuffer(side, np.int16, ncol, 2 * nrow).copy(), self.device)
        self.scl = _dev(np.frombuffer(side, np.int8, ncol, 2 * nrow + 2 * ncol).copy(), self.device)
        self.ntab = layout["nroles"] * TPT
        freq, used = load_tables(parts["tables"], PB, self.ntab)
        helper = BF16v2(device=self.device.index)
        self.enc, self.lut = helper._tables(freq, used, self.ntab, lut=True)
        lens = np.frombuffer(zstd.decompress(bytes(parts["lens"]), 1 << 32), np.uint32)
        self.nrows_c = meta["nrows_c"]
        nseg = [-(-self.nrows_c[i] * rl // SEG) for i, (_, _, rl, _) in enumerate(t)]
        self.seg0 = np.zeros(len(t) + 1, np.int64); self.seg0[1:] = np.cumsum(nseg)
        if self.seg0[-1] != len(lens):
            raise ValueError("R2: segment lengths do not match the layout")
        self.soff = np.zeros(len(lens) + 1, np.uint64); self.soff[1:] = np.cumsum(lens, dtype=np.uint64)
        self.stream = np.frombuffer(parts["stream"], np.uint8)
        if int(self.soff[-1]) != len(self.stream):
            raise ValueError("R2: segment lengths do not add up to the stream length")
        self.dups = {}
        for i, r, s in meta["dups"]:
            self.dups.setdefault(i, []).append((r, s))
        rmap_all, self.rmap_off = [], {}
        for i in range(len(t)):
            if i in self.dups:
                rl = t[i][2]; nr = t[i][1] // 2 // rl
                isdup = np.zeros(nr, bool); isdup[[r for r, _ in self.dups[i]]] = True
                self.rmap_off[i] = sum(len(x) for x in rmap_all); rmap_all.append(np.flatnonzero(~isdup).astype(np.int32))
        self.rowmap = _dev(np.concatenate(rmap_all), self.device) if rmap_all else torch.zeros(1, dtype=torch.int32, device=self.device)

    def decode(self, idxs):
        """coded tensors idxs (layout indices) -> (device uint8 tensor, byte offset of each tensor in it)"""
        t = self.layout["t"]
        idxs = list(idxs)
        d, st = self.device.index, ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        tb = np.zeros(len(idxs), TB_DT)
        segs, in_off, in_end, outs, doff, chunks, spos = [], [], [], [], 0, [], 0
        for k, i in enumerate(idxs):
            off, nb, rl, _ = t[i]
            tb[k] = (doff, rl, self.rb[i], self.cb[i], self.layout["role"][i] * TPT, self.rmap_off.get(i, -1), 0)
            n = self.nrows_c[i] * rl
            sg = np.zeros(-(-n // SEG), SG_DT)
            sg["t"] = k; sg["i0"] = np.arange(0, n, SEG); sg["n"] = np.minimum(SEG, n - sg["i0"])
            segs.append(sg)
            s = self.soff[self.seg0[i]:self.seg0[i + 1] + 1].astype(np.int64)
            chunks.append(self.stream[s[0]:s[-1]])
            in_off.append(s[:-1] - s[0] + spos); in_end.append(s[1:] - s[0] + spos)
            spos += int(s[-1] - s[0])
            outs.append(doff); doff += -(-nb // 256) * 256
        sg = np.concatenate(segs) if segs else np.zeros(0, SG_DT)
        dev = torch.empty(max(doff, 1), dtype=torch.uint8, device=self.device)
        keep = []
        if len(sg):
            sb = np.zeros((spos + 31) // 16 * 16, np.uint8)
            sb[:spos] = np.concatenate(chunks)
            # every device buffer of the launch stays referenced until the kernel has run: a temporary handed to the
            # caching allocator would be reused by the next upload
            keep = [_dev(sb, self.device), _dev(np.concatenate(in_off), self.device), _dev(np.concatenate(in_end), self.device),
                    _dev(tb.view(np.uint8), self.device), _dev(sg.view(np.uint8), self.device)]
            with _lib.timed("r2_decode"):
                _lib.check(self.lib.sg_r2_decode(d, st, _p(keep[0]), _p(keep[1]), _p(keep[2]), _p(dev), _p(keep[3]), _p(keep[4]), len(sg),
                                                 _p(self.rfi), _p(self.cfi), _p(self.scl), _p(self.rowmap), _p(self.enc), _p(self.lut)),
                           "sg_r2_decode")
        for k, i in enumerate(idxs):
            if i in self.dups:
                off, nb, rl, _ = t[i]
                pairs = _dev(np.array(self.dups[i], np.int64).reshape(-1), self.device)
                keep.append(pairs)
                _lib.check(self.lib.sg_copy_rows(d, st, _p(dev[outs[k]:]), rl, _p(pairs), len(self.dups[i])), "sg_copy_rows")
        bits = ctypes.c_int(0)
        _lib.check(self.lib.sg_status_fetch(d, st, ctypes.byref(bits)), "sg_status_fetch")
        if bits.value & 4:
            raise ValueError("R2: corrupt stream")
        return dev, outs
