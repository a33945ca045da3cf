"""Bindings of the reference's kernel names to the seedgrow C ABI.

`function(name)` returns a callable with CuPy's launch signature `f(grid, block, args, shared_mem=0)`; `args` are
the arguments the reference passes to its own kernel of that name (device arrays of refbind.cupy_shim, NumPy
scalars).  Grid and block are ignored: each C-ABI entry point chooses its own launch.  A name without a binding
raises, so nothing of the reference's CUDA source can run by accident.

    reference kernel (file:line)                       C-ABI entry point
    v2_hist / v2_enc / v2_dec   bf16v2.py:63-137       sg_r2_hist / sg_r2_encode / sg_r2_decode
    bf_hist / bf_enc / bf_dec   gpu_bf16.py:63-137     sg_m24_hist / sg_m24_encode / sg_m24_decode
    row_hash                    bf16v2.py:148-155      sg_row_hash
    build_lut                   bf16v2.py:139, qr.py:889   folded into the decoders' table preparation (sg_rans_tables)
    gather                      qr.py:880-887, gpu2.py     sg_scan_gather
    qr_hist / qr_enc / qr_dec   qr.py:674-807          sg_residual_blocks + sg_qr_hist / sg_qr_encode / sg_qr_decode
    block_fields / blocks_from_fields / intervals / weq / grid_h   qr.py:811-878   sg_qr_block_fields / ..._from_fields /
                                                       sg_qr_intervals / sg_qr_weight_equal / sg_qr_grid_half_step
    dm_log2 / dm_exp2 / dm_rows / dm_cols   detmath.py:67-106   sg_dm_log2 / sg_dm_exp2 / sg_dm_rows / sg_dm_cols
    dm_rows_d / dm_gram / dm_bdot / dm_solve  detmath.py:86-153  sg_dm_rows_f64 / sg_dm_gram / sg_dm_bdot / sg_dm_solve
    hist / encode / decode      gpu_codec.py:73-159    sg_m6_hist / sg_m6_encode / sg_m6_decode
    half_step / est_add / est_seed   siblings.py:51-77   sg_sib_half_step / sg_sib_est_add / sg_sib_est_seed
    hist_a / enc_a / dec_a / hist_b / enc_b / dec_b   gpu2.py:100-262   sg_m21_hist_a / ... / sg_m21_decode_b
    predict / predict_multi / hist_c / enc_c / dec_c  gpu3.py:90-232    sg_m21_predict / ... / sg_m21_decode_c
                                (their modules' #define switches - SIGN, RANK, HICF, PREDA, SEGA, SEGB - become arguments)
    k_dq_<type>                 gpuquant.py:215-219    sg_dequantize
    vq_bf16_to_f32 (elementwise) gpuquant.py:248-249   sg_convert_float

The coders' tables: the reference hands its kernels (remap, freq, cum[, lut]); the C ABI wants the entries
sg_rans_tables makes from the full frequency array.  `_tables` scatters the used rows into the full array on the
device and keeps the result for the arrays it was made from (a coding pass launches several times with the same
tables).
"""
import ctypes
from collections import OrderedDict

import numpy as np
import torch

from .. import _lib
from ..requant import QFUN

QR_NTAB, QR_PB, R2_PB = 294, 12, 15
QR_BS = {2: 18, 3: 20, 6: 22, 7: 24, 8: 34, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210, 20: 18, 23: 136, 42: 18,
         16: 66, 17: 74, 18: 98, 19: 50, 21: 110, 22: 82, 29: 56}
GRID_TYPES = {16, 17, 18, 19, 21, 22, 29}


def _dev():
    from .cupy_shim import device_index
    return device_index()


def _st():
    return ctypes.c_void_p(torch.cuda.current_stream(_dev()).cuda_stream)


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _i(x):
    return int(x)


_TABS = OrderedDict()


def _tables(remap, freq, pb, lut):
    """(remap int32[ntab], freq uint16[nused][256]) -> (encoder entries, decoder symbol table or None) on the device"""
    key = (id(remap.st), remap.off, id(freq.st), freq.off, pb)
    hit = _TABS.get(key)
    if hit is not None and (hit[1] is not None or not lut):
        _TABS.move_to_end(key)
        return hit[0], hit[1]
    ntab = remap.size
    sums = freq._h().reshape(-1, 256).sum(1, dtype=np.int64)
    if freq.size and (sums != (1 << pb)).any():
        raise ValueError("coder tables: a row of frequencies does not sum to 2^PB (damaged table part)")
    r = remap.dev_in().view(torch.int32).to(torch.int64)
    f = freq.dev_in().view(torch.int16).view(-1, 256)
    full = torch.zeros((ntab, 256), dtype=torch.int16, device=f.device)
    used = torch.nonzero(r >= 0).reshape(-1)
    if used.numel():
        full[used] = f[r[used]]
    enc = torch.empty(ntab * 256 * 2, dtype=torch.int32, device=f.device)
    l = torch.zeros(ntab * 1280 if pb == 15 else ntab << pb, dtype=torch.uint8, device=f.device) if lut else None
    _lib.check(_lib.lib().sg_rans_tables(_dev(), _st(), _p(full), ntab, pb, _p(enc), _p(l)), "sg_rans_tables")
    _TABS[key] = (enc, l, remap, freq)           # the source arrays stay alive with the entry: their ids stay theirs
    while len(_TABS) > 6:
        _TABS.popitem(last=False)
    return enc, l


def _seg_ends(off_t, total):
    """first bytes of the segments (any order, together covering [0, total)) -> one past their last bytes"""
    srt, idx = torch.sort(off_t)
    end_sorted = torch.cat([srt[1:], torch.tensor([total], dtype=srt.dtype, device=srt.device)])
    end = torch.empty_like(off_t)
    end[idx] = end_sorted
    return end


# ---- R2 -----------------------------------------------------------------------------------------------------------
def _v2_hist(args):
    dev, tb, sg, nseg, rfi, cfi, scl, rm, counts = args
    _lib.check(_lib.lib().sg_r2_hist(_dev(), _st(), _p(dev.dev_in()), _p(tb.dev_in()), _p(sg.dev_in()), _i(nseg), _p(rfi.dev_in()),
                                     _p(cfi.dev_in()), _p(scl.dev_in()), _p(rm.dev_in()), _p(counts.dev_inout())), "sg_r2_hist")


def _v2_enc(args):
    dev, tb, sg, nseg, rfi, cfi, scl, rowmap, remap, freq, cum, out, cap, out_len = args
    enc, _ = _tables(remap, freq, R2_PB, False)
    _lib.check(_lib.lib().sg_r2_encode(_dev(), _st(), _p(dev.dev_in()), _p(tb.dev_in()), _p(sg.dev_in()), _i(nseg), _p(rfi.dev_in()),
                                       _p(cfi.dev_in()), _p(scl.dev_in()), _p(rowmap.dev_in()), _p(enc), _p(out.dev_out()), _i(cap),
                                       _p(out_len.dev_out())), "sg_r2_encode")


def _v2_dec(args):
    stream, offs, dev, tb, sg, nseg, rfi, cfi, scl, rowmap, remap, freq, cum, lut = args
    enc, l = _tables(remap, freq, R2_PB, True)
    o = offs.dev_in().view(torch.int64)
    e = _seg_ends(o, stream.size)
    _lib.check(_lib.lib().sg_r2_decode(_dev(), _st(), _p(stream.dev_in()), _p(o), _p(e), _p(dev.dev_out()), _p(tb.dev_in()), _p(sg.dev_in()),
                                       _i(nseg), _p(rfi.dev_in()), _p(cfi.dev_in()), _p(scl.dev_in()), _p(rowmap.dev_in()), _p(enc), _p(l)),
               "sg_r2_decode")
    _corrupt("R2")


# ---- M24 ----------------------------------------------------------------------------------------------------------
def _bf_hist(args):
    dev, tb, sg, nseg, rfi, cfi, scl, counts = args
    _lib.check(_lib.lib().sg_m24_hist(_dev(), _st(), _p(dev.dev_in()), _p(tb.dev_in()), _p(sg.dev_in()), _i(nseg), _p(rfi.dev_in()),
                                      _p(cfi.dev_in()), _p(scl.dev_in()), _p(counts.dev_inout())), "sg_m24_hist")


def _bf_enc(args):
    dev, tb, sg, nseg, rfi, cfi, scl, remap, freq, cum, out, cap, out_len = args
    enc, _ = _tables(remap, freq, QR_PB, False)
    _lib.check(_lib.lib().sg_m24_encode(_dev(), _st(), _p(dev.dev_in()), _p(tb.dev_in()), _p(sg.dev_in()), _i(nseg), _p(rfi.dev_in()),
                                        _p(cfi.dev_in()), _p(scl.dev_in()), _p(enc), _p(out.dev_out()), _i(cap), _p(out_len.dev_out())),
               "sg_m24_encode")


def _bf_dec(args):
    stream, offs, dev, tb, sg, nseg, rfi, cfi, scl, remap, freq, cum, lut = args
    enc, l = _tables(remap, freq, QR_PB, True)
    o = offs.dev_in().view(torch.int64)
    e = _seg_ends(o, stream.size)
    _lib.check(_lib.lib().sg_m24_decode(_dev(), _st(), _p(stream.dev_in()), _p(o), _p(e), _p(dev.dev_inout()), _p(tb.dev_in()), _p(sg.dev_in()),
                                        _i(nseg), _p(rfi.dev_in()), _p(cfi.dev_in()), _p(scl.dev_in()), _p(enc), _p(l)), "sg_m24_decode")
    _corrupt("M24")


# ---- M6 (gpu_codec.py: Q8_0 files without a base) ---------------------------------------------------------------------
def _m6_tables(freq, lut):
    """the reference's full frequency array (a row per table, unused rows zero) -> encoder entries and symbol table"""
    key = ("m6", id(freq.st), freq.off)
    hit = _TABS.get(key)
    if hit is not None and (hit[1] is not None or not lut):
        _TABS.move_to_end(key)
        return hit[0], hit[1]
    sums = freq._h().reshape(-1, 256).sum(1, dtype=np.int64)
    if ((sums != 0) & (sums != (1 << QR_PB))).any():
        raise ValueError("coder tables: a row of frequencies does not sum to 2^PB (damaged table part)")
    ntab = sums.size
    f = freq.dev_in()
    enc = torch.empty(ntab * 256 * 2, dtype=torch.int32, device=f.device)
    l = torch.zeros(ntab << QR_PB, dtype=torch.uint8, device=f.device) if lut else None
    _lib.check(_lib.lib().sg_rans_tables(_dev(), _st(), _p(f), ntab, QR_PB, _p(enc), _p(l)), "sg_rans_tables")
    _TABS[key] = (enc, l, freq)
    while len(_TABS) > 6:
        _TABS.popitem(last=False)
    return enc, l


def _m6_hist(args):
    blocks, pos, meta, tfirst, ntens, colmap, n, counts = args
    _lib.check(_lib.lib().sg_m6_hist(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), _p(meta.dev_in()), _p(tfirst.dev_in()), _i(ntens),
                                     _p(colmap.dev_in()), _i(n), _p(counts.dev_inout())), "sg_m6_hist")


def _m6_enc(args):
    blocks, pos, meta, tfirst, ntens, colmap, n, freq, cum, out, cap, out_len = args
    enc, _ = _m6_tables(freq, False)
    _lib.check(_lib.lib().sg_m6_encode(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), _p(meta.dev_in()), _p(tfirst.dev_in()), _i(ntens),
                                       _p(colmap.dev_in()), _i(n), _p(enc), _p(out.dev_out()), _i(cap), _p(out_len.dev_out())), "sg_m6_encode")
    lens = out_len._h()
    if (lens == 0xffffffff).any():
        raise ValueError("M6: a segment's code outgrew its slot")


def _m6_dec(args):
    stream, offs, meta, tfirst, ntens, colmap, n, freq, cum, lut, blocks = args
    enc, l = _m6_tables(freq, True)
    o = offs.dev_in().view(torch.int64)
    e = _seg_ends(o, stream.size)
    _lib.check(_lib.lib().sg_m6_decode(_dev(), _st(), _p(stream.dev_in()), _p(o), _p(e), _p(meta.dev_in()), _p(tfirst.dev_in()), _i(ntens),
                                       _p(colmap.dev_in()), _i(n), _p(enc), _p(l), _p(blocks.dev_out())), "sg_m6_decode")
    _corrupt("M6")


def _corrupt(what):
    bits = ctypes.c_int(0)
    _lib.check(_lib.lib().sg_status_fetch(_dev(), _st(), ctypes.byref(bits)), "sg_status_fetch")
    if bits.value & 4:
        raise ValueError(f"{what}: corrupt coded stream")


def _row_hash(args):
    u, nr, rl, h = args
    _lib.check(_lib.lib().sg_row_hash(_dev(), _st(), _p(u.dev_in()), _i(nr), _i(rl), _p(h.dev_out())), "sg_row_hash")


def _build_lut(args):
    pass                                   # the decoders' symbol table is made with their encoder entries (_tables)


def _gather(args):
    out, cap, out_len, offs, nseg, dst = args
    if _i(nseg) == 0:
        return
    if (out_len._h() == 0xfffffffe).any():       # (the caller has read the lengths already: a host copy exists)
        raise ValueError("rANS encoder: a coded symbol has frequency 0 in its table")
    _lib.check(_lib.lib().sg_scan_gather(_dev(), _st(), _p(out.dev_in()), _i(cap), _p(out_len.dev_in()), _i(nseg), _p(dst.dev_out()),
                                         dst.size, _p(offs.dev_inout())), "sg_scan_gather")



# ---- QR (single-pass kernels) -------------------------------------------------------------------------------------
def _qr_common(T, F, P, imx):
    T = _i(T)
    if T in GRID_TYPES:
        from .. import tables
        tables.install(_dev())
    nb = F.size // QR_BS[T]
    ne = torch.empty(max(nb, 1), dtype=torch.uint8, device=F.dev_in().device)
    cnt = torch.zeros(1, dtype=torch.int64, device=ne.device)
    _lib.check(_lib.lib().sg_residual_blocks(_dev(), _st(), _p(F.dev_in()), _p(P.dev_in()), QR_BS[T], nb, _p(ne), _p(cnt)), "sg_residual_blocks")
    return T, ne


def _qr_hist(args):
    T, F, P, seed, tm, sg, nseg, counts, gk, imx, mv = args
    T, ne = _qr_common(T, F, P, imx)
    _lib.check(_lib.lib().sg_qr_hist(_dev(), _st(), T, _p(F.dev_in()), _p(P.dev_in()), _p(ne), _p(seed.dev_in()), _p(tm.dev_in()), _p(sg.dev_in()),
                                     _i(nseg), _p(imx.dev_in()), _p(counts.dev_inout()), _i(mv)), "sg_qr_hist")


def _qr_enc(args):
    T, F, P, seed, tm, sg, nseg, remap, freq, cum, out, cap, out_len, gk, imx, mv = args
    T, ne = _qr_common(T, F, P, imx)
    enc, _ = _tables(remap, freq, QR_PB, False)
    _lib.check(_lib.lib().sg_qr_encode(_dev(), _st(), T, _p(F.dev_in()), _p(P.dev_in()), _p(ne), _p(seed.dev_in()), _p(tm.dev_in()),
                                       _p(sg.dev_in()), _i(nseg), _p(imx.dev_in()), _p(enc), _p(out.dev_out()), _i(cap), _p(out_len.dev_out()),
                                       _i(mv)), "sg_qr_encode")


def _qr_dec(args):
    T, stream, offs, P, seed, tm, sg, nseg, remap, freq, cum, lut, F, gk, imx, mv = args
    T = _i(T)
    if T in GRID_TYPES:
        from .. import tables
        tables.install(_dev())
    enc, l = _tables(remap, freq, QR_PB, True)
    o = offs.dev_in().view(torch.int64)
    off = torch.cat([o, torch.tensor([stream.size], dtype=torch.int64, device=o.device)])
    _lib.check(_lib.lib().sg_qr_decode(_dev(), _st(), T, _p(stream.dev_in()), _p(off), _p(P.dev_in()), _p(seed.dev_in()), _p(tm.dev_in()),
                                       _p(sg.dev_in()), _i(nseg), _p(imx.dev_in()), _p(enc), _p(l), _p(F.dev_out()), _i(mv)), "sg_qr_decode")
    _corrupt("QR batch")


# ---- QR helpers for tensors without a BF16 seed ------------------------------------------------------------------------
def _block_fields(args):
    T, F, nblk, out = args
    _lib.check(_lib.lib().sg_qr_block_fields(_dev(), _st(), _i(T), _p(F.dev_in()), _i(nblk), _p(out.dev_out())), "sg_qr_block_fields")


def _blocks_from_fields(args):
    T, v, n, out = args
    _lib.check(_lib.lib().sg_qr_blocks_from_fields(_dev(), _st(), _i(T), _p(v.dev_in()), _i(n), _p(out.dev_out())), "sg_qr_blocks_from_fields")


def _intervals(args):
    T, F, nw, lo, hi = args
    _lib.check(_lib.lib().sg_qr_intervals(_dev(), _st(), _i(T), _p(F.dev_in()), _i(nw), _p(lo.dev_out()), _p(hi.dev_out())), "sg_qr_intervals")


def _weq(args):
    T, F, P, nw, out = args
    _lib.check(_lib.lib().sg_qr_weight_equal(_dev(), _st(), _i(T), _p(F.dev_in()), _p(P.dev_in()), _i(nw), _p(out.dev_out())), "sg_qr_weight_equal")


def _grid_h(args):
    T, F, nw, h = args
    if _i(T) in GRID_TYPES:
        from .. import tables
        tables.install(_dev())
    _lib.check(_lib.lib().sg_qr_grid_half_step(_dev(), _st(), _i(T), _p(F.dev_in()), _i(nw), _p(h.dev_out())), "sg_qr_grid_half_step")


# ---- M21 (gpu2.py / gpu3.py: Q8_0 files without a base) -------------------------------------------------------------------
def _m21_flags(d):
    return (1 if d.get("SIGN") else 0) | (2 if d.get("RANK") else 0) | (4 if d.get("HICF") else 0) | (8 if d.get("PREDA") else 0)


def _m21_tables(remap, freq, lut):
    return _tables(remap, freq, QR_PB, lut)


def _m21_lens(out_len, what):
    if (out_len._h() == 0xffffffff).any():
        raise RuntimeError(f"{what}: a segment's code outgrew its slot")


def _m21_hist_a(args, d):
    blocks, pos, skip, meta, ntens, n, bcf, spread, perm, rankof, scls, counts = args
    _lib.check(_lib.lib().sg_m21_hist_a(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), _p(skip.dev_in()), _p(meta.dev_in()), _i(ntens), _i(n),
                                        _p(bcf.dev_in()), _p(spread.dev_in()), _p(perm.dev_in()), _p(rankof.dev_in()), _p(scls.dev_in()),
                                        _m21_flags(d), d["SEGA"], _p(counts.dev_inout())), "sg_m21_hist_a")


def _m21_enc_a(args, d):
    blocks, pos, skip, meta, ntens, n, bcf, spread, perm, rankof, scls, remap, freq, cum, out, cap, out_len = args
    enc, _ = _m21_tables(remap, freq, False)
    _lib.check(_lib.lib().sg_m21_encode_a(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), _p(skip.dev_in()), _p(meta.dev_in()), _i(ntens), _i(n),
                                          _p(bcf.dev_in()), _p(spread.dev_in()), _p(perm.dev_in()), _p(rankof.dev_in()), _p(scls.dev_in()),
                                          _m21_flags(d), d["SEGA"], _p(enc), _p(out.dev_out()), _i(cap), _p(out_len.dev_out())), "sg_m21_encode_a")
    _m21_lens(out_len, "M21 phase A")


def _m21_dec_a(args, d):
    stream, offs, skip, meta, ntens, n, bcf, spread, perm, rankof, scls, remap, freq, cum, lut, blocks, pos = args
    enc, l = _m21_tables(remap, freq, True)
    o = offs.dev_in().view(torch.int64)
    e = _seg_ends(o, stream.size)
    _lib.check(_lib.lib().sg_m21_decode_a(_dev(), _st(), _p(stream.dev_in()), _p(o), _p(e), _p(skip.dev_in()), _p(meta.dev_in()), _i(ntens), _i(n),
                                          _p(bcf.dev_in()), _p(spread.dev_in()), _p(perm.dev_in()), _p(rankof.dev_in()), _p(scls.dev_in()),
                                          _m21_flags(d), d["SEGA"], _p(enc), _p(l), _p(blocks.dev_inout()), _p(pos.dev_inout())), "sg_m21_decode_a")
    _corrupt("M21 phase A")


def _m21_hist_b(args, d):
    blocks, pos, skip, meta, ntens, n, cfi, scls, row_m, qbase, G, counts = args
    _lib.check(_lib.lib().sg_m21_hist_b(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), _p(skip.dev_in()), _p(meta.dev_in()), _i(ntens), _i(n),
                                        _p(cfi.dev_in()), _p(scls.dev_in()), _p(row_m.dev_in()), _i(qbase), _i(G), _m21_flags(d), d["SEGB"],
                                        _p(counts.dev_inout())), "sg_m21_hist_b")


def _m21_enc_b(args, d):
    blocks, pos, skip, meta, ntens, n, cfi, scls, row_m, qbase, G, remap, freq, cum, out, cap, out_len = args
    enc, _ = _m21_tables(remap, freq, False)
    _lib.check(_lib.lib().sg_m21_encode_b(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), _p(skip.dev_in()), _p(meta.dev_in()), _i(ntens), _i(n),
                                          _p(cfi.dev_in()), _p(scls.dev_in()), _p(row_m.dev_in()), _i(qbase), _m21_flags(d), d["SEGB"], _p(enc),
                                          _p(out.dev_out()), _i(cap), _p(out_len.dev_out())), "sg_m21_encode_b")
    _m21_lens(out_len, "M21 phase B")


def _m21_dec_b(args, d):
    stream, offs, skip, meta, ntens, n, cfi, scls, row_m, qbase, G, remap, freq, cum, lut, blocks, pos = args
    enc, l = _m21_tables(remap, freq, True)
    o = offs.dev_in().view(torch.int64)
    e = _seg_ends(o, stream.size)
    _lib.check(_lib.lib().sg_m21_decode_b(_dev(), _st(), _p(stream.dev_in()), _p(o), _p(e), _p(skip.dev_in()), _p(meta.dev_in()), _i(ntens), _i(n),
                                          _p(cfi.dev_in()), _p(scls.dev_in()), _p(row_m.dev_in()), _i(qbase), _m21_flags(d), d["SEGB"], _p(enc), _p(l),
                                          _p(blocks.dev_inout()), _p(pos.dev_in())), "sg_m21_decode_b")
    _corrupt("M21 phase B")


def _m21_predict(args, d):
    blocks, first, nbr, C, rows, nrw, par, coef, K, mu, pint = args
    _lib.check(_lib.lib().sg_m21_predict(_dev(), _st(), _p(blocks.dev_in()), _i(first), _i(nbr), _i(C), _p(rows.dev_in()), _i(nrw), _p(par.dev_in()),
                                         _p(coef.dev_in()), _i(K), _p(mu.dev_in()), _p(pint.dev_inout())), "sg_m21_predict")


def _m21_predict_multi(args, d):
    blocks, ent_slot, ent_row, nent, CMAX, s_first, s_nbr, s_rbase, s_pbase, s_mubase, par, coef, K, mu, pint = args
    _lib.check(_lib.lib().sg_m21_predict_multi(_dev(), _st(), _p(blocks.dev_in()), _p(ent_slot.dev_in()), _p(ent_row.dev_in()), _i(nent), _i(CMAX),
                                               _p(s_first.dev_in()), _p(s_nbr.dev_in()), _p(s_rbase.dev_in()), _p(s_pbase.dev_in()),
                                               _p(s_mubase.dev_in()), _p(par.dev_in()), _p(coef.dev_in()), _i(K), _p(mu.dev_in()),
                                               _p(pint.dev_inout())), "sg_m21_predict_multi")


def _m21_c_common(a):
    skip, meta, st, sr, sn, ss, nseg, cfi, row_m, fbin, rbase, pint, pbase = a
    return (_p(skip.dev_in()), _p(meta.dev_in()), _p(st.dev_in()), _p(sr.dev_in()), _p(sn.dev_in()), _p(ss.dev_in()), _i(nseg), _p(cfi.dev_in()),
            _p(row_m.dev_in()), _p(fbin.dev_in()), _p(rbase.dev_in()), _p(pint.dev_in()), _p(pbase.dev_in()))


def _m21_hist_c(args, d):
    blocks, pos = args[:2]
    _lib.check(_lib.lib().sg_m21_hist_c(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), *_m21_c_common(args[2:15]), _m21_flags(d),
                                        _p(args[15].dev_inout())), "sg_m21_hist_c")


def _m21_enc_c(args, d):
    blocks, pos = args[:2]
    remap, freq, cum, out, cap, out_len = args[15:]
    enc, _ = _m21_tables(remap, freq, False)
    _lib.check(_lib.lib().sg_m21_encode_c(_dev(), _st(), _p(blocks.dev_in()), _p(pos.dev_in()), *_m21_c_common(args[2:15]), _m21_flags(d), _p(enc),
                                          _p(out.dev_out()), _i(cap), _p(out_len.dev_out())), "sg_m21_encode_c")
    _m21_lens(out_len, "M21 phase C")


def _m21_dec_c(args, d):
    stream, offs, seg0, pos = args[:4]
    remap, freq, cum, lut, blocks = args[17:]
    enc, l = _m21_tables(remap, freq, False)                  # the decoder keeps compact tables in shared memory: no symbol table
    o = offs.dev_in().view(torch.int64)
    e = _DEC_C_ENDS.get(id(offs.st))
    if e is None or e[0] is not offs.st:
        _DEC_C_ENDS.clear()
        e = (offs.st, _seg_ends(o, stream.size))
        _DEC_C_ENDS[id(offs.st)] = e
    _lib.check(_lib.lib().sg_m21_decode_c(_dev(), _st(), _p(stream.dev_in()), _p(o), _p(e[1]), _i(seg0), _p(pos.dev_inout()),
                                          *_m21_c_common(args[4:17]), _m21_flags(d), _p(enc), _p(l), _p(blocks.dev_inout())), "sg_m21_decode_c")
    _corrupt("M21 phase C")


_DEC_C_ENDS = {}           # the segment ends of the stream being decoded wave by wave (256 launches share them)


# ---- M30 (siblings.py) -----------------------------------------------------------------------------------------------
def _half_step(args):
    x, lo, hi, n, h = args
    _lib.check(_lib.lib().sg_sib_half_step(_dev(), _st(), _p(x.dev_in()), _p(lo.dev_in()), _p(hi.dev_in()), _i(n), _p(h.dev_out())),
               "sg_sib_half_step")


def _est_add(args):
    x, h, n, ws, wx = args
    _lib.check(_lib.lib().sg_sib_est_add(_dev(), _st(), _p(x.dev_in()), _p(h.dev_in()), _i(n), _p(ws.dev_inout()), _p(wx.dev_inout())),
               "sg_sib_est_add")


def _est_seed(args):
    ws, wx, x0, n, out = args
    _lib.check(_lib.lib().sg_sib_est_seed(_dev(), _st(), _p(ws.dev_in()), _p(wx.dev_in()), _p(x0.dev_in()), _i(n), _p(out.dev_out())),
               "sg_sib_est_seed")


# ---- detmath ---------------------------------------------------------------------------------------------------------
def _dm_log2(args):
    x, n, y = args
    _lib.check(_lib.lib().sg_dm_log2(_dev(), _st(), _p(x.dev_in()), _i(n), _p(y.dev_out())), "sg_dm_log2")


def _dm_exp2(args):
    x, n, y = args
    _lib.check(_lib.lib().sg_dm_exp2(_dev(), _st(), _p(x.dev_in()), _i(n), _p(y.dev_out())), "sg_dm_exp2")


def _dm_rows(args):
    x, nr, nc, square, out = args
    _lib.check(_lib.lib().sg_dm_rows(_dev(), _st(), _p(x.dev_in()), _i(nr), _i(nc), _i(square), _p(out.dev_out())), "sg_dm_rows")


def _dm_cols(args):
    x, nr, nc, square, m, has_mask, out = args
    _lib.check(_lib.lib().sg_dm_cols(_dev(), _st(), _p(x.dev_in()), _i(nr), _i(nc), _i(square), _p(m.dev_in()) if _i(has_mask) else None,
                                     _p(out.dev_out())), "sg_dm_cols")


def _dm_rows_d(args):
    x, nr, nc, square, out = args
    _lib.check(_lib.lib().sg_dm_rows_f64(_dev(), _st(), _p(x.dev_in()), _i(nr), _i(nc), _i(square), _p(out.dev_out())), "sg_dm_rows_f64")


def _dm_gram(args):
    X, nb, k, d, out = args
    _lib.check(_lib.lib().sg_dm_gram(_dev(), _st(), _p(X.dev_in()), _i(nb), _i(k), _i(d), _p(out.dev_out())), "sg_dm_gram")


def _dm_bdot(args):
    X, y, nb, k, d, out = args
    _lib.check(_lib.lib().sg_dm_bdot(_dev(), _st(), _p(X.dev_in()), _p(y.dev_in()), _i(nb), _i(k), _i(d), _p(out.dev_out())), "sg_dm_bdot")


def _dm_solve(args):
    A, b, nb, k, x = args
    _lib.check(_lib.lib().sg_dm_solve(_dev(), _st(), _p(A.dev_in()), _p(b.dev_in()), _i(nb), _i(k), _p(x.dev_out())), "sg_dm_solve")


# ---- dequantisers, float conversion ------------------------------------------------------------------------------------
def _dequant(T):
    qk, bs = QFUN[T][1], QFUN[T][2]

    def f(args):
        y, x, nrows, npr, rb = args
        n = _i(nrows) * _i(npr)
        if T in GRID_TYPES:
            from .. import tables
            tables.install(_dev())
        _lib.check(_lib.lib().sg_dequantize(_dev(), _st(), T, _p(y.dev_in()), _p(x.dev_out()), n), f"sg_dequantize(type {T})")
    return f


def _bf16_to_f32(a, y=None):
    from . import cupy_shim as cp
    if y is None:
        y = cp.empty(a.shape, np.float32)
    _lib.check(_lib.lib().sg_convert_float(_dev(), _st(), _p(a.dev_in()), _lib.DT_BF16, _p(y.dev_out()), _lib.DT_F32, a.size), "sg_convert_float")
    return y


_BOUND = {"bf_hist": _bf_hist, "bf_enc": _bf_enc, "bf_dec": _bf_dec, "v2_hist": _v2_hist, "v2_enc": _v2_enc, "v2_dec": _v2_dec, "row_hash": _row_hash, "build_lut": _build_lut,
          "gather": _gather, "qr_hist": _qr_hist, "qr_enc": _qr_enc, "qr_dec": _qr_dec, "block_fields": _block_fields,
          "blocks_from_fields": _blocks_from_fields, "intervals": _intervals, "weq": _weq, "grid_h": _grid_h,
          "dm_log2": _dm_log2, "dm_exp2": _dm_exp2, "dm_rows": _dm_rows, "dm_cols": _dm_cols, "dm_rows_d": _dm_rows_d,
          "dm_gram": _dm_gram, "dm_bdot": _dm_bdot, "dm_solve": _dm_solve,
          "hist": _m6_hist, "encode": _m6_enc, "decode": _m6_dec,
          "half_step": _half_step, "est_add": _est_add, "est_seed": _est_seed}
_BOUND_WITH_DEFINES = {"hist_a": _m21_hist_a, "enc_a": _m21_enc_a, "dec_a": _m21_dec_a, "hist_b": _m21_hist_b, "enc_b": _m21_enc_b,
                       "dec_b": _m21_dec_b, "predict": _m21_predict, "predict_multi": _m21_predict_multi, "hist_c": _m21_hist_c,
                       "enc_c": _m21_enc_c, "dec_c": _m21_dec_c}
for _t, (_name, _, _) in QFUN.items():
    _BOUND["k_dq_" + _name[len("quantize_"):]] = _dequant(_t)


def function(name, defines=None):
    f = _BOUND.get(name)
    g = _BOUND_WITH_DEFINES.get(name)
    if f is None and g is None:
        raise NotImplementedError(f"kernel '{name}' of the reference has no binding to libseedgrow.so "
                                  "(its CUDA source is never compiled here)")
    if g is not None:
        f = lambda args: g(args, defines or {})

    def launch(grid, block, args, shared_mem=0):
        f(args)
    launch.__name__ = name
    return launch


def elementwise(name):
    if name == "vq_bf16_to_f32":
        return _bf16_to_f32

    def missing(*a, **kw):
        raise NotImplementedError(f"elementwise kernel '{name}' of the reference has no binding")
    return missing
