"""Device twin of the row planner of the reference's M21 codec (seedpack/gpu3.py:252-346, `GPU3._row_matrix` and
`GPU3._plan_tensor`): for every row of a Q8_0 matrix (the token embedding) the K most similar rows of earlier waves and
the least-squares coefficients that predict the row from them.

The reference writes the planner as array operations (CuPy on its GPU path, NumPy on its CPU path): a matrix product of
int8-normalised rows against all earlier rows (151 936 x 151 936 / 2 x 1024 products for the 0.6B shape), masks and
arg-maxima over the products, gathers of the parents' rows.  Over the binding's array module those would run on the host,
for minutes.  Here the same steps run on the device with torch for the plumbing (element-wise IEEE float32 / float64
operations one at a time - no fused multiply-add -, exact integer products through an fp32 GEMM, as `detmath.sim8`
argues) and the reference's own `detmath` functions (bound kernels) for every sum, solve and logarithm.  The results are
the reference's bit for bit: the goldens of tests/test_archive_gpu.py with a Q8_0 file alone cover it.
"""
import ctypes

import numpy as np
import torch

from .. import _lib
from . import cupy_shim as cp

_NP = {torch.float32: np.float32, torch.float64: np.float64, torch.float16: np.float16, torch.int8: np.int8, torch.uint8: np.uint8,
       torch.int32: np.int32, torch.int64: np.int64, torch.bool: np.bool_}
_TT = {np.dtype(v): k for k, v in _NP.items()}
_LOW = -(1 << 62)              # key of a masked product


def dev(a, write=False):
    """binding array -> torch view of its device copy (uploaded if the host copy was the valid one)"""
    d = a.dev_inout() if write else a.dev_in()
    return d.view(_TT[np.dtype(a.dtype)]).reshape(a.shape)


def arr(t):
    """torch tensor -> binding array resident on the device"""
    a = cp.empty(tuple(t.shape), _NP[t.dtype])
    if t.numel():
        a.dev_out().view(t.dtype).reshape(t.shape).copy_(t)
    return a


def div(a, s):
    """a / s for a Python number s as a true IEEE division: torch turns a division by a host scalar into a
    multiplication by its reciprocal, which rounds differently"""
    return a / torch.tensor(s, dtype=a.dtype, device=a.device)


def row_matrix(self, allb, f, nb, rowlen):
    """the float32 weights of blocks f .. f + nb (gpu3.py:252-259): llama.cpp's dequantize_row_q8_0, code x scale"""
    W = cp.empty((nb * 32,), np.float32)
    d = cp.device_index()
    src = allb.dev_in()
    _lib.check(_lib.lib().sg_dequantize(d, ctypes.c_void_p(torch.cuda.current_stream(d).cuda_stream), 8,
                                        ctypes.c_void_p(src.data_ptr() + f * 34), ctypes.c_void_p(W.dev_out().data_ptr()), nb * 32),
               "sg_dequantize")
    return W.reshape(-1, rowlen)


def make(detmath):
    """-> plan_tensor(self, W, valid) over the reference's detmath module"""

    def f64(a):
        return dev(a).clone()

    def plan_tensor(self, W, valid):
        n, C = W.shape
        P, K, NC = self.WAVES, self.K, self.NCAND
        Wt = dev(W, write=True)
        vt = dev(valid.astype(np.bool_) if valid.dtype != np.bool_ else valid)
        D = Wt.device
        idx = torch.arange(n, device=D)
        wave = (idx * P) // n
        wstart = torch.searchsorted(wave, wave, right=False)                    # first row of the row's wave
        nvalid = float(int(vt.sum()))
        mu = div(f64(detmath.cols(W, mask=valid)), max(nvalid, 1.0)).to(torch.float32)
        col_w = detmath.cols(W, True, mask=valid)
        Wt -= mu                                                                # centred in place
        Wq = torch.empty((n, C), dtype=torch.int8, device=D)
        for i in range(0, n, 8192):
            x = Wt[i:i + 8192]
            nrm = torch.clamp_min(torch.sqrt(f64(detmath.rows(arr(x), True))), 1e-12)[:, None]
            Wq[i:i + 8192] = torch.clamp(torch.round(x.to(torch.float64) / nrm * 127), -127, 127).to(torch.int8)
        Wq[~vt] = 0
        # the K most similar valid rows of earlier waves; ties go to the lower row as arg-max over the products does
        par = torch.full((n, K), -1, dtype=torch.int32, device=D)
        CH = 512
        ws_host = wstart.cpu().numpy()
        sh = max(n.bit_length(), 1)                                             # key = product, then the lower row first
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False                           # the products must be exact
        Wf = [Wq[:, c0:c0 + detmath.SIM_COLS].float() for c0 in range(0, C, detmath.SIM_COLS)]
        for i in range(0, n, CH):
            j = min(i + CH, n)
            m = int(ws_host[j - 1])
            if m == 0:
                continue
            S = None
            for part in Wf:                                                     # every partial sum an integer below 2^24
                p = (part[i:j] @ part[:m].T).to(torch.int64)
                S = p if S is None else S + p
            key = S * (1 << sh) + ((1 << sh) - 1 - idx[:m])[None, :]
            ok = (idx[None, :m] < wstart[i:j, None]) & vt[None, :m]
            key = torch.where(ok, key, torch.full_like(key, _LOW))
            rows = torch.arange(j - i, device=D)
            for k in range(min(NC, K)):
                best, at = key.max(1)
                par[i:j, k] = torch.where(best > _LOW, at, torch.full_like(at, -1)).to(torch.int32)
                key[rows, at] = _LOW
            del S, key, ok
        del Wf
        torch.backends.cuda.matmul.allow_tf32 = tf32
        frac = torch.ones(n, dtype=torch.float32, device=D)
        coefs = torch.zeros((n, K), dtype=torch.float32, device=D)
        kuse = torch.zeros(n, dtype=torch.int32, device=D)
        col_res = torch.zeros(C, dtype=torch.float64, device=D)
        cost_side = 17 + self.COEF_BITS
        for i in range(0, n, 2048):
            j = min(i + 2048, n)
            r = j - i
            y = Wt[i:j]
            ya = arr(y)
            yy = torch.clamp_min(f64(detmath.rows(ya, True)), 1e-12)
            pj = par[i:j]
            Xa = Wt[torch.clamp_min(pj, 0).long()] * (pj >= 0)[..., None]
            best = torch.ones(r, dtype=torch.float64, device=D)
            bestk = torch.zeros(r, dtype=torch.int32, device=D)
            bestc = torch.zeros((r, K), dtype=torch.float32, device=D)
            best_cost = torch.zeros(r, dtype=torch.float64, device=D)           # cost (bits) of no parent
            res_best = y.clone()
            for k in (range(1, K + 1) if self.ADAPTIVE_K else (K,)):
                X = Xa[:, :k].contiguous()
                Xs = arr(X)
                A = dev(detmath.gram(Xs)) + (1e-3 * torch.eye(k, dtype=torch.float32, device=D))[None]
                c = dev(detmath.solve(arr(A), detmath.bdot(Xs, ya)))
                if self.COEF_BITS == 16:
                    c = c.to(torch.float16).to(torch.float32)
                else:
                    c = div(torch.clamp(torch.round(c * 64), -127, 127), 64)
                res = y.clone()
                for kk in range(k):                                             # in a fixed order, product and difference rounded apart
                    res = res - c[:, kk, None] * X[:, kk, :]
                f = torch.clamp(f64(detmath.rows(arr(res), True)) / yy, 1e-3, 4)
                cost = 0.5 * f64(detmath.log2(arr(f))) * (C - C // 32) + k * cost_side
                better = cost < best_cost
                best_cost = torch.where(better, cost, best_cost)
                best = torch.where(better, f, best)
                bestk = torch.where(better, torch.full_like(bestk, k), bestk)
                cpad = torch.zeros((r, K), dtype=torch.float32, device=D)
                cpad[:, :k] = c
                bestc = torch.where(better[:, None], cpad, bestc)
                res_best = torch.where(better[:, None], res, res_best)
            frac[i:j] = best.to(torch.float32)
            kuse[i:j] = bestk
            coefs[i:j] = bestc
            col_res += f64(detmath.cols(arr(res_best), True, mask=arr(vt[i:j])))
        valid_par = (torch.arange(K, device=D)[None, :] < kuse[:, None]) & vt[:, None]
        par = torch.where(valid_par, par, torch.full_like(par, -1))
        coefs = torch.where(valid_par, coefs, torch.zeros_like(coefs))
        frac = torch.where(kuse > 0, frac, torch.ones_like(frac))
        if self.COLRES:
            # column factor of the residual (1/8 octave of RMS) and row class relative to the mean
            cw = dev(col_w)
            gfrac = float(detmath.total(arr(col_res))) / max(float(detmath.total(col_w)), 1e-30)
            ratio = torch.clamp_min(col_res / torch.clamp_min(cw, 1e-30), 1e-6)
            cadj = torch.clamp(torch.round(4 * f64(detmath.log2(arr(ratio)))), -60, 0).to(torch.int8)
            fbin = torch.clamp(torch.round(f64(detmath.log2(arr(div(frac, max(gfrac, 1e-6))))) * 4), -40, 20).to(torch.int8)
        else:
            cadj = torch.zeros(C, dtype=torch.int8, device=D)
            fbin = torch.clamp(torch.round(f64(detmath.log2(arr(frac))) * 4), -40, 0).to(torch.int8)
        return arr(par), arr(coefs), arr(fbin), arr(mu), arr(cadj)

    return plan_tensor
