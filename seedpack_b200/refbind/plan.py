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


class Planner:
    """one matrix's plan, step by step on the device.  dm = the reference's detmath module (bound kernels); codec = the
    GPU3 instance whose class constants (WAVES, K, NCAND, COEF_BITS, ADAPTIVE_K, COLRES) choose the variant"""
    SEARCH_ROWS = 512          # rows whose products with all earlier rows are held at once
    FIT_ROWS = 2048            # rows fitted per batch of small systems
    UNIT_ROWS = 8192

    def __init__(self, dm, codec, W, valid):
        self.dm, self.codec, self.W = dm, codec, W
        self.n, self.cols = W.shape
        self.Wt = dev(W, write=True)
        self.valid = valid
        self.ok = dev(valid if valid.dtype == np.bool_ else valid.astype(np.bool_))
        self.D = self.Wt.device
        self.row = torch.arange(self.n, device=self.D)
        wave = (self.row * codec.WAVES) // self.n
        self.wave_first = torch.searchsorted(wave, wave, right=False)          # first row of each row's wave

    def sums(self, a, *more, **kw):
        """a detmath reduction -> float64 tensor of its result"""
        return dev(a(*more, **kw)).clone()

    def centre(self):
        """subtract the mean of the valid rows (in place) -> (mean float32, column energy before centring)"""
        count = max(float(int(self.ok.sum())), 1.0)
        mean = div(self.sums(self.dm.cols, self.W, mask=self.valid), count).to(torch.float32)
        energy = self.dm.cols(self.W, True, mask=self.valid)
        self.Wt -= mean
        return mean, energy

    def unit_rows(self):
        """rows scaled to unit length and rounded to int8 (exact similarities afterwards); rows left out are zero"""
        U = torch.empty((self.n, self.cols), dtype=torch.int8, device=self.D)
        for a in range(0, self.n, self.UNIT_ROWS):
            x = self.Wt[a:a + self.UNIT_ROWS]
            length = torch.clamp_min(torch.sqrt(self.sums(self.dm.rows, arr(x), True)), 1e-12)[:, None]
            U[a:a + self.UNIT_ROWS] = torch.clamp(torch.round(x.to(torch.float64) / length * 127), -127, 127).to(torch.int8)
        U[~self.ok] = 0
        return U

    def nearest(self, U):
        """-> (n, K) int32: the K most similar valid rows of earlier waves, best first, -1 where there is none.  A product
        of int8 rows over at most SIM_COLS columns is an integer below 2^24, exact in an fp32 GEMM whatever its order; the
        key puts the lower row first among equal products, as a first-maximum search does"""
        K = min(self.codec.NCAND, self.codec.K)
        parents = torch.full((self.n, self.codec.K), -1, dtype=torch.int32, device=self.D)
        first = self.wave_first.cpu().numpy()
        bits = max(self.n.bit_length(), 1)
        step = self.dm.SIM_COLS
        parts = [U[:, c:c + step].float() for c in range(0, self.cols, step)]
        keep = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for a in range(0, self.n, self.SEARCH_ROWS):
                b = min(a + self.SEARCH_ROWS, self.n)
                m = int(first[b - 1])
                if m == 0:
                    continue
                dots = None
                for part in parts:
                    d = (part[a:b] @ part[:m].T).to(torch.int64)
                    dots = d if dots is None else dots + d
                key = dots * (1 << bits) + ((1 << bits) - 1 - self.row[:m])[None, :]
                allowed = (self.row[None, :m] < self.wave_first[a:b, None]) & self.ok[None, :m]
                key = torch.where(allowed, key, torch.full_like(key, _LOW))
                line = torch.arange(b - a, device=self.D)
                for k in range(K):
                    top, at = key.max(1)
                    parents[a:b, k] = torch.where(top > _LOW, at, torch.full_like(at, -1)).to(torch.int32)
                    key[line, at] = _LOW
                del dots, key, allowed
        finally:
            torch.backends.cuda.matmul.allow_tf32 = keep
        return parents

    def stored(self, c):
        """coefficients as the archive holds them: fp16, or int8 in steps of 1/64"""
        if self.codec.COEF_BITS == 16:
            return c.to(torch.float16).to(torch.float32)
        return div(torch.clamp(torch.round(c * 64), -127, 127), 64)

    def fit(self, parents):
        """least squares of every row on its parents -> (energy left / energy float32, parents used int32,
        coefficients (n, K) float32, column energy of what is left float64)"""
        dm, K, D = self.dm, self.codec.K, self.D
        left = torch.ones(self.n, dtype=torch.float32, device=D)
        weights = torch.zeros((self.n, K), dtype=torch.float32, device=D)
        used = torch.zeros(self.n, dtype=torch.int32, device=D)
        col_left = torch.zeros(self.cols, dtype=torch.float64, device=D)
        side_bits = 17 + self.codec.COEF_BITS
        free = self.cols - self.cols // 32                                      # codes the prediction helps: all but one a block
        for a in range(0, self.n, self.FIT_ROWS):
            b = min(a + self.FIT_ROWS, self.n)
            y = self.Wt[a:b]
            y_arr = arr(y)
            energy = torch.clamp_min(self.sums(dm.rows, y_arr, True), 1e-12)
            pa = parents[a:b]
            P = self.Wt[torch.clamp_min(pa, 0).long()] * (pa >= 0)[..., None]
            win_left = torch.ones(b - a, dtype=torch.float64, device=D)
            win_k = torch.zeros(b - a, dtype=torch.int32, device=D)
            win_c = torch.zeros((b - a, K), dtype=torch.float32, device=D)
            win_bits = torch.zeros(b - a, dtype=torch.float64, device=D)       # no parent: 0 bits against itself
            win_rest = y.clone()
            for k in (range(1, K + 1) if self.codec.ADAPTIVE_K else (K,)):
                X = P[:, :k].contiguous()
                X_arr = arr(X)
                normal = dev(dm.gram(X_arr)) + (1e-3 * torch.eye(k, dtype=torch.float32, device=D))[None]
                c = self.stored(dev(dm.solve(arr(normal), dm.bdot(X_arr, y_arr))))
                rest = y.clone()
                for q in range(k):                                              # product and difference rounded apart, in index order
                    rest = rest - c[:, q, None] * X[:, q, :]
                share = torch.clamp(self.sums(dm.rows, arr(rest), True) / energy, 1e-3, 4)
                bits = 0.5 * self.sums(dm.log2, arr(share)) * free + k * side_bits
                wins = bits < win_bits
                win_bits = torch.where(wins, bits, win_bits)
                win_left = torch.where(wins, share, win_left)
                win_k = torch.where(wins, torch.full_like(win_k, k), win_k)
                padded = torch.zeros((b - a, K), dtype=torch.float32, device=D)
                padded[:, :k] = c
                win_c = torch.where(wins[:, None], padded, win_c)
                win_rest = torch.where(wins[:, None], rest, win_rest)
            left[a:b] = win_left.to(torch.float32)
            used[a:b] = win_k
            weights[a:b] = win_c
            col_left += self.sums(dm.cols, arr(win_rest), True, mask=arr(self.ok[a:b]))
        return left, used, weights, col_left

    def classes(self, left, col_left, energy):
        """-> (row class int8, column adjustment int8): quarter octaves of the energy the prediction leaves"""
        dm = self.dm
        if self.codec.COLRES:
            whole = float(dm.total(arr(col_left))) / max(float(dm.total(energy)), 1e-30)
            ratio = torch.clamp_min(col_left / torch.clamp_min(dev(energy), 1e-30), 1e-6)
            col_adj = torch.clamp(torch.round(4 * self.sums(dm.log2, arr(ratio))), -60, 0).to(torch.int8)
            row_cls = torch.clamp(torch.round(self.sums(dm.log2, arr(div(left, max(whole, 1e-6)))) * 4), -40, 20).to(torch.int8)
        else:
            col_adj = torch.zeros(self.cols, dtype=torch.int8, device=self.D)
            row_cls = torch.clamp(torch.round(self.sums(dm.log2, arr(left)) * 4), -40, 0).to(torch.int8)
        return row_cls, col_adj


def make(detmath):
    """-> the replacement of GPU3._plan_tensor(self, W, valid) over the reference's detmath module: parents (n, K) int32,
    coefficients (n, K) float32, row classes int8, column means float32, column adjustments int8"""

    def plan_tensor(self, W, valid):
        pl = Planner(detmath, self, W, valid)
        mean, energy = pl.centre()
        parents = pl.nearest(pl.unit_rows())
        left, used, weights, col_left = pl.fit(parents)
        live = (torch.arange(self.K, device=pl.D)[None, :] < used[:, None]) & pl.ok[:, None]
        parents = torch.where(live, parents, torch.full_like(parents, -1))
        weights = torch.where(live, weights, torch.zeros_like(weights))
        left = torch.where(used > 0, left, torch.ones_like(left))
        row_cls, col_adj = pl.classes(left, col_left, energy)
        return arr(parents), arr(weights), arr(row_cls), arr(mean), arr(col_adj)

    return plan_tensor
