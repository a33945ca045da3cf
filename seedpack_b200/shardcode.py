"""One coding batch over several GPUs: regrow, compare, code - each rank on its share, the exchange through the host.

The path shards by rANS segment (seedpack_b200.shard): a rank owns a contiguous range of a batch's segments, hence a
contiguous range of blocks, hence - per tensor - a range of rows (rounded outwards to whole rows; the quantisers work
row by row, so a few rows at the seams are regrown by two ranks).  A rank

  1. regrows its rows from the BF16 base on its GPU (GPUQuant) and compares them with the stored file's blocks
     (sg_residual_xor: how many bytes differ),
  2. models its segments and counts their symbols (QRCodec.hist),
  3. adds its counts to the other ranks' through the host (shard.sum_counts) and normalises the sum - every rank gets
     the same tables,
  4. codes its segments (QRCodec.code) and hands lengths and bytes to rank 0 (shard.gather_segments), which frames the
     batch (QRCodec.finish).

Nothing crosses from GPU to GPU; the batch's bytes do not depend on the number of ranks (tests/test_shard_gpu.py).
`make_case` builds a seeded stand-in for a window of a repository: BF16 tensors, an importance vector per tensor, and
stored files that were quantised with a slightly different importance vector and have some blocks disturbed.
"""
import numpy as np
import torch

from . import residual, shard
from .gpuquant import GPUQuant
from .qr import BS, GRID_TYPES, MODEL, QK, QRCodec, _layout
from .rans import normalize


class RowRange:
    """the bytes [first, first + len(data)) of a tensor of `total` bytes: what a rank holds of a tensor it shares;
    slices inside the held range come back as device tensors, anything else is an error"""

    def __init__(self, total, first, data):
        self.total, self.first, self.data = int(total), int(first), data

    def __len__(self):
        return self.total

    def __getitem__(self, s):
        a, z, step = s.indices(self.total)
        if step != 1 or a < self.first or z > self.first + self.data.numel():
            raise IndexError(f"bytes {a}..{z} are not in the rows this rank holds ({self.first}..{self.first + self.data.numel()})")
        return self.data[a - self.first:z - self.first]


def make_case(T, shapes, seed=1):
    """tensors [(rows, cols)] -> dict(bits: BF16 bits per tensor, imx / imx2: importance vectors for the prediction and for
    the stored file, T, shapes)"""
    rng = np.random.default_rng(seed)
    bits, imx, imx2 = [], [], []
    for nr, nc in shapes:
        x = rng.standard_normal((nr, nc), np.float32) * np.float32(0.02)
        u = np.ascontiguousarray(x).view(np.uint32)
        bits.append(((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16))
        w = np.exp(1.5 * rng.standard_normal(nc)).astype(np.float32)
        imx.append(w); imx2.append((w * np.exp(0.3 * rng.standard_normal(nc))).astype(np.float32))
    return dict(T=T, shapes=list(shapes), bits=bits, imx=imx, imx2=imx2)


def _disturb(f, first_block, bs):
    """XOR one byte of about every 200th block with a value that depends on the block's number in the batch only"""
    nb = f.numel() // bs
    b = torch.arange(first_block, first_block + nb, device=f.device, dtype=torch.int64)
    h = (b * 2654435761) & 0xffffffff
    pick = (h % 211) == 0
    idx = torch.nonzero(pick).reshape(-1)
    if idx.numel():
        pos = idx * bs + (h[idx] >> 8) % bs
        f[pos] ^= (1 + (h[idx] >> 16) % 255).to(torch.uint8)
    return f


class ShardedBatch:
    """this rank's share of one batch of type T over `world` ranks.  prepare() makes the stored file's blocks for the
    share (set-up: the file exists before anything is packed); run() is the path proper"""

    def __init__(self, case, rank, world, device=None, staged=True, group=None):
        """group: the torch.distributed group of the host exchange (gloo; default: the default group)"""
        self.case, self.rank, self.world, self.group = case, rank, world, group
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.gq, self.qc = GPUQuant(self.device.index), QRCodec(self.device.index, staged=staged)
        T = self.T = case["T"]
        bs, qk = BS[T], QK[T]
        self.nbs = [nr * nc // qk for nr, nc in case["shapes"]]
        tm, sg, _ = _layout(T, self.nbs)
        self.nseg = len(sg)
        self.segs = shard.segment_range(self.nseg, rank, world)
        s0, s1 = self.segs
        B0 = int(sg["b0"][s0]) if s1 > s0 else 0
        B1 = int(sg["b0"][s1 - 1] + sg["nb"][s1 - 1]) if s1 > s0 else 0
        self.rows = []                               # per tensor: (first row, rows) this rank regrows, (0, 0) if none
        for k, (nr, nc) in enumerate(case["shapes"]):
            g0, bpr = int(tm["blk0"][k]), nc // qk
            a, z = max(B0, g0) - g0, min(B1, g0 + self.nbs[k]) - g0
            self.rows.append((a // bpr, -(-z // bpr) - a // bpr) if z > a else (0, 0))
        # the seed buffer: the tensors' BF16 bits back to back (a window of the base file)
        self.seed_offs, o = [], 0
        for b in case["bits"]:
            self.seed_offs.append(o); o += b.nbytes
        self.seed = torch.from_numpy(np.concatenate([b.reshape(-1) for b in case["bits"]]).view(np.int16)).to(self.device)
        self.imx = torch.from_numpy(np.concatenate(case["imx"])).to(self.device)
        self.imx_offs, o = [], 0
        for w in case["imx"]:
            self.imx_offs.append(o); o += len(w)
        self.files = None

    def _rows_src(self, k):
        r0, n = self.rows[k]
        nc = self.case["shapes"][k][1]
        first = self.seed_offs[k] // 2 + r0 * nc
        return self.seed[first:first + n * nc], nc

    def _quantize(self, imxs):
        """this rank's rows of every tensor it shares, regrown -> {tensor: device bytes}"""
        ks = [k for k, (_, n) in enumerate(self.rows) if n]
        ys = self.gq.quantize_tensors(self.T, [self._rows_src(k) for k in ks], [imxs[k] for k in ks], device=True) if ks else []
        return dict(zip(ks, ys))

    def prepare(self):
        bs, qk = BS[self.T], QK[self.T]
        tm, _, _ = _layout(self.T, self.nbs)
        imx2 = [torch.from_numpy(w).to(self.device) for w in self.case["imx2"]]
        self.files = {}
        for k, y in self._quantize(imx2).items():
            nc = self.case["shapes"][k][1]
            first_block = int(tm["blk0"][k]) + self.rows[k][0] * (nc // qk)
            self.files[k] = _disturb(y.clone(), first_block, bs)
        torch.cuda.synchronize(self.device)
        return self

    def run(self, root=0, pool=None):
        """-> (the batch's bytes on rank `root`, None elsewhere; bytes of this rank's blocks that differ from their
        prediction).  With `pool` (a thread pool) the framing of the batch - level-19 zstd of its tables, host work that
        no other rank can help with - is handed to it and a future of the bytes comes back, so that the caller can go
        on to the next batch's GPU work; giving successive batches different roots spreads that work over the ranks"""
        T, bs, qk = self.T, BS[self.T], QK[self.T]
        use_imx = T in GRID_TYPES
        imxs = [self.imx[o:o + len(w)] for o, w in zip(self.imx_offs, self.case["imx"])]
        pred = self._quantize(imxs)
        differ = [residual.count_diff(self.files[k], pred[k], sync=False) for k in pred]
        items = []
        for k, (nr, nc) in enumerate(self.case["shapes"]):
            total = self.nbs[k] * bs
            if k in pred:
                first = self.rows[k][0] * (nc // qk) * bs
                f, p = RowRange(total, first, self.files[k]), RowRange(total, first, pred[k])
            else:
                f = p = RowRange(total, 0, torch.empty(0, dtype=torch.uint8, device=self.device))
            items.append((f, p, self.seed_offs[k], 30, nc, self.imx_offs[k] if use_imx else -1))
        state, counts = self.qc.hist(T, items, self.seed.view(torch.uint8), self.imx if use_imx else None, MODEL, self.segs)
        freq, used = normalize(shard.sum_counts(counts, self.group))
        lens, stream = self.qc.code(state, freq, used)
        lens, stream = shard.gather_segments(lens, stream, self.group, dst=root)
        ndiff = int(sum(int(d.item()) for d in differ))
        if lens is None:
            return None, ndiff
        if pool is not None:
            return pool.submit(self.qc.finish, freq, used, lens, stream, MODEL), ndiff
        return self.qc.finish(freq, used, lens, stream, MODEL), ndiff


def sharded_batch(T, case, rank, world, device=None):
    buf, _ = ShardedBatch(dict(case, T=T), rank, world, device).prepare().run()
    return buf
