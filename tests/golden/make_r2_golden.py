"""Writes tests/golden/r2_golden.npz: a small GGUF file of BF16 tensors (built with the reference's own minimal
writer, seedpack/seed.py gguf_bytes) and the parts of its R2 chunk as coded by the REFERENCE (seedpack/bf16v2.py
BF16v2.compress, --cpu path), plus detmath outputs on a sample.   python tests/golden/make_r2_golden.py <reference tree>"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import refimport  # noqa: E402

refimport.setup(sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"])
import numpy as np  # noqa: E402
from seedpack import bf16v2, detmath, seed  # noqa: E402
from seedpack.codecs_gguf import unpack  # noqa: E402
from tests import synth  # noqa: E402

rng = np.random.default_rng(5)


def bf(nr, npr, s, scale=1.0):
    b = synth.weights(nr, npr, seed=s, edge_cases=False)
    x = synth.bf16_bits_to_f32(b) * np.float32(scale)
    return synth.f32_to_bf16_bits(x).reshape(nr, npr)


emb = bf(200, 256, 1)
emb[150:] = emb[149]                      # untrained-token rows: exact duplicates
emb[7] = emb[3]
col_scale = np.exp(rng.normal(0, 0.5, 512)).astype(np.float32)
up = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(bf(96, 512, 4)).reshape(96, 512) * col_scale + np.float32(0.002)).reshape(96, 512)
tensors = [("token_embd.weight", (256, 200), 30, emb.tobytes()),
           ("blk.0.attn_norm.weight", (256,), 0, rng.normal(1, 0.05, 256).astype(np.float32).tobytes()),
           ("blk.0.attn_q.weight", (256, 128), 30, bf(128, 256, 2).tobytes()),
           ("blk.0.ffn_up.weight", (512, 96), 30, up.tobytes()),
           ("blk.1.attn_q.weight", (256, 128), 30, bf(128, 256, 3, 1.7).tobytes()),
           ("blk.1.ffn_up.weight", (512, 96), 30, bf(96, 512, 5).tobytes())]
data = seed.gguf_bytes(tensors)
codec = bf16v2.BF16v2(group_bytes=150_000)            # several groups
buf = codec.compress(data)
assert bytes(codec.decompress(buf)) == data
ch = unpack(buf)
out = {"data": np.frombuffer(data, np.uint8), "counts": np.asarray(codec.last_counts)}
for k in ("meta", "side", "tables", "lens", "stream"):
    out["part_" + k] = np.frombuffer(bytes(ch[k]), np.uint8)
x = np.concatenate([rng.normal(0, 1, 500), np.exp(rng.normal(0, 20, 500)), [0.0, 1.0, 2.0, 1e-310, 4.9e-324, np.inf]])
out["dm_x"] = x
out["dm_log2"] = np.asarray(detmath.log2(x))
y = np.concatenate([rng.normal(0, 30, 800), [0.0, 0.5, -0.5, 1023.9, -1074.5, 1024.0, -1080.0]])
out["dm_y"] = y
out["dm_exp2"] = np.asarray(detmath.exp2(y))
m = rng.normal(0, 1, (37, 53)).astype(np.float32)
out["dm_m"] = m
out["dm_rows"] = np.asarray(detmath.rows(m)); out["dm_rows_sq"] = np.asarray(detmath.rows(m, True))
out["dm_cols"] = np.asarray(detmath.cols(m)); out["dm_cols_sq"] = np.asarray(detmath.cols(m, True))
np.savez_compressed(os.path.join(HERE, "r2_golden.npz"), **out)
print("file", len(data), "coded stream", len(ch["stream"]), "parts", {k: len(ch[k]) for k in ch})
