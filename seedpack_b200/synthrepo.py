"""Seeded synthetic GGUF model repositories: a BF16 base model (optionally split in shards), quantised files derived
from it, and an importance-matrix file - the inputs of `pack` when the real repositories the reference was measured
on are not at hand.  Shapes and value laws:

    weights      float32 N(0, 0.02^2), 0.1 % of the positions replaced by +-20 sigma, rounded to BF16 (nearest even)
    norm vectors N(1, 0.05^2), stored as F32 in every file
    importance   exp(N(0, 1.5^2)) per input column, one vector per tensor, legacy .dat layout
                 (seedpack/requant.py:59-91: count; per entry name, ncall, nval, values; trailing chunk count)
    quant files  every 2-D tensor quantised with the type its file's map names, by the quantiser the caller passes
                 (tests: the reference's C code; bench: the CUDA kernels), then `flip` of the blocks get one byte
                 XOR-ed with a random value so that predictions leave a residual
    tensor names blk.{i}.attn_q / attn_k / attn_v / attn_output / ffn_gate / ffn_up / ffn_down .weight,
                 blk.{i}.attn_norm / ffn_norm .weight, token_embd.weight, output_norm.weight[, output.weight]

The per-file type maps are this module's own (they only imitate the look of llama.cpp's mixed files: two or three
types per file).  Every random draw comes from numpy's PCG64 seeded with a digest of (repository seed, tensor or
file name), so a repository is reproducible tensor by tensor whatever the order of generation.

GGUF v3 layout written here: magic, version 3, tensor count, key-value count, key-values, tensor infos (name,
dims in ggml order - dims[0] is the row length -, type, offset), padding to general.alignment (32), tensor data
each padded to the alignment (seedpack/gguf_reader.py:49-80 reads exactly this).
"""
import hashlib
import os
import struct

import numpy as np

F32, F16, BF16 = 0, 1, 30
# ggml type -> (weights per block, bytes per block)
BLOCK = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 10: (256, 84), 11: (256, 110),
         12: (256, 144), 13: (256, 176), 14: (256, 210), 16: (256, 66), 17: (256, 74), 18: (256, 98), 19: (256, 50),
         20: (32, 18), 21: (256, 110), 22: (256, 82), 23: (256, 136), 29: (256, 56), 42: (64, 18)}
NEEDS_IMATRIX = {16, 17, 19, 22, 29}
ALIGN = 32

CONFIGS = {
    # 0.6B shape (28 layers, hidden 1024, FFN 3072, 16 q / 8 kv heads of 128, vocab 151936, tied embeddings)
    "c1": dict(layers=28, hidden=1024, ffn=3072, q_heads=16, kv_heads=8, head_dim=128, vocab=151936, tied=True,
               imatrix=False, shards=1, flip=0.005, alter=0.0,
               files={"Q8_0": "q8_0", "Q4_K_M": "q4_k_m", "Q6_K": "q6_k"}),
    # the same with 4 layers and a 4096-token vocabulary: the archive-parity tests' repository
    "c1-mini": dict(layers=4, hidden=1024, ffn=3072, q_heads=16, kv_heads=8, head_dim=128, vocab=4096, tied=True,
                    imatrix=False, shards=1, flip=0.005, alter=0.0,
                    files={"Q8_0": "q8_0", "Q4_K_M": "q4_k_m", "Q6_K": "q6_k"}),
    # the same without disturbed blocks, for sibling coding without the BF16 file (--method m30): a flipped byte can turn
    # a block's fp16 scale into a NaN, M30's column statistics over the FILES then hold NaNs, and the payload bits of a
    # NaN that arithmetic hands on differ between x86 and the GPU (the side information differs in those bits only)
    "sib-mini": dict(layers=4, hidden=1024, ffn=3072, q_heads=16, kv_heads=8, head_dim=128, vocab=4096, tied=True,
                     imatrix=False, shards=1, flip=0.0, alter=0.0,
                     files={"Q8_0": "q8_0", "Q4_K_M": "q4_k_m", "Q6_K": "q6_k"}),
    # one layer of the 0.6B shape and a 4096-token vocabulary: the bounded sample the CPU baseline is timed on
    "c1-micro": dict(layers=1, hidden=1024, ffn=3072, q_heads=16, kv_heads=8, head_dim=128, vocab=4096, tied=True,
                     imatrix=False, shards=1, flip=0.005, alter=0.0,
                     files={"Q8_0": "q8_0", "Q4_K_M": "q4_k_m", "Q6_K": "q6_k"}),
    # a repository of a few megabytes for tests of the host logic
    "c1-nano": dict(layers=2, hidden=256, ffn=768, q_heads=2, kv_heads=1, head_dim=128, vocab=512, tied=True,
                    imatrix=False, shards=1, flip=0.005, alter=0.0,
                    files={"Q8_0": "q8_0", "Q4_K_M": "q4_k_m", "Q6_K": "q6_k"}),
    # 9B shape (36 layers, hidden 4096, FFN 12288, 32 q / 8 kv heads of 128, vocab 151936, untied), 21 imatrix quants
    "c4": dict(layers=36, hidden=4096, ffn=12288, q_heads=32, kv_heads=8, head_dim=128, vocab=151936, tied=False,
               imatrix=True, shards=1, flip=0.005, alter=0.0, files="imatrix21"),
    # its reduction: 2 layers, hidden 512, FFN 1536, vocabulary 2048
    "c4-mini": dict(layers=2, hidden=512, ffn=1536, q_heads=4, kv_heads=2, head_dim=128, vocab=2048, tied=False,
                    imatrix=True, shards=1, flip=0.005, alter=0.0, files="imatrix21"),
    # two legacy quants made with ANOTHER importance matrix than the one in the repository (their metadata names 45
    # chunks, the repository's file 100): packing fits their importance back from the files (seedpack/imxfit.py)
    "fit-mini": dict(layers=2, hidden=512, ffn=1536, q_heads=4, kv_heads=2, head_dim=128, vocab=2048, tied=False,
                     imatrix=True, shards=1, flip=0.0, alter=0.0, files={"Q4_0": "q4_0", "Q5_1": "q5_1", "Q4_K_S": "q4_k_s"},
                     other_imatrix=("Q4_0", "Q5_1")),
    # 27B shape in two shards (64 layers, hidden 5120, FFN 17408, 40 q / 8 kv heads of 128), 24 imatrix quants,
    # 2 % of the tensors quantised with another type than their file's map names
    "c5": dict(layers=64, hidden=5120, ffn=17408, q_heads=40, kv_heads=8, head_dim=128, vocab=151936, tied=False,
               imatrix=True, shards=2, flip=0.005, alter=0.02, files="imatrix24"),
    "c5-mini": dict(layers=4, hidden=512, ffn=1536, q_heads=4, kv_heads=2, head_dim=128, vocab=2048, tied=False,
                    imatrix=True, shards=2, flip=0.005, alter=0.02, files="imatrix24"),
}

# file label -> (main type, second type for the "more bits" tensors, type of token_embd / output)
_MIX = {
    "q8_0": (8, 8, 8), "q6_k": (14, 14, 14), "q5_k_m": (13, 14, 14), "q5_k_s": (13, 13, 13), "q4_k_m": (12, 14, 14),
    "q4_k_s": (12, 12, 12), "q3_k_m": (11, 12, 14), "q3_k_s": (11, 11, 11), "q2_k": (10, 11, 14), "q5_0": (6, 6, 8),
    "q5_1": (7, 7, 8), "q4_0": (2, 2, 14), "q4_1": (3, 3, 14), "iq4_xs": (23, 23, 14), "iq4_nl": (20, 20, 14),
    "iq3_s": (21, 21, 12), "iq3_xxs": (18, 21, 12), "iq2_s": (22, 21, 12), "iq2_xs": (17, 22, 12),
    "iq2_xxs": (16, 17, 12), "iq1_m": (29, 16, 12), "iq1_s": (19, 16, 12), "q2_0": (42, 42, 14), "iq2_m": (22, 18, 12),
}
_SETS = {
    "imatrix21": ["iq1_m", "iq2_xxs", "iq2_xs", "iq2_s", "iq3_xxs", "iq3_s", "q2_k", "q3_k_s", "q3_k_m", "iq4_xs",
                  "iq4_nl", "q4_0", "q4_1", "q4_k_s", "q4_k_m", "q5_0", "q5_1", "q5_k_s", "q5_k_m", "q6_k", "q8_0"],
    "imatrix24": ["iq1_s", "iq1_m", "iq2_xxs", "iq2_xs", "iq2_s", "iq2_m", "iq3_xxs", "iq3_s", "q2_k", "q3_k_s",
                  "q3_k_m", "iq4_xs", "iq4_nl", "q4_0", "q4_1", "q4_k_s", "q4_k_m", "q5_0", "q5_1", "q5_k_s", "q5_k_m",
                  "q6_k", "q8_0", "q2_0"],
}


def _rng(seed, name):
    h = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=16).digest()
    return np.random.Generator(np.random.PCG64(int.from_bytes(h, "little")))


def bf16_round(x):
    """float32 array -> BF16 bits (uint16), round to nearest even on the bits (seedpack/repo3.py:687-688)"""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def tensor_shapes(cfg):
    """[(name, (cols, rows) in ggml order or (n,) for vectors)] in file order"""
    h, f = cfg["hidden"], cfg["ffn"]
    q, kv = cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
    out = [("token_embd.weight", (h, cfg["vocab"]))]
    for i in range(cfg["layers"]):
        p = f"blk.{i}."
        out += [(p + "attn_norm.weight", (h,)), (p + "attn_q.weight", (h, q)), (p + "attn_k.weight", (h, kv)),
                (p + "attn_v.weight", (h, kv)), (p + "attn_output.weight", (q, h)), (p + "ffn_norm.weight", (h,)),
                (p + "ffn_gate.weight", (h, f)), (p + "ffn_up.weight", (h, f)), (p + "ffn_down.weight", (f, h))]
    out.append(("output_norm.weight", (h,)))
    if not cfg["tied"]:
        out.append(("output.weight", (h, cfg["vocab"])))
    return out


def weights(seed, name, shape):
    """the BF16 bits (2-D, uint16, rows x cols) or F32 values (1-D) of one base tensor"""
    r = _rng(seed, name)
    if len(shape) == 1:
        return (1.0 + 0.05 * r.standard_normal(shape[0], np.float32)).astype(np.float32)
    cols, rows = shape
    x = r.standard_normal((rows, cols), np.float32) * np.float32(0.02)
    n = x.size
    k = int(round(0.001 * n))
    if k:
        pos = r.choice(n, k, replace=False) if n < (1 << 26) else r.integers(0, n, k)
        x.reshape(-1)[pos] = np.where(r.integers(0, 2, k) == 1, np.float32(0.4), np.float32(-0.4))
    return bf16_round(x).reshape(rows, cols)


_draw_weights = weights


def importance(seed, name, cols):
    """the repository's importance vector of a tensor; tensors fed by the same activations (q / k / v of a layer, gate /
    up of a layer) get the same vector, as a calibration run gives them"""
    shared = name.replace("attn_k", "attn_q").replace("attn_v", "attn_q").replace("ffn_up", "ffn_gate")
    return np.exp(1.5 * _rng(seed, "imx:" + shared).standard_normal(cols)).astype(np.float32)


def file_labels(cfg):
    return dict(cfg["files"]) if isinstance(cfg["files"], dict) else {l.upper(): l for l in _SETS[cfg["files"]]}


def type_of(label, name, layer, layers):
    """this module's own per-tensor type map of a quant file"""
    main, more, emb = _MIX[label]
    if name.startswith(("token_embd", "output.")):
        return emb
    if ("attn_v" in name or "ffn_down" in name) and layer % 2 == 0:
        return more
    return main


def _kv(key, vtype, value):
    kb = key.encode()
    head = struct.pack("<Q", len(kb)) + kb + struct.pack("<I", vtype)
    if vtype == 8:
        vb = value.encode()
        return head + struct.pack("<Q", len(vb)) + vb
    return head + struct.pack({4: "<I", 5: "<i", 6: "<f", 10: "<Q"}[vtype], value)


def write_gguf(path, meta, tensors):
    """path: a file name or a writable binary file object.  meta: [(key, gguf value type, value)]; tensors: [(name, dims in ggml order, ggml type, nbytes, payload())];
    payload() -> the tensor's bytes (called in order while the file is written, so only one is held at a time)"""
    head = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta)))
    for k, t, v in meta:
        head += _kv(k, t, v)
    off = 0
    for name, dims, ty, nb, _ in tensors:
        nbn = name.encode()
        head += struct.pack("<Q", len(nbn)) + nbn + struct.pack("<I", len(dims))
        head += struct.pack(f"<{len(dims)}Q", *dims) + struct.pack("<IQ", ty, off)
        off += -(-nb // ALIGN) * ALIGN
    head += bytes(-len(head) % ALIGN)
    import contextlib
    with (open(path, "wb") if isinstance(path, str) else contextlib.nullcontext(path)) as f:
        f.write(head)
        for name, dims, ty, nb, payload in tensors:
            b = payload()
            b = b.tobytes() if isinstance(b, np.ndarray) else bytes(b)
            if len(b) != nb:
                raise ValueError(f"{name}: {len(b)} bytes for a tensor of {nb}")
            f.write(b)
            f.write(bytes(-nb % ALIGN))


def gguf_bytes(meta, tensors):
    """write_gguf into memory -> bytes"""
    import io
    f = io.BytesIO()
    write_gguf(f, meta, tensors)
    return f.getvalue()


def _flip(seed, key, q, bs, share):
    """XOR one random byte of `share` of the blocks of q (uint8 array, in place) with a random non-zero value"""
    nb = q.size // bs
    k = int(round(share * nb))
    if not k:
        return
    r = _rng(seed, "flip:" + key)
    blocks = r.choice(nb, k, replace=False)
    q[blocks * bs + r.integers(0, bs, k)] ^= r.integers(1, 256, k).astype(np.uint8)


def make_repo(root, config, quantize, seed=0, name="synth", only=None, keep_weights=False):
    """write the repository `config` (a key of CONFIGS or a dict of the same form) under `root` ->
    {"base": [paths], "files": {label: path}, "extras": [paths], "bytes": total}.
    quantize(ggml type, BF16 bits as a (rows, cols) uint16 array, importance vector or None) -> uint8 array.
    only: labels of the quant files to make (default: all of the configuration); keep_weights: hold every base tensor
    in memory while the files are written (each is drawn once instead of once per file)"""
    cfg = CONFIGS[config] if isinstance(config, str) else config
    os.makedirs(root, exist_ok=True)
    shapes = tensor_shapes(cfg)
    L = cfg["layers"]
    held = {}

    def weights(seed, n, s, _draw=_draw_weights):
        if not keep_weights:
            return _draw(seed, n, s)
        if n not in held:
            held[n] = _draw(seed, n, s)
        return held[n]

    out = {"base": [], "files": {}, "extras": []}

    def layer_of(n):
        return int(n.split(".")[1]) if n.startswith("blk.") else 0

    # base model: one file, or shards named <name>-0000k-of-0000N.gguf holding consecutive tensors
    ns = cfg["shards"]
    cut = [len(shapes) * k // ns for k in range(ns + 1)]
    for k in range(ns):
        fn = f"{name}-BF16.gguf" if ns == 1 else f"{name}-BF16-{k + 1:05d}-of-{ns:05d}.gguf"
        meta = [("general.architecture", 8, "synth"), ("general.name", 8, name), ("general.alignment", 4, ALIGN),
                ("general.file_type", 4, 32)]
        write_gguf(os.path.join(root, fn), meta,
                   [(n, s, F32 if len(s) == 1 else BF16, (4 if len(s) == 1 else 2) * int(np.prod(s)),
                     (lambda n=n, s=s: weights(seed, n, s))) for n, s in shapes[cut[k]:cut[k + 1]]])
        out["base"].append(os.path.join(root, fn))
    imx = {}
    if cfg["imatrix"]:
        ents = [(n, importance(seed, n, s[0])) for n, s in shapes if len(s) == 2]
        buf = bytearray(struct.pack("<i", len(ents)))
        for n, v in ents:
            nb = n.encode()
            buf += struct.pack("<i", len(nb)) + nb + struct.pack("<ii", 1, len(v)) + v.tobytes()
        buf += struct.pack("<i", 100)
        p = os.path.join(root, "imatrix_synth.dat")
        with open(p, "wb") as f:
            f.write(buf)
        out["extras"].append(p)
        imx = dict(ents)
    p = os.path.join(root, "README.md")
    with open(p, "w") as f:
        f.write(f"# {name}\n\nSeeded synthetic repository (seed {seed}).\n")
    out["extras"].append(p)
    labels = file_labels(cfg)
    alt_types = sorted(t for t in BLOCK if t not in NEEDS_IMATRIX or cfg["imatrix"])
    for lab, mix in labels.items():
        if only is not None and lab not in only:
            continue
        tens = []
        for n, s in shapes:
            if len(s) == 1:
                tens.append((n, s, F32, 4 * s[0], (lambda n=n, s=s: weights(seed, n, s))))
                continue
            ty = type_of(mix, n, layer_of(n), L)
            r = _rng(seed, f"alter:{lab}:{n}")
            if cfg["alter"] and r.random() < cfg["alter"]:
                ty = int(r.choice([t for t in alt_types if t != ty and s[0] % BLOCK[t][0] == 0]))
            qk, bs = BLOCK[ty]
            nb = int(np.prod(s)) // qk * bs

            def payload(n=n, s=s, ty=ty, bs=bs, lab=lab):
                w = imx.get(n)
                if w is not None and lab in cfg.get("other_imatrix", ()):
                    # the unpublished matrix such a file was made with; tensors with the same input (q / k / v, gate / up)
                    # share it, as a calibration run gives them the same activations
                    shared = n.replace("attn_k", "attn_q").replace("attn_v", "attn_q").replace("ffn_up", "ffn_gate")
                    w = (w * np.exp(0.7 * _rng(seed, "imx2:" + shared).standard_normal(len(w)))).astype(np.float32)
                if w is None and ty in NEEDS_IMATRIX:
                    raise ValueError(f"{n}: type {ty} needs an importance matrix")
                q = np.array(quantize(ty, weights(seed, n, s), w), np.uint8, copy=True).reshape(-1)
                _flip(seed, f"{lab}:{n}", q, bs, cfg["flip"])
                return q

            tens.append((n, s, ty, nb, payload))
        meta = [("general.architecture", 8, "synth"), ("general.name", 8, name), ("general.alignment", 4, ALIGN),
                ("general.file_type", 4, 7), ("general.quantization_version", 4, 2)]
        if cfg["imatrix"]:
            meta += [("quantize.imatrix.file", 8, "imatrix_synth.dat"), ("quantize.imatrix.entries_count", 5, len(imx)),
                     ("quantize.imatrix.chunks_count", 5, 45 if lab in cfg.get("other_imatrix", ()) else 100)]
        fp = os.path.join(root, f"{name}-{lab}.gguf")
        write_gguf(fp, meta, tens)
        out["files"][lab] = fp
    out["bytes"] = sum(os.path.getsize(p) for p in out["base"] + list(out["files"].values()) + out["extras"])
    return out
