"""Small Forilorn configurations for tests, and a writer of random weights for them.

The configurations differ from one another in every size and option: heads over one, some and as many key/value
heads; head sizes of 16 to 128; chunked masks shorter than a page, across page borders, of one position and none;
latent layers with windows of 1, across a page border and none, rotary parts narrower than, as wide as and wider
than the plain part, a rotation of all of the rotary part and of a part of it; layers without a feed-forward; with and
without the pair table; stream multipliers of 1 and other values; widths that are no multiple of 8.

Weights are drawn so that faults show: score scales that leave attention far from uniform (scores of standard
deviation about 1.5), norm weights stored around zero with a spread of 0.1.  They are stored in bfloat16, so a
32-bit run and a bfloat16 run compute on the same numbers.
"""
import json
import math
import os

import torch

from rustyllm_b200.weights.safetensors_io import write_safetensors


def rot(dims, base):
    return {"dims": dims, "base": base}


def attention(heads, kv_heads, dim, chunk=None, r=None, ff=None, sharp=1.5):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": sharp / math.sqrt(dim)}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if r is not None:
        m["rot"] = r
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, r=None, ff=None, sharp=1.5):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": sharp / math.sqrt(dim + rot_dim)}
    if window is not None:
        m["mask"] = {"size": window}
    if r is not None:
        m["rot"] = r
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # small heads, chunks shorter than a page and across a page border, a window shorter than a page, a layer without a
    # feed-forward, a pair table, a rotation of half of a head
    "P": {"architecture": "Forilorn", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
          "embedding": {"scale": 3.0, "bigram": {"buckets": 61, "mul_prev": 7, "mul_cur": 13}},
          "layers": [attention(4, 2, 16, chunk=9, r=rot(8, 100.0), ff=40),
                     latent(3, 24, 8, 20, 40, 32, window=5, r=rot(8, 10000.0), ff=24),
                     attention(2, 2, 32, chunk=70, r=rot(32, 10000.0)),
                     latent(2, 8, 16, 8, 16, 24, window=70, r=rot(16, 500.0), ff=56)]},
    # head sizes 64 and 128 (the tensor-core attention shapes), one key/value head for four query heads, chunks across
    # two page borders and of exactly a page, a layer that sees everything, no pair table, a window across a page border
    "Q": {"architecture": "Forilorn", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
          "embedding": {"scale": 11.0},
          "layers": [attention(4, 1, 64, chunk=130, r=rot(64, 10000.0), ff=96),
                     latent(2, 32, 16, 48, 24, 64, window=65, r=rot(16, 10000.0), ff=64),
                     attention(2, 2, 128, chunk=64, r=rot(32, 1.0e6), ff=72),
                     attention(4, 2, 64, chunk=None, r=rot(16, 5000.0), ff=None)]},
    # a width that is no multiple of 8, an odd vocabulary, a latent layer first, windows of 1 and none, a chunk of 1 and
    # none, no rotation in one layer of each kind, a rotation of a part of the rotary part, multipliers of 1
    "R": {"architecture": "Forilorn", "vocab": 53, "width": 44, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
          "embedding": {"scale": 1.0, "bigram": {"buckets": 5, "mul_prev": 1, "mul_cur": 1}},
          "layers": [latent(4, 12, 8, 16, 20, 40, window=1, r=rot(4, 100.0), ff=16),
                     attention(6, 3, 18, chunk=1, r=None, ff=20),
                     latent(1, 40, 6, 10, 36, 12, window=None, r=None, ff=None),
                     attention(3, 3, 16, chunk=None, r=rot(16, 10000.0), ff=32)]},
}


def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "final.norm": (d,)}
    bg = cfg.get("embedding", {}).get("bigram")
    if bg:
        out["bigram"] = (bg["buckets"] + 1, d)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (d,)
        q = p + "mix."
        if l["type"] == "attention":
            H, G, hd = m["heads"], m["kv_heads"], m["dim"]
            out[q + "q"], out[q + "k"], out[q + "g"], out[q + "o"] = (H * hd, d), (G * hd, d), (H * hd, d), (d, H * hd)
        else:
            H, hd, rd, vd, rq, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out[q + "dq"], out[q + "dq.norm"], out[q + "uq"] = (rq, d), (rq,), (H * (hd + rd), rq)
            out[q + "dkv"], out[q + "dkv.norm"] = (rk + rd, d), (rk,)
            out[q + "uk"], out[q + "uv"], out[q + "g"], out[q + "o"] = (H * hd, rk), (H * vd, rk), (H, d), (d, H * vd)
        if l["mlp"] is not None:
            out[p + "norm2"] = (d,)
            out[p + "mlp.up"], out[p + "mlp.down"] = (l["mlp"]["ff"], d), (d, l["mlp"]["ff"])
    return out


def draw_weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * z                                    # stored around zero: the model multiplies by 1 + w
        elif name.endswith("dq.norm") or name.endswith("dkv.norm"):
            t = 1.0 + 0.1 * z                              # plain weights
        elif name == "embed":
            t = z / max(1.0, cfg.get("embedding", {}).get("scale", 1.0)) * 1.0
        elif name == "bigram":
            t = 0.5 * z
        elif leaf == "g":
            t = 1.5 * z / math.sqrt(shape[1])
        else:
            t = z / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16)
    return out


def random_config(seed):
    """A configuration with every size drawn at random."""
    import random
    rng = random.Random(seed)
    width = rng.choice([24, 36, 40, 56, 72, 100, 136])
    layers = []
    for _ in range(rng.randrange(1, 5)):
        ff = rng.choice([None, 8, 20, 48, 100])
        if rng.random() < 0.55:
            heads = rng.choice([1, 2, 3, 4, 6, 8])
            kv = rng.choice([g for g in range(1, heads + 1) if heads % g == 0])
            dim = rng.choice([8, 16, 18, 24, 32, 50, 64, 128])
            r = None
            if rng.random() < 0.8:
                r = rot(rng.choice([x for x in (2, 4, 8, 16, dim) if x <= dim and x % 2 == 0]), rng.choice([100.0, 10000.0, 200000.0]))
            layers.append(attention(heads, kv, dim, chunk=rng.choice([None, 1, 2, 5, 33, 63, 64, 65, 100, 128, 129]), r=r, ff=ff,
                                    sharp=rng.choice([0.5, 1.5, 3.0])))
        else:
            rd = rng.choice([0, 2, 4, 8, 16, 32])
            r = None
            if rd and rng.random() < 0.85:
                r = rot(rng.choice([x for x in (2, 4, rd) if x <= rd]), rng.choice([100.0, 10000.0]))
            layers.append(latent(rng.choice([1, 2, 3, 5, 8]), rng.choice([8, 12, 16, 32, 64]), rd, rng.choice([4, 8, 12, 24, 64]),
                                 rng.choice([8, 12, 24, 40]), rng.choice([8, 16, 24, 48, 96, 128]),
                                 window=rng.choice([None, 1, 2, 5, 33, 63, 64, 65, 100, 129]), r=r, ff=ff, sharp=rng.choice([0.5, 1.5, 3.0])))
    cfg = {"architecture": "Forilorn", "vocab": rng.choice([17, 64, 101, 300]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "residual_mult": rng.choice([0.3, 0.5, 1.0, 1.4]),
           "embedding": {"scale": rng.choice([1.0, 4.0, 9.5])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["embedding"]["bigram"] = {"buckets": rng.choice([1, 7, 64, 499]), "mul_prev": rng.choice([0, 1, 29, 1000003]),
                                      "mul_cur": rng.choice([0, 1, 19, 999983])}
    return cfg


def write_model(name, path, seed=None, cfg=None):
    cfg = cfg or CONFIGS[name]
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), draw_weights(cfg, seed if seed is not None else sum(map(ord, name))))
    return path
