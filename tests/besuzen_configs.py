"""Small Besuzen configurations for tests, and a writer of random weights for them.

The configurations differ from one another in every size and option: parallel layers first, last and in the middle;
attention heads over one, some and as many key/value heads; key heads narrower than, wider than and equal to value
heads; rotation of a part of a head and of all of it; one, two and three layers that blend their values (and none);
time mixers of one head and several, head sizes 8 to 64, decay projections 3 to 16 wide; mixer factors of 1 and
others; dense feed-forwards, experts in groups (keep one, keep some, no groups), top = 1 and top = all, with and
without the shared expert, layers without a feed-forward; widths that are and are not multiples of 8; embedding and
logit factors of 1 and others.

Weights are drawn so that faults show: queries and keys large enough that attention is far from uniform, router
logits of standard deviation 1.5, decays whose offsets reach from -6 (a memory of hundreds of tokens) to 0.5 (a few
tokens), bonuses of both signs, blending factors between 0.2 and 0.8.  They are stored in bfloat16, so a 32-bit run and a
bfloat16 run compute on the same numbers.

``router_std``: the standard deviation of the router's logits.  1.5 (the default) makes lively routers whose scores
often lie close together; the bfloat16 runs of the engine tests draw 6, decisive routers: a close call that falls
the other way once the router's input is rounded replaces an expert (with one expert a token, the token's whole
feed-forward), which is no fault of a kernel and would drown the bound that a wrong key or a lost state must break.
The 32-bit runs keep the lively routers, and the router's kernels are tested on lively inputs by themselves.
"""
import json
import math
import os

import torch

from rustyllm_b200.weights.safetensors_io import write_safetensors


def att(heads, kv_heads, dim, vdim, scale, rot=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if v_mix:
        m["v_mix"] = True
    return m


def attention(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def parallel(left, right_heads, right_dim, ls, rs, mlp):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": {"heads": right_heads, "dim": right_dim}, "left_scale": ls, "right_scale": rs}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": r, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


# the inner width of the decay projections is in no key of config.json (the tensors' shapes give it): per configuration
DECAY_RANK = {"A": 5, "B": 3, "C": 16}

CONFIGS = {
    # a parallel layer first (one key/value head, value heads narrower than key heads), then two blending layers with
    # half the head rotated, the second without a feed-forward; experts in three groups of which two are kept
    "A": {"architecture": "Besuzen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5}, "logit_scale": 0.7,
          "layers": [parallel(att(4, 1, 16, 8, 0.3), 2, 16, 0.8, 1.3, dense(48)),
                     attention(att(6, 3, 24, 16, 0.25, rot=(12, 10000.0), v_mix=True), moe(6, 2, 16, groups=(3, 2), shared=24)),
                     attention(att(3, 3, 8, 16, 0.4, rot=(8, 100.0), v_mix=True), None)]},
    # a width that is no multiple of 8 (no tensor-core product takes it); an attention layer without blending first, all
    # experts chosen, no groups, no shared expert; mixer factors, embedding factor and logit factor of 1; as many
    # key/value heads as heads; value heads wider than key heads; a time mixer of one head
    "B": {"architecture": "Besuzen", "vocab": 53, "width": 44, "norm": {"eps": 1e-6},
          "layers": [attention(att(2, 2, 12, 20, 0.35, rot=(12, 500.0)), moe(3, 3, 12)),
                     parallel(att(2, 2, 10, 12, 0.3), 1, 20, 1.0, 1.0, None),
                     parallel(att(3, 1, 8, 8, 0.5), 3, 8, 0.5, 2.0, dense(36))]},
    # heads of 64 with values as wide as keys (the tensor-core attention kernels take the element-wise gate), three
    # blending layers around a parallel layer with a time mixer of 64-wide heads, experts in four groups of which one
    # is kept, one expert a token
    "C": {"architecture": "Besuzen", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5}, "logit_scale": 1.8,
          "layers": [attention(att(4, 2, 64, 64, 0.125, rot=(64, 300000.0), v_mix=True), dense(96)),
                     attention(att(2, 2, 64, 64, 0.125, rot=(32, 10000.0), v_mix=True), moe(8, 1, 32, groups=(4, 1), shared=32)),
                     parallel(att(2, 2, 64, 64, 0.11), 2, 64, 0.75, 0.45, moe(4, 2, 24, groups=(2, 2))),
                     attention(att(4, 2, 64, 64, 0.125, rot=(64, 300000.0), v_mix=True), dense(64))]},
}


def tensor_shapes(cfg: dict, rank: int) -> dict:
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = (d,)
        out[p + "norm2"] = (d,)

        def att_shapes(q, m, per_head):
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * dk, d), q + "q.b": (H * dk,), q + "k": (G * dk, d), q + "k.b": (G * dk,),
                        q + "v": (G * dv, d), q + "v.b": (G * dv,), q + "g": (H if per_head else H * dv, d),
                        q + "o": (d, H * dv)})
        if l["type"] == "attention":
            att_shapes(p + "mix.", l["mixer"], False)
            if l["mixer"].get("v_mix"):
                out[p + "mix.vmix"] = ()
        else:
            att_shapes(p + "mix.left.", l["mixer"]["left"], True)
            r = l["mixer"]["right"]
            inner = r["heads"] * r["dim"]
            q = p + "mix.right."
            for s in "rkvgw":
                out[q + "mu." + s] = (d,)
            for s in "rkvg":
                out[q + s] = (inner, d)
            out.update({q + "w1": (rank, d), q + "w2": (inner, rank), q + "w0": (inner,), q + "u": (r["heads"], r["dim"]),
                        q + "norm": (inner,), q + "o": (d, inner)})
        mlp = l["mlp"]
        if mlp is None:
            continue
        q = p + "mlp."
        if mlp["kind"] == "dense":
            out.update({q + "gate": (mlp["ff"], d), q + "up": (mlp["ff"], d), q + "down": (d, mlp["ff"])})
        else:
            F = mlp["expert"]["ff"]
            out[q + "router"] = (mlp["router"]["experts"], d)
            for e in range(mlp["router"]["experts"]):
                out.update({f"{q}e{e}.gate": (F, d), f"{q}e{e}.up": (F, d), f"{q}e{e}.down": (d, F)})
            if mlp.get("shared") is not None:
                S = mlp["shared"]["ff"]
                out.update({q + "shared.gate": (S, d), q + "shared.up": (S, d), q + "shared.down": (d, S), q + "shared.sg": (1, d)})
    return out


def draw_weights(cfg: dict, rank: int, seed: int, router_std: float = 1.5) -> dict:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        last = name.rsplit(".", 1)[-1]

        def normal(std):
            return torch.randn(shape, generator=g, dtype=torch.float64) * std
        if last in ("norm1", "norm2") or name == "final.norm" or name.endswith("right.norm"):
            t = 1.0 + normal(0.15)
        elif name.endswith(".b"):
            t = normal(0.3)
        elif last == "vmix":
            t = 0.2 + 0.6 * torch.rand((), generator=g, dtype=torch.float64)
        elif ".mu." in name:
            t = torch.rand(shape, generator=g, dtype=torch.float64)
        elif last == "w0":
            t = -6.0 + 6.5 * torch.rand(shape, generator=g, dtype=torch.float64)
        elif last == "u":
            t = normal(0.5)
        elif last == "w2":
            t = normal(1.0 / math.sqrt(shape[1]))
        elif last == "router":
            t = normal(router_std / math.sqrt(shape[1]))
        elif last == "sg":
            t = normal(2.0 / math.sqrt(shape[1]))
        elif name == "embed":
            t = normal(1.0)
        elif last in ("q", "k") and ".right." not in name:
            t = normal(2.0 / math.sqrt(shape[1]))        # sharp attention
        else:
            t = normal(1.0 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(name: str, model_dir: str, seed: int = 0, cfg: dict = None, rank: int = None, router_std: float = 1.5) -> str:
    cfg = CONFIGS[name] if cfg is None else cfg
    rank = DECAY_RANK[name] if rank is None else rank
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), draw_weights(cfg, rank, seed, router_std))
    return model_dir


def random_config(seed: int):
    """A configuration with every size drawn: (config, decay rank)."""
    r = torch.Generator().manual_seed(1000 + seed)

    def pick(*xs):
        return xs[int(torch.randint(0, len(xs), (1,), generator=r))]
    d = pick(24, 36, 40, 50, 64, 72)

    def rand_att(v_mix_shape=None, rot_ok=True):
        G = pick(1, 2, 3)
        H = G * pick(1, 2, 3)
        dk = pick(8, 12, 16, 32)
        dv = pick(8, 16, 24)
        if v_mix_shape is not None:
            G, dv = v_mix_shape
            H = G * pick(1, 2)
        rot = (pick(4, 8, dk), pick(100.0, 10000.0, 300000.0)) if rot_ok else None
        return att(H, G, dk, dv, 1.0 / math.sqrt(dk), rot=rot, v_mix=v_mix_shape is not None)

    def rand_mlp():
        kind = pick("dense", "moe", "moe", None)
        if kind is None:
            return None
        if kind == "dense":
            return dense(pick(16, 40, 56))
        groups = pick(None, (2, 1), (2, 2), (3, 2))
        per = pick(1, 2, 3)
        E = per * (groups[0] if groups else pick(2, 3, 5))
        top = pick(*range(1, (per * groups[1] if groups else E) + 1))
        return moe(E, top, pick(8, 16, 24), groups=groups, shared=pick(None, 16, 24))
    mix_shape = (pick(1, 2), pick(8, 16))
    layers = []
    for _ in range(pick(2, 3, 4)):
        if pick(0, 1):
            layers.append(parallel(rand_att(rot_ok=False), pick(1, 2, 3), pick(8, 16, 24), pick(1.0, 0.65), pick(1.0, 0.45, 1.5), rand_mlp()))
        else:
            layers.append(attention(rand_att(v_mix_shape=mix_shape if pick(0, 1, 1) else None), rand_mlp()))
    cfg = {"architecture": "Besuzen", "vocab": pick(31, 64, 150), "width": d, "norm": {"eps": pick(1e-5, 1e-6)},
           "embedding": {"scale": pick(1.0, 2.0, 3.5)}, "logit_scale": pick(1.0, 0.5, 3.0), "layers": layers}
    return cfg, pick(2, 4, 8)
