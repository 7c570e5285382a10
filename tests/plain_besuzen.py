"""A plain, slow implementation of the Besuzen decoder: whole sequences, no cache, one function
for each mechanism, float64 on the CPU, loops over time where a recurrence says it most plainly.

It shares no code with the package under test: it reads config.json and model.safetensors
itself and states every mechanism from its definition (t: time, h: a sublayer's input).

  layer norm     ln(y) = (y - mean(y)) / sqrt(mean((y - mean(y))^2) + eps) * w
  layer          x += mixer(ln1(x)) + ff(ln2(x))           (both sublayers read norms of the same x)
  attention      q, k, v = W h + b; rotary on the neighbouring pairs (2i, 2i + 1) of the first ``dims``
                 dimensions of q and k; s_ij = (q_i . k_j) * scale for j <= i; softmax; values mixed with
                 the first mixing layer's, v <- (1 - lam) v + lam v_first; the heads times sigmoid(Wg h)
                 (an element each, or one number a head); Wo
  time mix       h' = the previous token's h (zero at the start); m_s = h + (h' - h) mu_s for s in r, k, v, g, w;
                 r, k, v = W m; gate = silu(Wg m_g); w = exp(-exp(W2 tanh(W1 m_w) + w0));
                 o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t;  S_t = diag(w_t) S_{t-1} + k_t v_t^T;
                 out = Wo (unit_rms_per_head(o) * norm * gate)
  parallel       a * attention(h) + b * time_mix(h)
  dense ff       Wd (gelu_tanh(Wg h) * (Wu h))
  experts        s = softmax(Wr h) over all experts; a group's score is its largest s; only the best groups'
                 experts can be chosen; the ``top`` largest s are chosen; weights s / (sum of the chosen + 1e-20);
                 expert: Wd (silu(Wg h) * (Wu h)); plus sigmoid(w_sg . h) * shared(h)
  output         head (ln(x)) * logit_scale
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    dt = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
          "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[b:e]), dtype=dt[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def load_model_dir(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: v.to(F64) for k, v in w.items()}


# --------------------------------------------------------------------------- small functions
def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    c = x - x.mean(dim=-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(dim=-1, keepdim=True) + eps) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# --------------------------------------------------------------------------- rotary positions
def rotate_pairs(x: torch.Tensor, positions: Sequence[int], dims: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: dimension 2i pairs with 2i + 1 among the first ``dims``; the rest pass."""
    out = x.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


# --------------------------------------------------------------------------- attention
def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; query head h reads key/value head h // (H / G);
    position i sees every j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        for i in range(T):
            row = s[i, :i + 1]
            p = torch.exp(row - row.max())
            out[i, h] = (p / p.sum()) @ v[:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, v_first: Optional[torch.Tensor],
                    mixes: bool, gate_per_head: bool):
    """The attention mixer of a layer; returns (output [T, d], this layer's values as cached [T, G, dv])."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_pairs(q, range(T), rot["dims"], rot["base"])
        k = rotate_pairs(k, range(T), rot["dims"], rot["base"])
    if mixes and v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    o = softmax_attention(q, k, v, m["scale"])
    gate = sigmoid(h @ w[p + "g"].T)
    if gate_per_head:
        o = o * gate.view(T, H, 1)
    else:
        o = o * gate.view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T, v


# --------------------------------------------------------------------------- time mixing with a matrix state
def time_mix(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T, d = h.shape
    H, n = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros((1, d), dtype=F64), h[:-1]], dim=0)

    def mix(s: str) -> torch.Tensor:
        return h + (prev - h) * w[p + "mu." + s]
    r = (mix("r") @ w[p + "r"].T).view(T, H, n)
    k = (mix("k") @ w[p + "k"].T).view(T, H, n)
    v = (mix("v") @ w[p + "v"].T).view(T, H, n)
    gate = silu(mix("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, n)
    u = w[p + "u"]                                   # [H, n]: the bonus of the current token
    o = torch.zeros((T, H, n), dtype=F64)
    for hd in range(H):
        S = torch.zeros((n, n), dtype=F64)           # [key channel, value channel]
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S + u[hd].unsqueeze(1) * kv).T @ r[t, hd]
            S = decay[t, hd].unsqueeze(1) * S + kv
    o = unit_rms(o, eps).reshape(T, H * n) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forwards
def gated_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, act) -> torch.Tensor:
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(scores: torch.Tensor, top: int, groups: int, keep: int):
    """scores [E] (softmax over all experts) -> (chosen ids in falling order of score, their weights)."""
    E = scores.shape[0]
    allowed = torch.ones(E, dtype=torch.bool)
    if groups > 1:
        per = E // groups
        best = scores.view(groups, per).max(dim=1).values
        order = sorted(range(groups), key=lambda g: (-best[g].item(), g))
        allowed = torch.zeros(E, dtype=torch.bool)
        for g in order[:keep]:
            allowed[g * per:(g + 1) * per] = True
    cand = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-scores[e].item(), e))[:top]
    chosen = scores[cand]
    return cand, chosen / (chosen.sum() + 1e-20)


def experts_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict, forced: Optional[Dict[int, List[int]]] = None) -> torch.Tensor:
    """``forced`` {position: expert ids}: the experts of these tokens are given instead of chosen (their weights are
    still the plain scores, renormalised): a comparison with a run in fewer bits takes that run's choices where a
    close call may have fallen the other way, so that it measures rounding and not the choice."""
    r = mlp["router"]
    g = r.get("groups") or {}
    out = torch.zeros_like(h)
    logits = h @ w[p + "router"].T
    for t in range(h.shape[0]):
        z = logits[t]
        s = torch.exp(z - z.max())
        s = s / s.sum()
        ids, weights = route(s, r["top"], g.get("count", 1), g.get("keep", 1))
        if forced is not None and t in forced:
            ids = list(forced[t])
            weights = s[ids] / (s[ids].sum() + 1e-20)
        for e, wt in zip(ids, weights):
            out[t] += wt * gated_ff(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if mlp.get("shared") is not None:
        out = out + sigmoid(h @ w[p + "shared.sg"].T) * gated_ff(h, w, p + "shared.", silu)
    return out


# --------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[List[torch.Tensor]] = None,
            forced: Optional[Dict[int, Dict[int, List[int]]]] = None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence; ``layers_out`` collects the stream after every layer; ``forced``
    {layer: {position: expert ids}}: see ``experts_ff``."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][list(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h1 = layer_norm(x, w[p + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v = attention_mixer(h1, w, p + "mix.", m, v_first, mixes, gate_per_head=False)
            if mixes and v_first is None:
                v_first = v
        elif layer["type"] == "parallel":
            left, _ = attention_mixer(h1, w, p + "mix.left.", m["left"], None, False, gate_per_head=True)
            right = time_mix(h1, w, p + "mix.right.", m["right"], eps)
            y = m["left_scale"] * left + m["right_scale"] * right
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = layer_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = y + gated_ff(h2, w, p + "mlp.", gelu_tanh)
            else:
                y = y + experts_ff(h2, w, p + "mlp.", mlp, None if forced is None else forced.get(i))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return (layer_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg.get("logit_scale", 1.0)
