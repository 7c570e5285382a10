"""A plain, slow implementation of the Forilorn decoder: whole sequences, no cache, one function
for each mechanism, float64 on the CPU.

It shares no code with the package under test: it reads config.json and model.safetensors
itself and states every mechanism from its definition (t: time, h: the sublayer's input,
n(y) = y / sqrt(mean(y^2) + eps)).

  embedding      x_t = s E[tok_t] + B[(a tok_{t-1} + b tok_t) mod buckets]; for t = 0 the row behind the buckets
  layer          x += m n(mixer(x)) (1 + w1);  x += m n(ff(x)) (1 + w2)     (the sublayers read x itself)
  rotary         pairs (2i, 2i + 1) of the first r dimensions turn by p f_i, f_i = base^(-2i/r)
  attention      q = Wq h, k = Wk h, v = k (as projected); q, k <- n(rotary(q)), n(rotary(k)) a head, no weight;
                 s_ij = (q_i . k_j) scale for j <= i in the same chunk (i // C == j // C); softmax;
                 out = Wo (concat(heads) * sigmoid(Wg h))
  latent         cq = n(Wdq h) wq;  q = Wuq cq, a head [plain | rotated];  [c | kr] = Wdkv h, c <- n(c) wkv,
                 kr <- rotary(kr), shared by the heads;  k_h = Wuk_h c, v_h = Wuv_h c;
                 s_ij = (q_plain . k_h + rotary(q_rot) . kr) scale for 0 <= i - j < window; softmax;
                 head h's output times sigmoid((Wg h)_h); Wo
  feed-forward   Wdown gelu_tanh(Wup h)
  output         E (n(x) (1 + wf))
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
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, positions: Sequence[int], rot: Optional[dict]) -> torch.Tensor:
    """x [T, ..., width]: neighbours (2i, 2i + 1) among the first ``dims`` turn by position * base^(-2i/dims);
    ``rot`` = {"dims", "base"} or None (nothing turns)."""
    out = x.clone()
    if not rot:
        return out
    dims, base = rot["dims"], rot["base"]
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * c - v * s
            out[t, ..., 2 * i + 1] = v * c + u * s
    return out


def softmax_rows(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """scores, visible [T, T]: softmax over the visible keys of every row."""
    s = scores.masked_fill(~visible, -math.inf)
    s = s - s.max(dim=-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(dim=-1, keepdim=True)


def chunk_mask(T: int, size: Optional[int]) -> torch.Tensor:
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    if size is None:
        return j <= i
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    if size is None:
        return j <= i
    return (j <= i) & (i - j < size)


# --------------------------------------------------------------------------- the parts
def embed(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    e = cfg.get("embedding") or {}
    x = w["embed"][list(tokens)] * e.get("scale", 1.0)
    bg = e.get("bigram")
    if bg:
        rows = [bg["buckets"]] + [(tokens[t - 1] * bg["mul_prev"] + tokens[t] * bg["mul_cur"]) % bg["buckets"]
                                  for t in range(1, len(tokens))]
        x = x + w["bigram"][rows]
    return x


def attention_mixer(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, hd = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(T, H, hd)
    k = (h @ w[p + "k"].T).reshape(T, G, hd)
    v = k.clone()                                        # the values are the keys as projected
    pos = list(range(T))
    q = unit_rms(rotate_pairs(q, pos, m.get("rot")), eps)
    k = unit_rms(rotate_pairs(k, pos, m.get("rot")), eps)
    visible = chunk_mask(T, (m.get("mask") or {}).get("size"))
    heads = []
    for a in range(H):
        g = a // (H // G)
        pr = softmax_rows((q[:, a] @ k[:, g].T) * m["scale"], visible)
        heads.append(pr @ v[:, g])
    y = torch.cat(heads, dim=-1) * sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def latent_mixer(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, hd, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = list(range(T))
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, hd + rd)
    q_plain, q_rot = q[..., :hd], rotate_pairs(q[..., hd:], pos, m.get("rot"))
    ckr = h @ w[p + "dkv"].T
    c = unit_rms(ckr[:, :r], eps) * w[p + "dkv.norm"]
    kr = rotate_pairs(ckr[:, r:], pos, m.get("rot"))          # [T, rd], one for all heads
    k = (c @ w[p + "uk"].T).reshape(T, H, hd)
    v = (c @ w[p + "uv"].T).reshape(T, H, vd)
    gate = sigmoid(h @ w[p + "g"].T)                     # [T, H]: one number a head
    visible = window_mask(T, (m.get("mask") or {}).get("size"))
    heads = []
    for a in range(H):
        s = (q_plain[:, a] @ k[:, a].T + q_rot[:, a] @ kr.T) * m["scale"]
        heads.append((softmax_rows(s, visible) @ v[:, a]) * gate[:, a:a + 1])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def dense_ff(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


# --------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer, [layers, T, width])."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = embed(cfg, w, tokens)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "attention":
            y = attention_mixer(layer["mixer"], w, p + "mix.", x, eps)
        elif layer["type"] == "latent_attention":
            y = latent_mixer(layer["mixer"], w, p + "mix.", x, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + mult * unit_rms(y, eps) * (1.0 + w[p + "norm1"])
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            x = x + mult * unit_rms(dense_ff(w, p + "mlp.", x), eps) * (1.0 + w[p + "norm2"])
        after.append(x.clone())
    logits = (unit_rms(x, eps) * (1.0 + w["final.norm"])) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(new_tokens):
        nxt = int(torch.argmax(forward(cfg, w, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
