"""Attention through a latent: keys and values of all heads are projections of one small vector a token, and
only that vector and one rotary key part shared by the heads are cached.

h: the mixer's input; n(y) w = y / sqrt(mean(y^2) + eps) * w.  With H heads of a plain width hd, a rotary width
rd and a value width vd, a query latent of q_rank and a key/value latent of kv_rank dimensions:

    cq = n(Wdq h) wq;   q = Wuq cq, a head laid out [plain (hd) | rotary (rd)]
    [c | kr] = Wdkv h;  c <- n(c) wkv (kv_rank);  kr (rd) is turned by the position and serves every head
    k_a = Wuk_a c,  v_a = Wuv_a c                                   (head a; neither is ever materialised)
    s_ij = (q_plain_i . k_a,j + rot(q_rot_i) . rot(kr_j)) * scale,  0 <= i - j < window;  softmax
    out = Wo concat_a(sigmoid((Wg h)_a) * sum_j p_ij v_a,j)         (one gate number a head)

What runs is the same sum reordered so that the cache is read as it is stored: q_plain . (Wuk_a c) =
(Wuk_a^T q_plain) . c, so head a's query becomes [Wuk_a^T q_plain | rot(q_rot)] of kv_rank + rd dimensions and
meets the cached rows [c | rot(kr)] directly - attention of H query heads over ONE key head whose values are the
first kv_rank elements of the key rows; sum_j p_ij v_a,j = Wuv_a (sum_j p_ij c_j) brings a head's result back
from the latent, and the head's gate, a number, is applied to the latent sum.  Prompt steps and single tokens
take the same route, so a position's result does not depend on how its sequence was cut.

The cache holds kv_rank + rd numbers a token and layer (``KVNeed(1, kv_rank + rd, window, value_dim=0)``: no value
pool).  Wdq, Wdkv and Wg are one matrix so that one product serves the three.  Wuk is kept head by head transposed
([H, kv_rank, hd]) so that the query's way into the latent is an ordinary product a head.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..cache.sequence_cache import KVNeed
from ..config.spec import ParamSource, ParamSpec, PartSpec
from .base import Mixer, Runtime
from .linear import OUT_ADD_F32, OUT_F32, OUT_SAME, linear
from .registry import build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 q_rank: int, kv_rank: int, scale: float, norm_eps: float, position: PartSpec, names: Dict[str, str],
                 window: Optional[int] = None, head_gate: bool = True):
        if min(hidden_size, num_heads, head_dim, value_dim, q_rank, kv_rank) <= 0 or rot_dim < 0:
            raise ValueError("latent attention: sizes must be positive")
        if window is not None and window <= 0:
            raise ValueError("window must be > 0 or None")
        self.runtime = runtime
        self.d, self.H, self.hd, self.rd, self.vd = hidden_size, num_heads, head_dim, rot_dim, value_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale, self.eps = float(scale), float(norm_eps)
        self.window = window
        self.names = names
        self.head_gate = bool(head_gate)
        self.position = build_part("position", position, runtime)     # over the rd-wide rotary part
        if self.position.rotary_dim > rot_dim:
            raise ValueError(f"{self.position.rotary_dim} rotated dimensions exceed the rotary part's {rot_dim}")
        self.w_in = self.wuq = self.wuk = self.wuv = self.wo = self.q_norm_w = self.kv_norm_w = None

    FEW_TOKENS = 64        # up to here a step's per-head products run on the CUDA cores as one launch

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, H, hd, rd, vd, n = self.d, self.H, self.hd, self.rd, self.vd, self.names
        sfx = n.get("suffix", ".weight")
        w_in = (ParamSource(n["dq"] + sfx, (self.q_rank, d)), ParamSource(n["dkv"] + sfx, (self.kv_rank + rd, d)))
        if self.head_gate:
            w_in += (ParamSource(n["g"] + sfx, (H, d)),)
        return {
            "w_in": ParamSpec(w_in),
            "wuq": ParamSpec((ParamSource(n["uq"] + sfx, (H * (hd + rd), self.q_rank)),)),
            "wuk": ParamSpec((ParamSource(n["uk"] + sfx, (H * hd, self.kv_rank)),)),
            "wuv": ParamSpec((ParamSource(n["uv"] + sfx, (H * vd, self.kv_rank)),)),
            "wo": ParamSpec((ParamSource(n["o"] + sfx, (d, H * vd)),)),
            "q_norm_w": ParamSpec((ParamSource(n["dq_norm"], (self.q_rank,)),), role="vector", init="ones"),
            "kv_norm_w": ParamSpec((ParamSource(n["dkv_norm"], (self.kv_rank,)),), role="vector", init="ones"),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.get("wuk")
        if w is not None and w.dim() == 2:
            # [H * hd, kv_rank] -> [H, kv_rank, hd]: head a's rows are the weight of the product q_plain_a -> latent
            tensors = dict(tensors, wuk=w.view(self.H, self.hd, self.kv_rank).transpose(1, 2).contiguous())
        super().bind(tensors)

    def kv_need(self) -> KVNeed:
        return KVNeed(1, self.kv_rank + self.rd, self.window, 0)

    def forward_out(self, xn, step, cache):
        y = torch.empty((xn.shape[0], self.d), dtype=torch.float32, device=xn.device)
        self.forward(xn, y, step, cache, _out_mode=OUT_F32)
        return [(y, 1.0)]

    def forward(self, xn, residual: torch.Tensor, step, cache, _out_mode=OUT_ADD_F32):
        H, hd, rd, vd, r, qr = self.H, self.hd, self.rd, self.vd, self.kv_rank, self.q_rank
        M, dt, dev = xn.shape[0], xn.dtype, xn.device
        pos = self.position
        group, layer = cache.kv_group, cache.kv_layer
        k_pool = group.k_pool(layer)
        u = torch.empty((M, self.w_in.shape[0]), dtype=dt, device=dev)
        linear(xn, self.w_in, u, OUT_SAME)                              # [query latent | c | kr | gates]
        cq = torch.empty((M, qr), dtype=dt, device=dev)
        K.latent_prepare(u, qr, r, rd, self.q_norm_w, self.kv_norm_w, self.eps, cq, step.positions, step.slot_of_token,
                         group.page_table, pos.inv_freq, pos.rotary_dim, pos.interleaved, k_pool if cache.writes else None)
        q = torch.empty((M, H * (hd + rd)), dtype=dt, device=dev)
        linear(cq, self.wuq, q, OUT_SAME)
        ql = torch.empty((M, H * (r + rd)), dtype=dt, device=dev)       # a head: [Wuk^T q_plain | rot(q_rot)]
        K.latent_query(q, ql, H, hd, rd, r, step.positions, pos.inv_freq, pos.rotary_dim, pos.interleaved)
        # a product a head: with few tokens they only stream weights and run as one launch; with many, one tensor-core
        # product a head
        few = M <= self.FEW_TOKENS and self.wuk.dtype == dt and self.wuv.dtype == dt
        if few and hd <= K.HEADS_LINEAR_MAX_K:
            K.heads_linear(q, hd + rd, self.wuk, ql, r + rd)
        else:
            for a in range(H):
                linear(q[:, a * (hd + rd):a * (hd + rd) + hd], self.wuk[a], ql[:, a * (r + rd):a * (r + rd) + r], OUT_SAME)
        ol = torch.empty((M, H * r), dtype=dt, device=dev)              # a head: its gate * sum_j p_ij c_j
        K.attention(ql, k_pool, k_pool, group.page_table, step, ol, H, 1, r + rd, self.scale, self.window or 0, value_dim=r,
                    gate=u[:, qr + r + rd:] if self.head_gate else None, gate_per_head=self.head_gate, values_in_keys=True)
        o = torch.empty((M, H * vd), dtype=dt, device=dev)
        if few and r <= K.HEADS_LINEAR_MAX_K:
            K.heads_linear(ol, r, self.wuv.view(H, vd, r), o, vd)
        else:
            for a in range(H):
                linear(ol[:, a * r:(a + 1) * r], self.wuv[a * vd:(a + 1) * vd], o[:, a * vd:(a + 1) * vd], OUT_SAME)
        return linear(o, self.wo, residual, _out_mode)
