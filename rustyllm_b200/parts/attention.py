"""Grouped-query attention over the paged cache: the mixer of the Llama decoder.

Per layer, in the reference's order (SimonWaldherr/RustyLLM src/model.rs:7207-7318):
q = Wq xn, k = Wk xn, v = Wv xn (+ biases if the tensors exist); rotary encoding of
q and k; K[pos] = k, V[pos] = v; per query head h with KV head g = h / (H/G):
softmax over t <= pos of (q_h . K[t, g]) / sqrt(head_dim), times V; then
x += Wo attn.  Options other designs use, each a constructor parameter: another score
scale than 1/sqrt(head_dim) (``scale``); a sliding ``window`` (a query at position i reads
positions j with 0 <= i - j < window); a ``sink`` (the softmax's denominator has one more
term, of score 0 and without a value: p_j = e^{s_j} / (1 + sum_t e^{s_t})); an output gate
(``names["g"]``: the concatenated heads are multiplied by sigmoid(Wg xn) before Wo); a short causal
convolution over time on every channel of q, k and v, directly behind the projection (``conv_taps``; the
last taps - 1 projected rows of a sequence are per-sequence state); an RMS norm of every query and key head
with one weight vector for all heads, before the rotation (``names["q_norm"]``, ``names["k_norm"]``,
``qk_norm_eps``); scores squashed to softcap * tanh(s / softcap) (``softcap``); first positions that stay
visible behind a window (``keep_first``); a chunked mask instead of a window (``chunk`` = C: a query at position i
sees j <= i with i // C == j // C, blocks counted from the sequence's start); query and key heads divided by their
root mean square after the rotation, without a weight (``unit_qk_eps``); values that are the keys as projected,
before rotation and norm, with no value projection (``value_from_key``); an output gate of one number a head
instead of one an element (``gate_per_head``: Wg has H rows); values blended with another layer's values of the same
token before they are cached, v <- (1 - lam) v + lam v_other (``value_mix`` = {"key": k, "role": "source" or "blend"}:
the "source" layer of a key leaves its values of the step's tokens for the "blend" layers that run after it; lam is
the learned scalar ``names["vmix"]``).  Here Wq, Wk, Wv are one matrix [(H + 2G) hd x d] so that one product
serves all three, rotation and cache write are one kernel, and all tokens of the
step (several sequences, prompt or single tokens) run together.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import kernels as K
from ..cache.sequence_cache import KVNeed, StateNeed
from ..config.spec import ParamSource, ParamSpec, PartSpec
from .base import Mixer, NormedInput, Runtime
from .linear import OUT_ADD_F32, OUT_F32, OUT_SAME, can_fold_norms, linear
from .registry import build_part, register_mixer


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, position: PartSpec, names: Dict[str, str], bias: bool = False,
                 window: Optional[int] = None, value_dim: Optional[int] = None,
                 scale: Optional[float] = None, sink: bool = False, conv_taps: int = 0,
                 qk_norm_eps: Optional[float] = None, softcap: Optional[float] = None, keep_first: int = 0,
                 bias_o: Optional[bool] = None, chunk: Optional[int] = None, unit_qk_eps: Optional[float] = None,
                 value_from_key: bool = False, gate_per_head: bool = False, value_mix: Optional[Dict[str, str]] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} KV heads")
        if head_dim % 2 or not (0 < head_dim <= 256):
            raise ValueError(f"head_dim {head_dim} must be even and at most 256")
        if window is not None and window <= 0:
            raise ValueError("window must be > 0 or None")
        vd = head_dim if value_dim is None else value_dim      # the reference keeps value_dim apart, src/model.rs:33, 67-69
        if vd % 2 or not (0 < vd <= 256):
            raise ValueError(f"value_dim {vd} must be even and at most 256")
        self.vd = vd
        self.runtime = runtime
        self.d, self.H, self.G, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.bias = bias
        self.window = window
        self.names = names
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)     # src/model.rs:7239
        self.sink = bool(sink)
        self.gated = "g" in names          # an output gate: its rows ride behind q, k, v in the one product
        self.position = build_part("position", position, runtime)
        self.wqkv = self.wo = self.bqkv = self.bo = None
        if conv_taps < 0 or conv_taps > 8:
            raise ValueError(f"conv_taps {conv_taps} outside [0, 8]")
        self.conv_taps = int(conv_taps)                      # 0: no convolution (1 would be a gain a channel)
        self.qk_norm = "q_norm" in names or "k_norm" in names
        if self.qk_norm and qk_norm_eps is None:
            raise ValueError("query and key norms need qk_norm_eps")
        self.qk_norm_eps = 0.0 if qk_norm_eps is None else float(qk_norm_eps)
        if softcap is not None and not softcap > 0:
            raise ValueError(f"softcap {softcap} must be > 0 or None")
        self.softcap = 0.0 if softcap is None else float(softcap)
        if keep_first < 0:
            raise ValueError("keep_first must be >= 0")
        self.keep_first = int(keep_first) if window is not None else 0
        self.bias_o = bias if bias_o is None else bool(bias_o)
        if self.gated and (self.conv_taps or self.qk_norm):
            raise ValueError("an output gate together with a convolution or head norms is not built")
        self.channels = (num_heads + num_kv_heads) * head_dim + num_kv_heads * vd
        self.conv_w = self.q_norm_w = self.k_norm_w = None
        if chunk is not None and (chunk <= 0 or window is not None):
            raise ValueError("chunk must be > 0 or None, and excludes a window")
        self.chunk = chunk
        self.unit_qk_eps = None if unit_qk_eps is None else float(unit_qk_eps)
        self.value_from_key = bool(value_from_key)
        if self.value_from_key and vd != head_dim:
            raise ValueError(f"values that are the keys need value_dim = head_dim, got {vd} and {head_dim}")
        if (self.value_from_key or self.unit_qk_eps is not None) and (bias or self.conv_taps or self.qk_norm):
            raise ValueError("unit-size heads or values from keys together with biases, a convolution or weighted head norms are not built")
        self.gate_per_head = bool(gate_per_head)
        if self.gate_per_head and not self.gated:
            raise ValueError("gate_per_head needs an output gate (names['g'])")
        self.gate_rows = 0 if not self.gated else (num_heads if self.gate_per_head else num_heads * vd)
        if value_mix is not None:
            if value_mix.get("role") not in ("source", "blend") or not value_mix.get("key"):
                raise ValueError("value_mix needs a key and the role 'source' or 'blend'")
            if value_mix["role"] == "blend" and "vmix" not in names:
                raise ValueError("a layer that blends its values needs names['vmix']")
            if self.value_from_key or self.conv_taps or self.qk_norm:
                raise ValueError("blended values together with values from keys, a convolution or head norms are not built")
        self.value_mix = dict(value_mix) if value_mix is not None else None
        self.vmix = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, H, G, hd, vd, n = self.d, self.H, self.G, self.hd, self.vd, self.names
        sfx = n.get("suffix", ".weight")     # what follows a projection's name in the checkpoint
        qkv = (ParamSource(n["q"] + sfx, (H * hd, d)), ParamSource(n["k"] + sfx, (G * hd, d)))
        if not self.value_from_key:
            qkv += (ParamSource(n["v"] + sfx, (G * vd, d)),)
        if self.gated:
            qkv += (ParamSource(n["g"] + sfx, (self.gate_rows, d)),)
        specs = {"wqkv": ParamSpec(qkv), "wo": ParamSpec((ParamSource(n["o"] + sfx, (d, H * vd)),))}
        bsfx = n.get("bias_suffix", ".bias")
        if self.bias:
            specs["bqkv"] = ParamSpec((ParamSource(n["q"] + bsfx, (H * hd,)),
                                       ParamSource(n["k"] + bsfx, (G * hd,)),
                                       ParamSource(n["v"] + bsfx, (G * vd,))), role="vector")
        if self.bias_o:
            specs["bo"] = ParamSpec((ParamSource(n["o"] + bsfx, (d,)),), role="vector")
        if self.conv_taps:
            csfx, t = n.get("conv_suffix", ".conv"), self.conv_taps
            specs["conv_w"] = ParamSpec((ParamSource(n["q"] + csfx, (H * hd, t)), ParamSource(n["k"] + csfx, (G * hd, t)),
                                         ParamSource(n["v"] + csfx, (G * vd, t))), role="vector")
        if self.value_mix is not None and self.value_mix["role"] == "blend":
            specs["vmix"] = ParamSpec((ParamSource(n["vmix"], ()),), role="vector", init="zeros")
        if "q_norm" in n:
            specs["q_norm_w"] = ParamSpec((ParamSource(n["q_norm"], (hd,)),), role="vector", init="ones")
        if "k_norm" in n:
            specs["k_norm_w"] = ParamSpec((ParamSource(n["k_norm"], (hd,)),), role="vector", init="ones")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        b = tensors.get("bqkv")
        if b is not None and self.gated:
            # the gate's rows ride behind q, k, v in the one product and have no bias
            tensors = dict(tensors, bqkv=torch.cat([b, torch.zeros(self.gate_rows, dtype=b.dtype, device=b.device)]))
        super().bind(tensors)

    def kv_need(self) -> KVNeed:
        return KVNeed(self.G, self.hd, self.window, None if self.vd == self.hd else self.vd, self.keep_first, self.chunk)

    def state_need(self) -> Optional[StateNeed]:
        # the last taps - 1 projected rows of a sequence, float32
        return StateNeed(4 * (self.conv_taps - 1) * self.channels) if self.conv_taps > 1 else None

    folds_norms = True

    def takes_normed_input(self, num_tokens: int) -> bool:
        return can_fold_norms(self.wqkv, self.runtime.compute_dtype, num_tokens)

    def forward_out(self, xn, step, cache):
        """The mixer's output as float32 [M, d] of its own (for a block that norms it before it joins the stream):
        a list of (tensor, factor) terms."""
        y = torch.empty((xn.shape[0], self.d), dtype=torch.float32, device=xn.device)
        self.forward(xn, y, step, cache, _out_mode=OUT_F32)
        return [(y, 1.0)]

    def forward(self, xn, residual: torch.Tensor, step, cache, then_norm=None, _out_mode=OUT_ADD_F32):
        H, G, hd, vd = self.H, self.G, self.hd, self.vd
        M = xn.shape[0]
        dt = xn.dtype
        n_qkv = (H + G) * hd + (0 if self.value_from_key else G * vd)
        width = n_qkv + self.gate_rows
        # rows a multiple of 8 elements apart (the tensor-core attention kernels read queries by 16-byte pieces): a gate of
        # one number a head can leave the row's length odd
        qkv = torch.empty((M, -(-width // 8) * 8 if self.gate_per_head else width), dtype=dt, device=xn.device)[:, :width]
        v_other = v_mix = None
        if self.value_mix is not None and self.value_mix["role"] == "blend":
            v_other = getattr(step, "derived", {}).get(("values", self.value_mix["key"]))
            if v_other is None:
                raise K.KernelError(f"no layer has left values under {self.value_mix['key']!r} in this step for this one to blend with")
            if v_other.shape != (M, G * vd):
                raise K.KernelError(f"values to blend with are {tuple(v_other.shape)}, this layer's {(M, G * vd)}")
            v_mix = self.vmix
        group, layer = cache.kv_group, cache.kv_layer
        k_pool, v_pool = group.k_pool(layer), group.v_pool(layer)
        pos = self.position
        x = xn.weighted if isinstance(xn, NormedInput) else xn
        magnitude = getattr(pos, "magnitude", 1.0)      # a position kind of its own need not know the attribute
        prepared = self.conv_taps or self.qk_norm or magnitude != 1.0
        q = qkv
        if self.value_from_key or self.unit_qk_eps is not None:
            # rotation first, then heads of unit size; the keys as projected are the values: one kernel behind the product
            linear(xn, self.wqkv, qkv, OUT_SAME, self.bqkv)
            if not self.value_from_key:
                raise K.KernelError("unit-size heads with a value projection of their own are not built")
            K.qk_rotate_unit(qkv, qkv, step.positions, step.slot_of_token, group.page_table, pos.inv_freq, pos.rotary_dim,
                             pos.interleaved, self.unit_qk_eps, H, G, hd, k_pool if cache.writes else None,
                             v_pool if cache.writes else None, value_from_key=True)
        elif prepared:
            # convolution, head norms, rotation and the cache write in one kernel behind the product
            linear(xn, self.wqkv, qkv, OUT_SAME, self.bqkv)
            q = torch.empty((M, H * hd), dtype=dt, device=xn.device)
            if pos.interleaved:
                raise K.KernelError("interleaved rotary pairs behind a convolution or head norms are not built")
            K.qkv_prepare(qkv, q, self.conv_w if self.conv_taps else None, cache.state if self.conv_taps > 1 else None,
                          self.q_norm_w, self.k_norm_w, self.qk_norm_eps, step.positions, step.slot_of_token, group.page_table,
                          pos.inv_freq, pos.rotary_dim, magnitude, H, G, hd, vd,
                          k_pool if cache.writes else None, v_pool if cache.writes else None)
            if self.conv_taps > 1 and cache.writes:
                K.short_conv_state(qkv, self.conv_taps, step.cu_seqlens, step.seq_slots, cache.state)
        elif (v_other is None and dt == torch.bfloat16 and vd == hd and not self.gated and self.wqkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16
                and K.gemm_tc_qkv_rope_supported(x, self.wqkv, H, G, hd, pos.rotary_dim)):
            # few tokens: rotation and cache write ride in the product's epilogue
            kw = dict(row_sumsq=xn.sumsq, row_eps=xn.eps) if isinstance(xn, NormedInput) else {}
            K.gemm_tc_qkv_rope(x, self.wqkv, qkv, self.bqkv, step.positions, step.slot_of_token, group.page_table,
                               pos.inv_freq, pos.interleaved, H, G,
                               k_pool if cache.writes else None, v_pool if cache.writes else None, **kw)
        else:
            linear(xn, self.wqkv, qkv, OUT_SAME, self.bqkv)
            K.rope_kv_write(qkv, step.positions, step.slot_of_token, group.page_table, pos.inv_freq, H, G, hd,
                            pos.rotary_dim, pos.interleaved,
                            k_pool if cache.writes else None, v_pool if cache.writes else None, value_dim=vd,
                            v_other=v_other, v_mix=v_mix)
        if self.value_mix is not None and self.value_mix["role"] == "source" and hasattr(step, "derived"):
            # this layer's values of the step's tokens, as cached, for the layers that blend theirs with them
            step.derived[("values", self.value_mix["key"])] = qkv[:, (H + G) * hd:(H + G) * hd + G * vd]
        attn = torch.empty((M, H * vd), dtype=dt, device=xn.device)
        K.attention(q, k_pool, v_pool, group.page_table, step, attn, H, G, hd, self.scale,
                    self.window or 0, value_dim=vd, sink=self.sink, gate=qkv[:, n_qkv:] if self.gated else None,
                    softcap=self.softcap, keep_first=self.keep_first, chunk=self.chunk or 0, gate_per_head=self.gate_per_head)
        return linear(attn, self.wo, residual, _out_mode, self.bo, then_norm=then_norm)
