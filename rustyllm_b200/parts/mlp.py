"""Gated feed-forward (SwiGLU): x += Wdown (silu(Wgate xn) * (Wup xn)).

SimonWaldherr/RustyLLM src/model.rs:7321-7347 with the activation of src/simd.rs:2403-2408
(``g / (1 + exp(-g)) * u``).  Wgate and Wup are one matrix [2I x d] so that one
product serves both (the reference reads a fused ``ffn_up`` of 2I rows, gate rows
first, src/model.rs:3933-3967).  In a bf16 run the rows are interleaved (gate_0, up_0,
gate_1, up_1, ...): a gate and its up value then sit in neighbouring lanes of the
tensor-core product's epilogue, which applies the activation and writes the
[M x I] product directly - the [M x 2I] intermediate is never stored.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec
from .base import FeedForward, NormedInput, Runtime
from .linear import OUT_ADD_F32, OUT_SAME, can_fold_norms, linear
from .registry import register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, names: Dict[str, str],
                 activation: str = "silu", bias: bool = False):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"activation {activation!r} is not supported; known: 'silu', 'gelu_tanh'")
        self.activation = activation       # on the gate: silu(g) * u, or the tanh form of gelu, gelu_tanh(g) * u
        self.runtime = runtime
        self.d, self.I = hidden_size, intermediate_size
        self.names = names
        self.bias = bias
        self.interleaved = runtime.compute_dtype == torch.bfloat16
        self.wgu = self.wdown = self.bgu = self.bdown = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, I, n = self.d, self.I, self.names
        layout = "interleave" if self.interleaved else "concat"
        sfx = n.get("suffix", ".weight")     # what follows a projection's name in the checkpoint
        specs = {
            "wgu": ParamSpec((ParamSource(n["gate"] + sfx, (I, d)),
                              ParamSource(n["up"] + sfx, (I, d))), layout=layout),
            "wdown": ParamSpec((ParamSource(n["down"] + sfx, (d, I)),)),
        }
        if self.bias:
            specs["bgu"] = ParamSpec((ParamSource(n["gate"] + ".bias", (I,)),
                                      ParamSource(n["up"] + ".bias", (I,))), role="vector", layout=layout)
            specs["bdown"] = ParamSpec((ParamSource(n["down"] + ".bias", (d,)),), role="vector")
        return specs

    folds_norms = True

    def takes_normed_input(self, num_tokens: int) -> bool:
        return self.interleaved and can_fold_norms(self.wgu, self.runtime.compute_dtype, num_tokens)

    def forward_out(self, xn, step):
        """The output as float32 [M, d] of its own (for whoever scales it before it joins the stream)."""
        y = torch.empty((xn.shape[0], self.d), dtype=torch.float32, device=xn.device)
        self.forward(xn, y, step, _out_mode=K.OUT_F32)
        return [(y, 1.0)]

    def forward(self, xn, residual: torch.Tensor, step, then_norm=None, _out_mode=OUT_ADD_F32):
        M = xn.shape[0]
        h = torch.empty((M, self.I), dtype=xn.dtype, device=xn.device)
        gelu = self.activation == "gelu_tanh"
        # The activation runs in the product's epilogue: with few tokens the kernel streams
        # weights and the epilogue is idle time anyway; with many, the persistent kernel drains
        # one accumulator while the tensor cores fill the other.
        x = xn.weighted if isinstance(xn, NormedInput) else xn
        if self.interleaved and self.wgu.dtype == torch.bfloat16 and K.gemm_tc_supported(x, self.wgu, None):
            kw = dict(row_sumsq=xn.sumsq, row_eps=xn.eps) if isinstance(xn, NormedInput) else {}
            K.gemm_tc(x, self.wgu, h, K.OUT_GEGLU if gelu else K.OUT_SWIGLU, self.bgu, **kw)
        else:
            gu = torch.empty((M, 2 * self.I), dtype=xn.dtype, device=xn.device)
            linear(xn, self.wgu, gu, OUT_SAME, self.bgu)
            (K.geglu if gelu else K.swiglu)(gu, h, interleaved=self.interleaved)
        return linear(h, self.wdown, residual, _out_mode, self.bdown, then_norm=then_norm)


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """Feed-forward without a gate: Wdown act(Wup xn), act the tanh form of gelu,
    0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), computed in 32-bit from the product's output."""

    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, names: Dict[str, str],
                 activation: str = "gelu_tanh"):
        if activation != "gelu_tanh":
            raise ValueError(f"activation {activation!r} is not supported; known: 'gelu_tanh'")
        self.runtime = runtime
        self.d, self.I = hidden_size, intermediate_size
        self.names = names
        self.wup = self.wdown = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, I, n = self.d, self.I, self.names
        sfx = n.get("suffix", ".weight")
        return {"wup": ParamSpec((ParamSource(n["up"] + sfx, (I, d)),)),
                "wdown": ParamSpec((ParamSource(n["down"] + sfx, (d, I)),))}

    def forward_out(self, xn, step):
        y = torch.empty((xn.shape[0], self.d), dtype=torch.float32, device=xn.device)
        self.forward(xn, y, step, _out_mode=K.OUT_F32)
        return [(y, 1.0)]

    def forward(self, xn, residual: torch.Tensor, step, _out_mode=OUT_ADD_F32):
        h = torch.empty((xn.shape[0], self.I), dtype=xn.dtype, device=xn.device)
        if xn.dtype == torch.bfloat16 and self.wup.dtype == torch.bfloat16 and K.gemm_tc_supported(xn, self.wup, None):
            K.gemm_tc(xn, self.wup, h, K.OUT_GELU)         # the activation rides in the product's epilogue
        else:
            linear(xn, self.wup, h, OUT_SAME)
            K.gelu_tanh(h, h)
        return linear(h, self.wdown, residual, _out_mode)


@register_feed_forward("none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward: the block skips its second half."""
    absent = True

    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def forward(self, xn, residual: torch.Tensor, step) -> None:
        return None
