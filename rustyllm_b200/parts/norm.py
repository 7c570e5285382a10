"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, in 32-bit.

SimonWaldherr/RustyLLM src/model.rs:5429-5437 (``rms_norm_into``): no mean subtraction, no
bias, the weight used as it is (no ``1 + w``).  Used before the mixer, before the
feed-forward and before the head (src/model.rs:7205, 7321, 7351).

``offset``: a design that stores its norm weights around zero and multiplies by ``offset + w``
(``offset`` = 1) says so; the sum is formed once, in float32, when the weight is bound, and every
kernel sees an ordinary weight.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec
from .base import Norm, NormRequest, Runtime
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, runtime: Runtime, size: int, eps: float, name: str, offset: float = 0.0):
        self.runtime = runtime
        self.size = size
        self.eps = float(eps)
        self.name = name
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        # a weight stored around zero is drawn around zero in the random-weights mode
        return {"weight": ParamSpec((ParamSource(self.name, (self.size,)),), role="vector",
                                    init="normal" if self.offset else "ones")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.get("weight")
        if w is not None and self.offset:
            tensors = dict(tensors, weight=w.to(torch.float32) + self.offset)
        super().bind(tensors)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        K.rmsnorm(x, self.weight, out, self.eps, rows)
        return out

    def request(self) -> Optional[NormRequest]:
        return NormRequest(self.weight, self.eps) if self.weight is not None else None


@register_norm("layer_norm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w: the mean is taken off, the variance is the mean of
    the squared deviations, there is a weight and no bias; all in 32-bit.  ``forward_with`` norms the same rows with
    a second norm of this kind in the same kernel (a layer whose two sublayers read norms of one stream)."""

    def __init__(self, runtime: Runtime, size: int, eps: float, name: str):
        self.runtime = runtime
        self.size = size
        self.eps = float(eps)
        self.name = name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((ParamSource(self.name, (self.size,)),), role="vector", init="ones")}

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        K.layer_norm(x, self.weight, out, self.eps, rows)
        return out

    def pairs_with(self, other: Norm) -> bool:
        return isinstance(other, LayerNorm) and other.size == self.size and other.eps == self.eps

    def forward_with(self, other: "LayerNorm", x: torch.Tensor, out_dtype: torch.dtype):
        out = torch.empty((2, x.shape[0], self.size), dtype=out_dtype, device=x.device)
        K.layer_norm(x, self.weight, out[0], self.eps, None, other.weight, out[1])
        return out[0], out[1]


@register_norm("none")
class NoNorm(Norm):
    """The norm in front of a part that does not exist (a layer without a feed-forward)."""

    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def forward(self, x, out_dtype, rows=None):
        raise RuntimeError("a norm of kind 'none' stands in front of nothing and is never run")
