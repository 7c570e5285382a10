"""Mixture-of-experts feed-forward: a router picks ``top`` of ``experts`` small gated feed-forwards
per token; their outputs are summed with the router's weights; a shared expert, where the model
has one, runs for every token and is added.

    z = Wr xn + b                       (32-bit)
    C = the ``top`` experts of largest z; w_c = softmax over z restricted to C
    x += sum_{c in C} w_c * Wdown_c (silu(Wgate_c xn) * (Wup_c xn))  [+ shared(xn)]

The experts' matrices are stacked: gate and up as [E, 2, F, d] (in a bfloat16 run [E, F, 2, d]: a gate row
and its up row in turn, as the tensor-core product's SwiGLU epilogue wants them), down as [E, d, F], so one
kernel indexes any expert.  A bfloat16 step orders its (token, choice) pairs by expert and runs two grouped
tensor-core products (every chosen expert's weights are read once, whatever the number of tokens it got); the
32-bit path, and shapes the tensor-core product cannot address, run every pair against its expert's rows on the
CUDA cores.  The shared expert is an ordinary gated feed-forward part of its own sizes.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec, PartSpec
from .base import FeedForward, Runtime
from .linear import OUT_F32, linear
from .registry import build_part, register_feed_forward


@register_feed_forward("moe_mlp")
class MoEMLP(FeedForward):
    def __init__(self, runtime: Runtime, hidden_size: int, expert_size: int, num_experts: int, top: int,
                 names: Dict[str, str], router_bias: bool = True, shared: Optional[PartSpec] = None,
                 scoring: str = "softmax", groups: int = 1, keep_groups: int = 1):
        """``names``: "router" (the router's matrix; its bias is that name + ``names["bias_suffix"]``),
        "expert" (a format string with ``{e}`` for the expert's number, giving the prefix of its
        "gate", "up" and "down" tensors), "suffix" (what follows a projection's name)."""
        if not (0 < top <= num_experts):
            raise ValueError(f"top {top} must lie in [1, {num_experts}]")
        if top > 32:
            raise ValueError("at most 32 experts a token")
        if scoring not in ("softmax", "sigmoid", "softmax_all"):
            raise ValueError(f"scoring {scoring!r} is not known; known: 'softmax', 'sigmoid', 'softmax_all'")
        # "softmax_all": scores s = softmax(z) over all experts; the ``top`` largest are chosen among the ``keep_groups``
        # best of ``groups`` equal groups of neighbours (a group's score: its largest score); the weights are the chosen
        # scores divided by their sum (+ 1e-20)
        # "sigmoid": scores s = sigmoid(z); experts are chosen by s + correction (``names["correction"]``, a value an
        # expert) among the ``keep_groups`` best of ``groups`` equal groups of neighbours (a group's score: its two
        # largest choice scores); the weights are the chosen experts' s, not renormalised
        self.scoring, self.groups, self.keep_groups = scoring, int(groups), int(keep_groups)
        if scoring in ("sigmoid", "softmax_all"):
            if router_bias:
                raise ValueError(f"a router with {scoring} scores has no bias (sigmoid scores may have a correction of the choice)")
            if groups < 1 or num_experts % groups or not (1 <= keep_groups <= groups):
                raise ValueError(f"{groups} groups (keep {keep_groups}) do not fit {num_experts} experts")
            if keep_groups * (num_experts // groups) < top:
                raise ValueError(f"{keep_groups} groups of {num_experts // groups} experts hold fewer than top = {top}")
        elif groups != 1:
            raise ValueError("groups of experts exist with sigmoid scoring only")
        self.correction = None
        self.runtime = runtime
        self.d, self.F, self.E, self.top = hidden_size, expert_size, num_experts, top
        self.names = names
        self.router_bias = router_bias
        self.shared = build_part("feed_forward", shared, runtime) if shared is not None else None
        # names["shared_gate"] (a [1, d] matrix): the shared expert's output times sigmoid(gate . xn), one number a token
        self.shared_gated = "shared_gate" in names
        if self.shared_gated and self.shared is None:
            raise ValueError("a gate of the shared expert without a shared expert")
        if self.shared_gated and not hasattr(self.shared, "forward_out"):
            raise ValueError("a gated shared expert must return its output (forward_out)")
        self.shared_gate = None
        self.interleaved = runtime.compute_dtype == torch.bfloat16
        self.router = self.router_b = self.wgu = self.wdown = None

    def sub_parts(self):
        return {"shared": self.shared} if self.shared is not None else {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, F, E, n = self.d, self.F, self.E, self.names
        sfx = n.get("suffix", ".weight")
        ex = [n["expert"].format(e=e) for e in range(E)]
        gu = tuple(ParamSource(p + "." + part + sfx, (F, d)) for p in ex for part in ("gate", "up"))
        specs = {
            "router": ParamSpec((ParamSource(n["router"] + sfx, (E, d)),)),
            "wgu": ParamSpec(gu),                                                   # [E * 2 * F, d], see ``bind``
            "wdown": ParamSpec(tuple(ParamSource(p + ".down" + sfx, (d, F)) for p in ex)),   # [E * d, F]
        }
        if self.scoring == "sigmoid" and "correction" in n:
            specs["correction"] = ParamSpec((ParamSource(n["correction"], (E,)),), role="vector", init="zeros")
        if self.shared_gated:
            specs["shared_gate"] = ParamSpec((ParamSource(n["shared_gate"] + sfx, (1, d)),))
        if self.router_bias:
            specs["router_b"] = ParamSpec((ParamSource(n["router"] + n.get("bias_suffix", ".bias"), (E,)),),
                                          role="vector", init="zeros")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.interleaved and "wgu" in tensors:
            # [E, 2, F, d] as loaded -> [E, F, 2, d]: a gate row and its up row in turn
            t = tensors["wgu"]
            tensors = dict(tensors)
            tensors["wgu"] = t.view(self.E, 2, self.F, self.d).transpose(1, 2).contiguous().view(self.E * 2 * self.F, self.d)
        super().bind(tensors)

    # from this many tokens on the router's logits are a matrix product and a selection kernel; below, one kernel
    # that does both a token a block (two launches cost more than they save there)
    ROUTER_PRODUCT_FROM = 128
    # False: every step on the per-pair kernels (for measurements and tests)
    use_grouped = True

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step) -> None:
        M = xn.shape[0]
        ids = torch.empty((M, self.top), dtype=torch.int32, device=xn.device)
        weights = torch.empty((M, self.top), dtype=torch.float32, device=xn.device)
        router = self.router
        if router.dtype != xn.dtype:
            raise K.KernelError(f"the router's matrix is {router.dtype} in a {xn.dtype} run")
        if self.scoring in ("sigmoid", "softmax_all"):
            variant = dict(softmax_all=self.scoring == "softmax_all", group_top=1 if self.scoring == "softmax_all" else 2,
                           renorm=self.scoring == "softmax_all")
            if M >= self.ROUTER_PRODUCT_FROM:
                logits = torch.empty((M, self.E), dtype=torch.float32, device=xn.device)
                linear(xn, router, logits, OUT_F32)
                K.moe_select_scored(logits, self.correction, self.top, self.groups, self.keep_groups, ids, weights, **variant)
            else:
                K.moe_route_scored(xn, router, self.correction, self.top, self.groups, self.keep_groups, ids, weights, **variant)
        elif M >= self.ROUTER_PRODUCT_FROM and self.E <= 1024:
            # many tokens: the logits as one matrix product (32-bit accumulation, the bias in its epilogue)
            logits = torch.empty((M, self.E), dtype=torch.float32, device=xn.device)
            linear(xn, router, logits, OUT_F32, self.router_b)
            K.moe_select(logits, self.top, ids, weights)
        else:
            K.moe_route(xn, router, self.router_b, self.top, ids, weights)
        wd = self.wdown.view(self.E, self.d, self.F)
        if self.interleaved:
            wgu = self.wgu.view(self.E, self.F, 2, self.d)
            if self.use_grouped and K.moe_experts_grouped_supported(xn, wgu, wd):
                K.moe_experts_grouped(xn, wgu, wd, ids, weights, residual)
            else:
                K.moe_experts(xn, wgu, wd, ids, weights, residual, interleaved=True)
        else:
            K.moe_experts(xn, self.wgu.view(self.E, 2, self.F, self.d), wd, ids, weights, residual)
        if self.shared_gated and self.shared is not None:
            (y, _), = self.shared.forward_out(xn, step)
            K.row_gate_add(residual, y, xn, self.shared_gate)
        elif self.shared is not None:
            self.shared.forward(xn, residual, step)
