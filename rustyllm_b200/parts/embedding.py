"""Token embedding and output head.

SimonWaldherr/RustyLLM: ``x = token_embd.row(token)`` (src/model.rs:7193, no scaling) and
``logits = output . rms_norm(x)`` (src/model.rs:7351-7357); an absent output matrix
is the embedding matrix (tied, src/model.rs:3654-3667) - here the head then shares
the embedding's storage instead of cloning it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..cache.sequence_cache import StateNeed
from ..config.spec import ParamSource, ParamSpec
from .base import Part, Runtime
from .linear import OUT_F32, linear
from .registry import register


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str):
        self.runtime = runtime
        self.V, self.d, self.name = vocab_size, hidden_size, name
        self.weight: Optional[torch.Tensor] = None
        self.bad_token = torch.zeros(1, dtype=torch.int32, device=runtime.device)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((ParamSource(self.name, (self.V, self.d)),), role="table")}

    def forward(self, step) -> torch.Tensor:
        """The step's tokens (``step.tokens``, int32 [M]) -> float32 residual [M, d].  An embedding
        part is handed the whole step, so that one which also needs the tokens' positions (a
        learned absolute position table) finds them in ``step.positions``."""
        tokens = step.tokens
        x = torch.empty((tokens.numel(), self.d), dtype=torch.float32, device=tokens.device)
        K.embedding(self.weight, tokens, x, self.bad_token)
        return x


@register("embedding", "token_position_embedding")
class TokenPositionEmbedding(TokenEmbedding):
    """Token embedding plus a learned absolute position vector: x = E[token] + P[position], neither
    scaled, summed in 32-bit.  Positions count from 0 in each sequence; the table has
    ``max_positions`` rows."""

    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str, max_positions: int,
                 position_name: str):
        super().__init__(runtime, vocab_size, hidden_size, name)
        self.P, self.position_name = max_positions, position_name
        self.positions: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = super().param_specs()
        specs["positions"] = ParamSpec((ParamSource(self.position_name, (self.P, self.d)),), role="table")
        return specs

    def forward(self, step) -> torch.Tensor:
        tokens = step.tokens
        x = torch.empty((tokens.numel(), self.d), dtype=torch.float32, device=tokens.device)
        K.embedding_pos(self.weight, self.positions, tokens, step.positions, x, self.bad_token)
        return x


@register("embedding", "scaled_pair_embedding")
class ScaledPairEmbedding(TokenEmbedding):
    """x = scale * E[token] + P[(mul_prev * previous token + mul_cur * token) mod buckets], summed in 32-bit; a
    sequence's first token takes row ``buckets`` of P, which has buckets + 1 rows.  The previous token belongs to
    the sequence's state: an int32 a slot in the cache's state area (``state_need``), read where a step's first
    token of a sequence continues one that is under way, and left behind by every step.  Without ``buckets``:
    the scaled token embedding alone."""

    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str, scale: float = 1.0,
                 buckets: Optional[int] = None, mul_prev: int = 0, mul_cur: int = 0, pair_name: Optional[str] = None):
        super().__init__(runtime, vocab_size, hidden_size, name)
        if buckets is not None and (buckets <= 0 or mul_prev < 0 or mul_cur < 0 or not pair_name):
            raise ValueError("a pair table needs buckets > 0, multipliers >= 0 and a tensor name")
        self.scale = float(scale)
        self.buckets, self.mul_prev, self.mul_cur, self.pair_name = buckets, int(mul_prev), int(mul_cur), pair_name
        self.pairs: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = super().param_specs()
        if self.buckets is not None:
            specs["pairs"] = ParamSpec((ParamSource(self.pair_name, (self.buckets + 1, self.d)),), role="table")
        return specs

    def state_need(self) -> StateNeed:
        return StateNeed(4)        # the last token the sequence was fed

    def forward(self, step, state: torch.Tensor) -> torch.Tensor:
        tokens = step.tokens
        x = torch.empty((tokens.numel(), self.d), dtype=torch.float32, device=tokens.device)
        K.embedding_pair(self.weight, self.pairs, tokens, step.positions, step.slot_of_token, step.cu_seqlens, state, self.scale,
                         self.mul_prev, self.mul_cur, self.buckets or 1, x, self.bad_token)
        return x


@register("head", "lm_head")
class LMHead(Part):
    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str,
                 tied_to: Optional[str] = None, softcap: Optional[float] = None, scale: float = 1.0):
        if softcap is not None and not softcap > 0:
            raise ValueError(f"softcap {softcap} must be > 0 or None")
        self.scale = float(scale)        # logits <- logits * scale (a constant of the model), before any soft cap
        self.softcap = None if softcap is None else float(softcap)    # logits <- cap * tanh(logits / cap)
        self.runtime = runtime
        self.V, self.d, self.name, self.tied_to = vocab_size, hidden_size, name, tied_to
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((ParamSource(self.name, (self.V, self.d)),), role="table",
                                    alias_of=self.tied_to)}

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        """xn: [W, d] compute dtype -> float32 logits [W, V]."""
        logits = torch.empty((xn.shape[0], self.V), dtype=torch.float32, device=xn.device)
        linear(xn, self.weight, logits, OUT_F32)
        if self.scale != 1.0:
            K.scale(logits, self.scale)
        if self.softcap is not None:
            K.softcap(logits, self.softcap)
        return logits
