"""Arrangement of a layer's parts.  "pre_norm" is the Llama layer
(SimonWaldherr/RustyLLM src/model.rs:7201-7348): x += mixer(norm(x)); x += ff(norm(x)).
"""
from __future__ import annotations

import torch

from .base import Block, FeedForward, Mixer, Norm, Runtime
from .registry import register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, runtime: Runtime, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward,
                 feed_forward_norm: Norm):
        self.runtime = runtime
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def sub_parts(self):
        return {"mixer": self.mixer, "mixer_norm": self.mixer_norm,
                "feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm}

    folds_norms = True

    def first_norm_request(self, num_tokens: int):
        if getattr(self.mixer, "folds_norms", False) and self.mixer.takes_normed_input(num_tokens):
            return self.mixer_norm.request()
        return None

    def forward(self, x: torch.Tensor, step, cache, pending=None, next_norm=None):
        dt = self.runtime.compute_dtype
        # A norm between two matrix products can ride in their epilogues (the product in
        # front starts it, the one behind finishes it) where both parts can; otherwise the
        # norm part runs its own kernel.
        xn = pending if pending is not None else self.mixer_norm.forward(x, dt)
        if getattr(self.feed_forward, "absent", False):
            # a layer of a mixer alone: its last product may start the next layer's norm
            if getattr(self.mixer, "folds_norms", False):
                return self.mixer.forward(xn, x, step, cache, then_norm=next_norm)
            self.mixer.forward(xn, x, step, cache)
            return None
        started = None
        if getattr(self.mixer, "folds_norms", False):
            want = None
            if getattr(self.feed_forward, "folds_norms", False) and self.feed_forward.takes_normed_input(x.shape[0]):
                want = self.feed_forward_norm.request()
            started = self.mixer.forward(xn, x, step, cache, then_norm=want)
        else:
            self.mixer.forward(xn, x, step, cache)
        xn2 = started if started is not None else self.feed_forward_norm.forward(x, dt)
        if getattr(self.feed_forward, "folds_norms", False):
            return self.feed_forward.forward(xn2, x, step, then_norm=next_norm)
        self.feed_forward.forward(xn2, x, step)
        return None


@register_block("parallel_pre_norm")
class ParallelPreNormBlock(Block):
    """A layer whose two sublayers both read norms of the same stream and join it together:

        x += mixer(norm1(x)) + feed_forward(norm2(x))

    Both norms are taken before either sublayer adds anything; two norms that can share a kernel
    (``pairs_with`` / ``forward_with``: the row's statistics once, two weights) do.  A layer without a
    feed-forward is x += mixer(norm1(x))."""

    def __init__(self, runtime: Runtime, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward,
                 feed_forward_norm: Norm):
        self.runtime = runtime
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def sub_parts(self):
        return {"mixer": self.mixer, "mixer_norm": self.mixer_norm,
                "feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm}

    def forward(self, x: torch.Tensor, step, cache, pending=None, next_norm=None):
        dt = self.runtime.compute_dtype
        if getattr(self.feed_forward, "absent", False):
            self.mixer.forward(self.mixer_norm.forward(x, dt), x, step, cache)
            return None
        pairs = getattr(self.mixer_norm, "pairs_with", None)
        if pairs is not None and pairs(self.feed_forward_norm):
            h1, h2 = self.mixer_norm.forward_with(self.feed_forward_norm, x, dt)
        else:
            h1, h2 = self.mixer_norm.forward(x, dt), self.feed_forward_norm.forward(x, dt)
        self.mixer.forward(h1, x, step, cache)
        self.feed_forward.forward(h2, x, step)
        return None


@register_block("post_norm")
class PostNormBlock(Block):
    """A layer whose sublayers read the stream itself and whose norms sit on what they return:

        x += m norm1(mixer(x));  x += m norm2(feed_forward(x))  (m = ``residual_scale``, 1 unless the model says
        otherwise);  then, where the layer has one, ``after`` (a part of role "inject", e.g. a per-token side input)
        changes x once more.

    The stream is float32; a bfloat16 run hands the sublayers its rounding, which the kernel that adds a normed
    output into the stream leaves behind for the next reader.  A mixer that offers ``forward_out`` returns its
    output as float32 terms (tensor, factor) - mixers side by side return two - and the sum, the norm and the
    addition are one kernel; any other part adds into a zeroed buffer.
    """

    def __init__(self, runtime: Runtime, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward,
                 feed_forward_norm: Norm, after=None, residual_scale: float = 1.0):
        from .registry import build_part
        self.runtime = runtime
        self.residual_scale = float(residual_scale)     # x += residual_scale * norm(sublayer(x)): a constant of the model
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.after = build_part("inject", after, runtime) if after is not None else None
        if not hasattr(mixer_norm, "eps") or not (getattr(feed_forward, "absent", False) or hasattr(feed_forward_norm, "eps")):
            raise ValueError("a post_norm block needs RMS norms (a weight and an eps)")

    def sub_parts(self):
        parts = {"mixer": self.mixer, "mixer_norm": self.mixer_norm,
                 "feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm}
        if self.after is not None:
            parts["after"] = self.after
        return parts

    def _input(self, x: torch.Tensor, rounded):
        """What a sublayer reads: x itself in a 32-bit run, its bfloat16 rounding otherwise."""
        if self.runtime.compute_dtype == torch.float32:
            return x
        if rounded is not None:
            return rounded
        from .. import kernels as K
        h = torch.empty(x.shape, dtype=self.runtime.compute_dtype, device=x.device)
        K.convert(x, h)
        return h

    def _join(self, x, terms, norm):
        """x += residual_scale * norm(sum of factor * tensor); returns the new x's bfloat16 rounding in a bfloat16 run."""
        from .. import kernels as K
        if len(terms) > 2:
            raise K.KernelError("more than two terms under one norm are not built")
        rounded = None
        if self.runtime.compute_dtype == torch.bfloat16:
            rounded = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        (y0, s0), (y1, s1) = terms[0], (terms[1] if len(terms) > 1 else (None, 0.0))
        K.norm_add(x, y0, s0, y1, s1, norm.weight, norm.eps, rounded, out_scale=self.residual_scale)
        return rounded

    def forward(self, x: torch.Tensor, step, cache, pending=None, next_norm=None):
        h = self._input(x, getattr(step, "derived", {}).pop(("stream_rounded", id(x)), None))
        if hasattr(self.mixer, "forward_out"):
            terms = self.mixer.forward_out(h, step, cache)
        else:
            y = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            self.mixer.forward(h, y, step, cache)
            terms = [(y, 1.0)]
        rounded = self._join(x, terms, self.mixer_norm)
        if not getattr(self.feed_forward, "absent", False):
            h = self._input(x, rounded)
            if hasattr(self.feed_forward, "forward_out"):
                terms = self.feed_forward.forward_out(h, step)
            else:
                y = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
                self.feed_forward.forward(h, y, step)
                terms = [(y, 1.0)]
            rounded = self._join(x, terms, self.feed_forward_norm)
        if self.after is not None:
            rounded = self.after.forward(x, None, step, rounded=self._input(x, rounded))
        if rounded is not None and hasattr(step, "derived"):
            step.derived[("stream_rounded", id(x))] = rounded      # the next layer's first reader takes it
        return None
