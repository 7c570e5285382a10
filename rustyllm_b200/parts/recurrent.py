"""Mixers that carry a matrix state per head from token to token instead of caching keys and values.

Both are the same recurrence, S_t = a_t S_{t-1} + b_t k_t v_t^T with the output o_t = S_t^T q_t (csrc/linear_scan.cu),
with different decays and different parts around it:

``decay_linear_attention``
    q, k, v = silu(W h); a head's decay is a constant of the model, b = 1; the concatenated heads are RMS-normed
    together, multiplied by sigmoid(Wg h) and projected by Wo.
``selective_state_space``
    [z | x | B | C | dt] = W_in h; x, B and C pass a short causal convolution over time (with bias) and silu;
    dt = softplus(dt + dt_bias); per head a = exp(-exp(A_log) dt), b = dt, k = B, q = C (shared by the heads of a
    group), v = x; o += D x; then o * silu(z), an RMS norm in equal parts of the row, the weight, Wo.

The state (and the convolution's last taps - 1 inputs) lives in the cache's per-sequence state area as float32,
zero for a fresh sequence.  Decays, step sizes, the state and the norms are 32-bit in every run; projections and
the convolution's output take the run's compute dtype.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import kernels as K
from ..cache.sequence_cache import StateNeed
from ..config.spec import ParamSource, ParamSpec
from .base import Mixer, Runtime
from .linear import OUT_ADD_F32, OUT_F32, OUT_SAME, linear
from .registry import register_mixer


def _aligned(nbytes: int) -> int:
    return -(-nbytes // 256) * 256


class _StateMixer(Mixer):
    """What the two mixers share: they own no keys or values, and return their output either added into the
    stream or as a tensor of its own."""

    def forward_out(self, xn, step, cache):
        y = torch.empty((xn.shape[0], self.d), dtype=torch.float32, device=xn.device)
        self.forward(xn, y, step, cache, _out_mode=OUT_F32)
        return [(y, 1.0)]

    @staticmethod
    def _state(cache):
        if cache.state is None:
            raise K.KernelError("a mixer with per-sequence state was given a cache entry without state")
        if not cache.writes:
            raise K.KernelError("a mixer with per-sequence state cannot read another layer's cache entry")
        return cache.state


@register_mixer("decay_linear_attention")
class DecayLinearAttention(_StateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, head_dim: int, value_dim: int,
                 decay: Sequence[float], norm_eps: float, names: Dict[str, str]):
        """``names``: "q", "k", "v", "g", "o" (matrices), "norm" (weight of the norm over the heads), "suffix"."""
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        if not (0 < head_dim <= 256) or value_dim <= 0:
            raise ValueError(f"head_dim {head_dim} must lie in (0, 256] and value_dim {value_dim} be positive")
        self.runtime = runtime
        self.d, self.H, self.dk, self.dv = hidden_size, num_heads, head_dim, value_dim
        self.eps = float(norm_eps)
        self.names = names
        self.decay = torch.tensor([float(a) for a in decay], dtype=torch.float32, device=runtime.device)
        self.wqkvg = self.wo = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, H, dk, dv, n = self.d, self.H, self.dk, self.dv, self.names
        sfx = n.get("suffix", ".weight")
        return {
            "wqkvg": ParamSpec((ParamSource(n["q"] + sfx, (H * dk, d)), ParamSource(n["k"] + sfx, (H * dk, d)),
                                ParamSource(n["v"] + sfx, (H * dv, d)), ParamSource(n["g"] + sfx, (H * dv, d)))),
            "wo": ParamSpec((ParamSource(n["o"] + sfx, (d, H * dv)),)),
            "norm_w": ParamSpec((ParamSource(n["norm"], (H * dv,)),), role="vector", init="ones"),
        }

    def state_need(self) -> StateNeed:
        return StateNeed(4 * self.H * self.dk * self.dv)

    def forward(self, xn, residual: torch.Tensor, step, cache, _out_mode=OUT_ADD_F32):
        H, dk, dv = self.H, self.dk, self.dv
        M = xn.shape[0]
        state = self._state(cache)
        proj = torch.empty((M, 2 * H * dk + 2 * H * dv), dtype=xn.dtype, device=xn.device)
        linear(xn, self.wqkvg, proj, OUT_SAME)
        q, k = proj[:, :H * dk], proj[:, H * dk:2 * H * dk]
        v, g = proj[:, 2 * H * dk:2 * H * dk + H * dv], proj[:, 2 * H * dk + H * dv:]
        o = torch.empty((M, H * dv), dtype=torch.float32, device=xn.device)
        K.linear_scan(q, k, v, o, state, step.cu_seqlens, step.seq_slots, H, 1, dk, dv, self.decay, silu=True)
        on = torch.empty((M, H * dv), dtype=xn.dtype, device=xn.device)
        K.gated_norm(o, g, self.norm_w, self.eps, on, groups=1, gate_act="sigmoid", gate_first=False)
        linear(on, self.wo, residual, _out_mode)


@register_mixer("selective_state_space")
class SelectiveStateSpace(_StateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int,
                 conv_taps: int, norm_groups: int, norm_eps: float, names: Dict[str, str]):
        """``names``: "in", "o" (matrices), "conv" (filters [channels, taps]; bias: + ``names["bias_suffix"]``),
        "dt_bias", "A_log", "D" (a value a head), "norm" (weight of the norm in parts), "suffix"."""
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads are no multiple of {groups} groups")
        if (num_heads * head_dim) % norm_groups:
            raise ValueError(f"{norm_groups} norm groups do not divide {num_heads * head_dim} channels")
        if not (1 <= conv_taps <= 8):
            raise ValueError(f"conv_taps {conv_taps} outside [1, 8]")
        if not (0 < state_size <= 256):
            raise ValueError(f"state_size {state_size} outside (0, 256]")
        self.runtime = runtime
        self.d, self.H, self.P, self.N, self.G = hidden_size, num_heads, head_dim, state_size, groups
        self.taps, self.norm_groups, self.eps = int(conv_taps), int(norm_groups), float(norm_eps)
        self.inner = num_heads * head_dim
        self.conv_channels = self.inner + 2 * groups * state_size
        self.names = names
        self._conv_bytes = _aligned(4 * (self.taps - 1) * self.conv_channels)
        self.w_in = self.wo = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, H = self.names, self.H
        sfx = n.get("suffix", ".weight")
        rows = 2 * self.inner + 2 * self.G * self.N + H
        return {
            "w_in": ParamSpec((ParamSource(n["in"] + sfx, (rows, self.d)),)),
            "wo": ParamSpec((ParamSource(n["o"] + sfx, (self.d, self.inner)),)),
            "conv_w": ParamSpec((ParamSource(n["conv"], (self.conv_channels, self.taps)),), role="vector"),
            "conv_b": ParamSpec((ParamSource(n["conv"] + n.get("bias_suffix", ".bias"), (self.conv_channels,)),), role="vector",
                                init="zeros"),
            "dt_bias": ParamSpec((ParamSource(n["dt_bias"], (H,)),), role="vector", init="zeros"),
            "a_log": ParamSpec((ParamSource(n["A_log"], (H,)),), role="vector", init="zeros"),
            "skip": ParamSpec((ParamSource(n["D"], (H,)),), role="vector", init="ones"),
            "norm_w": ParamSpec((ParamSource(n["norm"], (self.inner,)),), role="vector", init="ones"),
        }

    def state_need(self) -> StateNeed:
        # the convolution's last taps - 1 inputs, then the heads' matrix states
        return StateNeed(self._conv_bytes + 4 * self.H * self.N * self.P)

    def forward(self, xn, residual: torch.Tensor, step, cache, _out_mode=OUT_ADD_F32):
        H, P, N, G, inner, C = self.H, self.P, self.N, self.G, self.inner, self.conv_channels
        M = xn.shape[0]
        state = self._state(cache)
        conv_state, scan_state = state[:, :self._conv_bytes], state[:, self._conv_bytes:]
        proj = torch.empty((M, 2 * inner + 2 * G * N + H), dtype=xn.dtype, device=xn.device)
        linear(xn, self.w_in, proj, OUT_SAME)
        z, u, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
        xbc = torch.empty((M, C), dtype=xn.dtype, device=xn.device)
        K.short_conv(u, self.conv_w, self.conv_b, True, step.slot_of_token, conv_state, xbc)
        K.short_conv_state(u, self.taps, step.cu_seqlens, step.seq_slots, conv_state)
        x, b, c = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
        y = torch.empty((M, inner), dtype=torch.float32, device=xn.device)
        K.linear_scan(c, b, x, y, scan_state, step.cu_seqlens, step.seq_slots, H, H // G, N, P, self.a_log,
                      dt_raw=dt, dt_bias=self.dt_bias, skip=self.skip)
        yn = torch.empty((M, inner), dtype=xn.dtype, device=xn.device)
        K.gated_norm(y, z, self.norm_w, self.eps, yn, groups=self.norm_groups, gate_act="silu", gate_first=True)
        linear(yn, self.wo, residual, _out_mode)


@register_mixer("shifted_decay_recurrence")
class ShiftedDecayRecurrence(_StateMixer):
    """Time mixing over a token's input h_t and its predecessor's h_{t-1} (zero before the sequence starts):

        m_s = h_t + (h_{t-1} - h_t) * mu_s                for s in r, k, v, g, w (five learned vectors)
        r, k, v = W_r m_r, W_k m_k, W_v m_v               (heads x head_dim each);   gate = silu(W_g m_g)
        w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))           a decay a head and key channel, in (0, 1)
        o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t         per head; the bonus u weighs the current token alone
        S_t = diag(w_t) S_{t-1} + k_t v_t^T
        out = W_o (o / rms(o, per head) * norm * gate)

    The per-sequence state is the last input the sequence was fed ([d]) and the heads' matrix states, float32, zero
    for a fresh sequence.  The blends, the decay's logarithm from the second projection on, the decay, the state, the
    sums and the head norm are 32-bit in every run; the projections and their activations take the compute dtype."""

    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, norm_eps: float,
                 names: Dict[str, str]):
        """``names``: "mu" (prefix of the five blend vectors: + "r", "k", "v", "g", "w"), "r", "k", "v", "g", "o"
        (matrices), "w1", "w2" (the decay's two projections), "w0" (its offset, a value a channel), "u" (the bonus,
        [heads, head_dim]), "norm" (weight behind the head norm), "suffix"."""
        if not (0 < head_dim <= 256) or num_heads <= 0 or decay_rank <= 0:
            raise ValueError(f"head_dim {head_dim} must lie in (0, 256], heads {num_heads} and decay_rank {decay_rank} be positive")
        self.runtime = runtime
        self.d, self.H, self.n, self.rank = hidden_size, num_heads, head_dim, int(decay_rank)
        self.eps = float(norm_eps)
        self.names = names
        self._shift_bytes = _aligned(4 * hidden_size)
        self.mu = self.wrkvg = self.w1 = self.w2 = self.w0 = self.u = self.norm_w = self.wo = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, inner, n = self.d, self.H * self.n, self.names
        sfx = n.get("suffix", ".weight")
        specs = {"mu": ParamSpec(tuple(ParamSource(n["mu"] + s, (d,)) for s in self.MIXES), role="vector", init="normal")}
        # the four projections one behind the other, [4 * inner, d]: one grouped product reads each blend with its own rows
        specs["wrkvg"] = ParamSpec(tuple(ParamSource(n[key] + sfx, (inner, d)) for key in ("r", "k", "v", "g")))
        specs.update({
            "w1": ParamSpec((ParamSource(n["w1"] + sfx, (self.rank, d)),)),
            "w2": ParamSpec((ParamSource(n["w2"] + sfx, (inner, self.rank)),)),
            "w0": ParamSpec((ParamSource(n["w0"], (inner,)),), role="vector", init="normal"),
            "u": ParamSpec((ParamSource(n["u"], (self.H, self.n)),), role="vector", init="normal"),
            "norm_w": ParamSpec((ParamSource(n["norm"], (inner,)),), role="vector", init="ones"),
            "wo": ParamSpec((ParamSource(n["o"] + sfx, (d, inner)),)),
        })
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if "mu" in tensors:          # five vectors one after another -> [5, d]
            tensors = dict(tensors, mu=tensors["mu"].view(len(self.MIXES), self.d))
        super().bind(tensors)

    def state_need(self) -> StateNeed:
        # the last input the sequence was fed, then the heads' matrix states
        return StateNeed(self._shift_bytes + 4 * self.H * self.n * self.n)

    def forward(self, xn, residual: torch.Tensor, step, cache, _out_mode=OUT_ADD_F32):
        H, n, inner = self.H, self.n, self.H * self.n
        M = xn.shape[0]
        dt, dev = xn.dtype, xn.device
        state = self._state(cache)
        shift_state, scan_state = state[:, :self._shift_bytes], state[:, self._shift_bytes:]
        w4 = self.wrkvg.view(4, inner, self.d)
        grouped = K.gemm_tc_row_groups_supported(xn, w4) and inner % 8 == 0
        tile = K.gemm_tc_row_groups_tile(M) if grouped else 1
        # every blend's rows padded to whole tiles of the grouped product; what the padding holds is never looked at
        # (every row of a product is computed by itself, and the padding's results are not read)
        rows = -(-M // tile) * tile
        mixes = torch.empty((len(self.MIXES), rows, self.d), dtype=dt, device=dev)
        K.token_shift_mix(xn, self.mu, step.positions, step.slot_of_token, step.cu_seqlens, shift_state, mixes)
        proj = torch.empty((4, rows, inner), dtype=dt, device=dev)          # r, k, v, g
        if grouped:
            K.gemm_tc_row_groups(mixes[:4], w4, proj, tile)
        else:
            for i in range(4):
                linear(mixes[i], w4[i], proj[i], OUT_SAME)
        mixes, proj = mixes[:, :M], proj[:, :M]
        # the decay: the first projection's output and its tanh in 32-bit, the second projection's output (the decay's
        # logarithm's logarithm, with its offset) in 32-bit; the scan forms exp(-exp(.)) itself
        low = torch.empty((M, self.rank), dtype=torch.float32, device=dev)
        linear(mixes[4], self.w1, low, OUT_F32)
        low_t = torch.empty((M, self.rank), dtype=dt, device=dev)
        K.tanh_cast(low, low_t)
        wlog = torch.empty((M, inner), dtype=torch.float32, device=dev)
        linear(low_t, self.w2, wlog, OUT_F32, self.w0)
        o = torch.empty((M, inner), dtype=torch.float32, device=dev)
        K.channel_decay_scan(proj[0], proj[1], proj[2], wlog, self.u, o, scan_state, step.cu_seqlens, step.seq_slots, H, n, n)
        on = torch.empty((M, inner), dtype=dt, device=dev)
        K.gated_norm(o, proj[3], self.norm_w, self.eps, on, groups=H, gate_act="silu", gate_first=False)
        linear(on, self.wo, residual, _out_mode)


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    """Two mixers side by side on the same input: left_scale * left(h) + right_scale * right(h).  At most one of
    them caches keys and values; their per-sequence states lie one behind the other in the layer's state entry."""

    def __init__(self, runtime: Runtime, left, right, left_scale: float = 1.0, right_scale: float = 1.0):
        from .registry import build_part
        self.runtime = runtime
        self.left = build_part("mixer", left, runtime)
        self.right = build_part("mixer", right, runtime)
        self.scales = (float(left_scale), float(right_scale))
        if self.left.kv_need() is not None and self.right.kv_need() is not None:
            raise ValueError("two mixers side by side that both cache keys and values are not built")
        sizes = [m.state_need().nbytes if m.state_need() is not None else 0 for m in (self.left, self.right)]
        self._state_at = (0, _aligned(sizes[0]))
        self._state_sizes = tuple(sizes)

    def sub_parts(self):
        return {"left": self.left, "right": self.right}

    def kv_need(self):
        return self.left.kv_need() or self.right.kv_need()

    def state_need(self) -> Optional[StateNeed]:
        total = self._state_at[1] + self._state_sizes[1]
        return StateNeed(total) if total else None

    def _views(self, cache):
        from dataclasses import replace
        out = []
        for at, n in zip(self._state_at, self._state_sizes):
            out.append(replace(cache, state=cache.state[:, at:at + n] if n else None))
        return out

    def forward_out(self, xn, step, cache):
        terms = []
        for m, view, s in zip((self.left, self.right), self._views(cache), self.scales):
            if hasattr(m, "forward_out"):
                terms += [(y, f * s) for y, f in m.forward_out(xn, step, view)]
            else:
                y = torch.zeros((xn.shape[0], xn.shape[1]), dtype=torch.float32, device=xn.device)
                m.forward(xn, y, step, view)
                terms.append((y, s))
        return terms

    def forward(self, xn, residual: torch.Tensor, step, cache):
        if self.scales != (1.0, 1.0):
            # the two outputs as tensors of their own, then residual += a * left + b * right in one pass
            terms = self.forward_out(xn, step, cache)
            if len(terms) != 2:
                raise K.KernelError("mixers side by side with factors: each must return one term")
            (y0, s0), (y1, s1) = terms
            K.scaled_add(residual, y0, s0, y1, s1)
            return
        for m, view in zip((self.left, self.right), self._views(cache)):
            m.forward(xn, residual, step, view)
