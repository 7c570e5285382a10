"""Typed configuration of the Besuzen decoder, read from its config.json.

The file describes the model layer by layer; every layer names its mixer by "type":

    {"architecture": "Besuzen", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s}, "logit_scale": c,
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": hd, "vdim": vd, "scale": s, "rot": {"base": B, "dims": r}, "v_mix": true},
        "mlp": {"kind": "dense", "ff": I}
             | {"kind": "moe", "router": {"experts": E, "top": k, "groups": {"count": c, "keep": m}}, "expert": {"ff": F},
                "shared": {"ff": S}}
             | null},
       {"type": "parallel",
        "mixer": {"left_scale": a, "right_scale": b,
                  "left":  {"heads": H, "kv_heads": G, "dim": hd, "vdim": vd, "scale": s},
                  "right": {"heads": Hr, "dim": n}},
        "mlp": ...}]}

Every size and constant that can differ between two models of the design is read here; nothing downstream
hard-codes one.  May be absent (or null): a layer's ``mlp`` (a mixer alone), ``rot`` (no rotation), ``v_mix`` (the
values are not blended), the router's ``groups``, ``shared`` (no shared expert), ``embedding`` and ``logit_scale``
(factors of 1).  One size is in no key of the file: the inner width of the right mixer's decay projection, which
the shape of its tensor gives (``with_checkpoint_sizes``); a configuration that is to be written out with random
weights names it under ``right.decay_rank``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Mapping, Optional, Tuple, Union

from .files import ConfigError
from .mosurax import _int, _num, _obj


def _opt_obj(d: Mapping[str, Any], key: str, where: str) -> Optional[Mapping[str, Any]]:
    return None if d.get(key) is None else _obj(d, key, where)


@dataclass(frozen=True)
class Rotary:
    base: float
    dims: int

    def to_dict(self) -> dict:
        return {"base": self.base, "dims": self.dims}


@dataclass(frozen=True)
class Attention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotary] = None
    v_mix: bool = False

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.v_mix:
            d["v_mix"] = True
        return d


@dataclass(frozen=True)
class TimeMix:
    heads: int
    dim: int
    decay_rank: Optional[int] = None      # inner width of the decay's two projections; None: the checkpoint's shapes say

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        return d


@dataclass(frozen=True)
class ParallelMixer:
    left: Attention
    right: TimeMix
    left_scale: float
    right_scale: float

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class FeedForward:
    kind: str                          # "dense" or "moe"
    ff: int                            # dense: intermediate size; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: Optional[int] = None

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        r = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        d = {"kind": "moe", "router": r, "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class BesuzenLayer:
    type: str                                        # "attention" or "parallel"
    mixer: Union[Attention, ParallelMixer]
    mlp: Optional[FeedForward]

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class BesuzenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BesuzenLayer, ...]
    embedding_scale: float = 1.0
    logit_scale: float = 1.0

    # the names other parts of the library read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return 1 << 24           # the design sets no limit; positions stay exact in float32 up to here

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        return {"architecture": "Besuzen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "layers": [l.to_dict() for l in self.layers]}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BesuzenConfig":
        where = "config.json"
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_in):
            lw = f"{where}: layers[{i}]"
            if not isinstance(l, Mapping):
                raise ConfigError(f"{lw} must be an object")
            kind = l.get("type")
            m = _obj(l, "mixer", lw)
            if kind == "attention":
                mixer = _attention(m, lw + ".mixer")
            elif kind == "parallel":
                left = _attention(_obj(m, "left", lw + ".mixer"), lw + ".mixer.left")
                if left.v_mix:
                    raise ConfigError(f"{lw}.mixer.left: the attention beside a time mixer does not blend its values")
                r = _obj(m, "right", lw + ".mixer")
                right = TimeMix(heads=_int(r, "heads", lw + ".mixer.right"), dim=_int(r, "dim", lw + ".mixer.right"),
                                decay_rank=None if r.get("decay_rank") is None else _int(r, "decay_rank", lw + ".mixer.right"))
                mixer = ParallelMixer(left=left, right=right, left_scale=_num(m, "left_scale", lw + ".mixer"),
                                      right_scale=_num(m, "right_scale", lw + ".mixer"))
            else:
                raise ConfigError(f"{lw}: mixer type {kind!r} is not known; known: 'attention', 'parallel'")
            layers.append(BesuzenLayer(kind, mixer, _feed_forward(l.get("mlp"), lw + ".mlp")))
        blended = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        for a in blended[1:]:
            if (a.kv_heads, a.vdim) != (blended[0].kv_heads, blended[0].vdim):
                raise ConfigError(f"{where}: layers that blend their values with the first such layer's need its "
                                  f"{blended[0].kv_heads} value heads of {blended[0].vdim}, got {a.kv_heads} of {a.vdim}")
        emb = _opt_obj(d, "embedding", where)
        return cls(vocab=_int(d, "vocab", where), width=_int(d, "width", where),
                   norm_eps=_num(_obj(d, "norm", where), "eps", where + ": norm"), layers=tuple(layers),
                   embedding_scale=1.0 if emb is None or emb.get("scale") is None else _num(emb, "scale", where + ": embedding"),
                   logit_scale=1.0 if d.get("logit_scale") is None else _num(d, "logit_scale", where))

    def with_checkpoint_sizes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "BesuzenConfig":
        """The sizes that only the checkpoint's tensor shapes give: the inner width of every right mixer's decay
        projection (rows of '<layer>.mix.right.w1')."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == "parallel" and l.mixer.right.decay_rank is None:
                shape = shapes.get(f"l{i}.mix.right.w1")
                if shape is not None and len(shape) == 2:
                    l = replace(l, mixer=replace(l.mixer, right=replace(l.mixer.right, decay_rank=int(shape[0]))))
            layers.append(l)
        return replace(self, layers=tuple(layers))


def _attention(m: Mapping[str, Any], w: str) -> Attention:
    rot_in = _opt_obj(m, "rot", w)
    rot = None
    if rot_in is not None:
        rot = Rotary(base=_num(rot_in, "base", w + ".rot"), dims=_int(rot_in, "dims", w + ".rot", 0))
        if rot.dims % 2 or rot.base <= 1.0:
            raise ConfigError(f"{w}.rot: 'dims' must be even and 'base' above 1")
        if rot.dims == 0:
            rot = None
    v_mix = m.get("v_mix")
    if v_mix is not None and not isinstance(v_mix, bool):
        raise ConfigError(f"{w}: 'v_mix' must be true or false, got {v_mix!r}")
    a = Attention(heads=_int(m, "heads", w), kv_heads=_int(m, "kv_heads", w), dim=_int(m, "dim", w), vdim=_int(m, "vdim", w),
                  scale=_num(m, "scale", w), rot=rot, v_mix=bool(v_mix))
    if a.heads % a.kv_heads:
        raise ConfigError(f"{w}: {a.heads} heads are no multiple of {a.kv_heads} kv_heads")
    if rot is not None and rot.dims > a.dim:
        raise ConfigError(f"{w}.rot: {rot.dims} rotated dimensions exceed the head's {a.dim}")
    return a


def _feed_forward(mlp_in: Any, w: str) -> Optional[FeedForward]:
    if mlp_in is None:
        return None
    if not isinstance(mlp_in, Mapping):
        raise ConfigError(f"{w} must be an object or null")
    kind = mlp_in.get("kind")
    if kind == "dense":
        return FeedForward("dense", ff=_int(mlp_in, "ff", w))
    if kind != "moe":
        raise ConfigError(f"{w}: kind {kind!r} is not known; known: 'dense', 'moe'")
    r = _obj(mlp_in, "router", w)
    g = _opt_obj(r, "groups", w + ".router")
    shared = _opt_obj(mlp_in, "shared", w)
    e = FeedForward("moe", ff=_int(_obj(mlp_in, "expert", w), "ff", w + ".expert"),
                    experts=_int(r, "experts", w + ".router"), top=_int(r, "top", w + ".router"),
                    groups=1 if g is None else _int(g, "count", w + ".router.groups"),
                    keep=1 if g is None else _int(g, "keep", w + ".router.groups"),
                    shared_ff=None if shared is None else _int(shared, "ff", w + ".shared"))
    if e.top > e.experts:
        raise ConfigError(f"{w}.router: top {e.top} exceeds experts {e.experts}")
    if e.experts % e.groups or e.keep > e.groups:
        raise ConfigError(f"{w}.router.groups: {e.groups} groups (keep {e.keep}) do not fit {e.experts} experts")
    if e.keep * (e.experts // e.groups) < e.top:
        raise ConfigError(f"{w}.router.groups: the {e.keep} kept groups hold fewer than top = {e.top} experts")
    return e
