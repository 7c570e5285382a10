"""Typed configuration of the Forilorn decoder, read from its config.json.

The file describes the model layer by layer; every layer names its mixer by "type":

    {"architecture": "Forilorn", "vocab": V, "width": d, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"scale": s, "bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": s, "mask": {"size": C},
                  "rot": {"base": B, "dims": r}},
        "mlp": {"kind": "dense", "ff": I} | null},
       {"type": "latent_attention",
        "mixer": {"heads": H, "dim": hd, "rot_dim": rd, "vdim": vd, "q_rank": rq, "kv_rank": rkv, "scale": s,
                  "mask": {"size": W}, "rot": {"base": B, "dims": rd}},
        "mlp": ...}]}

"attention": ``mask.size`` is the length of the blocks of a chunked mask; its values are its keys as projected, so
``vdim`` equals ``dim``.  "latent_attention": ``mask.size`` is a sliding window.  Every size and constant that can
differ between two models of the design is read here; nothing downstream hard-codes one.  May be absent (or
null): ``embedding.bigram`` (no pair table), a layer's ``mlp`` (a mixer alone), ``mask`` (all earlier positions are
seen), ``rot`` (no rotation), ``residual_mult`` (1), ``embedding.scale`` (1).
"""
from __future__ import annotations

from dataclasses import dataclass
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


def _rotary(m: Mapping[str, Any], w: str, most: int) -> Optional[Rotary]:
    r = _opt_obj(m, "rot", w)
    if r is None:
        return None
    rot = Rotary(base=_num(r, "base", w + ".rot"), dims=_int(r, "dims", w + ".rot", 0))
    if rot.dims % 2 or rot.dims > most or rot.base <= 0:
        raise ConfigError(f"{w}.rot: 'dims' must be even and at most {most}, 'base' positive")
    return rot


def _mask(m: Mapping[str, Any], w: str) -> Optional[int]:
    mask = _opt_obj(m, "mask", w)
    return None if mask is None else _int(mask, "size", w + ".mask")


@dataclass(frozen=True)
class ChunkedAttention:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    chunk: Optional[int] = None          # mask.size
    rot: Optional[Rotary] = None

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.dim, "scale": self.scale}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int] = None         # mask.size
    rot: Optional[Rotary] = None

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
             "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class ForilornLayer:
    type: str                                        # "attention" or "latent_attention"
    mixer: Union[ChunkedAttention, LatentAttention]
    ff: Optional[int]                                # the dense feed-forward's inner width; None: no feed-forward

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int

    def to_dict(self) -> dict:
        return {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}


@dataclass(frozen=True)
class ForilornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ForilornLayer, ...]
    residual_mult: float = 1.0
    embedding_scale: float = 1.0
    bigram: Optional[PairTable] = None

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
        emb: dict = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = self.bigram.to_dict()
        return {"architecture": "Forilorn", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "embedding": emb, "layers": [l.to_dict() for l in self.layers]}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ForilornConfig":
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
            mw = lw + ".mixer"
            if kind == "attention":
                mixer = ChunkedAttention(heads=_int(m, "heads", mw), kv_heads=_int(m, "kv_heads", mw), dim=_int(m, "dim", mw),
                                         scale=_num(m, "scale", mw), chunk=_mask(m, mw), rot=_rotary(m, mw, _int(m, "dim", mw)))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{mw}: {mixer.heads} heads are no multiple of {mixer.kv_heads} kv_heads")
                if m.get("vdim") is not None and _int(m, "vdim", mw) != mixer.dim:
                    raise ConfigError(f"{mw}: the values are the keys as projected, so 'vdim' must equal 'dim' = {mixer.dim}")
            elif kind == "latent_attention":
                mixer = LatentAttention(heads=_int(m, "heads", mw), dim=_int(m, "dim", mw), rot_dim=_int(m, "rot_dim", mw, 0),
                                        vdim=_int(m, "vdim", mw), q_rank=_int(m, "q_rank", mw), kv_rank=_int(m, "kv_rank", mw),
                                        scale=_num(m, "scale", mw), window=_mask(m, mw), rot=_rotary(m, mw, _int(m, "rot_dim", mw, 0)))
            else:
                raise ConfigError(f"{lw}: mixer type {kind!r} is not known; known: 'attention', 'latent_attention'")
            mlp = l.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{lw}.mlp must be an object or null")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{lw}.mlp: kind {mlp.get('kind')!r} is not known; known: 'dense'")
                ff = _int(mlp, "ff", lw + ".mlp")
            layers.append(ForilornLayer(kind, mixer, ff))
        emb = _opt_obj(d, "embedding", where) or {}
        bg = _opt_obj(emb, "bigram", where + ": embedding")
        pairs = None
        if bg is not None:
            bw = where + ": embedding.bigram"
            pairs = PairTable(buckets=_int(bg, "buckets", bw), mul_prev=_int(bg, "mul_prev", bw, 0), mul_cur=_int(bg, "mul_cur", bw, 0))
        return cls(vocab=_int(d, "vocab", where), width=_int(d, "width", where),
                   norm_eps=_num(_obj(d, "norm", where), "eps", where + ": norm"), layers=tuple(layers),
                   residual_mult=1.0 if d.get("residual_mult") is None else _num(d, "residual_mult", where),
                   embedding_scale=1.0 if emb.get("scale") is None else _num(emb, "scale", where + ": embedding"),
                   bigram=pairs)
