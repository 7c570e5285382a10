"""The Forilorn decoder as a ``ModelSpec``: which parts, with which constants and which tensor names.

    x = scale * embed[token] + bigram[hash(previous token, token)]
    a layer:  x += m * rms_norm(mixer(x)) * (1 + norm1);  x += m * rms_norm(ff(x)) * (1 + norm2)
              (the sublayers read x itself; the norms sit on what they return)
    mixer "attention":        grouped-query attention whose values are its keys as projected (no value projection);
                              rotary positions on neighbouring pairs, then q and k heads of unit size; a chunked mask;
                              an output gate an element
    mixer "latent_attention": queries through a normed latent; keys and values from one normed latent a token plus
                              one rotary key part for all heads (parts/latent.py); a sliding window; a gate a head
    ff:       down(gelu_tanh(up(x)))
    logits = embed (rms_norm(x) * (1 + final.norm))     (the embedding table itself, unscaled)

Tensor names: "embed", "bigram", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.{q,k,g,o}" or
"l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}", "l<i>.mlp.{up,down}", "final.norm"; matrices [out, in].
"""
from __future__ import annotations

from ..config.forilorn import ForilornConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec


def _position(head_dim: int, rot) -> PartSpec:
    if rot is None or not rot.dims:
        return PartSpec("none", {"head_dim": head_dim})
    return PartSpec("rope", {"head_dim": head_dim, "rotary_dim": rot.dims, "theta": rot.base, "pairing": "interleaved"})


def forilorn_spec(cfg: ForilornConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers, ignored = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        if l.type == "attention":
            mixer = PartSpec("gqa_attention", {
                "hidden_size": d, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
                "chunk": m.chunk, "unit_qk_eps": eps, "value_from_key": True, "position": _position(m.dim, m.rot),
                "names": {"q": p + "mix.q", "k": p + "mix.k", "g": p + "mix.g", "o": p + "mix.o", "suffix": ""}})
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": d, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "window": m.window,
                "position": _position(m.rot_dim, m.rot) if m.rot_dim else PartSpec("none", {"head_dim": 2}),
                "names": {"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv",
                          "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv", "g": p + "mix.g",
                          "o": p + "mix.o", "suffix": ""}})
        if l.ff is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
            ignored.append(p + "norm2")
        else:
            ff = PartSpec("dense_mlp", {"hidden_size": d, "intermediate_size": l.ff, "activation": "gelu_tanh",
                                        "names": {"up": p + "mlp.up", "down": p + "mlp.down", "suffix": ""}})
            ff_norm = PartSpec("rms_norm", {"size": d, "eps": eps, "name": p + "norm2", "offset": 1.0})
        layers.append(LayerSpec(block=PartSpec("post_norm", {"residual_scale": cfg.residual_mult}), mixer=mixer,
                                mixer_norm=PartSpec("rms_norm", {"size": d, "eps": eps, "name": p + "norm1", "offset": 1.0}),
                                feed_forward=ff, feed_forward_norm=ff_norm))
    emb = {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed", "scale": cfg.embedding_scale}
    if cfg.bigram is not None:
        emb.update(buckets=cfg.bigram.buckets, mul_prev=cfg.bigram.mul_prev, mul_cur=cfg.bigram.mul_cur, pair_name="bigram")
    spec = ModelSpec(
        architecture="Forilorn", vocab_size=cfg.vocab, hidden_size=d, max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("scaled_pair_embedding", emb),
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        final_norm=PartSpec("rms_norm", {"size": d, "eps": eps, "name": "final.norm", "offset": 1.0}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "head", "tied_to": "embedding.weight"}),
        ignored_tensors=tuple(ignored))
    spec.validate()
    return spec


FORILORN = register_architecture(("Forilorn", "forilorn"), ForilornConfig.from_dict, forilorn_spec)
