"""The Besuzen decoder as a ``ModelSpec``: which parts, with which constants and which tensor names.

    x = embed[token] * embedding.scale
    a layer:  x += mixer(ln1(x)) + ff(ln2(x))      (ln: layer norm with a weight and no bias; both of the same x)
    mixer "attention":  biased q, k, v; rotary positions on neighbouring pairs of the first rot.dims dimensions; causal
              softmax attention; in layers that say v_mix, but for the first of them, the values are blended with that
              first layer's values of the same token before they are cached; the heads times sigmoid(Wg h), an element
              each; Wo
    mixer "parallel":   left_scale * attention(h) + right_scale * time_mix(h); the attention has no rotation and a gate
              of one number a head; the time mixer blends every token's input with its predecessor's and carries a
              matrix state a head with a decay a key channel (parts/recurrent.py, ``shifted_decay_recurrence``)
    ff "dense":  Wd (gelu_tanh(Wg h) * (Wu h))
    ff "moe":    softmax scores over all experts, the best groups' experts eligible, weights renormalised; experts
              Wd (silu(Wg h) * (Wu h)); a shared expert times sigmoid(w_sg . h)
    logits = head (ln(x) * final.norm) * logit_scale

Tensor names: "embed", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.{q,k,v}" (+ ".b"), "l<i>.mix.{g,o,vmix}",
"l<i>.mix.left.*" likewise, "l<i>.mix.right.{mu.r,mu.k,mu.v,mu.g,mu.w,r,k,v,g,w1,w2,w0,u,norm,o}",
"l<i>.mlp.{gate,up,down}" or "l<i>.mlp.{router,e<j>.{gate,up,down},shared.{gate,up,down,sg}}", "final.norm", "head";
matrices [out, in].
"""
from __future__ import annotations

from ..config.besuzen import BesuzenConfig
from ..config.files import ConfigError
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec

_VALUES_KEY = "first_blending_layer"


def _attention_spec(d: int, a, p: str, gate_per_head: bool, value_mix=None) -> PartSpec:
    if a.rot is not None:
        position = PartSpec("rope", {"head_dim": a.dim, "rotary_dim": a.rot.dims, "theta": a.rot.base, "pairing": "interleaved"})
    else:
        position = PartSpec("none", {"head_dim": a.dim})
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o", "suffix": "", "bias_suffix": ".b"}
    params = {"hidden_size": d, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
              "scale": a.scale, "bias": True, "bias_o": False, "position": position, "gate_per_head": gate_per_head, "names": names}
    if value_mix is not None:
        params["value_mix"] = {"key": _VALUES_KEY, "role": value_mix}
        if value_mix == "blend":
            names["vmix"] = p + "vmix"
    return PartSpec("gqa_attention", params)


def _time_mix_spec(d: int, r, p: str, eps: float, where: str) -> PartSpec:
    if r.decay_rank is None:
        raise ConfigError(f"{where}: the inner width of the decay projection is in no key of config.json; the checkpoint's "
                          "tensor shapes give it, or 'decay_rank' names it")
    return PartSpec("shifted_decay_recurrence", {
        "hidden_size": d, "num_heads": r.heads, "head_dim": r.dim, "decay_rank": r.decay_rank, "norm_eps": eps,
        "names": {"mu": p + "mu.", "r": p + "r", "k": p + "k", "v": p + "v", "g": p + "g", "w1": p + "w1", "w2": p + "w2",
                  "w0": p + "w0", "u": p + "u", "norm": p + "norm", "o": p + "o", "suffix": ""}})


def _feed_forward_spec(d: int, f, p: str) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": f.ff, "activation": "gelu_tanh",
                                      "names": {"gate": p + "gate", "up": p + "up", "down": p + "down", "suffix": ""}})
    names = {"router": p + "router", "expert": p + "e{e}", "suffix": ""}
    shared = None
    if f.shared_ff is not None:
        shared = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": f.shared_ff, "activation": "silu",
                                        "names": {"gate": p + "shared.gate", "up": p + "shared.up", "down": p + "shared.down",
                                                  "suffix": ""}})
        names["shared_gate"] = p + "shared.sg"
    return PartSpec("moe_mlp", {"hidden_size": d, "expert_size": f.ff, "num_experts": f.experts, "top": f.top, "router_bias": False,
                                "scoring": "softmax_all", "groups": f.groups, "keep_groups": f.keep, "shared": shared, "names": names})


def besuzen_spec(cfg: BesuzenConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers, ignored = [], []
    blending_seen = False
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        if l.type == "attention":
            role = None
            if m.v_mix:
                role = "blend" if blending_seen else "source"
                if not blending_seen:
                    ignored.append(p + "mix.vmix")        # the first blending layer's factor is in the file and unused
                blending_seen = True
            mixer = _attention_spec(d, m, p + "mix.", gate_per_head=False, value_mix=role)
        else:
            mixer = PartSpec("parallel_mixers", {"left": _attention_spec(d, m.left, p + "mix.left.", gate_per_head=True),
                                                 "right": _time_mix_spec(d, m.right, p + "mix.right.", eps, f"layers[{i}].mixer.right"),
                                                 "left_scale": m.left_scale, "right_scale": m.right_scale})
        if l.mlp is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
            ignored.append(p + "norm2")
        else:
            ff = _feed_forward_spec(d, l.mlp, p + "mlp.")
            ff_norm = PartSpec("layer_norm", {"size": d, "eps": eps, "name": p + "norm2"})
        layers.append(LayerSpec(block=PartSpec("parallel_pre_norm"), mixer=mixer,
                                mixer_norm=PartSpec("layer_norm", {"size": d, "eps": eps, "name": p + "norm1"}),
                                feed_forward=ff, feed_forward_norm=ff_norm))
    spec = ModelSpec(
        architecture="Besuzen", vocab_size=cfg.vocab, hidden_size=d, max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("scaled_pair_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed",
                                                     "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        final_norm=PartSpec("layer_norm", {"size": d, "eps": eps, "name": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "head", "scale": cfg.logit_scale}),
        ignored_tensors=tuple(ignored))
    spec.validate()
    return spec


BESUZEN = register_architecture(("Besuzen", "besuzen"), BesuzenConfig.from_dict, besuzen_spec,
                                sizes_from_checkpoint=BesuzenConfig.with_checkpoint_sizes)
