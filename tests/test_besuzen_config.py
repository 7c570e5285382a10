"""The Besuzen configuration, its description as parts and the plain implementation's own mechanisms (no GPU)."""
import copy
import math

import pytest
import torch

import besuzen_configs as C
import plain_besuzen as P
from rustyllm_b200 import ConfigError, resolve_architecture
from rustyllm_b200.cache.sequence_cache import KVNeed
from rustyllm_b200.config.besuzen import BesuzenConfig
from rustyllm_b200.models.decoder import DecoderModel
from rustyllm_b200.parts import Runtime
from rustyllm_b200.weights.loader import check_checkpoint
from rustyllm_b200.weights.safetensors_io import Checkpoint

F64 = torch.float64


@pytest.mark.parametrize("name", list(C.CONFIGS) + list(range(12)))
def test_configuration_round_trip_and_tensor_names(tmp_path, name):
    cfg, rank = (C.CONFIGS[name], C.DECAY_RANK[name]) if isinstance(name, str) else C.random_config(name)
    arch = resolve_architecture(cfg)
    d = C.write_model(str(name), str(tmp_path / "m"), seed=1, cfg=cfg, rank=rank)
    ck = Checkpoint(d)
    typed = arch.parse_for(cfg, {n: tuple(e.shape) for n, e in ck.entries.items()})
    assert isinstance(typed, BesuzenConfig) and arch.parse_config(typed.to_dict()) == typed
    spec = arch.build_spec(typed)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    check_checkpoint(model.param_specs(), ck.entries, spec.ignored_tensors, d)     # every tensor named, none left over
    # the first blending layer's factor is the only tensor that is in the file and not read
    blending = [i for i, l in enumerate(cfg["layers"]) if l["type"] == "attention" and l["mixer"].get("v_mix")]
    unread = [f"l{i}.norm2" for i, l in enumerate(cfg["layers"]) if l["mlp"] is None]
    assert sorted(spec.ignored_tensors) == sorted(unread + ([f"l{blending[0]}.mix.vmix"] if blending else []))
    for layer, (kv, state) in zip(cfg["layers"], model.entry_needs[:len(cfg["layers"])]):
        if layer["type"] == "parallel":
            a, r = layer["mixer"]["left"], layer["mixer"]["right"]
            assert kv == KVNeed(a["kv_heads"], a["dim"], None, a["vdim"])
            assert state.nbytes >= 4 * cfg["width"] + 4 * r["heads"] * r["dim"] * r["dim"]
        else:
            a = layer["mixer"]
            assert kv == KVNeed(a["kv_heads"], a["dim"], None, a["vdim"]) and state is None


def test_the_decay_width_comes_from_the_checkpoint_or_from_its_own_key():
    cfg = C.CONFIGS["A"]
    arch = resolve_architecture(cfg)
    with pytest.raises(ConfigError, match="decay"):
        arch.build_spec(arch.parse_config(cfg))
    named = copy.deepcopy(cfg)
    named["layers"][0]["mixer"]["right"]["decay_rank"] = 7
    assert arch.parse_config(named).layers[0].mixer.right.decay_rank == 7
    arch.build_spec(arch.parse_config(named))
    assert arch.parse_for(cfg, {"l0.mix.right.w1": (9, 64)}).layers[0].mixer.right.decay_rank == 9


def test_configuration_errors_name_the_key():
    base = C.CONFIGS["A"]

    def broken(change):
        cfg = copy.deepcopy(base)
        change(cfg)
        return cfg
    cases = [
        (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "mixer type"),
        (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
        (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 4), "groups"),
        (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
        (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
        (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 26), "rot"),
        (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
        (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), "value heads"),
        (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
        (lambda c: c["layers"][0]["mixer"]["right"].pop("dim"), "dim"),
        (lambda c: c.pop("norm"), "norm"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError, match=word):
            BesuzenConfig.from_dict(broken(change))
    plain = copy.deepcopy(base)
    plain.pop("embedding"), plain.pop("logit_scale")
    typed = BesuzenConfig.from_dict(plain)
    assert typed.embedding_scale == 1.0 and typed.logit_scale == 1.0


# --------------------------------------------------------------------------- the plain implementation's mechanisms
def test_plain_layer_norm_takes_the_mean_off():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=F64)
    y = P.layer_norm(x, w, 0.0)
    c = x - 3.0
    torch.testing.assert_close(y, c / math.sqrt(3.5) * w)          # deviations -2, -1, 0, 3: mean square 3.5
    torch.testing.assert_close(P.layer_norm(x + 100.0, w, 0.0), y)   # a shift of the row changes nothing
    assert P.layer_norm(torch.zeros(1, 4, dtype=F64), w, 1e-6).abs().max() == 0


def test_plain_rotation_pairs_neighbours_and_leaves_the_rest():
    x = torch.arange(1.0, 9.0, dtype=F64).view(1, 1, 8).repeat(3, 1, 1)
    y = P.rotate_pairs(x, [0, 1, 5], 4, 100.0)
    torch.testing.assert_close(y[0], x[0])                          # position 0: no turn
    torch.testing.assert_close(y[:, :, 4:], x[:, :, 4:])            # beyond the rotated dimensions: as they were
    a0, a1 = 5 * 1.0, 5 * 100.0 ** (-2.0 / 4)
    want = [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
            3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1)]
    torch.testing.assert_close(y[2, 0, :4], torch.tensor(want, dtype=F64))


def test_plain_routing_keeps_the_best_groups_and_renormalises():
    s = torch.tensor([0.05, 0.30, 0.10, 0.08, 0.25, 0.22], dtype=F64)       # groups of two: maxima 0.30, 0.10, 0.25
    ids, w = P.route(s, 2, 3, 2)
    assert ids == [1, 4]
    torch.testing.assert_close(w, torch.tensor([0.30, 0.25], dtype=F64) / 0.55)
    ids, w = P.route(s, 2, 3, 1)                                             # one group kept: both of its experts
    assert ids == [1, 0]
    ids, _ = P.route(s, 3, 1, 1)
    assert ids == [1, 4, 5]
    ids, _ = P.route(torch.tensor([0.2, 0.2, 0.2, 0.4], dtype=F64), 2, 2, 1)   # ties go to the lower index
    assert ids == [3, 2]


def test_plain_time_mix_state_and_bonus():
    """One head of two channels, by hand: the output reads the state before the token enters it, plus the bonus on
    the token's own product; the state then decays a key channel."""
    d, n = 2, 2
    eye = torch.eye(2, dtype=F64)
    w = {"p.mu." + s: torch.zeros(d, dtype=F64) for s in "rkvgw"}
    w.update({"p.r": eye, "p.k": eye, "p.v": eye, "p.g": eye * 50.0, "p.o": eye, "p.w1": torch.zeros(1, d, dtype=F64),
              "p.w2": torch.zeros(n, 1, dtype=F64), "p.w0": torch.tensor([0.0, -30.0], dtype=F64),
              "p.u": torch.tensor([[0.5, 2.0]], dtype=F64), "p.norm": torch.ones(n, dtype=F64)})
    h = torch.tensor([[1.0, 2.0], [3.0, 1.0]], dtype=F64)
    # token 0: o = diag(u) k v^T applied to r = [[0.5*1*1, 0.5*1*2], [2*2*1, 2*2*2]]^T r = (0.5 + 8, 1 + 16)
    # state after token 0: k v^T = [[1, 2], [2, 4]] (rows: key channels); decays exp(-1) and exp(-exp(-30)) ~ 1
    # token 1 (r = k = v = (3, 1)): o = (S0 + diag(u) k v^T)^T r with S0 = [[1, 2], [2, 4]], diag(u) k v^T = [[4.5, 1.5], [6, 2]]
    o0 = torch.tensor([8.5, 17.0], dtype=F64)
    o1 = torch.tensor([3 * 5.5 + 1 * 8.0, 3 * 3.5 + 1 * 6.0], dtype=F64)
    want = torch.stack([P.unit_rms(o0, 0.0), P.unit_rms(o1, 0.0)]) * P.silu(h * 50.0)
    torch.testing.assert_close(P.time_mix(h, w, "p.", {"heads": 1, "dim": 2}, 0.0), want)
    # the predecessor's input enters through mu: with mu = 1 every blend is the previous token's input
    for s in "rkvgw":
        w["p.mu." + s] = torch.ones(d, dtype=F64)
    shifted = P.time_mix(h, w, "p.", {"heads": 1, "dim": 2}, 1e-6)
    assert shifted[0].abs().max() == 0                              # the first token's predecessor is zero
