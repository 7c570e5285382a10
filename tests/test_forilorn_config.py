"""The Forilorn design without a GPU: configuration round trip and errors, tensor names against the parts' parameters,
the cache's pages under a chunked mask, the value-less storage of a latent layer, and the plain implementation's own
properties (a prefix's logits do not depend on what follows; the masks)."""
import copy

import pytest
import torch

import forilorn_configs as C
import plain_forilorn as P
from rustyllm_b200 import ConfigError, resolve_architecture
from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache
from rustyllm_b200.models.decoder import DecoderModel
from rustyllm_b200.parts import Runtime


def _model(cfg):
    arch = resolve_architecture(cfg)
    return DecoderModel(arch.build_spec(arch.parse_config(cfg)), Runtime(torch.device("cpu"), torch.float32))


@pytest.mark.parametrize("name", list(C.CONFIGS) + list(range(8)))
def test_configuration_round_trip_and_tensor_names(name):
    cfg = C.CONFIGS[name] if isinstance(name, str) else C.random_config(name)
    arch = resolve_architecture(cfg)
    assert arch.name == "Forilorn"
    typed = arch.parse_config(cfg)
    assert arch.parse_config(typed.to_dict()) == typed
    m = _model(cfg)
    names = {s.name: tuple(s.shape) for ps in m.param_specs().values() if ps.alias_of is None for s in ps.sources}
    assert names == C.tensor_shapes(cfg)
    # the head is the embedding table itself
    assert m.param_specs()["head.weight"].alias_of == "embedding.weight"
    # every layer run has keys; the embedding keeps one token of state a sequence
    assert all(n is not None for n in m.kv_needs()[:-1]) and m.kv_needs()[-1] is None
    assert m.state_needs()[-1].nbytes == 4


def test_what_may_be_absent_and_what_is_refused():
    base = C.CONFIGS["P"]
    cfg = copy.deepcopy(base)
    del cfg["residual_mult"], cfg["embedding"]
    typed = resolve_architecture(cfg).parse_config(cfg)
    assert typed.residual_mult == 1.0 and typed.embedding_scale == 1.0 and typed.bigram is None
    for change, word in ((lambda c: c["layers"][0].update(type="conv"), "not known"),
                         (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
                         (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "at most"),
                         (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not known"),
                         (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
                         (lambda c: c.update(layers=[]), "layers")):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError, match=word):
            resolve_architecture(cfg).parse_config(cfg)


def test_norm_weights_stored_around_zero_are_bound_as_one_plus_weight():
    from rustyllm_b200.parts.norm import RMSNorm
    n = RMSNorm(Runtime(torch.device("cpu"), torch.float32), size=4, eps=1e-6, name="w", offset=1.0)
    n.bind({"weight": torch.tensor([0.0, -0.25, 0.5, 1.0])})
    assert n.weight.tolist() == [1.0, 0.75, 1.5, 2.0]
    plain = RMSNorm(Runtime(torch.device("cpu"), torch.float32), size=4, eps=1e-6, name="w")
    plain.bind({"weight": torch.tensor([0.0, -0.25, 0.5, 1.0])})
    assert plain.weight.tolist() == [0.0, -0.25, 0.5, 1.0]


@pytest.mark.parametrize("chunk", [1, 5, 64, 70, 128, 200])
def test_pages_under_a_chunked_mask_go_back_once_their_block_has_passed(chunk):
    cache = SequenceCache([KVNeed(2, 16, None, None, 0, chunk), KVNeed(1, 40, 70, 0)], [None, None], 64 * 12, torch.float32, "cpu", max_slots=2)
    assert cache.groups[1].values.numel() == 0            # a latent layer stores no values of its own
    s = cache.alloc_slot()
    g = cache.groups[0]
    n = 0
    for cnt in (3, 61, 1, 1, 130, 1, 70, 1, 1, 200, 1):
        cache.prepare([s], [cnt])
        cache.commit([s], [cnt])
        cache.check()
        n += cnt
        first_needed = n - n % chunk                       # the next query's block starts here
        for page, held in enumerate(g.slot_pages[s]):
            if (page + 1) * 64 <= first_needed:
                assert held == -1, (n, page)
            else:
                assert held >= 0, (n, page)
    cache.free_slot(s)
    cache.check()
    assert g.pages.held_count == 0
    with pytest.raises(ValueError):
        KVNeed(1, 8, 4, None, 0, 4)


def test_plain_implementation_a_prefix_does_not_depend_on_what_follows(tmp_path):
    d = C.write_model("P", str(tmp_path / "P"))
    cfg, w = P.load_model_dir(d)
    toks = [int(t) for t in torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(3))]
    whole = P.forward(cfg, w, toks)
    part = P.forward(cfg, w, toks[:17])
    assert torch.allclose(whole[:17], part, rtol=0, atol=1e-12)
    # the pair table matters, and so does the order of the pair
    swapped = toks[:]
    swapped[4], swapped[5] = swapped[5], swapped[4]
    assert not torch.allclose(P.embed(cfg, w, toks)[6], P.embed(cfg, w, swapped)[6])
    assert torch.equal(P.embed(cfg, w, toks)[7], P.embed(cfg, w, swapped)[7])


def test_plain_masks():
    m = P.chunk_mask(10, 4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert m[8].tolist() == [False] * 8 + [True, False]
    w = P.window_mask(10, 3)
    assert w[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4
    assert P.chunk_mask(4, None).tolist() == P.window_mask(4, None).tolist() == torch.ones(4, 4).tril().bool().tolist()
