"""The Forilorn design on the GPU against the plain implementation (tests/plain_forilorn.py): each mechanism alone at
its kernel's own interface, then the engine - the residual stream after every layer, whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, slots, pages and
state used again, the edges of chunks and windows in prompts and in decoding, long decoding - and greedy generation
through ``Runner.generate``."""
import functools
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import forilorn_configs as C
import plain_forilorn as P
from gpu_helpers import BF16_REL_MAX, BF16_REL_MEAN, F32_REL, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = list(C.CONFIGS)
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("forilorn")
    return {n: C.write_model(n, str(root / n)) for n in NAMES}


@functools.lru_cache(maxsize=None)
def _plain(d):
    return P.load_model_dir(d)


_LOGITS = {}


def plain_logits(d, tokens):
    key = (d, tuple(tokens))
    if key not in _LOGITS:
        cfg, w = _plain(d)
        _LOGITS[key] = P.forward(cfg, w, list(tokens))
    return _LOGITS[key]


@functools.lru_cache(maxsize=None)
def runner(d, dtype, max_cache_tokens=64 * 40, max_batch=8):
    from rustyllm_b200 import Runner
    return Runner.from_path(d, dtype=dtype, max_cache_tokens=max_cache_tokens, max_batch=max_batch)[0]


def close(got, ref, dtype, cfg, what):
    """32-bit: 3e-5 of a logit row's rms.  bfloat16: the bounds of gpu_helpers (derived for three pre-norm layers,
    whose sublayers add a small term to the stream) times three and grown with the square root of the layers: here
    every sublayer's output is normed to unit size, rounding noise included, before it joins the stream."""
    got, ref = got.detach().to("cpu", F64), ref.detach().to("cpu", F64)
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = (got - ref).abs() / ref.pow(2).mean(dim=-1, keepdim=True).sqrt().clamp_min(1e-30)
    rows = err.max(dim=-1).values
    if dtype == "float32":
        assert rows.max().item() <= F32_REL, f"{what}: {rows.max().item():.3e} (row {rows.argmax().item()})"
    else:
        grow = 3.0 * math.sqrt(max(1.0, len(cfg["layers"]) / 3.0))
        over = (rows > BF16_REL_MAX * grow).double().sum().item()
        assert over <= max(2.0, 0.03 * rows.numel()), f"{what}: {over:.0f} of {rows.numel()} rows above {BF16_REL_MAX * grow:.3f} (worst {rows.max().item():.3e})"
        assert rows.max().item() <= 3.0 * BF16_REL_MAX * grow, f"{what}: max {rows.max().item():.3e} (row {rows.argmax().item()})"
        assert err.mean().item() <= BF16_REL_MEAN * grow, f"{what}: mean {err.mean().item():.3e}"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def tdt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def rounded(x, dtype):
    """What the kernel is given: the float64 test data rounded to the run's storage type."""
    return x.to(tdt(dtype)).to(F64)


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=1.2e-2, atol=1.2e-2)


def step_state(slot, at, cnt, tokens=None):
    from rustyllm_b200.engine.step import StepState
    return StepState(cnt, 1, i32(tokens if tokens is not None else [0] * cnt), i32(list(range(at, at + cnt))), i32([slot] * cnt),
                     i32([0, cnt]), i32([slot]), i32([at + cnt]), i32([]), [cnt], [at + cnt], cnt, at + cnt, cnt == 1)


def inv_freq(dims, base):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)] or [0.0], dtype=torch.float32, device=DEV)


# =========================================================================== mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(61, 7, 13), (1, 1, 1), (499, 1000003, 999983), (5, 0, 3), (None, 0, 0)])
def test_scaled_pair_embedding_across_steps(dtype, buckets, mul_prev, mul_cur):
    """Two sequences packed in every step and cut differently; the previous token crosses the cuts through the slot's
    state, a sequence's first token takes the row behind the buckets, and a slot that is used again starts anew."""
    from rustyllm_b200 import kernels as K
    V, d, scale = 300, 40, 3.5
    g = torch.Generator().manual_seed(5)
    E = rounded(torch.randn(V, d, generator=g, dtype=F64), dtype)
    B = None if buckets is None else rounded(torch.randn(buckets + 1, d, generator=g, dtype=F64), dtype)
    cfg = {"embedding": {"scale": scale}}
    if buckets is not None:
        cfg["embedding"]["bigram"] = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    w = {"embed": E, "bigram": B}
    area = torch.zeros((4, 256 + 4 + 256), dtype=torch.uint8, device=DEV)
    state = area[:, 256:260]
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    for rnd, portions in enumerate(([(5, 1, 1, 2, 30), (1, 1, 1, 1, 7)], [(1, 9), (12, 1)])):
        seqs = [random_tokens(V, sum(p), 10 * rnd + s) for s, p in enumerate(portions)]
        ref = [P.embed(cfg, w, t) for t in seqs]
        slots, at, got = [3, 1], [0, 0], [[], []]
        state[slots] = 0                                      # what the cache does when it hands a slot out
        for step in range(max(len(p) for p in portions)):
            live = [s for s in range(2) if step < len(portions[s])]
            cnt = [portions[s][step] for s in live]
            toks = [t for s, c in zip(live, cnt) for t in seqs[s][at[s]:at[s] + c]]
            pos = [p for s, c in zip(live, cnt) for p in range(at[s], at[s] + c)]
            out = torch.empty((len(toks), d), dtype=torch.float32, device=DEV)
            K.embedding_pair(E.to(tdt(dtype)).to(DEV), None if B is None else B.to(tdt(dtype)).to(DEV), i32(toks), i32(pos),
                             i32([slots[s] for s, c in zip(live, cnt) for _ in range(c)]), i32([0] + list(np.cumsum(cnt))), state,
                             scale, mul_prev, mul_cur, buckets or 1, out, err)
            o = 0
            for s, c in zip(live, cnt):
                got[s].append(out[o:o + c].double().cpu())
                o += c
                at[s] += c
        for s in range(2):
            torch.testing.assert_close(torch.cat(got[s]), ref[s], rtol=1e-6, atol=1e-6)
    assert int(err.item()) == 0
    K.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,dims,base", [(4, 2, 16, 8, 100.0), (4, 1, 64, 64, 10000.0), (2, 2, 128, 32, 1.0e6), (6, 3, 18, 0, 1.0),
                                               (3, 3, 50, 50, 200000.0), (2, 1, 17, 8, 100.0)])
def test_rotation_of_neighbours_then_unit_heads_values_from_keys(dtype, H, G, hd, dims, base):
    """q and k heads: neighbouring pairs of the first ``dims`` dimensions turn by the position, then the head is divided
    by its root mean square; the keys' pages take that, the values' pages the keys as they were projected.  Positions
    up to 70,000 (the angle is computed in 32-bit from an exact position)."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache
    torch.manual_seed(hd)
    eps = 1e-5
    for start, cnt in ((0, 70), (1000, 11)):
        cache = SequenceCache([KVNeed(G, hd, None, None)], [None], 64 * 6, tdt(dtype), DEV, max_slots=3)
        cache.alloc_slot()
        slot = cache.alloc_slot()
        group, layer = cache.kv_entry(0)
        writes = start == 0                                   # far positions: the queries alone, without pages
        if writes:
            cache.prepare([slot], [cnt])
        u = rounded(torch.randn(cnt, (H + G) * hd + 5, dtype=F64), dtype)
        pos = list(range(start, start + cnt))
        rot = {"dims": dims, "base": base} if dims else None
        q = P.unit_rms(P.rotate_pairs(u[:, :H * hd].reshape(cnt, H, hd), pos, rot), eps)
        k = P.unit_rms(P.rotate_pairs(u[:, H * hd:(H + G) * hd].reshape(cnt, G, hd), pos, rot), eps)
        v = u[:, H * hd:(H + G) * hd].reshape(cnt, G, hd)
        dev_u = u.to(tdt(dtype)).to(DEV)
        st = step_state(slot, start, cnt)
        K.qk_rotate_unit(dev_u, dev_u, st.positions, st.slot_of_token, group.page_table, inv_freq(dims, base), dims, True, eps,
                         H, G, hd, group.k_pool(layer) if writes else None, group.v_pool(layer) if writes else None, value_from_key=True)
        K.check_device_errors()
        # a position of 1,000 times a frequency rounded to 24 bits: the angle is good to 1e-4
        t = (dict(rtol=3e-5, atol=3e-5) if writes else dict(rtol=3e-4, atol=3e-4)) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(dev_u[:, :H * hd].double().cpu().view(cnt, H, hd), q, **t)
        assert torch.equal(dev_u[:, (H + G) * hd:].double().cpu(), u[:, (H + G) * hd:])       # what lies behind stays
        if not writes:
            continue
        pages = group.page_table[slot].tolist()
        for j, p in enumerate(pos):
            row_k = group.k_pool(layer)[pages[p // 64], :, p % 64].double().cpu()
            row_v = group.v_pool(layer)[pages[p // 64], :, p % 64].double().cpu()
            torch.testing.assert_close(row_k, k[j], **t)
            assert torch.equal(row_v, v[j])
        cache.commit([slot], [cnt])
        cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,hd,rd,r,qr,dims", [(3, 24, 8, 32, 40, 8), (2, 8, 16, 24, 16, 16), (4, 12, 8, 40, 20, 4), (1, 40, 6, 12, 36, 0),
                                               (2, 32, 0, 64, 24, 0), (3, 9, 4, 15, 11, 4)])
def test_latents_are_normed_and_the_shared_key_part_turned(dtype, H, hd, rd, r, qr, dims):
    """From one projected row [query latent | key/value latent | rotary key | gates]: both latents normed with their plain
    weights, the rotary key turned, the key row [latent | rotary key] in its page; and the query's rotary part turned
    into its place behind the latent columns of every head."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache
    torch.manual_seed(r + rd)
    eps, base, cnt, start = 1e-6, 500.0, 75, 60
    cache = SequenceCache([KVNeed(1, r + rd, 200, 0)], [None], 64 * 6, tdt(dtype), DEV, max_slots=2)
    slot = cache.alloc_slot()
    group, layer = cache.kv_entry(0)
    cache.prepare([slot], [start]); cache.commit([slot], [start])
    cache.prepare([slot], [cnt])
    u = rounded(2.0 * torch.randn(cnt, qr + r + rd + H, dtype=F64), dtype)
    wq, wkv = 1.0 + 0.1 * torch.randn(qr, dtype=F64).float().double(), 1.0 + 0.1 * torch.randn(r, dtype=F64).float().double()
    pos = list(range(start, start + cnt))
    rot = {"dims": dims, "base": base} if dims else None
    cq_ref = P.unit_rms(u[:, :qr], eps) * wq
    c_ref = P.unit_rms(u[:, qr:qr + r], eps) * wkv
    kr_ref = P.rotate_pairs(u[:, qr + r:qr + r + rd], pos, rot)
    st = step_state(slot, start, cnt)
    cq = torch.empty((cnt, qr), dtype=tdt(dtype), device=DEV)
    fr = inv_freq(dims, base)
    K.latent_prepare(u.to(tdt(dtype)).to(DEV), qr, r, rd, wq.float().to(DEV), wkv.float().to(DEV), eps, cq, st.positions,
                     st.slot_of_token, group.page_table, fr, dims, True, group.k_pool(layer))
    t = dict(rtol=3e-5, atol=3e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(cq.double().cpu(), cq_ref, **t)
    pages = group.page_table[slot].tolist()
    rows = torch.stack([group.k_pool(layer)[pages[p // 64], 0, p % 64] for p in pos]).double().cpu()
    torch.testing.assert_close(rows[:, :r], c_ref, **t)
    torch.testing.assert_close(rows[:, r:], kr_ref, **t)
    q = rounded(torch.randn(cnt, H * (hd + rd), dtype=F64), dtype)
    out = torch.full((cnt, H * (r + rd)), 7.0, dtype=tdt(dtype), device=DEV)
    K.latent_query(q.to(tdt(dtype)).to(DEV), out, H, hd, rd, r, st.positions, fr, dims, True)
    K.check_device_errors()
    got = out.double().cpu().view(cnt, H, r + rd)
    assert (got[:, :, :r] == 7.0).all()                         # the latent columns are the next product's to fill
    torch.testing.assert_close(got[:, :, r:], P.rotate_pairs(q.view(cnt, H, hd + rd)[:, :, hd:], pos, rot), **t)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_and_the_scaled_norm_that_joins_the_stream(dtype):
    from rustyllm_b200 import kernels as K
    torch.manual_seed(3)
    z = rounded(3.0 * torch.randn(50, 44, dtype=F64), dtype)
    out = torch.empty((50, 44), dtype=tdt(dtype), device=DEV)
    K.gelu_tanh(z.to(tdt(dtype)).to(DEV), out)
    torch.testing.assert_close(out.double().cpu(), P.gelu_tanh(z), **tol(dtype))
    x, y = torch.randn(9, 44, dtype=F64).float(), (40.0 * torch.randn(9, 44, dtype=F64)).float()
    w = (0.1 * torch.randn(44, dtype=F64)).float()
    xd = x.clone().to(DEV)
    xb = torch.empty((9, 44), dtype=torch.bfloat16, device=DEV)
    K.norm_add(xd, y.to(DEV), 1.0, None, 0.0, (1.0 + w).to(DEV), 1e-5, xb, out_scale=0.7)
    ref = x.double() + 0.7 * P.unit_rms(y.double(), 1e-5) * (1.0 + w.double())
    torch.testing.assert_close(xd.double().cpu(), ref, rtol=1e-5, atol=1e-5)
    assert torch.equal(xb.cpu(), xd.cpu().to(torch.bfloat16))
    K.check_device_errors()


def _through_cache(dtype, need, portions, write, attend, width):
    """One sequence fed in ``portions`` through the cache: ``write(step, at, cnt, group, layer)`` fills the step's rows,
    ``attend(step, at, cnt, group, layer, out)`` runs the attention dispatcher; returns [n, width] float64.  The sequence
    lives in slot 1, behind a slot that stays empty."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import SequenceCache
    n = sum(portions)
    cache = SequenceCache([need], [None], 64 * (n // 64 + 3), tdt(dtype), DEV, max_slots=3)
    cache.alloc_slot()
    slot = cache.alloc_slot()
    group, layer = cache.kv_entry(0)
    outs, at = [], 0
    for cnt in portions:
        cache.prepare([slot], [cnt])
        st = step_state(slot, at, cnt)
        held = write(st, at, cnt, group, layer)
        out = torch.empty((cnt, width), dtype=tdt(dtype), device=DEV)
        attend(st, at, cnt, group, layer, out, held)
        cache.commit([slot], [cnt])
        outs.append(out.double().cpu())
        at += cnt
    K.check_device_errors()
    cache.check()
    return torch.cat(outs)


def chunked_attention(dtype, H, G, hd, chunk, scale, q, k, gate, portions, rot=None, eps=1e-6):
    """q [n, H*hd], k [n, G*hd], gate [n, H*hd] as projected (float64): rotation, unit heads, values from keys and the
    chunked mask, as the mixer runs them."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import KVNeed
    dims, base = (rot["dims"], rot["base"]) if rot else (0, 1.0)
    fr = inv_freq(dims, base)

    def write(st, at, cnt, group, layer):
        u = torch.cat([q[at:at + cnt], k[at:at + cnt], gate[at:at + cnt]], dim=1).to(tdt(dtype)).to(DEV).contiguous()
        K.qk_rotate_unit(u, u, st.positions, st.slot_of_token, group.page_table, fr, dims, True, eps, H, G, hd,
                         group.k_pool(layer), group.v_pool(layer), value_from_key=True)
        return u

    def attend(st, at, cnt, group, layer, out, u):
        K.attention(u, group.k_pool(layer), group.v_pool(layer), group.page_table, st, out, H, G, hd, scale, 0, value_dim=hd,
                    gate=u[:, (H + G) * hd:], chunk=chunk or 0)

    return _through_cache(dtype, KVNeed(G, hd, None, None, 0, chunk), portions, write, attend, H * hd)


def plain_chunked(H, G, hd, chunk, scale, q, k, gate, rot=None, eps=1e-6):
    n = q.shape[0]
    pos = list(range(n))
    qq = P.unit_rms(P.rotate_pairs(q.view(n, H, hd), pos, rot), eps)
    kk = P.unit_rms(P.rotate_pairs(k.view(n, G, hd), pos, rot), eps)
    vv = k.view(n, G, hd)
    vis = P.chunk_mask(n, chunk)
    heads = [P.softmax_rows((qq[:, a] @ kk[:, a // (H // G)].T) * scale, vis) @ vv[:, a // (H // G)] for a in range(H)]
    return torch.cat(heads, dim=-1) * P.sigmoid(gate)


CHUNK_SHAPES = [(4, 2, 16), (4, 1, 64), (2, 2, 128), (6, 3, 18), (8, 2, 32)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd", CHUNK_SHAPES)
@pytest.mark.parametrize("chunk", [None, 1, 9, 64, 70, 130])
def test_chunked_attention_with_unit_heads_values_from_keys_and_gate_alone(dtype, H, G, hd, chunk):
    """A prompt portion across the blocks' and the pages' borders, a short portion, single tokens, a portion again."""
    torch.manual_seed(H * hd + (chunk or 0))
    n = 275
    q, k, g = (rounded(torch.randn(n, w, dtype=F64), dtype) for w in (H * hd, G * hd, H * hd))
    rot = {"dims": hd if hd % 4 == 0 else 2 * (hd // 4), "base": 1000.0}
    scale = 2.5 / math.sqrt(hd)
    got = chunked_attention(dtype, H, G, hd, chunk, scale, q, k, g, [150, 2] + [1] * 70 + [53], rot)
    ref = plain_chunked(H, G, hd, chunk, scale, q, k, g, rot)
    torch.testing.assert_close(got, ref, **(dict(rtol=3e-5, atol=3e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd", [(4, 1, 64), (2, 2, 128), (4, 2, 16)])
@pytest.mark.parametrize("chunk,n", [(None, 700), (9, 60), (64, 200), (70, 220), (130, 400)])
def test_one_key_that_stands_out_is_seen_exactly_inside_its_block(dtype, H, G, hd, chunk, n):
    """Every query points along one direction and the key at position j lies along it (a score far above the others)
    with a value of its own, 100 in every element: a query's output is near 100 where it sees j and of order 1 where it
    does not.  j is the first position of a block, so the block's last query still sees it and the next block's first
    does not; without blocks j lies hundreds of positions back.  Read in a prompt portion and token by token."""
    torch.manual_seed(n)
    C = chunk or n
    j = C * ((n - 1) // C - 1) if chunk else 3              # the start of the block before the last
    u = torch.randn(hd, dtype=F64)
    u = u / u.pow(2).mean().sqrt()
    q = rounded(u.repeat(n, H) + 0.05 * torch.randn(n, H * hd, dtype=F64), dtype)
    k = rounded(torch.randn(n, G * hd, dtype=F64), dtype)
    k[j] = rounded(100.0 * u.repeat(G), dtype)               # as projected: the value; unit size makes the key u
    g = torch.full((n, H * hd), 20.0, dtype=F64)             # gates open
    scale = 30.0 / hd                                        # the aligned score is 30, the others of order 30 / sqrt(hd)
    ref = plain_chunked(H, G, hd, chunk, scale, q, k, g)
    sees = torch.tensor([(i >= j) and (chunk is None or i // C == j // C) for i in range(n)])
    along = (ref.view(n, H, hd) * u).mean(-1) / 100.0        # 1 where the key at j carries the row
    assert (along[sees] > 0.9).all() and (along[~sees].abs() < 0.2).all()
    last_block = n - 1 - (n - 1) % C if chunk else n - 40
    for portions in ([n], [last_block - 3] + [1] * (n - last_block + 3), [j + 1, C - 1 if chunk else 5, n - j - (C if chunk else 6)]):
        got = chunked_attention(dtype, H, G, hd, chunk, scale, q, k, g, portions)
        # bfloat16: values of 100 leave roundings of 0.25 in an output and of 0.4 % in a weight
        torch.testing.assert_close(got, ref, **(dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=3e-2, atol=1e-1)))


def latent_scan(dtype, H, r, rd, window, scale, ql, rows, gate, portions):
    """ql [n, H*(r+rd)]: the queries in the cache's own coordinates; rows [n, r+rd]: the cached rows; gate [n, H]."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import KVNeed

    def write(st, at, cnt, group, layer):
        pool = group.k_pool(layer)
        pages = group.page_table[int(st.seq_slots[0])].tolist()
        for p in range(at, at + cnt):
            pool[pages[p // 64], 0, p % 64] = rows[p].to(tdt(dtype)).to(DEV)
        return None

    def attend(st, at, cnt, group, layer, out, _):
        pool = group.k_pool(layer)
        K.attention(ql[at:at + cnt].to(tdt(dtype)).to(DEV).contiguous(), pool, pool, group.page_table, st, out, H, 1, r + rd, scale,
                    window or 0, value_dim=r, gate=gate[at:at + cnt].to(tdt(dtype)).to(DEV).contiguous(), gate_per_head=True,
                    values_in_keys=True)

    return _through_cache(dtype, KVNeed(1, r + rd, window, 0), portions, write, attend, H * r)


def plain_latent_scan(H, r, rd, window, scale, ql, rows, gate):
    n = ql.shape[0]
    vis = P.window_mask(n, window)
    qh = ql.view(n, H, r + rd)
    heads = [(P.softmax_rows((qh[:, a] @ rows.T) * scale, vis) @ rows[:, :r]) * P.sigmoid(gate[:, a:a + 1]) for a in range(H)]
    return torch.cat(heads, dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,r,rd", [(3, 32, 8), (2, 24, 16), (16, 64, 32), (1, 12, 6), (4, 256, 32), (2, 320, 0), (5, 64, 16), (20, 32, 16),
                                    (4, 80, 16), (8, 40, 8), (1, 512, 64)])
@pytest.mark.parametrize("window", [None, 1, 5, 64, 65, 130])
def test_heads_over_one_cached_row_whose_front_is_the_value(dtype, H, r, rd, window):
    torch.manual_seed(r + rd + (window or 0))
    n = 215
    ql = rounded(torch.randn(n, H * (r + rd), dtype=F64), dtype)
    rows = rounded(torch.randn(n, r + rd, dtype=F64), dtype)
    gate = rounded(2.0 * torch.randn(n, H, dtype=F64), dtype)
    scale = 2.0 / math.sqrt(r + rd)
    got = latent_scan(dtype, H, r, rd, window, scale, ql, rows, gate, [140, 2] + [1] * 40 + [33])
    ref = plain_latent_scan(H, r, rd, window, scale, ql, rows, gate)
    torch.testing.assert_close(got, ref, **(dict(rtol=3e-5, atol=3e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,r,rd", [(4, 32, 16), (2, 96, 8), (3, 80, 16)])
@pytest.mark.parametrize("window,n", [(None, 600), (5, 80), (64, 200), (65, 200), (150, 360)])
def test_one_row_that_stands_out_is_seen_exactly_inside_the_window(dtype, H, r, rd, window, n):
    """The row at position j carries a score far above the others and a value of 50 in every element: queries at
    j .. j + window - 1 return about 50, the query at j + window about 0.  Through a prompt, and with the window passing
    over j while tokens are decoded one by one."""
    torch.manual_seed(n + r)
    j = n - window - 20 if window else 2
    u = torch.randn(r + rd, dtype=F64)
    u[:r] = u[:r] - u[:r].mean()                              # so that the standing-out row's value can be set apart
    noise = 0.05 * torch.randn(n, H, r + rd, dtype=F64)
    noise[..., :r] -= noise[..., :r].mean(-1, keepdim=True)  # the row at j adds 50 to every value element: keep its score at 30
    ql = rounded(u.repeat(n, H) + noise.reshape(n, H * (r + rd)), dtype)
    rows = rounded(0.3 * torch.randn(n, r + rd, dtype=F64), dtype)
    rows[j] = rounded(torch.cat([50.0 + u[:r], u[r:]]), dtype)
    gate = torch.full((n, H), 20.0, dtype=F64)
    scale = 30.0 / float(u @ u)
    ref = plain_latent_scan(H, r, rd, window, scale, ql, rows, gate)
    sees = torch.tensor([i >= j and (window is None or i - j < window) for i in range(n)])
    level = ref.view(n, H, r).mean(-1) / 50.0
    assert (level[sees] > 0.9).all() and (level[~sees].abs() < 0.1).all()
    edge = j + (window or 40)
    for portions in ([n], [edge - 4] + [1] * (n - edge + 4), [j + 1, 2, n - j - 3]):
        got = latent_scan(dtype, H, r, rd, window, scale, ql, rows, gate, portions)
        torch.testing.assert_close(got, ref, **(dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=3e-2, atol=5e-2)))


# =========================================================================== the model, layer by layer
@pytest.mark.parametrize("name", NAMES)
def test_the_residual_after_every_layer_in_32_bit(dirs, name):
    d = dirs[name]
    cfg, w = _plain(d)
    r = runner(d, "float32")
    toks = random_tokens(cfg["vocab"], 150, 11)
    _, want = P.forward(cfg, w, toks, True)
    got = []
    blocks = r.model.blocks
    originals = [b.forward for b in blocks]
    try:
        for b, f in zip(blocks, originals):
            def wrapped(x, step, cache, *a, _f=f, **kw):
                out = _f(x, step, cache, *a, **kw)
                got.append(x.double().cpu())
                return out
            b.forward = wrapped
        s = r.engine.alloc_slot()
        r.engine.step([s], [toks], None)
        r.engine.free_slot(s)
    finally:
        for b, f in zip(blocks, originals):
            b.forward = f
    assert len(got) == len(want) == len(cfg["layers"])
    for i, (a, b_) in enumerate(zip(got, want)):
        assert (a - b_).abs().max().item() <= 3e-5 * b_.abs().max().item(), f"{name}: after layer {i}"


# =========================================================================== the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_first_tokens(dirs, name, dtype):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    for seed, n in enumerate([1, 2, 3, 17, 64, 65, 129, 150]):
        toks = random_tokens(cfg["vocab"], n, 100 + seed)
        s = r.engine.alloc_slot()
        got = r.engine.step([s], [toks], "all")
        r.engine.free_slot(s)
        close(got, plain_logits(d, toks), dtype, cfg, f"{name} whole n={n}")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token_over_the_edges_of_blocks_and_windows(dirs, name, dtype):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    for n, tail in ((40, 39), (150, 90), (200, 32), (275, 150)):
        toks = random_tokens(cfg["vocab"], n, 200 + n)
        s = r.engine.alloc_slot()
        rows = [r.engine.step([s], [toks[:n - tail]], "all")]
        for t in toks[n - tail:]:
            rows.append(r.engine.step([s], [[t]], "last"))
        r.engine.free_slot(s)
        close(torch.cat(rows), plain_logits(d, toks), dtype, cfg, f"{name} n={n} last {tail} one by one")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 100])
def test_a_prompt_in_portions(dirs, name, dtype, portion):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    n = 141 if portion < 7 else 207
    toks = random_tokens(cfg["vocab"], n, 300 + portion)
    s = r.engine.alloc_slot()
    rows = [r.engine.step([s], [toks[i:i + portion]], "all") for i in range(0, n, portion)]
    r.engine.free_slot(s)
    close(torch.cat(rows), plain_logits(d, toks), dtype, cfg, f"{name} portions of {portion}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_equal_each_request_alone_and_reuse_slots_pages_and_state(dirs, name, dtype):
    """Two batches through a cache that only just holds one: prompts of unequal lengths in one step, decoded together,
    the shorter requests ending earlier; the second batch gets the first one's slots (with the previous token they
    held) and pages."""
    d = dirs[name]
    cfg, _ = _plain(d)
    from rustyllm_b200 import Runner
    r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 7, max_batch=4)
    eng = r.engine
    for batch_no, (lens, total) in enumerate([([5, 70, 17, 1], [13, 140, 17, 30]), ([64, 3, 130], [66, 90, 141])]):
        seqs = [random_tokens(cfg["vocab"], t, 400 + 10 * batch_no + i) for i, t in enumerate(total)]
        slots = [eng.alloc_slot() for _ in seqs]
        assert sorted(slots) == list(range(len(seqs))), "freed slots are handed out again, lowest first"
        got = [[] for _ in seqs]
        out = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        o = 0
        for i, n in enumerate(lens):
            got[i].append(out[o:o + n])
            o += n
        at = list(lens)
        live = [i for i in range(len(seqs)) if at[i] < total[i]]
        for i in range(len(seqs)):
            if i not in live:
                eng.free_slot(slots[i])
        while live:
            out = eng.step([slots[i] for i in live], [[seqs[i][at[i]]] for i in live], "last")
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                at[i] += 1
            for i in [i for i in live if at[i] == total[i]]:
                eng.free_slot(slots[i])
            live = [i for i in live if at[i] < total[i]]
        for i, s in enumerate(seqs):
            close(torch.cat(got[i]), plain_logits(d, s), dtype, cfg, f"{name} batch {batch_no} request {i}")
        r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_from_the_first_token(dirs, name, dtype):
    """One token, then 280 more one by one: across four page borders, every block's and window's edge, with pages given
    back on the way; the captured single-token step takes over after the first eager one."""
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    toks = random_tokens(cfg["vocab"], 281, 77)
    s = r.engine.alloc_slot()
    rows = [r.engine.step([s], [[t]], "last") for t in toks]
    r.engine.free_slot(s)
    close(torch.cat(rows), plain_logits(d, toks), dtype, cfg, f"{name} 281 single tokens")
    r.cache.check()


@pytest.mark.parametrize("name", NAMES)
def test_logits_do_not_depend_on_the_batch_or_the_cut_in_32_bit(dirs, name):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, "float32")
    a, b, c = (random_tokens(cfg["vocab"], n, 500 + n) for n in (90, 33, 141))
    s = r.engine.alloc_slot()
    alone = r.engine.step([s], [a], "all")
    r.engine.free_slot(s)
    slots = [r.engine.alloc_slot() for _ in range(3)]
    first = r.engine.step(slots, [b, a[:50], c], [[], list(range(50)), []])
    second = r.engine.step(slots[1:], [a[50:], [1, 2]], [list(range(40)), []])
    for s in slots:
        r.engine.free_slot(s)
    both = torch.cat([first, second])
    assert (both - alone).abs().max().item() <= 1e-5 * alone.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_configurations_with_every_size_drawn_at_random(tmp_path, dtype, seed):
    """A prompt, a second portion, then single tokens, beside a shorter request in the same steps."""
    cfg = C.random_config(1000 + seed)
    d = C.write_model(None, str(tmp_path / "m"), seed=seed, cfg=cfg)
    from rustyllm_b200 import Runner
    r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 12, max_batch=3)
    a, b = random_tokens(cfg["vocab"], 170, seed), random_tokens(cfg["vocab"], 75, seed + 50)
    sa, sb = r.engine.alloc_slot(), r.engine.alloc_slot()
    rows_a = [r.engine.step([sa, sb], [a[:100], b[:70]], [list(range(100)), []])]
    rows_a.append(r.engine.step([sa], [a[100:131]], "all"))
    rows_b = []
    for i in range(5):
        out = r.engine.step([sa, sb], [[a[131 + i]], [b[70 + i]]], "last")
        rows_a.append(out[0:1]); rows_b.append(out[1:2])
    r.engine.free_slot(sb)
    for t in a[136:]:
        rows_a.append(r.engine.step([sa], [[t]], "last"))
    r.engine.free_slot(sa)
    close(torch.cat(rows_a), plain_logits(d, a), dtype, cfg, f"random configuration {seed}: {json.dumps(cfg)}")
    close(torch.cat(rows_b), plain_logits(d, b)[70:75], dtype, cfg, f"random configuration {seed}, second request")
    r.cache.check()


@pytest.mark.parametrize("M,N,K", [(1, 256, 176), (8, 520, 2048), (64, 1024, 512), (200, 384, 136), (1000, 2048, 256), (3000, 520, 1024)])
def test_gelu_in_the_epilogue_of_the_tensor_core_product(M, N, K):
    """Few tokens (weights streamed, the product split over K), many (the persistent kernel), ragged edges."""
    from rustyllm_b200 import kernels as K_
    torch.manual_seed(M + N)
    a = torch.randn(M, K, dtype=F64).to(torch.bfloat16)
    w = (torch.randn(N, K, dtype=F64) / math.sqrt(K) * 2.0).to(torch.bfloat16)
    ad, wd = a.to(DEV), w.to(DEV)
    if not K_.gemm_tc_supported(ad, wd, None):
        pytest.skip("the tensor-core product does not take this shape")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    K_.gemm_tc(ad, wd, out, K_.OUT_GELU)
    K_.check_device_errors()
    ref = P.gelu_tanh(a.double() @ w.double().T)
    torch.testing.assert_close(out.double().cpu(), ref, rtol=1e-2, atol=1e-2)


# =========================================================================== generation, replay, command line
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_runner(dirs, name, dtype):
    """Prompts of unequal lengths through ``Runner.generate`` (its batches, prompt step, captured decode steps, sampler
    at temperature 0) against the plain greedy loop.  In bfloat16 a step whose two best logits lie within rounding of
    one another may pick the other token; the comparison ends there (and must not end at once)."""
    from rustyllm_b200 import GenerationOptions, SamplerConfig
    d = dirs[name]
    cfg, w = _plain(d)
    r = runner(d, dtype, 64 * 12, 3)
    prompts = [random_tokens(cfg["vocab"], n, 600 + n) for n in (1, 40, 9, 75, 12)]
    new = 12
    results = r.generate(prompts, GenerationOptions(max_tokens=new, sampler=SamplerConfig.greedy(), seed=1, ignore_eos=True))
    for p, res in zip(prompts, results):
        got = list(res.token_ids)
        assert len(got) == new
        if dtype == "float32":
            assert got == P.greedy(cfg, w, p, new)
        else:
            toks = list(p)
            for i, t in enumerate(got):
                row = P.forward(cfg, w, toks)[-1]
                best = int(row.argmax())
                if t != best:
                    assert float(row[best] - row[t]) <= 0.05 * float(row.std()), (name, i)
                    break
                toks.append(t)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_of_unequal_requests(dirs, tmp_path, dtype):
    """``bin/trace_run`` as a subprocess: requests of 3 to 150 tokens in one batch, decoded together, the shorter ones
    ending earlier, then a new request alone in the slots and pages that came back."""
    from test_trace_gpu import read_step, run_trace
    d = dirs["P"]
    cfg, _ = _plain(d)
    V = cfg["vocab"]
    lens = [3, 150, 7, 66, 5]
    extra = [0, 6, 2, 9, 1]
    reqs = [random_tokens(V, n + e, 900 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    steps = [{"step": 0, "entries": [{"id": f"q{i}", "tokens": r[:n], "want": [0, n - 1]} for i, (r, n) in enumerate(zip(reqs, lens))],
              "end": [f"q{i}" for i, e in enumerate(extra) if e == 0]}]
    expect = {0: [(i, [0, n - 1]) for i, n in enumerate(lens)]}
    for k in range(max(extra)):
        live = [i for i, e in enumerate(extra) if e > k]
        steps.append({"step": k + 1, "entries": [{"id": f"q{i}", "tokens": [reqs[i][lens[i] + k]], "want": [0]} for i in live],
                      "end": [f"q{i}" for i in live if extra[i] == k + 1]})
        expect[k + 1] = [(i, [lens[i] + k]) for i in live]
    late = random_tokens(V, 80, 950)
    reqs.append(late)
    steps.append({"step": 20, "entries": [{"id": "late", "tokens": late[:78], "want": [77]}], "end": []})
    steps.append({"step": 21, "entries": [{"id": "late", "tokens": late[78:79], "want": []}], "end": []})
    steps.append({"step": 22, "entries": [{"id": "late", "tokens": late[79:], "want": [0]}], "end": ["late"]})
    expect[20], expect[22] = [(5, [77])], [(5, [79])]
    out_dir = str(tmp_path / dtype)
    run_trace(d, dtype, steps, out_dir, max_tokens=sum(len(r) for r in reqs[:5]))
    assert not os.path.exists(os.path.join(out_dir, "21.f32"))
    for step, exp in expect.items():
        got = read_step(out_dir, step, V)
        ref = torch.cat([plain_logits(d, reqs[i])[pos] for i, pos in exp])
        close(got, ref, dtype, cfg, f"step {step}")


def test_command_line_generates_benchmarks_and_times_kernels(dirs, capsys):
    """``bin/rustyllm``'s entry point on a Forilorn folder: greedy ids equal the plain loop's; the benchmark and the kernel
    benchmark run, the latter on a layer of each kind of mixer."""
    from rustyllm_b200 import cli
    d = dirs["Q"]
    cfg, w = _plain(d)
    prompt = random_tokens(cfg["vocab"], 9, 81)
    assert cli.main([d, "--dtype", "float32", "-p", " ".join(map(str, prompt)), "-n", "5", "-t", "0", "--ignore-eos"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == P.greedy(cfg, w, prompt, 5)
    assert cli.main([d, "--bench-json", "--bench-runs", "2", "--batch", "3", "--prompt-len", "20", "-n", "4", "--seed", "5", "--ignore-eos"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["architecture"] == "Forilorn" and rep["results"][0]["prompt_tokens"] == 60 and rep["results"][0]["generated_tokens"] == 12
    for layer, names in ((0, ("attn_qkv.fused", "attn_output", "ffn_up_gelu_down", "attn_scan.ctx128", "output")),
                         (1, ("mixer_in.fused", "mixer_output", "ffn_up_gelu_down"))):
        assert cli.main([d, "--random", "--kernel-bench-json", "--kernel-bench-runs", "3", "--kernel-bench-layer", str(layer)]) == 0
        rows = {r["name"]: r for r in json.loads(capsys.readouterr().out)["rows"]}
        for n in names:
            assert rows[n]["avg_us"] > 0, n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,H,N,K,x_head,out_head", [(1, 3, 32, 24, 32, 40), (17, 16, 512, 128, 192, 576), (64, 4, 48, 96, 96, 48), (33, 1, 7, 5, 5, 9)])
def test_a_product_a_head_in_one_launch(dtype, M, H, N, K, x_head, out_head):
    from rustyllm_b200 import kernels as K_
    torch.manual_seed(M + N)
    x = rounded(torch.randn(M, (H - 1) * x_head + K + 3, dtype=F64), dtype)
    w = rounded(torch.randn(H, N, K, dtype=F64) / math.sqrt(K), dtype)
    out = torch.full((M, (H - 1) * out_head + N + 2), 7.0, dtype=tdt(dtype), device=DEV)
    K_.heads_linear(x.to(tdt(dtype)).to(DEV), x_head, w.to(tdt(dtype)).to(DEV), out, out_head)
    K_.check_device_errors()
    got = out.double().cpu()
    for a in range(H):
        ref = x[:, a * x_head:a * x_head + K] @ w[a].T
        torch.testing.assert_close(got[:, a * out_head:a * out_head + N], ref, **tol(dtype))
    assert (got[:, (H - 1) * out_head + N:] == 7.0).all()


@pytest.mark.parametrize("H,r,rd", [(16, 64, 32), (4, 96, 16), (3, 32, 16), (32, 64, 32), (40, 32, 16)])
@pytest.mark.parametrize("window", [None, 130])
def test_heads_over_one_cached_row_with_unequal_sequences_in_one_step(H, r, rd, window):
    """Five sequences of unequal lengths as one prompt step (blocks of two tiles that end inside a sequence), then four
    single-token steps of all of them (a sequence's keys in several runs, some of them empty), each against the
    sequence alone in the plain implementation."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache
    from rustyllm_b200.engine.step import StepState
    dtype, extra = "bfloat16", 4
    lens = [200, 37, 1, 129, 64]
    torch.manual_seed(H + r)
    scale = 2.0 / math.sqrt(r + rd)
    ql = [rounded(torch.randn(n + extra, H * (r + rd), dtype=F64), dtype) for n in lens]
    rows = [rounded(torch.randn(n + extra, r + rd, dtype=F64), dtype) for n in lens]
    gate = [rounded(2.0 * torch.randn(n + extra, H, dtype=F64), dtype) for n in lens]
    cache = SequenceCache([KVNeed(1, r + rd, window, 0)], [None], 64 * 12, tdt(dtype), DEV, max_slots=6)
    cache.alloc_slot()
    slots = [cache.alloc_slot() for _ in lens]
    group, layer = cache.kv_entry(0)
    got = [[] for _ in lens]
    at = [0] * len(lens)
    for cnts in [lens] + [[1] * len(lens)] * extra:
        cache.prepare(slots, cnts)
        pool = group.k_pool(layer)
        for b, (s, a, c) in enumerate(zip(slots, at, cnts)):
            pages = group.page_table[s].tolist()
            for p in range(a, a + c):
                pool[pages[p // 64], 0, p % 64] = rows[b][p].to(tdt(dtype)).to(DEV)
        M = sum(cnts)
        kv = [a + c for a, c in zip(at, cnts)]
        cu = [0]
        for c in cnts:
            cu.append(cu[-1] + c)
        st = StepState(M, len(lens), i32([0] * M), i32([p for a, c in zip(at, cnts) for p in range(a, a + c)]),
                       i32([s for s, c in zip(slots, cnts) for _ in range(c)]), i32(cu), i32(slots), i32(kv), i32([]), list(cnts), kv,
                       max(cnts), max(kv), all(c == 1 for c in cnts))
        q = torch.cat([ql[b][a:a + c] for b, (a, c) in enumerate(zip(at, cnts))]).to(tdt(dtype)).to(DEV).contiguous()
        gt = torch.cat([gate[b][a:a + c] for b, (a, c) in enumerate(zip(at, cnts))]).to(tdt(dtype)).to(DEV).contiguous()
        out = torch.empty((M, H * r), dtype=tdt(dtype), device=DEV)
        K.attention(q, pool, pool, group.page_table, st, out, H, 1, r + rd, scale, window or 0, value_dim=r, gate=gt,
                    gate_per_head=True, values_in_keys=True)
        o = out.double().cpu()
        for b, c in enumerate(cnts):
            got[b].append(o[cu[b]:cu[b] + c])
        cache.commit(slots, cnts)
        at = kv
    K.check_device_errors()
    for b in range(len(lens)):
        ref = plain_latent_scan(H, r, rd, window, scale, ql[b], rows[b], gate[b])
        torch.testing.assert_close(torch.cat(got[b]), ref, rtol=2e-2, atol=2e-2)
