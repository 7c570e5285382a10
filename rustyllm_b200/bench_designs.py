"""Prompt and single-token throughput of the Mosurax, Mogutar and Forilorn designs beside the Llama decoder at equal layer sizes
(random bfloat16 weights, synthetic tokens): ``python bench.py --designs`` or
``python -m rustyllm_b200.bench_designs [--size NAME] [--steps K] [--warmup W]``.

For every size three models of the same width, heads, head size, feed-forward width (the experts that a token
uses together with the shared one are as wide as the dense feed-forward), vocabulary and depth:
  llama          grouped-query attention with rotary encoding, dense SwiGLU feed-forward
  mosurax-dense  learned positions, attention with a sink term and an output gate (one more projection of
                 heads x head size rows), dense feed-forward, soft-capped logits
  mosurax-moe    the same with every second layer's feed-forward a mixture of experts with a shared expert
  mogutar        post-norm layers, two in four with attention (convolved, normed, rotated q and k; soft-capped scores; a
                 window of 1,024 with 8 kept tokens) beside a selective state-space mixer of the model's width, two in
                 four with linear attention with decay; every feed-forward 16 experts in 4 groups (2 kept), 4 a token,
                 each a quarter of the dense width; a per-layer token input of 256 columns
  forilorn       post-norm layers with a scaled stream; three in four with grouped-query attention whose values are its
                 keys (no value projection), rotated neighbours, unit-size q and k heads, blocks of 2,048 positions as the
                 mask and an output gate an element; one in four with attention through latents (queries 3/8 of the
                 width, at most 1,536; keys and values 1/4 of it, at most 512, plus a rotary key part of 64 for all heads, a window of 1,024, a gate
                 a head); dense gelu feed-forwards; a hashed pair table of 65,536 rows beside the embedding; tied head
  besuzen        layers x += mixer(ln1(x)) + ff(ln2(x)) with layer norms; every second layer attention without rotation
                 (a gate a head) beside a time mixer over the token and its predecessor with a matrix state a head and a
                 decay a key channel (heads of 64, the model's width); the others rotated attention with an output gate an
                 element whose values are blended with the first such layer's; feed-forwards in turn dense (gelu on the gate)
                 and 16 experts in 4 groups (2 kept), 3 a token, softmax scores over all, with a gated shared expert
``--besuzen-kernels`` times the Besuzen design's kernels alone, each beside the like kernel of the closest designs.
``--kernels`` times the Mogutar design's own kernels alone at the sizes of a layer (a JSON line a kernel, with the
bytes it must move and their share of the measured copy bandwidth).
Measured with CUDA events after warm-up: one prompt of ``prompt`` tokens as one step; then single-token steps of
``batch`` sequences that hold ``context`` tokens each (the captured step, as generation runs it).  One JSON line
a model and a summary line a size.  Weights of a size exceed the L2 cache; the prompt's activations do too.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List

SIZES = {
    # width 2,048: 16 heads over 4 KV heads of 128, feed-forward 8,192, 8 layers
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, layers=8, vocab=32768,
                  experts=16, top=3, expert_ff=2048, shared_ff=2048),
    # width 4,096: the layer of an 8B model (32 heads over 8 KV heads of 128, feed-forward 14,336), 4 layers
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, layers=4, vocab=32768,
                  experts=16, top=3, expert_ff=3584, shared_ff=3584),
}
MAX_POSITIONS = 4096
MODELS = ("llama", "mosurax-dense", "mosurax-moe", "mogutar", "forilorn", "besuzen")


def llama_config(s: dict) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": s["vocab"], "hidden_size": s["width"],
            "intermediate_size": s["ff"], "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"], "max_position_embeddings": MAX_POSITIONS,
            "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False}


def mosurax_config(s: dict, experts: bool, window=None) -> dict:
    mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5}
    if window:
        mixer["mask"] = {"size": window}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]},
           "shared": {"ff": s["shared_ff"]}}
    layers = [{"type": "attention", "mixer": dict(mixer), "mlp": moe if (experts and i % 2) else dense} for i in range(s["layers"])]
    return {"architecture": "Mosurax", "vocab": s["vocab"], "width": s["width"], "max_positions": MAX_POSITIONS,
            "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": layers}


def mogutar_config(s: dict, window: int = 1024) -> dict:
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5, "conv": 4,
            "softcap": 30.0, "mask": {"size": window, "keep_first": 8},
            "rot": {"base": 1.0e6, "dims": s["dim"] // 2, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}
    right = {"heads": s["width"] // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}
    mlp = {"kind": "moe", "router": {"experts": s["experts"], "top": 4, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": s["expert_ff"]}}
    layers = []
    for i in range(s["layers"]):
        if i % 4 < 2:
            layers.append({"type": "parallel", "mixer": {"left": dict(left), "right": dict(right), "left_scale": 1.0, "right_scale": 1.0},
                           "mlp": dict(mlp)})
        else:
            layers.append({"type": "lightning", "mixer": {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"],
                                                           "decay": [1.0 - 2.0 ** -(5 + 4 * h / s["heads"]) for h in range(s["heads"])]},
                           "mlp": dict(mlp)})
    return {"architecture": "Mogutar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "token_side": {"dim": 256},
            "layers": layers}


def forilorn_config(s: dict, window: int = 1024) -> dict:
    d, H, hd = s["width"], s["heads"], s["dim"]
    # blocks of twice the window: the 2,048-token prompt and the single tokens behind 1,024 see what the other models' see
    plain = {"heads": H, "kv_heads": s["kv_heads"], "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": 2 * window},
             "rot": {"base": 10000.0, "dims": hd}}
    lat = {"heads": H, "dim": hd, "rot_dim": 64, "vdim": hd, "q_rank": min(1536, 3 * d // 8), "kv_rank": min(512, d // 4), "scale": (hd + 64) ** -0.5,
           "mask": {"size": window}, "rot": {"base": 10000.0, "dims": 64}}
    layers = [{"type": "latent_attention" if i % 4 == 2 else "attention", "mixer": dict(lat if i % 4 == 2 else plain),
               "mlp": {"kind": "dense", "ff": s["ff"]}} for i in range(s["layers"])]
    return {"architecture": "Forilorn", "vocab": s["vocab"], "width": d, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": d ** 0.5, "bigram": {"buckets": 65536, "mul_prev": 1000003, "mul_cur": 999983}}, "layers": layers}


def besuzen_config(s: dict) -> dict:
    d, H, G, hd = s["width"], s["heads"], s["kv_heads"], s["dim"]
    att = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5}
    rotated = dict(att, rot={"base": 1.0e6, "dims": hd}, v_mix=True)
    right = {"heads": d // 64, "dim": 64, "decay_rank": 64}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]}}
    layers = []
    for i in range(s["layers"]):
        mlp = moe if i % 2 else dense
        if i % 2 == 0:
            layers.append({"type": "parallel", "mlp": mlp,
                           "mixer": {"left": dict(att), "right": dict(right), "left_scale": 0.7, "right_scale": 0.4}})
        else:
            layers.append({"type": "attention", "mixer": dict(rotated), "mlp": mlp})
    return {"architecture": "Besuzen", "vocab": s["vocab"], "width": d, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
            "logit_scale": 0.5, "layers": layers}


def measure(config: dict, prompt: int, batches: List[int], context: int, steps: int, warmup: int) -> Dict[str, float]:
    import numpy as np
    import torch
    from . import Runner
    max_b = max(batches)
    runner = Runner.from_config(config, seed=0, dtype="bfloat16", device="cuda:0",
                                max_cache_tokens=max(max_b * (context + 64 + steps + warmup), prompt + 64), max_batch=max_b,
                                max_context=MAX_POSITIONS)
    eng = runner.engine
    rng = np.random.default_rng(0)
    V = runner.model.spec.vocab_size
    out: Dict[str, float] = {"parameter_gb": round(runner.model.parameter_bytes() / 1e9, 3)}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # ---- one prompt as one step ----
    times = []
    for i in range(3 + 3):
        s = eng.alloc_slot()
        toks = rng.integers(0, V, size=prompt).tolist()
        e0.record()
        eng.step([s], [toks], "last")
        e1.record()
        torch.cuda.synchronize()
        eng.free_slot(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    out["prefill_ms"] = round(min(times), 3)
    out["prefill_tok_s"] = round(prompt * 1000.0 / min(times), 1)
    # ---- single-token steps ----
    for B in batches:
        slots = [eng.alloc_slot() for _ in range(B)]
        for s in slots:
            eng.step([s], [rng.integers(0, V, size=context).tolist()], None)
        toks = [[int(t)] for t in rng.integers(0, V, size=B)]
        for _ in range(max(warmup, 3)):
            eng.step(slots, toks, "last")
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            eng.step(slots, toks, "last")
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[f"decode_b{B}_ms"] = round(ms, 4)
        out[f"decode_b{B}_tok_s"] = round(B * 1000.0 / ms, 1)
        for s in slots:
            eng.free_slot(s)
    from . import kernels
    kernels.check_device_errors()
    del runner, eng
    torch.cuda.empty_cache()
    return out


def run(sizes: List[str], prompt: int = 2048, batches=(8, 64), context: int = 1024, steps: int = 32, warmup: int = 8,
        window: int = 0, models=None) -> List[dict]:
    lines = []
    models = tuple(models or MODELS)
    for name in sizes:
        s = SIZES[name]
        got = {}
        for model in models:
            cfg = llama_config(s) if model == "llama" else besuzen_config(s) if model == "besuzen" else mogutar_config(s, window or 1024) if model == "mogutar" \
                else forilorn_config(s, window or 1024) if model == "forilorn" else mosurax_config(s, model == "mosurax-moe", window or None)
            got[model] = measure(cfg, prompt, list(batches), context, steps, warmup)
            line = {"size": name, "model": model, "prompt_tokens": prompt, "context": context, "window": window or None,
                    "dtype": "bf16", "data": "synthetic", **got[model]}
            print(json.dumps(line), flush=True)
            lines.append(line)
        if "llama" in got:
            for model in models:
                if model == "llama":
                    continue
                ratio = {k: round(got[model][k] / got["llama"][k], 3) for k in got[model] if k.endswith("tok_s")}
                line = {"size": name, "model": model, "throughput_over_llama": ratio}
                print(json.dumps(line), flush=True)
                lines.append(line)
    return lines


def kernel_times(sizes: List[str], prompt: int = 2048, batch: int = 64, runs: int = 20) -> List[dict]:
    """The recurrent and fused kernels of the Mogutar design alone, bfloat16, at a layer's sizes: ``prompt`` tokens of
    one sequence, and one token of each of ``batch`` sequences.  Bytes: what the kernel must read and write once."""
    import json as _json
    import os
    import torch
    from . import kernels as K
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = _json.load(f)
    except OSError:
        pass
    gbs = float(peaks.get("hbm_gbs", 6650.0))
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(runs):
            flush.zero_()                      # a buffer larger than L2 between runs
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2] * 1e3   # us

    lines = []

    def report(size, kernel, shape, us, nbytes):
        line = {"size": size, "kernel": kernel, "shape": shape, "us": round(us, 2), "gb": round(nbytes / 1e9, 4),
                "tb_s": round(nbytes / us / 1e6, 3), "of_copy_bandwidth": round(nbytes / us / 1e3 / gbs, 3)}
        print(_json.dumps(line), flush=True)
        lines.append(line)

    for name in sizes:
        s = SIZES[name]
        d, H, hd = s["width"], s["heads"], s["dim"]
        for what, M, B in (("prompt", prompt, 1), ("single tokens", batch, batch)):
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
            per = M // B
            cu, slots = i32([per * b for b in range(B + 1)]), i32(list(range(B)))
            slot_of_token = i32([b for b in range(B) for _ in range(per)])
            # linear attention with decay: heads of (hd, hd)
            state = torch.zeros((B, 4 * H * hd * hd), dtype=torch.uint8, device=dev)
            qkv = torch.randn((M, 3 * H * hd), dtype=torch.float32, device=dev).to(bf)
            o = torch.empty((M, H * hd), dtype=torch.float32, device=dev)
            decay = torch.full((H,), 0.99, dtype=torch.float32, device=dev)
            us = timed(lambda: K.linear_scan(qkv[:, :H * hd], qkv[:, H * hd:2 * H * hd], qkv[:, 2 * H * hd:], o, state, cu, slots, H, 1, hd, hd,
                                             decay, silu=True))
            report(name, "linear_scan (decay)", f"{what}: {M} tokens, {B} seq, {H} heads of {hd} x {hd}", us,
                   qkv.numel() * 2 + o.numel() * 4 + 2 * state.numel())
            # selective state space: width / 64 heads of (128, 64), 8 groups
            Hs, P, N, G = d // 64, 64, 128, 8
            state = torch.zeros((B, 4 * Hs * N * P), dtype=torch.uint8, device=dev)
            xbc = torch.randn((M, Hs * P + 2 * G * N), dtype=torch.float32, device=dev).to(bf)
            dt = torch.randn((M, Hs), dtype=torch.float32, device=dev).to(bf)
            y = torch.empty((M, Hs * P), dtype=torch.float32, device=dev)
            z32 = torch.zeros(Hs, dtype=torch.float32, device=dev)
            us = timed(lambda: K.linear_scan(xbc[:, Hs * P + G * N:], xbc[:, Hs * P:Hs * P + G * N], xbc[:, :Hs * P], y, state, cu, slots, Hs,
                                             Hs // G, N, P, z32, dt_raw=dt, dt_bias=z32, skip=z32))
            report(name, "linear_scan (selective)", f"{what}: {M} tokens, {B} seq, {Hs} heads of {N} x {P}", us,
                   xbc.numel() * 2 + dt.numel() * 2 + y.numel() * 4 + 2 * state.numel())
            # the convolution of x, B, C with its state
            C = Hs * P + 2 * G * N
            cstate = torch.zeros((B, 4 * 3 * C), dtype=torch.uint8, device=dev)
            w = torch.randn((C, 4), dtype=torch.float32, device=dev)
            out = torch.empty((M, C), dtype=bf, device=dev)
            us = timed(lambda: (K.short_conv(xbc, w, None, True, slot_of_token, cstate, out), K.short_conv_state(xbc, 4, cu, slots, cstate)))
            report(name, "short_conv + state", f"{what}: {M} tokens, {C} channels, 4 taps", us, 2 * xbc.numel() * 2 + 2 * cstate.numel())
            # the attention's preparation: convolution, head norms, rotation, cache write (keys and values to pages)
            G = s["kv_heads"]
            Cq = (H + 2 * G) * hd
            pstate = torch.zeros((B, 4 * 3 * Cq), dtype=torch.uint8, device=dev)
            u = torch.randn((M, Cq), dtype=torch.float32, device=dev).to(bf)
            qo = torch.empty((M, H * hd), dtype=bf, device=dev)
            pages = -(-per // K.PAGE_SIZE)
            k_pool = torch.zeros((B * pages, G, K.PAGE_SIZE, hd), dtype=bf, device=dev)
            v_pool = torch.zeros_like(k_pool)
            table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages)
            positions = i32([t for b in range(B) for t in range(per)])
            wq = torch.randn((Cq, 4), dtype=torch.float32, device=dev)
            nw = torch.ones(hd, dtype=torch.float32, device=dev)
            inv = torch.rand(hd // 4, dtype=torch.float32, device=dev)
            us = timed(lambda: (K.qkv_prepare(u, qo, wq, pstate, nw, nw, 1e-5, positions, slot_of_token, table, inv, hd // 2, 1.1, H, G, hd, hd,
                                              k_pool, v_pool), K.short_conv_state(u, 4, cu, slots, pstate)))
            report(name, "qkv_prepare + state", f"{what}: {M} tokens, {H} + 2 x {G} heads of {hd}, 4 taps", us, 2 * u.numel() * 2 + 2 * pstate.numel())
            # gate, norm in groups
            yn = torch.empty((M, Hs * P), dtype=bf, device=dev)
            gate = torch.randn((M, Hs * P), dtype=torch.float32, device=dev).to(bf)
            wn = torch.ones(Hs * P, dtype=torch.float32, device=dev)
            us = timed(lambda: K.gated_norm(y, gate, wn, 1e-5, yn, groups=8))
            report(name, "gated_norm", f"{what}: {M} x {Hs * P}", us, y.numel() * 4 + 2 * gate.numel() * 2)
            # x += norm(y0 + y1) * w, with the bfloat16 copy
            x = torch.randn((M, d), dtype=torch.float32, device=dev)
            y0, y1 = torch.randn_like(x), torch.randn_like(x)
            xb = torch.empty((M, d), dtype=bf, device=dev)
            wd = torch.ones(d, dtype=torch.float32, device=dev)
            us = timed(lambda: K.norm_add(x, y0, 1.0, y1, 1.0, wd, 1e-5, xb))
            report(name, "norm_add (two terms)", f"{what}: {M} x {d}", us, 4 * x.numel() * 4 + xb.numel() * 2)
    K.check_device_errors()
    return lines


def forilorn_kernel_times(sizes: List[str], prompt: int = 2048, batch: int = 64, context: int = 1024, mask: int = 1024,
                          runs: int = 20) -> List[dict]:
    """The Forilorn design's kernels alone beside the like kernel of the Mosurax design, bfloat16, at a layer's sizes:
    ``prompt`` tokens of one sequence, and one token of each of ``batch`` sequences that hold ``context`` tokens with it.  A
    row gives the bytes the kernel must move and the operations it must do, the time both would take at the measured
    copy bandwidth and matrix throughput, and the larger of the two over the measured time (``of_roofline``)."""
    import json as _json
    import os
    import torch
    from . import kernels as K
    from .cache.sequence_cache import KVNeed, SequenceCache
    from .engine.step import StepState
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = _json.load(f)
    except OSError:
        pass
    gbs, tflops = float(peaks.get("hbm_gbs", 6650.0)), float(peaks.get("bf16_tflops", 1590.0))
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(runs):
            flush.zero_()                      # a buffer larger than L2 between runs
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2] * 1e3   # us

    lines = []

    def report(size, design, kernel, shape, us, nbytes, flops=0.0):
        floor = max(nbytes / (gbs * 1e3), flops / (tflops * 1e6))        # us
        line = {"size": size, "design": design, "kernel": kernel, "shape": shape, "us": round(us, 2), "gb": round(nbytes / 1e9, 4),
                "gflop": round(flops / 1e9, 3), "floor_us": round(floor, 2), "of_roofline": round(floor / us, 3),
                "bound": "bandwidth" if nbytes / (gbs * 1e3) >= flops / (tflops * 1e6) else "matrix"}
        print(_json.dumps(line), flush=True)
        lines.append(line)

    def steps_for(cache, B, held, cnt):
        """B sequences that hold ``held`` tokens and bring ``cnt`` more: the cache prepared, and the step's description."""
        slots = [cache.alloc_slot() for _ in range(B)]
        if held:
            cache.prepare(slots, [held] * B); cache.commit(slots, [held] * B)
        cache.prepare(slots, [cnt] * B)
        M = B * cnt
        return StepState(M, B, i32([0] * M), i32([held + t for _ in range(B) for t in range(cnt)]),
                         i32([s for s in slots for _ in range(cnt)]), i32([cnt * b for b in range(B + 1)]), i32(slots),
                         i32([held + cnt] * B), i32([]), [cnt] * B, [held + cnt] * B, cnt, held + cnt, cnt == 1)

    for name in sizes:
        s = SIZES[name]
        d, H, G, hd, ff = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
        r, rd, qr = min(512, d // 4), 64, min(1536, 3 * d // 8)
        scale = hd ** -0.5
        # the single token is the last of a block of the mask: it sees ``mask`` keys under either kind of mask
        for what, B, held, cnt in (("prompt", 1, 0, prompt), ("single tokens", batch, context - 1, 1)):
            M = B * cnt
            pages = 64 * (-(-(held + cnt) // 64) + 1) * B
            seen = lambda lo: sum(p - lo(p) + 1 for p in range(held, held + cnt)) * B      # (query, key) pairs
            pairs_chunk = seen(lambda p: p - p % mask)
            pairs_window = seen(lambda p: max(0, p + 1 - mask))
            # ---- attention over keys and values of their own: the chunked mask beside the sliding window ----
            for design, kw, pairs in (("forilorn", dict(chunk=mask), pairs_chunk), ("mosurax", dict(window=mask), pairs_window)):
                need = KVNeed(G, hd, kw.get("window"), None, 0, kw.get("chunk"))
                cache = SequenceCache([need], [None], pages, bf, dev, max_slots=B)
                st = steps_for(cache, B, held, cnt)
                group, layer = cache.kv_entry(0)
                group.k_pool(layer).normal_(); group.v_pool(layer).normal_()
                u = torch.randn((M, (2 * H + 2 * G) * hd), dtype=torch.float32, device=dev).to(bf)
                o = torch.empty((M, H * hd), dtype=bf, device=dev)
                us = timed(lambda: K.attention(u, group.k_pool(layer), group.v_pool(layer), group.page_table, st, o, H, G, hd, scale,
                                               kw.get("window", 0), gate=u[:, (H + 2 * G) * hd:], chunk=kw.get("chunk", 0)))
                keys = (pairs // cnt if cnt == 1 else min(held + cnt, 10 ** 9) * B)         # key rows read at least once
                if cnt > 1 and "window" not in kw:
                    keys = (held + cnt) * B
                report(name, design, "attention, gated, " + ("chunked mask" if "chunk" in kw else "window"),
                       f"{what}: {M} tokens, {B} seq of {held + cnt}, {H} heads over {G} of {hd}, mask {mask}", us,
                       keys * G * 2 * hd * 2 + 3 * M * H * hd * 2, 4.0 * pairs * H * hd)
                del cache
            # ---- all heads over one cached row whose front is the value (the latent layer), a sliding window ----
            cache = SequenceCache([KVNeed(1, r + rd, mask, 0)], [None], pages, bf, dev, max_slots=B)
            st = steps_for(cache, B, held, cnt)
            group, layer = cache.kv_entry(0)
            group.k_pool(layer).normal_()
            ql = torch.randn((M, H * (r + rd)), dtype=torch.float32, device=dev).to(bf)
            gate = torch.randn((M, H), dtype=torch.float32, device=dev).to(bf)
            o = torch.empty((M, H * r), dtype=bf, device=dev)
            us = timed(lambda: K.attention(ql, group.k_pool(layer), group.k_pool(layer), group.page_table, st, o, H, 1, r + rd, scale, mask,
                                           value_dim=r, gate=gate, gate_per_head=True, values_in_keys=True))
            keys = pairs_window // cnt if cnt == 1 else (held + cnt) * B
            report(name, "forilorn", "attention over one latent row, gate a head, window",
                   f"{what}: {M} tokens, {B} seq of {held + cnt}, {H} heads over rows of {r} + {rd}, window {mask}", us,
                   keys * (r + rd) * 2 + M * H * (2 * r + rd) * 2, 2.0 * pairs_window * H * (2 * r + rd))
            del cache
            # ---- what stands between the input product and the attention ----
            cache = SequenceCache([KVNeed(G, hd, None, None, 0, mask), KVNeed(1, r + rd, mask, 0)], [None, None], 2 * pages, bf, dev, max_slots=B)
            st = steps_for(cache, B, held, cnt)
            (g0, l0), (g1, l1) = cache.kv_entry(0), cache.kv_entry(1)
            inv = torch.rand(hd // 2, dtype=torch.float32, device=dev)
            u = torch.randn((M, (2 * H + G) * hd), dtype=torch.float32, device=dev).to(bf)
            us = timed(lambda: K.qk_rotate_unit(u, u, st.positions, st.slot_of_token, g0.page_table, inv, hd, True, 1e-6, H, G, hd,
                                                g0.k_pool(l0), g0.v_pool(l0), value_from_key=True))
            report(name, "forilorn", "rotation of pairs, unit heads, keys and values to pages", f"{what}: {M} tokens, {H} + {G} heads of {hd}", us,
                   M * (2 * H + 3 * G) * hd * 2)
            u3 = torch.randn((M, (H + 2 * G) * hd), dtype=torch.float32, device=dev).to(bf)
            us = timed(lambda: K.rope_kv_write(u3, st.positions, st.slot_of_token, g0.page_table, inv, H, G, hd, hd, False,
                                               g0.k_pool(l0), g0.v_pool(l0), value_dim=hd))
            report(name, "mosurax", "rotation, keys and values to pages", f"{what}: {M} tokens, {H} + 2 x {G} heads of {hd}", us,
                   M * (2 * H + 4 * G) * hd * 2)
            ul = torch.randn((M, qr + r + rd + H), dtype=torch.float32, device=dev).to(bf)
            cq = torch.empty((M, qr), dtype=bf, device=dev)
            ones_q, ones_k = torch.ones(qr, dtype=torch.float32, device=dev), torch.ones(r, dtype=torch.float32, device=dev)
            us = timed(lambda: K.latent_prepare(ul, qr, r, rd, ones_q, ones_k, 1e-6, cq, st.positions, st.slot_of_token, g1.page_table,
                                                inv, rd, True, g1.k_pool(l1)))
            report(name, "forilorn", "latents normed, rotary key turned, row to its page", f"{what}: {M} tokens, latents {qr} and {r} + {rd}", us,
                   M * (2 * qr + 2 * (r + rd)) * 2)
            qh = torch.randn((M, H * (hd + rd)), dtype=torch.float32, device=dev).to(bf)
            qlat = torch.empty((M, H * (r + rd)), dtype=bf, device=dev)
            us = timed(lambda: K.latent_query(qh, qlat, H, hd, rd, r, st.positions, inv, rd, True))
            report(name, "forilorn", "query's rotary parts turned into place", f"{what}: {M} tokens, {H} heads of {hd} + {rd}", us, 2 * M * H * rd * 2)
            del cache
            # ---- the embedding with its pair table beside the plain one ----
            V = s["vocab"]
            table = torch.randn((V, d), dtype=torch.float32, device=dev).to(bf)
            pair = torch.randn((65537, d), dtype=torch.float32, device=dev).to(bf)
            ids = torch.randint(0, V, (M,), dtype=torch.int32, device=dev)
            x = torch.empty((M, d), dtype=torch.float32, device=dev)
            area = torch.zeros((B, 256), dtype=torch.uint8, device=dev)
            err = torch.zeros(1, dtype=torch.int32, device=dev)
            slots_tok, pos = i32([b for b in range(B) for _ in range(cnt)]), i32([held + t for _ in range(B) for t in range(cnt)])
            cu = i32([cnt * b for b in range(B + 1)])
            us = timed(lambda: K.embedding_pair(table, pair, ids, pos, slots_tok, cu, area[:, :4], 3.0, 31, 17, 65536, x, err))
            report(name, "forilorn", "scaled embedding + hashed pair row", f"{what}: {M} tokens of {d}", us, M * d * (2 + 2 + 4))
            us = timed(lambda: K.embedding(table, ids, x, err))
            report(name, "mosurax", "embedding", f"{what}: {M} tokens of {d}", us, M * d * (2 + 4))
            # ---- the feed-forward's first product with its activation in the epilogue ----
            xn = torch.randn((M, d), dtype=torch.float32, device=dev).to(bf)
            w1 = (torch.randn((ff, d), dtype=torch.float32, device=dev) * d ** -0.5).to(bf)
            w2 = (torch.randn((2 * ff, d), dtype=torch.float32, device=dev) * d ** -0.5).to(bf)
            h = torch.empty((M, ff), dtype=bf, device=dev)
            us = timed(lambda: K.gemm_tc(xn, w1, h, K.OUT_GELU))
            report(name, "forilorn", "up product, gelu in the epilogue", f"{what}: {M} x {d} -> {ff}", us, (w1.numel() + xn.numel() + h.numel()) * 2,
                   2.0 * M * d * ff)
            us = timed(lambda: K.gemm_tc(xn, w2, h, K.OUT_SWIGLU))
            report(name, "mosurax", "gate and up product, silu * up in the epilogue", f"{what}: {M} x {d} -> 2 x {ff}", us,
                   (w2.numel() + xn.numel() + h.numel()) * 2, 4.0 * M * d * ff)
            # ---- a sublayer's normed output, scaled, into the stream ----
            xs, y0 = torch.randn((M, d), dtype=torch.float32, device=dev), torch.randn((M, d), dtype=torch.float32, device=dev)
            xb = torch.empty((M, d), dtype=bf, device=dev)
            wd = torch.ones(d, dtype=torch.float32, device=dev)
            us = timed(lambda: K.norm_add(xs, y0, 1.0, None, 0.0, wd, 1e-6, xb, out_scale=0.5))
            report(name, "forilorn", "stream += m * norm(sublayer)", f"{what}: {M} x {d}", us, 3 * xs.numel() * 4 + xb.numel() * 2)
    K.check_device_errors()
    return lines


def besuzen_kernel_times(sizes: List[str], prompt: int = 2048, batch: int = 64, context: int = 1024, runs: int = 20) -> List[dict]:
    """The Besuzen design's kernels alone, each beside the like kernel of the closest designs (Mosurax: gated attention,
    rotation and cache write, RMS norm, gated product; Mogutar: recurrence, a pass over rows with per-sequence state, router
    with groups), bfloat16, at a layer's sizes: ``prompt`` tokens of one sequence, and one token of each of ``batch``
    sequences that hold ``context`` tokens with it.  A row gives the bytes the kernel must move and the operations it
    must do, the time both would take at the measured copy bandwidth and matrix throughput, and the larger of the two
    over the measured time (``of_roofline``)."""
    import json as _json
    import os
    import torch
    from . import kernels as K
    from .cache.sequence_cache import KVNeed, SequenceCache
    from .engine.step import StepState
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = _json.load(f)
    except OSError:
        pass
    gbs, tflops = float(peaks.get("hbm_gbs", 6650.0)), float(peaks.get("bf16_tflops", 1590.0))
    dev, bf = torch.device("cuda:0"), torch.bfloat16
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    rnd = lambda *shape: torch.randn(shape, dtype=torch.float32, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(runs):
            flush.zero_()                      # a buffer larger than L2 between runs
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2] * 1e3   # us

    lines = []

    def report(size, design, kernel, shape, us, nbytes, flops=0.0):
        floor = max(nbytes / (gbs * 1e3), flops / (tflops * 1e6))        # us
        line = {"size": size, "design": design, "kernel": kernel, "shape": shape, "us": round(us, 2), "gb": round(nbytes / 1e9, 4),
                "gflop": round(flops / 1e9, 3), "floor_us": round(floor, 2), "of_roofline": round(floor / us, 3),
                "bound": "bandwidth" if nbytes / (gbs * 1e3) >= flops / (tflops * 1e6) else "matrix"}
        print(_json.dumps(line), flush=True)
        lines.append(line)

    for name in sizes:
        s = SIZES[name]
        d, H, G, hd, ff = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
        scale = hd ** -0.5
        for what, B, held, cnt in (("prompt", 1, 0, prompt), ("single tokens", batch, context - 1, 1)):
            M = B * cnt
            shape = f"{what}: {M} tokens, {B} seq of {held + cnt}"
            pairs = sum(p + 1 for p in range(held, held + cnt)) * B
            cache = SequenceCache([KVNeed(G, hd)], [None], 64 * (-(-(held + cnt) // 64) + 1) * B, bf, dev, max_slots=B)
            slots = [cache.alloc_slot() for _ in range(B)]
            if held:
                cache.prepare(slots, [held] * B); cache.commit(slots, [held] * B)
            cache.prepare(slots, [cnt] * B)
            st = StepState(M, B, i32([0] * M), i32([held + t for _ in range(B) for t in range(cnt)]),
                           i32([sl for sl in slots for _ in range(cnt)]), i32([cnt * b for b in range(B + 1)]), i32(slots),
                           i32([held + cnt] * B), i32([]), [cnt] * B, [held + cnt] * B, cnt, held + cnt, cnt == 1)
            group, layer = cache.kv_entry(0)
            kp, vp = group.k_pool(layer), group.v_pool(layer)
            kp.normal_(); vp.normal_()
            # ---- attention: a gate a head beside a gate an element ----
            u = rnd(M, (2 * H + 2 * G) * hd).to(bf)
            o = torch.empty((M, H * hd), dtype=bf, device=dev)
            att_bytes = (held + cnt) * B * G * 2 * hd * 2 + 2 * M * H * hd * 2
            for design, kw, extra in (("besuzen", dict(gate=u[:, (H + 2 * G) * hd:(H + 2 * G) * hd + H], gate_per_head=True), M * H * 2),
                                      ("mosurax", dict(gate=u[:, (H + 2 * G) * hd:]), M * H * hd * 2)):
                us = timed(lambda: K.attention(u, kp, vp, group.page_table, st, o, H, G, hd, scale, **kw))
                report(name, design, "attention, " + ("gate a head" if "gate_per_head" in kw else "gate an element"),
                       f"{shape}, {H} heads over {G} of {hd}", us, att_bytes + extra, 4.0 * pairs * H * hd)
            # ---- rotation of neighbours, values blended, keys and values to pages; beside the half-split rotation ----
            inv = torch.rand(hd // 2, dtype=torch.float32, device=dev)
            u3 = rnd(M, (H + 2 * G) * hd).to(bf)
            other, lam = rnd(M, G * hd).to(bf), torch.tensor(0.4, dtype=torch.float32, device=dev)
            us = timed(lambda: K.rope_kv_write(u3, st.positions, st.slot_of_token, group.page_table, inv, H, G, hd, hd, True, kp, vp,
                                               value_dim=hd, v_other=other, v_mix=lam))
            report(name, "besuzen", "rotation of neighbours, values blended, keys and values to pages", f"{shape}, {H} + 2 x {G} heads of {hd}", us,
                   M * (2 * H + 5 * G) * hd * 2)
            us = timed(lambda: K.rope_kv_write(u3, st.positions, st.slot_of_token, group.page_table, inv, H, G, hd, hd, False, kp, vp, value_dim=hd))
            report(name, "mosurax", "rotation, keys and values to pages", f"{shape}, {H} + 2 x {G} heads of {hd}", us, M * (2 * H + 4 * G) * hd * 2)
            del cache
            # ---- the recurrence with a decay a key channel beside the one with a decay a head ----
            Hr, n = d // 64, 64
            state = torch.zeros((B, 4 * Hr * n * n), dtype=torch.uint8, device=dev)
            rkv = rnd(M, 3 * Hr * n).to(bf)
            wlog, bonus = rnd(M, Hr * n) - 3.0, rnd(Hr, n)
            o32 = torch.empty((M, Hr * n), dtype=torch.float32, device=dev)
            us = timed(lambda: K.channel_decay_scan(rkv[:, :Hr * n], rkv[:, Hr * n:2 * Hr * n], rkv[:, 2 * Hr * n:], wlog, bonus, o32, state,
                                                    st.cu_seqlens, st.seq_slots, Hr, n, n))
            report(name, "besuzen", "recurrence, decay a key channel, bonus", f"{shape}, {Hr} heads of {n} x {n}", us,
                   rkv.numel() * 2 + wlog.numel() * 4 + o32.numel() * 4 + 2 * state.numel(), 6.0 * M * Hr * n * n)
            decay = torch.full((Hr,), 0.99, dtype=torch.float32, device=dev)
            us = timed(lambda: K.linear_scan(rkv[:, :Hr * n], rkv[:, Hr * n:2 * Hr * n], rkv[:, 2 * Hr * n:], o32, state, st.cu_seqlens,
                                             st.seq_slots, Hr, 1, n, n, decay, silu=True))
            report(name, "mogutar", "recurrence, decay a head", f"{shape}, {Hr} heads of {n} x {n}", us,
                   rkv.numel() * 2 + o32.numel() * 4 + 2 * state.numel(), 4.0 * M * Hr * n * n)
            # ---- the blends with the previous token beside the short convolution (a pass over rows with per-sequence state) ----
            h = rnd(M, d).to(bf)
            mu = torch.rand(5, d, dtype=torch.float32, device=dev)
            sstate = torch.zeros((B, 4 * d), dtype=torch.uint8, device=dev)
            mixes = torch.empty((5, M, d), dtype=bf, device=dev)
            us = timed(lambda: K.token_shift_mix(h, mu, st.positions, st.slot_of_token, st.cu_seqlens, sstate, mixes))
            report(name, "besuzen", "five blends with the previous token + state", f"{shape}, width {d}", us, 6 * M * d * 2 + 2 * sstate.numel())
            cstate = torch.zeros((B, 4 * 3 * d), dtype=torch.uint8, device=dev)
            wconv = rnd(d, 4)
            cout = torch.empty((M, d), dtype=bf, device=dev)
            us = timed(lambda: (K.short_conv(h, wconv, None, True, st.slot_of_token, cstate, cout), K.short_conv_state(h, 4, st.cu_seqlens, st.seq_slots, cstate)))
            report(name, "mogutar", "short convolution + state", f"{shape}, {d} channels, 4 taps", us, 2 * M * d * 2 + 2 * cstate.numel())
            # ---- the head norm with the gate behind the recurrence (the kernel is Mogutar's) ----
            gate = rnd(M, Hr * n).to(bf)
            ones = torch.ones(Hr * n, dtype=torch.float32, device=dev)
            on = torch.empty((M, Hr * n), dtype=bf, device=dev)
            us = timed(lambda: K.gated_norm(o32, gate, ones, 1e-6, on, groups=Hr, gate_act="silu", gate_first=False))
            report(name, "besuzen", "unit heads, weight, silu gate", f"{shape}, {Hr} heads of {n}", us, M * Hr * n * (4 + 2 + 2))
            us = timed(lambda: K.gated_norm(o32, gate, ones, 1e-6, on, groups=8, gate_act="silu", gate_first=True))
            report(name, "mogutar", "gate, norm in 8 parts, weight", f"{shape}, width {Hr * n}", us, M * Hr * n * (4 + 2 + 2))
            # ---- both layer norms of a layer in one kernel beside two RMS norms ----
            x = rnd(M, d)
            w0, w1 = torch.ones(d, dtype=torch.float32, device=dev), torch.ones(d, dtype=torch.float32, device=dev)
            pair = torch.empty((2, M, d), dtype=bf, device=dev)
            us = timed(lambda: K.layer_norm(x, w0, pair[0], 1e-6, None, w1, pair[1]))
            report(name, "besuzen", "two layer norms of one stream", f"{shape}, width {d}", us, M * d * (4 + 2 + 2))
            us = timed(lambda: (K.rmsnorm(x, w0, pair[0], 1e-6), K.rmsnorm(x, w1, pair[1], 1e-6)))
            report(name, "mosurax", "two RMS norms", f"{shape}, width {d}", us, M * d * (4 + 4 + 2 + 2))
            # ---- the joins ----
            y0, y1 = rnd(M, d), rnd(M, d)
            us = timed(lambda: K.scaled_add(x, y0, 0.6, y1, 0.5))
            report(name, "besuzen", "stream += a * left + b * right", f"{shape}, width {d}", us, M * d * 16)
            xb = torch.empty((M, d), dtype=bf, device=dev)
            us = timed(lambda: K.norm_add(x, y0, 0.6, y1, 0.5, w0, 1e-6, xb))
            report(name, "mogutar", "stream += norm(a * left + b * right) w", f"{shape}, width {d}", us, M * d * 18)
            gvec = rnd(d).to(bf)
            us = timed(lambda: K.row_gate_add(x, y0, h, gvec))
            report(name, "besuzen", "stream += sigmoid(h . g) * shared", f"{shape}, width {d}", us, M * d * 14)
            # ---- routers ----
            E, top = s["experts"], s["top"]
            wr = (rnd(E, d) * d ** -0.5).to(bf)
            ids = torch.empty((M, top), dtype=torch.int32, device=dev)
            wts = torch.empty((M, top), dtype=torch.float32, device=dev)
            if M < 128:
                us = timed(lambda: K.moe_route_scored(h, wr, None, top, 4, 2, ids, wts, softmax_all=True, group_top=1, renorm=True))
                report(name, "besuzen", "router, softmax over all, groups by their best", f"{shape}, {E} experts", us, M * d * 2 + E * d * 2)
                us = timed(lambda: K.moe_route_sigmoid(h, wr, None, top, 4, 2, ids, wts))
                report(name, "mogutar", "router, sigmoid scores, groups by their two best", f"{shape}, {E} experts", us, M * d * 2 + E * d * 2)
            else:
                logits = rnd(M, E)
                us = timed(lambda: K.moe_select_scored(logits, None, top, 4, 2, ids, wts, softmax_all=True, group_top=1, renorm=True))
                report(name, "besuzen", "choice from logits, softmax over all", f"{shape}, {E} experts", us, M * E * 4 + M * top * 8)
                us = timed(lambda: K.moe_select_sigmoid(logits, None, top, 4, 2, ids, wts))
                report(name, "mogutar", "choice from logits, sigmoid scores", f"{shape}, {E} experts", us, M * E * 4 + M * top * 8)
            # ---- the feed-forward's first product with its activation in the epilogue ----
            w2 = (rnd(2 * ff, d) * d ** -0.5).to(bf)
            hh = torch.empty((M, ff), dtype=bf, device=dev)
            for design, mode in (("besuzen", K.OUT_GEGLU), ("mosurax", K.OUT_SWIGLU)):
                us = timed(lambda: K.gemm_tc(h, w2, hh, mode))
                report(name, design, "gate-up product, " + ("gelu" if mode == K.OUT_GEGLU else "silu") + " on the gate in the epilogue",
                       f"{shape}, {d} -> 2 x {ff}", us, w2.numel() * 2 + M * (d + ff) * 2, 4.0 * M * d * ff)
    K.check_device_errors()
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--size", action="append", choices=sorted(SIZES), help="default: all")
    ap.add_argument("--model", action="append", choices=list(MODELS), help="default: all")
    ap.add_argument("--kernels", action="store_true", help="time the Mogutar design's own kernels alone instead")
    ap.add_argument("--forilorn-kernels", action="store_true",
                    help="time the Forilorn design's kernels alone, each beside the like kernel of the Mosurax design, instead")
    ap.add_argument("--besuzen-kernels", action="store_true",
                    help="time the Besuzen design's kernels alone, each beside the like kernel of the Mosurax or Mogutar design, instead")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--batch", type=int, action="append", help="default: 8 and 64")
    ap.add_argument("--window", type=int, default=0, help="sliding window of the Mosurax layers (0: none, as Llama)")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    a = ap.parse_args(argv)
    if a.forilorn_kernels:
        forilorn_kernel_times(a.size or sorted(SIZES), a.prompt, max(a.batch or (64,)), a.context, a.window or 1024)
        return 0
    if a.besuzen_kernels:
        besuzen_kernel_times(a.size or sorted(SIZES), a.prompt, max(a.batch or (64,)), a.context)
        return 0
    if a.kernels:
        kernel_times(a.size or sorted(SIZES), a.prompt, max(a.batch or (64,)))
        return 0
    run(a.size or sorted(SIZES), a.prompt, tuple(a.batch or (8, 64)), a.context, a.steps, a.warmup, a.window,
        tuple(a.model or MODELS))
    return 0


if __name__ == "__main__":
    sys.exit(main())
