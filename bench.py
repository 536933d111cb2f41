#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Phi-mini-MoE layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 (a "step" is
one decode step of the whole batch, timed on the device with CUDA events); ``e2e`` is
the same through ``Engine.step`` with host tokens in and out; ``prefill`` is one
2,048-token prompt; ``roofline`` relates the bytes a decode step must read to its time;
``points`` has decode at batch 1 and 64.  The engine runs on one GPU: for ``--gpus N``
with N > 1 it says so and exits with 2.
"""
import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Phi-mini-MoE layer sizes (the third configuration of BASELINE.json)
MINI = {
    "architectures": ["PhimoeForCausalLM"], "model_type": "phimoe",
    "vocab_size": 32064, "hidden_size": 4096, "intermediate_size": 960, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 131072, "original_max_position_embeddings": 4096, "rope_theta": 10000.0,
    "sliding_window": 131072, "rms_norm_eps": 1e-5, "hidden_act": "silu",
    "attention_bias": True, "lm_head_bias": True, "tie_word_embeddings": False,
    "num_local_experts": 16, "num_experts_per_tok": 2, "router_jitter_noise": 0.01,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


def mini_config(layers=None, expert_intermediate=None, sizes=None):
    """The Phi-mini-MoE sizes, with any of them replaced (``sizes``: config.json key -> value)."""
    cfg = dict(MINI)
    if expert_intermediate:
        cfg["intermediate_size"] = int(expert_intermediate)
    for key, value in (sizes or {}).items():
        if value:
            cfg[key] = int(value)
    r = random.Random(7)
    half = cfg["head_dim"] // 2
    cfg["rope_scaling"] = {"type": "longrope",
                           "short_factor": [round(r.uniform(1, 4), 4) for _ in range(half)],
                           "long_factor": [round(r.uniform(1, 4), 4) for _ in range(half)]}
    if layers:
        cfg["num_hidden_layers"] = layers
    return cfg


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_model(cfg, max_slots, ctx, device="cuda:0", n_pages=None):
    import torch
    from flint_b200.engine.loading import expected_from_config
    from flint_b200.engine.model import Model
    from flint_b200.weights.sources import RandomSource
    spec, expected = expected_from_config(cfg)
    src = RandomSource(expected, seed=0, dtype=torch.bfloat16, on_device=True)
    return Model(spec, src, dtype="bfloat16", device=device, page_size=64, n_pages=n_pages or max_slots * (ctx // 64),
                 max_slots=max_slots, max_context=ctx, max_step_tokens=2048 + max_slots)


def checked(model, logits, what):
    """A timed region counts only if no kernel raised a flag in it (a bounded wait that ran out, a position
    without a page) and its last logits are finite numbers."""
    import torch
    model.check_status()
    if logits is not None and not bool(torch.isfinite(logits).all()):
        raise SystemExit(f"bench.py: {what} produced logits that are not finite; no number is reported")


def step_flops(cfg, n_tokens, kv_lens):
    """Multiply-add flops x2 of one step: projections, attention over the cache, router, two experts."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nq, nkv, hd, E = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_local_experts"]
    per_tok = 2 * H * (nq + 2 * nkv) * hd + 2 * nq * hd * H + 2 * H * E + 2 * (3 * H * I) * 2
    attn = sum(4 * nq * hd * k for k in kv_lens)       # QK^T and PV per (token, keys seen)
    return L * (n_tokens * per_tok + attn)


def decode_bytes(cfg, model, batch_kv_lens, distinct_experts):
    """Bytes a decode step must read: every weight it uses once, and the live requests' cache."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nq, nkv, hd, E, V = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["num_local_experts"], cfg["vocab_size"])
    attn_w = ((nq + 2 * nkv) * hd * H + nq * hd * H) * 2
    router = E * H * 2
    expert = 3 * H * I * 2
    weights = L * (attn_w + router) + sum(distinct_experts) * expert + V * H * 2
    kv = sum(batch_kv_lens) * nkv * hd * 2 * 2 * L
    return weights + kv


def run_decode(model, cfg, batch, prompt_len, steps, warmup, rng, count_experts=True):
    """Prefill ``batch`` requests of ``prompt_len`` random tokens, then time decode steps."""
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    slots = [model.cache.admit() for _ in range(batch)]
    for s in slots:
        model.cache.ensure(s, 0, prompt_len)
        for p0 in range(0, prompt_len, 2048):          # in portions, as the scheduler would
            n = min(2048, prompt_len - p0)
            model.step([StepEntry(s, p0, [rng.randrange(V) for _ in range(n)], [])])
    pos = prompt_len
    distinct = None
    if count_experts:
        rec = {}
        for s in slots:
            model.cache.ensure(s, pos, pos + 1)
        model.step([StepEntry(s, pos, [rng.randrange(V)], [0]) for s in slots], record=rec)
        distinct = [int(torch.unique(ids).numel()) for ids in rec["experts"]]
        pos += 1

    def one():
        nonlocal pos
        for s in slots:
            model.cache.ensure(s, pos, pos + 1)
        out = model.step([StepEntry(s, pos, [rng.randrange(V)], [0]) for s in slots])
        pos += 1
        return out
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    l0 = model.ops.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        last = one()
    e1.record()
    torch.cuda.synchronize()
    checked(model, last, f"decoding at batch {batch}")
    ms = e0.elapsed_time(e1) / steps
    launches = model.ops.launches - l0
    kv_lens = [pos] * batch
    for s in slots:
        model.cache.release(s)
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches": launches, "distinct": distinct, "kv_lens": kv_lens}


def run_prefill(model, cfg, n_tokens, reps, warmup, rng):
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    times = []
    for i in range(warmup + reps):
        s = model.cache.admit()
        toks = [rng.randrange(V) for _ in range(n_tokens)]
        model.cache.ensure(s, 0, n_tokens)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = model.step([StepEntry(s, 0, toks, [n_tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        checked(model, last, f"the prefill of {n_tokens} tokens")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
        model.cache.release(s)
    return statistics.median(times)


def run_e2e(model, cfg, batch, prompt_len, steps, warmup, rng):
    """The same decode through the public entry point: Engine.step, host tokens in and out."""
    import torch
    from flint_b200.engine.engine import Engine
    from flint_b200.sampling.params import SamplingParams
    eng = Engine(model, SamplingParams.greedy(), seed=1, prefill_chunk=2048, max_step_tokens=2048 + batch)
    V = cfg["vocab_size"]
    # prompts go in one portion per step, so the first request has decoded batch * portions tokens before the
    # last one is in: give all of them room to keep decoding through the timed region
    portions = -(-prompt_len // 2048)
    ids = [eng.create([rng.randrange(V) for _ in range(prompt_len)], steps + warmup + batch * (portions + 1) + 8)
           for _ in range(batch)]
    while any(r.remaining > 1 for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(steps):
        n_tok += eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = model.staging.host.numel() * 4
    for i in ids:
        eng.close(i)
    return {"tok_s": n_tok / dt, "h2d": h2d, "d2h": (batch + 2) * 4, "ms": dt * 1000 / steps}


def run_mixed(model, cfg, n_requests, lo, hi, decode_tokens, rng):
    """Continuous batching through the engine: requests with prompts of lo..hi random tokens, all submitted
    at once, each decoding ``decode_tokens`` tokens greedily; wall time from the first step to the last."""
    import torch
    from flint_b200.engine.engine import Engine
    from flint_b200.sampling.params import SamplingParams
    eng = Engine(model, SamplingParams.greedy(), seed=1, prefill_chunk=2048, max_step_tokens=2048 + n_requests)
    V = cfg["vocab_size"]
    lens = [rng.randint(lo, hi) for _ in range(n_requests)]
    ids = [eng.create([rng.randrange(V) for _ in range(n)], decode_tokens) for n in lens]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    stats = [eng.stats(i) for i in ids]
    for i in ids:
        eng.close(i)
    return {"seconds": dt, "steps": steps, "prompt_tokens": sum(lens), "decoded": sum(s.decode_tokens + 1 for s in stats),
            "preemptions": sum(s.preemptions for s in stats)}


def run_long(cfg, pk, rng, lengths, decode_tokens, chunk=2048):
    """Long contexts (the last configuration of BASELINE.json): prompts of ``lengths`` tokens run in portions of
    ``chunk`` through the step function, each portion timed with its depth; then ``decode_tokens`` steps of all
    requests together; then the same workload through ``Engine`` (continuous batching: a request decodes while
    the next one's prompt runs), wall clock."""
    import torch
    from flint_b200.engine.engine import Engine
    from flint_b200.engine.step import StepEntry
    from flint_b200.sampling.params import SamplingParams
    V = cfg["vocab_size"]
    ctx = max(lengths) + decode_tokens
    n_pages = sum(-(-(n + decode_tokens) // 64) for n in lengths) + 8
    model = build_model(cfg, len(lengths), ctx, n_pages=n_pages)
    by_depth = {}
    slots = []
    t_prefill = 0.0
    for n in lengths:
        s = model.cache.admit()
        slots.append(s)
        model.cache.ensure(s, 0, n)
        for p0 in range(0, n, chunk):
            m = min(chunk, n - p0)
            toks = [rng.randrange(V) for _ in range(m)]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            last = model.step([StepEntry(s, p0, toks, [m - 1] if p0 + m == n else [])])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            t_prefill += ms
            if m == chunk:
                by_depth.setdefault(p0, []).append(ms)
        checked(model, last, f"the prefill of {n} tokens")
    depth_points = {}
    for d in (0, 4096, 16384, 32768 - chunk, 65536, max(lengths) // chunk * chunk - chunk):
        if d in by_depth:
            depth_points[f"prefill_tok_s_at_depth_{d}"] = round(chunk * 1000.0 / statistics.median(by_depth[d]), 1)
    pos = list(lengths)

    def one(record=None):
        for i, s in enumerate(slots):
            model.cache.ensure(s, pos[i], pos[i] + 1)
        out = model.step([StepEntry(s, pos[i], [rng.randrange(V)], [0]) for i, s in enumerate(slots)], record=record)
        for i in range(len(pos)):
            pos[i] += 1
        return out
    rec = {}
    one(rec)
    distinct = [int(torch.unique(ids).numel()) for ids in rec["experts"]]
    for _ in range(3):
        one()
    torch.cuda.synchronize()
    n_timed = decode_tokens - 4
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_timed):
        last = one()
    e1.record()
    torch.cuda.synchronize()
    checked(model, last, "decoding at long contexts")
    ms = e0.elapsed_time(e1) / n_timed
    bytes_step = decode_bytes(cfg, model, pos, distinct)
    for s in slots:
        model.cache.release(s)
    # as served: all requests submitted at once
    eng = Engine(model, SamplingParams.greedy(), seed=1, prefill_chunk=chunk, max_step_tokens=chunk + len(lengths))
    ids = [eng.create([rng.randrange(V) for _ in range(n)], decode_tokens) for n in lengths]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while eng.has_work():
        eng.step()
    torch.cuda.synchronize()
    served = time.perf_counter() - t0
    stats = [eng.stats(i) for i in ids]
    errors = [eng.error(i) for i in ids if eng.error(i)]
    for i in ids:
        eng.close(i)
    if errors:
        raise SystemExit(f"bench.py: the served run failed: {errors[0]}")
    return {"metric": f"long contexts: prompts of {', '.join(f'{n:,}' for n in lengths)} tokens in portions of {chunk:,}, "
                      f"then {decode_tokens} decoded tokens each",
            "value": round(sum(lengths) * 1000.0 / t_prefill, 1), "unit": "prompt tokens/s (all portions, device time)",
            **depth_points,
            "decode_ms_per_step": round(ms, 3), "decode_tok_s": round(len(lengths) * 1000.0 / ms, 1),
            "decode_roofline_frac": round(bytes_step / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
            "decode_bytes_per_step": bytes_step, "cache_tokens": sum(pos),
            "served_seconds": round(served, 2), "served_tok_s": round((sum(lengths) + sum(s.decode_tokens + 1 for s in stats)) / served, 1),
            "config": config_of(cfg, len(lengths), max(lengths), ctx, pk)}


def run_sweep(cfg, pk, rng, steps, warmup):
    """``--sweep``: decode at further batch sizes and context lengths, each with its roofline fraction: batch 1 and
    8 at contexts of 16,384 and 65,536 tokens, batch 1 at 131,008, and batch 128 and 256 at 2,048.  One model, the
    cache sized for the largest point (about 70 GB)."""
    import torch
    points = [(1, 16384), (8, 16384), (1, 65536), (8, 65536), (1, 131072 - 64), (128, 2048), (256, 2048)]
    n_pages = max(b * -(-(c + 64) // 64) for b, c in points) + 8
    model = build_model(cfg, max(b for b, _ in points), 131072, n_pages=n_pages)
    out = {}
    for b, c in points:
        r = run_decode(model, cfg, b, c, steps, warmup, rng)
        frac = decode_bytes(cfg, model, r["kv_lens"], r["distinct"]) / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]
        out[f"decode_b{b}_ctx{c}"] = {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms"], 3),
                                      "roofline_frac": round(frac, 4)}
        torch.cuda.empty_cache()
    return {"metric": "decode tok/s at further batch sizes and context lengths", "points": out,
            "config": config_of(cfg, 0, 0, 131072, pk)}


def run_tiny(which, reps=5):
    """The tiny workloads of the two test configurations, in 32-bit: through ``Engine`` on the GPU (wall clock,
    host tokens in and out) and on the timed CPU baseline, the plain C++ implementation of the test-suite
    (tests/plain_phimoe.cpp: float32, whole-sequence forward pass for every token, one thread)."""
    import tempfile
    import torch
    sys.path.insert(0, os.path.join(REPO, "tests"))
    import plain_cpp
    import tiny
    from flint_b200.engine.engine import Engine
    from flint_b200.engine.model import load_model
    from flint_b200.sampling.params import SamplingParams
    cfg = tiny.CONFIGS[which]
    if which == "A":
        lens, n_tokens, params, chunk = (7, 13, 32), 16, SamplingParams.greedy(), 2048
    else:
        lens, n_tokens, params, chunk = (5, 40, 70, 100), 24, SamplingParams(temperature=0.8, top_k=20, top_p=0.8), 16
    prompts = [tiny.random_tokens(n, cfg["vocab_size"], 100 + n) for n in lens]
    with tempfile.TemporaryDirectory() as d:
        folder = tiny.write_tiny(os.path.join(d, "tiny"), which, seed=0, dtype=torch.float32)
        base_tokens, base_secs = plain_cpp.generate(folder, prompts, n_tokens, params.temperature, params.top_k,
                                                    params.top_p, seed=42)
        model = load_model(folder, dtype="float32", page_size=16, n_pages=64, max_slots=len(prompts), max_step_tokens=256)
        times = []
        for i in range(reps + 2):
            eng = Engine(model, params, seed=42, prefill_chunk=chunk, stop=())
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = eng.generate(prompts, n_tokens)
            torch.cuda.synchronize()
            if i >= 2:
                times.append(time.perf_counter() - t0)
        model.check_status()
    n_out = sum(len(g) for g in got)
    ours = n_out / statistics.median(times)
    base = sum(len(g) for g in base_tokens) / base_secs
    return {"metric": f"generated tokens/s, Tiny {which} workload ({len(prompts)} requests, prompts of "
                      f"{'/'.join(map(str, lens))} tokens, {n_tokens} tokens each, "
                      f"{'greedy' if params.temperature <= 0 else 'temperature 0.8, seed 42'})",
            "value": round(ours, 1), "unit": "tokens/s", "n_gpus": 1, "dtype": "fp32", "higher_is_better": True,
            "vs_baseline": round(ours / base, 2),
            "baseline": {"impl": "tests/plain_phimoe.cpp: plain float32 C++, whole-sequence forward pass per token, one CPU thread",
                         "value": round(base, 1), "seconds": round(base_secs, 4)},
            "tokens_match_baseline": got == base_tokens, "seconds": round(statistics.median(times), 5),
            "data": "synthetic: seeded random weights, uniform-random token ids", "impl": "ours"}


# ---------------------------------------------------------------------------------------------- Puledra beside Phi-MoE

def puledra_config(width, heads, dim, rot, vdim, kv_rank, ff, experts, top, groups, keep, layers, vocab, share_every=0):
    """A Puledra configuration of ``layers`` equal layers (every ``share_every``-th one reads the latent of the
    layer before it, 0: none does)."""
    out = []
    for i in range(layers):
        m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank,
             "rot": {"base": 10000.0, "dims": rot}, "scale": (dim + rot) ** -0.5}
        if share_every and i % share_every == share_every - 1:
            m["kv_from"] = i - 1
        out.append({"type": "latent_attention", "mixer": m,
                    "mlp": {"kind": "moe", "expert": {"ff": ff},
                            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}, "scale": 1.0}}})
    return {"architecture": "Puledra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31337, "mul_cur": 7919}}, "layers": out}


# layer sizes that resemble real models of this kind, and the Phi-MoE layer of equal width, head count, head size
# and active expert parameters that each is put beside
PULEDRA_SIZES = {
    "2048x16": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, kv_rank=512, ff=1408, experts=64, top=6, groups=8, keep=3,
                    phi=dict(hidden_size=2048, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
                             intermediate_size=4224, num_local_experts=16)),
    "4096x32": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, kv_rank=512, ff=960, experts=16, top=2, groups=1, keep=1,
                    phi=dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                             intermediate_size=960, num_local_experts=16)),
}


def gepadra_config(width, heads, kv_heads, dim, vdim, window, keep, rot, m_heads, m_dim, m_vdim, ff, experts, top, shared,
                   dense_ff, layers, vocab, every=3):
    """A Gepadra configuration of ``layers`` layers: every ``every``-th an attention layer (sliding window with kept
    first tokens, sinks, blended values), the others mLSTM layers; the first layer's feed-forward is the clamped
    gated unit, the others' a mixture of ungated experts with a shared one."""
    out = []
    for i in range(layers):
        if i % every == every - 1:
            kind, m = "attention", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
                                    "mask": {"size": window, "keep_first": keep}, "rot": {"dims": rot, "base": 5e5}, "v_mix": True}
        else:
            kind, m = "mlstm", {"heads": m_heads, "dim": m_dim, "vdim": m_vdim, "gate_cap": 15.0}
        mlp = {"kind": "dense", "ff": dense_ff, "limit": 7.0} if i == 0 else \
            {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared}}
        out.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Gepadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": out}


# layer sizes that resemble real models of this kind, beside the Phi-MoE layer of equal width, head count and head size
GEPADRA_SIZES = {
    "2048x16": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep=8, rot=64, m_heads=4, m_dim=256,
                    m_vdim=512, ff=2112, experts=16, top=2, shared=2112, dense_ff=5632,
                    phi=dict(hidden_size=2048, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
                             intermediate_size=1408, num_local_experts=16)),
    "4096x32": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, keep=8, rot=64, m_heads=8, m_dim=256,
                    m_vdim=512, ff=1440, experts=16, top=2, shared=1440, dense_ff=8192,
                    phi=dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                             intermediate_size=960, num_local_experts=16)),
}


def tefovik_config(width, heads, kv_heads, dim, vdim, chunk, rot, d_heads, d_kv_heads, d_dim, d_vdim, s_heads, s_vdim, s_state,
                   s_groups, ff, layers, vocab, taps=4):
    """A Tefovik configuration of ``layers`` layers: the even ones an attention branch (runs of ``chunk`` positions) beside
    a gated delta rule, the odd ones a state-space mixer; every layer with the ungated feed-forward."""
    out = []
    for i in range(layers):
        if i % 2 == 0:
            kind = "parallel"
            m = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "conv": taps,
                          "mask": {"size": chunk}, "rot": {"dims": rot, "base": 5e5}},
                 "right": {"heads": d_heads, "kv_heads": d_kv_heads, "dim": d_dim, "vdim": d_vdim, "conv": taps}}
        else:
            kind = "mamba2"
            m = {"heads": s_heads, "vdim": s_vdim, "state": s_state, "groups": s_groups, "norm_groups": s_groups, "conv": taps}
        out.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Tefovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
            "logit_softcap": 30.0, "layers": out}


# layer sizes that resemble real models of this kind, beside a Gepadra of equal width whose attention layers have the
# same heads and whose window is as long as the run, whose mLSTM heads hold a state of the delta rule's shape, and
# whose experts (two routed and the shared one) have the feed-forward's parameters.  With runs of 1,024 a decoded token
# behind a prompt of 2,048 sees the two keys of its own run; with runs of 4,096 it sees the whole prompt.
TEFOVIK_SIZES = {
    "2048x16": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, chunk=1024, rot=64, d_heads=16, d_kv_heads=8, d_dim=128,
                    d_vdim=128, s_heads=64, s_vdim=64, s_state=128, s_groups=8, ff=8192,
                    gepadra=dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep=8, rot=64, m_heads=16,
                                 m_dim=128, m_vdim=128, ff=2720, experts=8, top=2, shared=2720, dense_ff=5440, every=2)),
    "4096x32": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, chunk=4096, rot=64, d_heads=32, d_kv_heads=16, d_dim=128,
                    d_vdim=128, s_heads=128, s_vdim=64, s_state=128, s_groups=8, ff=16384,
                    gepadra=dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=4096, keep=8, rot=64, m_heads=32,
                                 m_dim=128, m_vdim=128, ff=5472, experts=8, top=2, shared=5472, dense_ff=10944, every=2)),
}

FP32_FMA_LANES = 148 * 128      # float32 lanes of the chip; times 2 flops, times the clock: the rate the scans are put against


def run_tefovik_pair(args, pk, rng):
    """Prefill and decode of Tefovik at layer sizes that resemble real models, beside Gepadra at equal width, heads and
    state shape: tokens/s, and for the attention and recurrence kernels of both the time a layer and the distance from
    the roofline (decode: cache or state bytes over the measured copy bandwidth; prefill attention: flops over the
    sustained library product rate; prefill recurrences, which walk tokens in float32 on the plain pipes: flops over
    the chip's float32 multiply-add rate at its highest clock)."""
    import torch
    layers = args.layers or 8
    vocab = args.vocab or 32064
    batch, ctx = args.batch, args.prompt_tokens
    fp32_rate = FP32_FMA_LANES * 2 * 1.965e9
    out = {"design": "Tefovik", "beside": "Gepadra", "layers": layers, "batch": batch, "prompt_tokens": ctx, "dtype": "bf16",
           "data": "synthetic: seeded random weights, uniform-random token ids",
           "peaks": {**{k: pk[k] for k in ("hbm_gbs", "bf16_tflops_sustained", "source")},
                     "fp32_tflops_nominal": round(fp32_rate / 1e12, 1)}, "sizes": {}}
    for name, sz in TEFOVIK_SIZES.items():
        if args.design_sizes and name not in args.design_sizes:
            continue
        cfgs = {"tefovik": tefovik_config(**{k: v for k, v in sz.items() if k != "gepadra"}, layers=layers, vocab=vocab),
                "gepadra": gepadra_config(**sz["gepadra"], layers=layers, vocab=vocab)}
        row = {}
        for which, cfg in cfgs.items():
            cfg.setdefault("vocab_size", cfg.get("vocab"))
            model = build_model(cfg, max(batch, 1), ctx + 256)
            pre_ms = run_prefill(model, cfg, ctx, reps=3, warmup=3, rng=rng)
            dec = run_decode(model, cfg, batch, ctx, args.steps, max(args.warmup, 3), rng, count_experts=False)
            pre_t, dec_t, _ = profile_tables(model, cfg, batch, ctx, rng)
            kv = ctx + 2
            mixers = [l.parts["mixer"] for l in model.layers]
            if which == "tefovik":
                pairs = [m for m in mixers if hasattr(m, "branches")]
                att, rec = (dict(pairs[0].branches)[n] for n in ("left", "right"))
                ssd = next(m for m in mixers if not hasattr(m, "branches"))
                seen = lambda k: (k - 1) % att.chunk + 1 if att.chunk else k
                n_att = len(pairs)
                # state elements of a layer's recurrence, and the multiply-adds (x2 flops) plus multiplies an element costs a token
                scans = {"delta": (rec.H * rec.D * rec.V, 9, n_att), "ssd": (ssd.H * ssd.N * ssd.V, 5, layers - n_att)}
                names = ("flint_sink_attention", "flint_qk_norm_write", "flint_head_finish", "flint_short_conv", "flint_recurrence_scan",
                         "flint_delta_prepare", "flint_ssd_prepare", "flint_gated_norm", "flint_branch_mean", "flint_post_norm",
                         "flint_depth_mix", "flint_row_act")
            else:
                att = next(m for m in mixers if hasattr(m, "keep_first"))
                rec = next(m for m in mixers if hasattr(m, "cap"))
                n_att = sum(1 for m in mixers if hasattr(m, "keep_first"))
                seen = lambda k: min(k, att.window + att.keep_first) if att.window else k
                scans = {"mlstm": (rec.H * (rec.D * rec.V + rec.D + 1), 5, layers - n_att)}
                names = ("flint_sink_attention", "flint_qkv_write", "flint_mlstm", "flint_row_norm", "flint_row_act")
            att_bytes = batch * seen(kv) * att.nkv * (att.hd + att.vd) * 2
            att_flops = sum(2 * att.nq * (att.hd + att.vd) * seen(k) for k in range(1, ctx + 1))
            kern = {}
            for kind, table in (("prefill", pre_t), ("decode", dec_t)):
                for kname, (n, ms) in sorted(table.items()):
                    if not kname.startswith(names):
                        continue
                    scan = next((s for s in scans if kname.startswith(("flint_recurrence_scan " + s, "flint_mlstm_scan"))), None)
                    per = layers
                    if scan is not None:
                        per = scans[scan][2]
                    elif any(t in kname for t in ("attention", "qkv_write", "qk_norm_write", "head_finish", "delta_prepare", "branch_mean")):
                        per = n_att
                    elif "mlstm" in kname or "ssd_prepare" in kname:
                        per = layers - n_att
                    secs = ms / per * 1e-3
                    e = {"launches": n, "us_per_layer": round(ms * 1000.0 / per, 2)}
                    if scan is not None:
                        elems, flops, _ = scans[scan]
                        if kind == "decode":        # the state is read and written once a token
                            e["frac_of_copy_bandwidth"] = round(batch * elems * 4 * 2 / secs / 1e9 / pk["hbm_gbs"], 4)
                        else:
                            e["frac_of_fp32_rate"] = round(ctx * elems * flops / secs / fp32_rate, 4)
                            e["ns_per_token"] = round(secs * 1e9 / ctx, 1)
                    elif kname.startswith("flint_sink_attention"):
                        if kind == "decode":
                            e["frac_of_copy_bandwidth"] = round(att_bytes / secs / 1e9 / pk["hbm_gbs"], 4)
                        else:
                            e["frac_of_sustained_product_rate"] = round(att_flops / secs / (pk["bf16_tflops_sustained"] * 1e12), 4)
                    kern[f"{kind}: {kname}"] = e
            row[which] = {"prefill_tok_s": round(ctx * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 3),
                          "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms"], 4),
                          "decode_launches": dec["launches"], "weight_gb": round(model.weight_bytes() / 1e9, 2), "kernels": kern}
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = row
    return out


def dumizen_config(width, heads, kv_heads, dim, vdim, window, pool, rot, r_heads, r_dim, r_vdim, ff, experts, top, groups, keep,
                   shared, layers, vocab):
    """A Dumizen configuration of ``layers`` layers in the order sigmoid attention, pooled-window attention, parallel
    mixer (gated sink attention beside a retention), pooled-window attention, ...; layers 2 .. 5 run twice (a model
    of 8 layers makes 12 layer runs); every layer with a mixture of squared-ReLU experts and a shared one."""
    yarn = {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    out = []
    for i in range(layers):
        head = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "scale": dim ** -0.5}
        if i % 4 == 0:
            kind, m = "attention_2", {**head, "vdim": vdim, "softcap": 30.0, "q_temp": {"coef": 0.1, "every": 1024}}
        elif i % 4 == 2:
            kind = "parallel"
            m = {"left": {**head, "vdim": dim, "rot": {"dims": dim, "base": 5e5, "scaling": yarn}},
                 "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "rot": {"dims": r_dim, "base": 1e6},
                           "decay": [1.0 - 2.0 ** (-5 - 5 * h / max(r_heads - 1, 1)) for h in range(r_heads)]},
                 "left_scale": 1.0, "right_scale": 1.0}
        else:
            kind, m = "attention", {**head, "vdim": vdim, "mask": {"size": window, "pool": pool},
                                    "rot": {"dims": rot, "base": 1e4, "scaling": yarn}}
        mlp = {"kind": "moe", "expert": {"ff": ff}, "shared": {"ff": shared},
               "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}}
        out.append({"type": kind, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Dumizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}
    if layers >= 6:
        cfg["loop"] = {"start": 2, "stop": 6, "times": 2}
    return cfg


# layer sizes that resemble real models of this kind, beside a Gepadra of equal width and as many layers as the Dumizen
# has layer runs, whose attention layers (every second one) have the same heads and window, whose mLSTM heads hold a
# state of the retention's shape, and whose experts have the same sizes
DUMIZEN_SIZES = {
    "2048x16": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, pool=64, rot=64, r_heads=16, r_dim=128,
                    r_vdim=128, ff=1408, experts=16, top=2, groups=4, keep=2, shared=2816,
                    gepadra=dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep=8, rot=64, m_heads=16,
                                 m_dim=128, m_vdim=128, ff=1408, experts=16, top=2, shared=2816, dense_ff=5632, every=2)),
    "4096x32": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, pool=64, rot=64, r_heads=32, r_dim=128,
                    r_vdim=128, ff=1408, experts=32, top=4, groups=4, keep=2, shared=2816,
                    gepadra=dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, keep=8, rot=64, m_heads=32,
                                 m_dim=128, m_vdim=128, ff=1408, experts=32, top=4, shared=2816, dense_ff=11264, every=2)),
}


def run_dumizen_pair(args, pk, rng):
    """Prefill and decode of Dumizen at layer sizes that resemble real models, beside Gepadra at equal width, heads,
    window and state shape and as many layers as the Dumizen has layer runs: tokens/s, and for the attention and
    recurrence kernels of both the time a layer run and the distance from the roofline (decode: cache or state bytes
    over the measured copy bandwidth; prefill attention: flops over the sustained library product rate; prefill
    recurrences, which walk tokens in float32 on the plain pipes: flops over the chip's float32 multiply-add rate)."""
    import torch
    layers = args.layers or 8
    vocab = args.vocab or 32064
    batch, ctx = args.batch, args.prompt_tokens
    fp32_rate = FP32_FMA_LANES * 2 * 1.965e9
    out = {"design": "Dumizen", "beside": "Gepadra", "layers": layers, "batch": batch, "prompt_tokens": ctx, "dtype": "bf16",
           "data": "synthetic: seeded random weights, uniform-random token ids",
           "peaks": {**{k: pk[k] for k in ("hbm_gbs", "bf16_tflops_sustained", "source")},
                     "fp32_tflops_nominal": round(fp32_rate / 1e12, 1)}, "sizes": {}}
    for name, sz in DUMIZEN_SIZES.items():
        if args.design_sizes and name not in args.design_sizes:
            continue
        dz = dumizen_config(**{k: v for k, v in sz.items() if k != "gepadra"}, layers=layers, vocab=vocab)
        runs = layers + (4 if "loop" in dz else 0)
        cfgs = {"dumizen": dz, "gepadra": gepadra_config(**sz["gepadra"], layers=runs, vocab=vocab)}
        row = {}
        for which, cfg in cfgs.items():
            cfg.setdefault("vocab_size", cfg.get("vocab"))
            model = build_model(cfg, max(batch, 1), ctx + 256)
            pre_ms = run_prefill(model, cfg, ctx, reps=3, warmup=3, rng=rng)
            dec = run_decode(model, cfg, batch, ctx, args.steps, max(args.warmup, 3), rng, count_experts=False)
            pre_t, dec_t, _ = profile_tables(model, cfg, batch, ctx, rng)
            kv = ctx + 2
            called = [model.layers[c.layer].parts["mixer"] for c in model.order]       # the mixer of every layer run
            kinds = {}          # label of the attention kernel's launches -> (mixer, layer runs, keys a row at k positions sees)
            if which == "dumizen":
                for m in called:
                    a = dict(m.branches)["left"] if hasattr(m, "branches") else m
                    label = "sigmoid" if a.weights_rule == "sigmoid" else ("pooled" if a.pool else "softmax")
                    seen = (lambda k, a=a: min(k, a.window) + max(0, (k - a.window) // a.pool)) if a.pool else (lambda k: k)
                    kinds[label] = (a, kinds.get(label, (None, 0))[1] + 1, seen)
                ret = next(dict(m.branches)["right"] for m in called if hasattr(m, "branches"))
                n_rec = sum(1 for m in called if hasattr(m, "branches"))
                scans = {"ssd": (ret.H * ret.D * ret.V, 5, n_rec)}
                names = ("flint_sink_attention", "flint_qk_norm_write", "flint_pool_write", "flint_head_finish",
                         "flint_recurrence_scan", "flint_retention_prepare", "flint_gated_norm", "flint_sum_norm_add",
                         "flint_router_sigmoid_grouped", "flint_row_act", "flint_row_norm")
            else:
                att = next(m for m in called if hasattr(m, "keep_first"))
                rec = next(m for m in called if hasattr(m, "cap"))
                n_att = sum(1 for m in called if hasattr(m, "keep_first"))
                kinds["softmax"] = (att, n_att, lambda k: min(k, att.window + att.keep_first))
                scans = {"mlstm": (rec.H * (rec.D * rec.V + rec.D + 1), 5, len(called) - n_att)}
                names = ("flint_sink_attention", "flint_qkv_write", "flint_mlstm", "flint_row_norm", "flint_row_act")
            kern = {}
            for kind, table in (("prefill", pre_t), ("decode", dec_t)):
                for kname, (n, ms) in sorted(table.items()):
                    if not kname.startswith(names):
                        continue
                    scan = next((s for s in scans if kname.startswith(("flint_recurrence_scan " + s, "flint_mlstm_scan"))), None)
                    label = next((l for l in kinds if kname.startswith("flint_sink_attention") and kname.endswith(" " + l)), None)
                    per = scans[scan][2] if scan is not None else (kinds[label][1] if label is not None else len(called))
                    secs = ms / per * 1e-3
                    e = {"launches": n, "us_per_layer_run": round(ms * 1000.0 / per, 2)}
                    if scan is not None:
                        elems, flops, _ = scans[scan]
                        if kind == "decode":        # the state is read and written once a token
                            e["frac_of_copy_bandwidth"] = round(batch * elems * 4 * 2 / secs / 1e9 / pk["hbm_gbs"], 4)
                        else:
                            e["frac_of_fp32_rate"] = round(ctx * elems * flops / secs / fp32_rate, 4)
                            e["ns_per_token"] = round(secs * 1e9 / ctx, 1)
                    elif label is not None and not kname.startswith("flint_sink_combine"):
                        a, _, seen = kinds[label]
                        if kind == "decode":
                            e["frac_of_copy_bandwidth"] = round(batch * seen(kv) * a.nkv * (a.hd + a.vd) * 2 / secs / 1e9 / pk["hbm_gbs"], 4)
                        else:
                            flops = sum(2 * a.nq * (a.hd + a.vd) * seen(k) for k in range(1, ctx + 1))
                            e["frac_of_sustained_product_rate"] = round(flops / secs / (pk["bf16_tflops_sustained"] * 1e12), 4)
                    kern[f"{kind}: {kname}"] = e
            row[which] = {"layer_runs": len(called), "prefill_tok_s": round(ctx * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 3),
                          "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms"], 4),
                          "decode_launches": dec["launches"], "weight_gb": round(model.weight_bytes() / 1e9, 2), "kernels": kern}
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = row
    return out


def run_design_pair(args, pk, rng):
    """Prefill and decode of Puledra or Gepadra at layer sizes that resemble real models, beside Phi-MoE at equal width, heads
    and active expert parameters: tokens/s, and for the attention kernels of both the time a layer and the
    fraction of the measured peak (decode: cache bytes over the copy bandwidth; prefill: flops over the sustained
    library product rate)."""
    import torch
    layers = args.layers or 8
    vocab = args.vocab or 32064
    batch, ctx = args.batch, args.prompt_tokens
    gep = args.design == "gepadra"
    out = {"design": "Gepadra" if gep else "Puledra", "beside": "PhimoeForCausalLM", "layers": layers, "batch": batch, "prompt_tokens": ctx,
           "dtype": "bf16", "data": "synthetic: seeded random weights, uniform-random token ids",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops_sustained", "source")}, "sizes": {}}
    for name, sz in (GEPADRA_SIZES if gep else PULEDRA_SIZES).items():
        if args.design_sizes and name not in args.design_sizes:
            continue
        phi = sz["phi"]
        make = gepadra_config if gep else puledra_config
        cfgs = {args.design: make(**{k: v for k, v in sz.items() if k != "phi"}, layers=layers, vocab=vocab),
                "phimoe": mini_config(layers, None, {**phi, "vocab_size": vocab})}
        row = {}
        for which, cfg in cfgs.items():
            cfg.setdefault("vocab_size", cfg.get("vocab"))
            model = build_model(cfg, max(batch, 1), ctx + 256)
            pre_ms = run_prefill(model, cfg, ctx, reps=3, warmup=3, rng=rng)
            dec = run_decode(model, cfg, batch, ctx, args.steps, max(args.warmup, 3), rng, count_experts=False)
            pre_t, dec_t, _ = profile_tables(model, cfg, batch, ctx, rng)
            kv = ctx + 2
            state_bytes = 0
            if which == "gepadra":
                att = next(l.parts["mixer"] for l in model.layers if hasattr(l.parts["mixer"], "keep_first"))
                rec = next(l.parts["mixer"] for l in model.layers if hasattr(l.parts["mixer"], "cap"))
                n_att = sum(1 for l in model.layers if l.parts["mixer"] is not None and hasattr(l.parts["mixer"], "keep_first"))
                seen = lambda k: min(k, att.window + att.keep_first) if att.window else k
                att_bytes = batch * seen(kv) * att.nkv * (att.hd + att.vd) * 2
                att_flops = sum(2 * att.nq * (att.hd + att.vd) * seen(k) for k in range(1, ctx + 1))
                state_bytes = batch * rec.H * (rec.D * rec.V + rec.D + 1) * 4 * 2       # read and written every token
                names = ("flint_sink_attention", "flint_qkv_write", "flint_mlstm", "flint_router_sigmoid", "flint_row_act",
                         "flint_gated_act", "flint_row_norm")
            elif which == "puledra":
                m = model.layers[0].parts["mixer"]
                att_bytes = batch * kv * m.row_w * 2
                att_flops = sum(2 * m.H * (m.Dk + m.C) * k for k in range(1, ctx + 1))
                names = ("flint_latent_attention", "flint_head_products", "flint_latent_prepare", "flint_router_topk", "flint_row_norm")
            else:
                nq, nkv, hd = phi["num_attention_heads"], phi["num_key_value_heads"], phi["head_dim"]
                att_bytes = batch * kv * nkv * hd * 2 * 2
                att_flops = sum(4 * nq * hd * k for k in range(1, ctx + 1))
                names = ("flint_attention", "flint_rope_kv_write", "flint_row_norm")
            kern = {}
            for kind, table in (("prefill", pre_t), ("decode", dec_t)):
                for kname, (n, ms) in sorted(table.items()):
                    if not kname.startswith(names):
                        continue
                    per = layers
                    if which == "gepadra":       # a kernel runs in the layers of its kind only
                        per = n_att if ("attention" in kname or "qkv_write" in kname) else (layers - n_att if "mlstm" in kname else layers)
                    e = {"launches": n, "us_per_layer": round(ms * 1000.0 / per, 2)}
                    if kname.startswith("flint_mlstm_scan") and kind == "decode":
                        e["frac_of_copy_bandwidth"] = round(state_bytes / (ms / per * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                    elif which == "gepadra" and kname.startswith("flint_sink_attention"):
                        if kind == "decode":
                            e["frac_of_copy_bandwidth"] = round(att_bytes / (ms / per * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                        else:
                            e["frac_of_sustained_product_rate"] = round(att_flops / (ms / per * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
                    elif which != "gepadra" and "attention" in kname and "prepare" not in kname:
                        if kind == "decode":
                            e["frac_of_copy_bandwidth"] = round(att_bytes / (ms / layers * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                        else:
                            e["frac_of_sustained_product_rate"] = round(att_flops / (ms / layers * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
                    kern[f"{kind}: {kname}"] = e
            row[which] = {"prefill_tok_s": round(ctx * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 3),
                          "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms"], 4),
                          "decode_launches": dec["launches"], "weight_gb": round(model.weight_bytes() / 1e9, 2), "kernels": kern}
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = row
    return out


def config_of(cfg, batch, prompt_tokens, ctx, pk):
    """Every size of a run, flat."""
    mini = all(cfg[k] == MINI[k] for k in MINI if k != "num_hidden_layers")
    return {"model": "Phi-mini-MoE sizes" if mini else
                     f"Phi-MoE sizes: hidden {cfg['hidden_size']}, experts of {cfg['intermediate_size']}",
            "layers": cfg["num_hidden_layers"], "layers_of_config": 32,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"],
            "top_k": 2, "expert_intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": batch, "prompt_tokens": prompt_tokens, "seq_len": ctx, "page_size": 64,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights streamed every step)",
            "peaks": pk["source"]}


def profile_tables(model, cfg, batch, prompt_len, rng):
    """Per-kernel device time (CUDA events around every launch, graphs off, so launches are serialised): one
    prefill of ``prompt_len`` tokens and one decode step of the batch at that context.  Returns
    (prefill table, decode table, distinct experts per layer of the decode step), tables as
    {launcher name and product shape: (launches, ms)}."""
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    graphs, model.use_graphs = model.use_graphs, False
    slots = [model.cache.admit() for _ in range(batch)]
    for i, s in enumerate(slots):
        model.cache.ensure(s, 0, prompt_len + 2)
        if i == len(slots) - 1:
            model.ops.start_profile()
        model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(prompt_len)], [prompt_len - 1])])
    prefill = model.ops.stop_profile()
    dec = lambda p, rec=None: model.step([StepEntry(s, p, [rng.randrange(V)], [0]) for s in slots], record=rec)
    dec(prompt_len)
    rec = {}
    model.ops.start_profile()
    dec(prompt_len + 1, rec)
    decode = model.ops.stop_profile()
    distinct = [int(torch.unique(ids).numel()) for ids in rec.get("experts", [])]
    for s in slots:
        model.cache.release(s)
    model.use_graphs = graphs
    return prefill, decode, distinct


def graph_step_table(model, cfg, batch, prompt_len, rng):
    """The kernels of one captured decode step with the time each adds to the step: inside the graph, kernels
    start early under programmatic dependent launch and wait for the one before, so a kernel's share is the time
    from the end of the kernel before it to its own end (device timestamps of one replay, read through
    torch.profiler).  Kernels are named by pairing them, in order, with the launches of one eager step of the
    same shape.  Returns ({label: (launches, ms)}, distinct experts per layer) or None if the profiler is not
    available or the two sequences do not pair up."""
    import torch
    from flint_b200.engine.step import StepEntry
    try:
        from torch.profiler import ProfilerActivity, profile as torch_profile
    except ImportError:
        return None
    V = cfg["vocab_size"]
    slots = [model.cache.admit() for _ in range(batch)]
    for s in slots:
        model.cache.ensure(s, 0, prompt_len + 8)
        model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(prompt_len)], [])])
    pos = prompt_len

    def dec(rec=None):
        nonlocal pos
        out = model.step([StepEntry(s, pos, [rng.randrange(V)], [0]) for s in slots], record=rec)
        pos += 1
        return out
    graphs, model.use_graphs = model.use_graphs, False
    dec()
    rec = {}
    model.ops.start_profile()
    dec(rec)
    labels = [name for name, _ in model.ops.stop_profile(ordered=True)]
    distinct = [int(torch.unique(ids).numel()) for ids in rec.get("experts", [])]
    model.use_graphs = graphs
    table = None
    if graphs:
        for _ in range(3):
            dec()
        torch.cuda.synchronize()
        try:
            with torch_profile(activities=[ProfilerActivity.CUDA]) as prof:
                dec()
                torch.cuda.synchronize()
            ev = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                         if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name and "Memset" not in e.name))
        except Exception:            # no CUPTI here: the caller falls back to the eager table
            ev = []
        followers = ("splitk_reduce", "attention_combine")      # second kernels of a launcher call
        paired, i = [], 0
        for start, end, name in ev:
            if any(f in name for f in followers) and paired:
                paired.append((paired[-1][0], end))
            elif i < len(labels):
                paired.append((labels[i], end))
                i += 1
            else:
                i += 1
        if ev and i == len(labels):
            table, prev = {}, ev[0][0]
            for label, end in paired:
                n, ms = table.get(label, (0, 0.0))
                table[label] = (n + 1, ms + max(0.0, end - prev) / 1000.0)
                prev = max(prev, end)
    for s in slots:
        model.cache.release(s)
    return (table, distinct) if table else None


def kernel_class(name, cfg):
    """The dominant kernels by what they compute; everything else is the small row-wise work."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    if "attention_prefill" in name:
        return "attention_prefill"
    if "attention" in name:
        return "attention_decode"
    if "gemm" in name and " " in name:
        shape = name.split(" ")[1]
        n, k = (int(x) for x in shape.split("x"))
        if "experts" in name:
            return "expert_gate_up" if k == H else "expert_down"
        if n == (nq + 2 * nkv) * hd and k == H:
            return "qkv"
        if n == V:
            return "head"
        if n == H and k == nq * hd:
            return "o_proj"
    return "other"


def kernel_fractions(table, cfg, pk, kind, n_tokens, kv_lens, distinct):
    """Flat {class.us, class.frac}: device time of each dominant kernel over a whole step and its fraction of the
    measured peak: bytes it must read over the copy bandwidth for a decode step, flops over the sustained library
    product rate for a prefill.  ``other`` (norms with routing, rotary write, plan, activation, embedding) has a
    time only."""
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    us = {}
    for name, (_, ms) in table.items():
        c = kernel_class(name, cfg)
        us[c] = us.get(c, 0.0) + ms * 1000.0
    keys = sum(kv_lens)
    if kind == "decode":
        work = {"qkv": L * (nq + 2 * nkv) * hd * H * 2, "o_proj": L * H * nq * hd * 2,
                "expert_gate_up": sum(distinct) * 2 * I * H * 2, "expert_down": sum(distinct) * H * I * 2,
                "attention_decode": keys * nkv * hd * 2 * 2 * L, "head": V * H * 2}
        peak = pk["hbm_gbs"] * 1e9
    else:
        T = n_tokens
        work = {"qkv": 2 * T * (nq + 2 * nkv) * hd * H * L, "o_proj": 2 * T * H * nq * hd * L,
                "expert_gate_up": 2 * (2 * T) * (2 * I) * H * L, "expert_down": 2 * (2 * T) * H * I * L,
                "attention_prefill": 4 * nq * hd * keys * L}
        peak = pk["bf16_tflops_sustained"] * 1e12
    out = {}
    for c, t in sorted(us.items(), key=lambda kv: -kv[1]):
        out[f"{kind}.{c}.us"] = round(t, 1)
        if c in work and t > 0:
            out[f"{kind}.{c}.frac"] = round(work[c] / (t * 1e-6) / peak, 3)
    return out


def profile(model, cfg, args, rng):
    """``--profile``: the tables to stderr."""
    prefill, decode, _ = profile_tables(model, cfg, args.batch, args.prompt_tokens, rng)

    def show(title, table):
        total = sum(ms for _, ms in table.values())
        print(f"--- {title}: {total:.3f} ms in {sum(n for n, _ in table.values())} launches", file=sys.stderr)
        for name, (n, ms) in sorted(table.items(), key=lambda kv: -kv[1][1]):
            print(f"{name:48s} {n:6d} launches {ms:10.3f} ms {100 * ms / total:6.1f} %", file=sys.stderr)
    show(f"prefill of {args.prompt_tokens} tokens", prefill)
    show(f"decode step, batch {args.batch}, context {args.prompt_tokens}", decode)
    return 0


def one_step(model, cfg, args, rng):
    """Set-up, one warm step and one more step of the asked kind, eagerly (no graph), for profilers."""
    import torch
    from flint_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    model.use_graphs = False
    n = args.prompt_tokens
    slots = [model.cache.admit() for _ in range(args.batch)]
    if args.one_step == "decode":
        for s in slots:
            model.cache.ensure(s, 0, n + 2)
            model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(n)], [])])
        step = lambda p: model.step([StepEntry(s, p, [rng.randrange(V)], [0]) for s in slots])
        step(n)
        torch.cuda.synchronize()
        before = model.ops.launches
        step(n + 1)
    else:
        run = lambda s: (model.cache.ensure(s, 0, n), model.step([StepEntry(s, 0, [rng.randrange(V) for _ in range(n)], [n - 1])]))
        run(slots[0])
        torch.cuda.synchronize()
        before = model.ops.launches
        run(slots[1 % len(slots)])
    torch.cuda.synchronize()
    print(f"launcher calls before the last step: {before}, in it: {model.ops.launches - before} "
          f"(a call with a split launches two kernels)", file=sys.stderr)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-tokens", type=int, default=2048)
    ap.add_argument("--ctx-size", type=int, default=4096)
    # the reference bench's own names for the sizes and the workload (crates/thuban_bench/src/main.rs:12-63)
    for flag in ("--hidden", "--intermediate", "--q-heads", "--kv-heads", "--head-dim", "--vocab", "--prefill-tokens",
                 "--decode-tokens", "--max-seq"):
        ap.add_argument(flag, type=int, default=None)
    ap.add_argument("--mixed", type=int, nargs=4, metavar=("REQUESTS", "MIN_PROMPT", "MAX_PROMPT", "DECODE"), default=None,
                    help="instead of the default run: continuous batching of this many requests through the engine")
    ap.add_argument("--expert-intermediate", type=int, default=None,
                    help="expert width (default 960, the Phi-mini-MoE sizes; 6400 gives the Phi-3.5-MoE sizes)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (both are named)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--one-step", choices=["decode", "prefill"], default=None,
                    help="run the set-up, then one warm and one measured eager step of this kind, and exit "
                         "(for a launch list under ncu: the launch counts to skip and capture go to stderr)")
    ap.add_argument("--tiny", choices=["A", "B"], default=None,
                    help="instead of the default run: the tiny workload of that test configuration, in 32-bit, against "
                         "the timed CPU baseline (the plain C++ implementation)")
    ap.add_argument("--long", action="store_true",
                    help="instead of the default run: prompts of 4 x 32,768 and one of 130,944 tokens (with its 128 decoded "
                         "tokens the model's 131,072 positions) in portions of 2,048, then 128 decoded tokens each; "
                         "use with --expert-intermediate 6400 for the Phi-3.5-MoE sizes")
    ap.add_argument("--long-prompts", type=int, nargs="+", default=None, help="other prompt lengths for --long")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel table")
    ap.add_argument("--sweep", action="store_true",
                    help="instead of the default run: decode at batch 1 and 8 with contexts of 16,384 and 65,536 tokens, "
                         "batch 1 with 131,008, and batch 128 and 256 with 2,048, each with its roofline fraction")
    ap.add_argument("--design", choices=["puledra", "gepadra", "tefovik", "dumizen"], default=None,
                    help="prefill and decode of this design at layer sizes that resemble real models, beside the closest "
                         "earlier model at equal sizes (Phi-MoE; for tefovik and dumizen Gepadra), with its kernels' shares of the peaks")
    ap.add_argument("--design-sizes", nargs="+", default=None, help="which of the design's size points to run")
    ap.add_argument("--profile", action="store_true",
                    help="print per-kernel device times of one prefill and one decode step to stderr and exit")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "formetaohy/Flint is a Rust workspace that reaches the GPU only through wgpu on Vulkan/Metal: "
                          "no Python package to install offline, no cargo here, no graphics API on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    pk = peaks()
    cfg = mini_config(args.layers, args.expert_intermediate or args.intermediate,
                      {"hidden_size": args.hidden, "num_attention_heads": args.q_heads, "num_key_value_heads": args.kv_heads,
                       "head_dim": args.head_dim, "vocab_size": args.vocab})
    if args.max_seq:
        args.ctx_size = args.max_seq
    if args.prefill_tokens:
        args.prompt_tokens = args.prefill_tokens
    if args.decode_tokens:
        args.steps = args.decode_tokens
    rng = random.Random(0)
    if args.tiny:
        print(json.dumps(run_tiny(args.tiny)))
        return 0
    if args.design:
        run = {"tefovik": run_tefovik_pair, "dumizen": run_dumizen_pair}.get(args.design, run_design_pair)
        print(json.dumps(run(args, pk, rng)))
        return 0
    if args.sweep:
        print(json.dumps(run_sweep(cfg, pk, rng, max(8, args.steps // 4), warmup)))
        return 0
    if args.long:
        print(json.dumps(run_long(cfg, pk, rng, args.long_prompts or [32768] * 4 + [131072 - 128], 128)))
        return 0
    max_batch = max(args.batch, 1 if args.no_points else 64, args.mixed[0] if args.mixed else 1)
    model = build_model(cfg, max_batch, args.ctx_size)

    if args.profile:
        return profile(model, cfg, args, rng)
    if args.one_step:
        return one_step(model, cfg, args, rng)
    if args.mixed:
        n, lo, hi, dec = args.mixed
        for _ in range(2):          # the first pass compiles kernels and captures graphs
            r = run_mixed(model, cfg, n, lo, hi, dec, rng)
        print(json.dumps({"metric": f"mixed serving: {n} requests, prompts of {lo}..{hi} tokens, {dec} decoded each",
                          "value": round((r["prompt_tokens"] + r["decoded"]) / r["seconds"], 1), "unit": "tokens/s (prompt + decoded)",
                          "decode_tok_s": round(r["decoded"] / r["seconds"], 1), **r}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    pre_ms = run_prefill(model, cfg, 2048, reps=3, warmup=3, rng=rng)
    dec = run_decode(model, cfg, args.batch, args.prompt_tokens, args.steps, warmup, rng)
    clock = clocks.stop()
    e2e = run_e2e(model, cfg, args.batch, args.prompt_tokens, args.steps, warmup, rng)
    points, points_frac = {}, {}
    if not args.no_points:
        for b in (1, 64):
            r = run_decode(model, cfg, b, args.prompt_tokens, max(8, args.steps // 2), warmup, rng)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            # the same roofline as the headline's: bytes the step must read over its time, of the copy peak
            points_frac[f"decode_b{b}"] = round(decode_bytes(cfg, model, r["kv_lens"], r["distinct"]) / (r["ms"] * 1e-3) / 1e9
                                                / pk["hbm_gbs"], 4)

    kernels = {}
    kernels_decode_how = "CUDA events around every launch of one eager step (launches serialised, host gaps included)"
    if not args.no_kernels:
        pre_t, dec_t, distinct = profile_tables(model, cfg, args.batch, args.prompt_tokens, rng)
        in_graph = graph_step_table(model, cfg, args.batch, args.prompt_tokens, rng)
        if in_graph is not None:
            dec_t, distinct = in_graph
            kernels_decode_how = ("device timestamps of one replay of the captured step: a kernel's time runs from the end "
                                  "of the kernel before it to its own end (kernels overlap under programmatic dependent launch)")
        kernels.update(kernel_fractions(dec_t, cfg, pk, "decode", args.batch, [args.prompt_tokens + 2] * args.batch, distinct))
        kernels.update(kernel_fractions(pre_t, cfg, pk, "prefill", args.prompt_tokens, range(1, args.prompt_tokens + 1), None))
    pre_flops = step_flops(cfg, 2048, range(1, 2049))
    bytes_step = decode_bytes(cfg, model, dec["kv_lens"], dec["distinct"])
    achieved = bytes_step / (dec["ms"] * 1e-3) / 1e9
    mini = all(cfg[k] == MINI[k] for k in MINI if k != "num_hidden_layers")
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({'Phi-mini-MoE layer sizes' if mini else 'other layer sizes, see config'}, "
                  f"{args.prompt_tokens:,}-token prompts, context {args.ctx_size:,})",
        "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(dec["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform-random token ids", "impl": "ours",
        "config": config_of(cfg, args.batch, args.prompt_tokens, args.ctx_size, pk),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms"], 4),
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": dec["launches"],
        "prefill": {"value": round(2048 * 1000.0 / pre_ms, 1), "tokens": 2048, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": bytes_step,
                     "distinct_experts_per_layer": round(sum(dec["distinct"]) / len(dec["distinct"]), 2)},
        "points": points,
        "points_roofline_frac": points_frac,
        "kernels": kernels,
        "kernels_how": "microseconds per step and fraction of the measured peak.  decode: " + kernels_decode_how +
                       "; fractions: bytes the kernel must read over the measured copy bandwidth.  prefill: CUDA events "
                       "around every launch of one eager step; fractions: flops over the measured sustained library "
                       "product rate",
        "clocks": clock,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
