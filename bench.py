#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-8B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A "step" is one decode step of the whole batch.  The timed region is exactly K replays of the
decode step's CUDA graph, bracketed by CUDA events and a synchronize on both sides, after W
untimed steps.  The K steps are centred on the benchmark's mean context (2,048-token prompts and
up to 2,048 generated tokens: mean 3,072), so the prompt fed before them has 3,072 - K/2 tokens;
with K = 2,047 that is the benchmark's own run.  `value` is decoded tokens a second (batch * K /
time); `e2e` is the same rate through `Model.generate` with host token lists in and out;
`prefill` is one 2,048-token prompt through the step function; `points` has decode at batch 1
and 64 and the milliseconds a 128-token and a 512-token prompt take through the step function; `roofline` places the decode step against the bytes it must read.  One JSON line is
printed.  This library runs on one GPU: for --gpus above 1 a line says so and the exit code is 2.

    python bench.py --design rovurax|tenetar|retuvik|barorax [--sizes 1.7b,8b] [--layers 8] [--chunk 1024] [--steps K]

instead runs that design beside Qwen3 (retuvik: beside Tenetar; barorax: beside Retuvik) at equal sizes (random bfloat16 weights, the same engine,
step function and decode graphs): one prompt of --prefill-tokens through the step function, then decode
at --batch, device-timed; one JSON line with a row per size and design.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
PUBLISHED_DECODE_TOK_S = None   # the reference publishes no B200 and no batched figure


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    src = "fallback"
    hbm, tf, tf_s = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, None
    def num(v, default):
        """A number, also when the file wraps it ({"value": ...}) or lists several (their median)."""
        if isinstance(v, dict):
            for key in ("value", "median", "mean", "gbs", "tflops"):
                if key in v:
                    return num(v[key], default)
            return default
        if isinstance(v, (list, tuple)) and v:
            vals = sorted(num(x, default) for x in v)
            return vals[len(vals) // 2]
        try:
            return float(v)
        except (TypeError, ValueError):
            return default

    try:
        with open(path) as f:
            d = json.load(f)
        if isinstance(d, dict) and ("hbm_gbs" in d or "bf16_tflops" in d):
            hbm = num(d.get("hbm_gbs"), hbm)
            tf = num(d.get("bf16_tflops"), tf)
            tf_s = num(d.get("bf16_tflops_sustained"), None) if "bf16_tflops_sustained" in d else None
            src = "measured"
    except (OSError, ValueError):
        pass
    if not (hbm > 0 and tf > 0):
        hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    return dict(hbm_gbs=hbm, bf16_tflops=tf, bf16_tflops_sustained=tf_s, source=src)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows = []
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synthetic_ids(n, vocab, seed):
    """splitmix64 ids below vocab (the generator x0ne-core/oracle/examples/core-bench.rs:26-43 uses)."""
    m = (1 << 64) - 1
    s, out = seed, []
    for _ in range(n):
        s = (s + 0x9E3779B97F4A7C15) & m
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        out.append(int((z ^ (z >> 31)) % vocab))
    return out


# ---------------------------------------------------------------------------------------------
# --design rovurax: the Rovurax design beside the Qwen3 design at equal sizes
# ---------------------------------------------------------------------------------------------
DESIGN_SIZES = {
    # width, feed-forward, q heads, kv heads, head size, latent rank, rotated part: the layer sizes of a 1.7B and of an 8B model
    "1.7b": dict(width=2048, ff=6144, heads=16, kv_heads=8, dim=128, kv_rank=256, rot_dim=64),
    "8b": dict(width=4096, ff=12288, heads=32, kv_heads=8, dim=128, kv_rank=256, rot_dim=64),
}


def tenetar_config(size: dict, layers: int, vocab: int, window: int):
    """A Tenetar configuration of the given layer sizes.  Of every four layers the first two keep keys and values
    and the other two read the second one's; the first layer of the model has a dense feed-forward of the full
    width, the others 16 experts of a quarter of it plus 2 identity experts in 6 groups of 3 of which 3 stay,
    4 chosen per token, and a gated shared expert of the same quarter: about the dense layer's work per token."""
    from x0ne_engine_b200.config import config_from_dict
    w, ff, H, G, d = size["width"], size["ff"], size["heads"], size["kv_heads"], size["dim"]
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4},
           "router": {"experts": 16, "identity": 2, "top": 4, "groups": {"count": 6, "keep": 3}}}
    out = []
    for i in range(layers):
        mixer = {"dim": d, "heads": H, "kv_heads": G, "vdim": d, "scale": d ** -0.5, "mask": {"size": window, "keep_first": 4},
                 "rot": {"base": 1000000.0, "dims": d}}
        if i % 4 >= 2:
            mixer["kv_from"] = i - i % 4 + 1
        out.append({"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if i == 0 else moe})
    return config_from_dict({"architecture": "Tenetar", "vocab": vocab, "width": w, "norm": {"eps": 1e-6},
                             "embedding": {"scale": float(w) ** 0.5}, "layers": out})


def retuvik_config(size: dict, layers: int, vocab: int, window: int):
    """A Retuvik configuration of the given layer sizes.  Of every four layers three are recurrent (heads of 64
    channels that fill the width, a decay of inner width 64) and the fourth is windowed attention with the distance
    bias, query temperature and output gate; the first layer has a dense feed-forward of the full width, the others
    16 gated experts of a sixth of it, 4 chosen per token: the dense layer's products per token.  The whole list is a
    stretch that runs once, so a pass opener runs; norms in 4 groups."""
    from x0ne_engine_b200.config import config_from_dict
    w, ff, H, G, d = size["width"], size["ff"], size["heads"], size["kv_heads"], size["dim"]
    moe = {"kind": "moe", "expert": {"ff": ff // 6}, "router": {"experts": 16, "top": 4}}
    out = []
    for i in range(layers):
        if i % 4 == 3:
            layer = {"type": "attention", "mixer": {"dim": d, "heads": H, "kv_heads": G, "vdim": d, "scale": d ** -0.5, "mask": {"size": window},
                                                    "q_temp": {"coef": 0.1, "every": 1024}}}
        else:
            layer = {"type": "wkv", "mixer": {"dim": 64, "heads": w // 64, "decay_rank": 64}}
        layer["mlp"] = {"kind": "dense", "ff": ff} if i == 0 else moe
        out.append(layer)
    return config_from_dict({"architecture": "Retuvik", "vocab": vocab, "width": w, "norm": {"eps": 1e-6, "groups": 4},
                             "embedding": {"scale": float(w) ** 0.5}, "layers": out, "loop": {"start": 0, "stop": layers, "times": 1}})


def barorax_config(size: dict, layers: int, vocab: int, chunk: int):
    """A Barorax configuration of the given layer sizes.  Of every four layers the first and third are selective
    state-space mixers (twice the width in channels, 16 states per channel, 4 taps, a step-size rank of a sixteenth of
    the width), the second is differential attention (half the heads, each with two maps of the head size and values
    of twice it, rotation over half of every map) and the fourth is chunked attention with rotation, unit-norm queries
    and keys and the sink; every layer has 16 gated experts of a sixth of the feed-forward width in 4 groups of which 2
    stay, 4 chosen per token, and a shared expert of the same size.  The whole list is a stretch that runs once, so a
    pass opener runs."""
    from x0ne_engine_b200.config import config_from_dict
    w, ff, H, G, d = size["width"], size["ff"], size["heads"], size["kv_heads"], size["dim"]
    moe = {"kind": "moe", "expert": {"ff": ff // 6}, "shared": {"ff": ff // 6},
           "router": {"experts": 16, "top": 4, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    out = []
    for i in range(layers):
        if i % 4 == 1:
            layer = {"type": "attention", "mixer": {"dim": d, "heads": H // 2, "kv_heads": max(1, G // 2), "vdim": 2 * d, "scale": d ** -0.5,
                                                    "diff": 0.3, "rot": {"base": 500000.0, "dims": d // 2}}}
        elif i % 4 == 3:
            layer = {"type": "attention_2", "mixer": {"dim": d, "heads": H, "kv_heads": G, "vdim": d, "scale": 8.0 / d, "mask": {"size": chunk},
                                                      "rot": {"base": 10000.0, "dims": d}}}
        else:
            layer = {"type": "mamba1", "mixer": {"inner": 2 * w, "state": 16, "conv": 4, "dt_rank": w // 16}}
        layer["mlp"] = moe
        out.append(layer)
    return config_from_dict({"architecture": "Barorax", "vocab": vocab, "width": w, "norm": {"eps": 1e-6}, "layers": out,
                             "loop": {"start": 0, "stop": layers, "times": 1}})


def design_configs(size: dict, layers: int, vocab: int, chunk: int, design: str = "rovurax"):
    """(the design's configuration, Qwen3 configuration) with the same width, heads, feed-forward, depth and
    vocabulary.  Of every four Rovurax layers three are chunk-masked attention with blended values and
    one is latent attention with YaRN-scaled rotation, a sink and a gate; Tenetar: see tenetar_config."""
    import x0ne_engine_b200 as x
    from x0ne_engine_b200.config import config_from_dict
    w, ff, H, G, d = size["width"], size["ff"], size["heads"], size["kv_heads"], size["dim"]
    old = x.Qwen3Config(hidden_size=w, intermediate_size=ff, num_hidden_layers=layers, num_attention_heads=H,
                        num_key_value_heads=G, head_dim=d, vocab_size=vocab, max_position_embeddings=40960,
                        rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, dtype="bfloat16")
    if design == "tenetar":
        return tenetar_config(size, layers, vocab, chunk), old
    if design == "retuvik":        # beside the closest design the library has: Tenetar (windowed attention, routed experts)
        return retuvik_config(size, layers, vocab, chunk), tenetar_config(size, layers, vocab, chunk)
    if design == "barorax":        # beside Retuvik: a recurrent mixer with a state, attention over a bounded span, gated experts, a stretch
        return barorax_config(size, layers, vocab, chunk), retuvik_config(size, layers, vocab, chunk)
    mlp = {"ff": ff, "kind": "dense", "limit": 7.0}
    att = {"type": "attention", "mlp": mlp, "mixer": {"dim": d, "heads": H, "kv_heads": G, "vdim": d, "scale": d ** -0.5,
                                                        "mask": {"size": chunk}, "v_mix": True}}
    lat = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "dim": d, "heads": H, "kv_rank": size["kv_rank"], "rot_dim": size["rot_dim"], "vdim": d, "scale": (d + size["rot_dim"]) ** -0.5,
        "rot": {"base": 1000000.0, "dims": size["rot_dim"], "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    new = config_from_dict({"architecture": "Rovurax", "vocab": vocab, "width": w, "norm": {"eps": 1e-6},
                            "layers": [lat if i % 4 == 3 else att for i in range(layers)]})
    return new, old


def design_bench(args) -> int:
    """Prefill and decode throughput of Rovurax and of Qwen3 at equal sizes, random bfloat16 weights, through the same
    engine, step function and decode graphs.  One JSON line."""
    import torch

    import x0ne_engine_b200 as x
    from x0ne_engine_b200.engine.decode import DeviceBatch
    from x0ne_engine_b200.engine.generate import Row
    from x0ne_engine_b200.sampling import SamplingParams
    pk = peaks()
    K, W, B, T = args.steps, max(args.warmup, 8), args.batch, args.prefill_tokens
    ctx = T + K + W + 64
    layers = args.layers or 8
    vocab = 32768
    rows_out = []
    other = {"retuvik": "tenetar", "barorax": "retuvik"}.get(args.design, "qwen3")
    for name in args.sizes.split(","):
        size = DESIGN_SIZES[name]
        for design, cfg in zip((args.design, other), design_configs(size, layers, vocab, args.chunk, args.design)):
            model = x.Model.random(cfg, seed=0, dtype="bfloat16", max_batch=B, max_ctx=ctx, max_step_tokens=max(T, 64))
            eng = model.engine
            ids = synthetic_ids(T, vocab, 20261104)
            times = []
            for i in range(W + 3):
                slot = eng.new_sequence(T)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                s.record()
                eng.step([slot], [ids])
                e.record()
                torch.cuda.synchronize()
                if i >= W:
                    times.append(s.elapsed_time(e))
                eng.free_sequence(slot)
            pre_ms = statistics.median(times)
            rows = [Row(i, synthetic_ids(T, vocab, 0x0C0E5EED + i), SamplingParams(max_tokens=ctx), ctx - T, i) for i in range(B)]
            runner = DeviceBatch(eng, B, cuda_graph=True)
            runner.run_ahead = False
            try:
                runner.start(rows)
                live = list(range(B))
                for _ in range(W):
                    runner.step(live)
                g = runner.last_graph
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                s.record()
                for _ in range(K):
                    g.replay()
                e.record()
                torch.cuda.synchronize()
                dec_ms = s.elapsed_time(e) / K
                for sl in runner.slots:
                    eng.cache.lengths[sl] += K
                launches = runner.launches_per_step
            finally:
                runner.close()
            weight_bytes, kv_per_tok = eng.model.step_weight_bytes(), eng.cache.bytes_per_token()
            # fixed-size states (a recurrent layer's matrices) are read and written once per sequence and step
            state_bytes = sum(t[0].numel() * 4 for t in {id(t): t for t in eng.cache.states.values()}.values())
            step_bytes = weight_bytes + B * (T + W + K / 2.0) * kv_per_tok + 2.0 * B * state_bytes
            rows_out.append({"size": name, "design": design, "layers": layers, "prefill_tokens": T, "prefill_ms": pre_ms,
                             "prefill_tok_s": T / (pre_ms / 1e3), "decode_batch": B, "decode_ms_per_step": dec_ms,
                             "decode_tok_s": B / (dec_ms / 1e3), "decode_bytes_per_step": step_bytes,
                             "decode_frac_of_hbm": step_bytes / (dec_ms / 1e3) / 1e9 / pk["hbm_gbs"],
                             "launches_per_decode_step": launches, "cache_bytes_per_token": kv_per_tok,
                             "state_bytes_per_sequence": state_bytes})
            print(f"[bench] {name} {design}: prefill {T} tokens {pre_ms:.2f} ms, decode b{B} {dec_ms:.3f} ms/step "
                  f"({rows_out[-1]['decode_frac_of_hbm']:.2f} of {pk['source']} copy bandwidth)", file=sys.stderr, flush=True)
            del runner, model, eng
            torch.cuda.empty_cache()
    print(json.dumps({"metric": f"prefill and decode tokens/s of {args.design.capitalize()} beside {other.capitalize()} at equal sizes (random bf16 weights)",
                      "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "dtype": "bf16", "data": "synthetic",
                      "impl": "ours", "chunk": args.chunk, "peaks": pk, "rows": rows_out}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the 36 of Qwen3-8B")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--design", default=None, choices=["rovurax", "tenetar", "retuvik", "barorax"],
                    help="instead of the default workload: this design beside Qwen3 (retuvik: beside Tenetar; barorax: beside Retuvik) "
                         "at equal sizes (prefill and decode)")
    ap.add_argument("--sizes", default="1.7b,8b", help="with --design: which of " + ", ".join(DESIGN_SIZES))
    ap.add_argument("--chunk", type=int, default=1024,
                    help="with --design: positions per chunk of the masked attention (rovurax, barorax) or of the sliding window (tenetar, retuvik)")
    args = ap.parse_args()
    if args.design is not None and args.impl == "ours" and args.gpus == 1:
        return design_bench(args)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace with no Python project (pip: neither setup.py nor "
                          "pyproject.toml) and this image has no cargo or rustc"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    # The prompts' pass runs the GPU into its power cap; for some 60 ms afterwards (about 14 decode steps
    # of this size) the SM clock is still below where decoding settles, and a step takes 4.5 ms instead
    # of 3.8 (the per-token gaps of the end-to-end run below show it).  The timed steps are the settled
    # rate, so at least 16 untimed steps come first; the number really run is the one reported.
    if args.warmup < 16:
        args.warmup = 16

    import torch

    import x0ne_engine_b200 as x
    from x0ne_engine_b200.engine.decode import DeviceBatch
    from x0ne_engine_b200.engine.generate import Row
    from x0ne_engine_b200.sampling import SamplingParams

    full_layers = 36
    layers = args.layers or full_layers
    cfg = x.Qwen3Config(hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers,
                        num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                        max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0,
                        tie_word_embeddings=False, dtype="bfloat16")
    pk = peaks()
    K, W, B, ctx = args.steps, args.warmup, args.batch, args.context
    mean_ctx = args.prefill_tokens + (ctx - args.prefill_tokens) // 2
    prompt_len = max(1, min(ctx - K - W - 1, mean_ctx - K // 2 - W))
    max_b = B if args.no_points else max(B, 64)
    t0 = time.time()
    model = x.Model.random(cfg, seed=0, dtype="bfloat16", max_batch=max_b, max_ctx=ctx, max_step_tokens=8192)
    eng = model.engine
    torch.cuda.synchronize()
    load_s = time.time() - t0
    print(f"[bench] model ready in {load_s:.1f} s: {eng.describe()}", file=sys.stderr, flush=True)

    weight_bytes = eng.model.step_weight_bytes()
    kv_per_tok = eng.cache.bytes_per_token()

    def decode_run(batch, steps, warmup, plen, with_clocks=False):
        """Device-timed: `steps` graph replays after `warmup` untimed ones."""
        rows = [Row(i, synthetic_ids(plen, cfg.vocab_size, 0x0C0E5EED + i), SamplingParams(max_tokens=ctx), ctx - plen, i)
                for i in range(batch)]
        runner = DeviceBatch(eng, batch, cuda_graph=True)
        runner.run_ahead = False        # the timed replays below are counted one by one
        try:
            runner.start(rows)
            live = list(range(batch))
            for _ in range(warmup):
                runner.step(live)
            g = runner.last_graph
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sampler = ClockSampler() if with_clocks else None
            if sampler:
                sampler.__enter__()
            torch.cuda.synchronize()
            start.record()
            for _ in range(steps):
                g.replay()
            end.record()
            torch.cuda.synchronize()
            if sampler:
                sampler.__exit__()
            ms = start.elapsed_time(end)
            first_ctx = plen + warmup + 1
            for s in runner.slots:
                eng.cache.lengths[s] += steps
            mean_keys = first_ctx + (steps - 1) / 2.0
            return dict(ms=ms, tok_s=batch * steps / (ms / 1e3), ctx_first=first_ctx, ctx_last=first_ctx + steps - 1,
                        bytes_per_step=weight_bytes + batch * mean_keys * kv_per_tok,
                        clocks=sampler.summary() if sampler else None, launches_per_step=runner.launches_per_step)
        finally:
            runner.close()

    # ---- prefill: one prompt of T tokens through the step function, logits at its last place
    def time_prompt(n_tokens):
        ids = synthetic_ids(n_tokens, cfg.vocab_size, 20261104)
        times = []
        for i in range(W + 3):
            slot = eng.new_sequence(n_tokens)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            eng.step([slot], [ids])
            e.record()
            torch.cuda.synchronize()
            if i >= W:
                times.append(s.elapsed_time(e))
            eng.free_sequence(slot)
        return statistics.median(times)

    T = args.prefill_tokens
    pre = time_prompt(T)
    flops = (2.0 * T * cfg.linear_params_per_layer * layers + 2.0 * cfg.vocab_size * cfg.hidden_size
             + 4.0 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2 * layers)
    prefill = {"value": T / (pre / 1e3), "tokens": T, "ms": pre,
               "frac": flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12)}
    print(f"[bench] prefill {T} tokens: {pre:.2f} ms", file=sys.stderr, flush=True)

    # ---- the headline: decode at the asked batch
    main_run = decode_run(B, K, W, prompt_len, with_clocks=True)
    print(f"[bench] decode b{B}: {main_run['tok_s']:.0f} tok/s, {main_run['ms'] / K:.3f} ms/step", file=sys.stderr, flush=True)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            k = min(K, 128)
            r = decode_run(b, k, W, max(1, mean_ctx - k // 2 - W))
            points[f"decode_b{b}"] = r["tok_s"]
            print(f"[bench] decode b{b}: {r['tok_s']:.0f} tok/s, {r['ms'] / k:.3f} ms/step", file=sys.stderr, flush=True)
        # a short prompt through the step function (its launches come from a graph after the second pass)
        points["prompt_t128_ms"] = time_prompt(128)
        points["prompt_t512_ms"] = time_prompt(512)

    # ---- end to end through the Python entry point: host token lists in, host token lists out
    e2e = None
    if not args.no_e2e:
        from x0ne_engine_b200.engine.generate import GenerationStats, percentiles
        prompts = [synthetic_ids(prompt_len, cfg.vocab_size, 0x0C0E5EED + i) for i in range(B)]
        n_new = K + W + 1

        def through_generate(n_tokens):
            model._generator.stats = st = GenerationStats()
            out = model.generate(prompts, max_tokens=n_tokens, stop_token_ids=())
            return out.tokens, st

        through_generate(4)                                                   # warms the batch's graph
        first, _ = through_generate(n_new)
        tokens, st = through_generate(n_new)
        if tokens != first:
            # two greedy runs of the same prompts must give the same tokens, or the timing is of
            # something else than generation (x0ne-core/oracle/examples/core-perf.rs:85-89)
            print("bench.py: two runs of the same greedy generation gave different tokens; no number is reported",
                  file=sys.stderr)
            return 3
        gaps = st.token_gaps
        print(f"[bench] e2e: {st.decode_tokens / st.decode_seconds:.0f} tok/s over {len(gaps)} steps; gaps ms: first "
              f"{[round(g * 1e3, 2) for g in gaps[:4]]} p50 {percentiles(gaps)['p50'] * 1e3:.3f} max {max(gaps) * 1e3:.3f}",
              file=sys.stderr, flush=True)
        e2e = {"value": st.decode_tokens / st.decode_seconds, "unit": "tokens/s",
               "h2d_bytes_per_step": round(B * prompt_len * 4 / n_new + 0.0, 1), "d2h_bytes_per_step": 4 * (B + 1),
               "steps": len(gaps), "token_gap_ms": {k: (v * 1e3 if k != "n" else v) for k, v in percentiles(gaps).items()},
               "note": "decode rate inside Model.generate: (tokens after the first) / (time from the first token's "
                       "arrival to the last one's); prompt ids go up once per batch, each step reads back one int32 "
                       "per live sequence and one status word"}
        long_steps = 192
        if K < long_steps and prompt_len + long_steps + 1 <= ctx:
            _, st = through_generate(long_steps + 1)
            e2e["long"] = {"value": st.decode_tokens / st.decode_seconds, "steps": len(st.token_gaps)}

    achieved = main_run["bytes_per_step"] / (main_run["ms"] / K / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {B} (Qwen3-8B shape, random bf16 weights), {ctx:,}-token context",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": main_run["ms"] / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_of_model": full_layers, "hidden": 4096,
                   "q_heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": 151936,
                   "global_batch": B, "seq_len": ctx, "prompt_len": prompt_len, "ctx_first_step": main_run["ctx_first"],
                   "ctx_last_step": main_run["ctx_last"], "parallelism": "single GPU", "decode": "cuda graph",
                   "l2": "each step reads all weights (>> L2)", "weights": "random N(0,0.02), norms 1", "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "e2e": e2e,
        "gpu_launches": main_run["launches_per_step"] * K,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
