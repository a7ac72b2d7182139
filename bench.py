#!/usr/bin/env python3
"""Headline measurement: GPT-2 124M, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--dtype bf16|fp32] [--impl reference]

A "step" is one decode step of a batch of 8 sequences near the model's full context.  The
line printed is one JSON object: ``value`` = decoded tokens per second on the device (CUDA
events around exactly K captured steps), ``e2e`` = the same through the Python entry point
``Engine.generate`` with host tokens in and out, plus ``prefill`` (2,048 tokens as 2 x 1024),
``roofline`` (bytes a decode step has to read / its time, against the measured copy
bandwidth), ``points`` (decode at batch 1 and 64), ``clocks`` and ``gpu_launches``.
Every decode step reads all weights (247 MB in bf16) and the cache of the live requests,
far more than the 126 MB L2, so no L2 flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# GPT-2 small, 124M parameters
MODEL = {"model_type": "gpt2", "vocab_size": 50257, "n_positions": 1024, "n_embd": 768,
         "n_layer": 12, "n_head": 12, "n_inner": 3072, "activation_function": "gelu_new",
         "layer_norm_epsilon": 1e-5, "tie_word_embeddings": True}
# the larger members of the family, for --model (side measurements, not the headline)
OTHER_MODELS = {
    "gpt2-medium": dict(MODEL, n_embd=1024, n_layer=24, n_head=16, n_inner=4096),
    "gpt2-xl": dict(MODEL, n_embd=1600, n_layer=48, n_head=25, n_inner=6400),
}
CONTEXT = 1024
BATCH = 8
PREFILL_TOKENS = 2048
REFERENCE_DECODE_TOK_S = 35.1      # the reference's published CPU figure (README.md:25), batch 1
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(s[0]))
                mx.append(int(s[1]))
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def prompts_for(batch, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(batch)]


def time_decode(engine, batch, context, steps, warmup, seed=0):
    """Device time of exactly `steps` decode steps of `batch` sequences whose contexts end at
    `context`; returns (ms per step, kernel launches in the timed region, mean context)."""
    import torch
    from nimbus_infer_rs_b200.engine.decode import DecodeSession
    start = context - steps - warmup
    assert start >= 1, "steps + warmup must stay below the context length"
    V = engine.spec.vocab_size
    slots = [engine.alloc_slot() for _ in range(batch)]
    prompts = prompts_for(batch, start, V, seed)
    # prefill in chunks of at most 16 sequences to bound activation memory
    for i in range(0, batch, 16):
        engine.step([(s, p, []) for s, p in zip(slots[i:i + 16], prompts[i:i + 16])])
    session = DecodeSession(engine, slots, [p[-1] for p in prompts])
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    launches0 = engine.ops.launches
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        session.step()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = engine.ops.launches - launches0
    for s in slots:
        engine.free_slot(s)
    mean_ctx = start + warmup + (steps - 1) / 2.0 + 1
    return ms, launches, mean_ctx


def time_e2e(engine, batch, context, steps, warmup, seed=1):
    """Decode tokens per second through Engine.generate: per step the host hands the step's
    state over and reads the sampled tokens back.  Timed from the first sampled token of the
    timed window to the last, on the host clock."""
    import torch
    from nimbus_infer_rs_b200 import SamplingParams
    start = context - steps - warmup - 1
    prompts = prompts_for(batch, start, engine.spec.vocab_size, seed)
    stamps = {}

    def on_token(i, tok, step):
        if i == batch - 1 and step in (warmup, warmup + steps):
            torch.cuda.synchronize()
            stamps[step] = time.perf_counter()

    engine.generate(prompts, SamplingParams(max_new_tokens=warmup + steps + 1, temperature=0.0),
                    on_token=on_token, max_batch=batch)
    dt = stamps[warmup + steps] - stamps[warmup]
    return batch * steps / dt


def time_prefill(engine, n_seqs, length, reps=5):
    import torch
    V = engine.spec.vocab_size
    best = None
    for r in range(reps + 1):
        slots = [engine.alloc_slot() for _ in range(n_seqs)]
        prompts = prompts_for(n_seqs, length, V, 100 + r)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        engine.step([(s, p, [length - 1]) for s, p in zip(slots, prompts)])
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1)
        for s in slots:
            engine.free_slot(s)
        if r > 0:   # the first run warms up
            best = ms if best is None else min(best, ms)
    return best


def model_flops_prefill(cfg, n_seqs, length):
    d, m, L, V = cfg.d_model, cfg.d_mlp, cfg.n_layers, cfg.vocab_size
    hq, hk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    T = n_seqs * length
    linear = 2 * T * L * (d * (hq + 2 * hk) + hq * d + 2 * d * m)
    attn = n_seqs * L * 2 * 2 * cfg.n_heads * cfg.head_dim * (length * (length + 1) // 2)
    head = 2 * n_seqs * d * V
    return linear + attn + head


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one phase only (for profiling); prints a reduced line")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of the decode step")
    ap.add_argument("--model", default="gpt2-124M", choices=["gpt2-124M", *OTHER_MODELS],
                    help="layer sizes; other than the default only with --only")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (Cargo.toml, no Python package); there is "
                          "no Rust toolchain on this box, so it cannot be built or installed"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (asked for {args.gpus}): this library has no "
              "multi-GPU path")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from nimbus_infer_rs_b200 import Engine
    from nimbus_infer_rs_b200.config import GPT2Config

    peaks = load_peaks()
    dtype = "bfloat16" if args.dtype == "bf16" else "float32"
    if args.model != "gpt2-124M" and args.only == "all":
        print("--model other than gpt2-124M needs --only decode or --only prefill")
        return 2
    cfg = GPT2Config.from_json(OTHER_MODELS.get(args.model, MODEL))
    cache_tokens = max(64, args.batch if args.only == "decode" else 64) * CONTEXT + 64
    engine = Engine.random(cfg, seed=0, dtype=dtype, cache_tokens=cache_tokens, std=0.02)
    elt = 2 if dtype == "bfloat16" else 4

    if args.only == "prefill":
        pre_ms = time_prefill(engine, PREFILL_TOKENS // CONTEXT, CONTEXT, reps=8)
        flops = model_flops_prefill(cfg, PREFILL_TOKENS // CONTEXT, CONTEXT)
        print(json.dumps({"only": "prefill", "model": args.model, "dtype": args.dtype,
                          "ms": round(pre_ms, 4),
                          "tokens_per_s": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1),
                          "tflops": round(flops / (pre_ms * 1e-3) / 1e12, 1)}))
        return 0
    if args.only == "decode":
        ms, launches, mean_ctx = time_decode(engine, args.batch, CONTEXT, args.steps, args.warmup)
        elt_ = 2 if dtype == "bfloat16" else 4
        nbytes = engine.model.weight_bytes() + args.batch * mean_ctx * (
            2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * elt_)
        print(json.dumps({"only": "decode", "model": args.model, "dtype": args.dtype,
                          "batch": args.batch, "ms_per_step": round(ms, 4),
                          "tokens_per_s": round(args.batch * 1000.0 / ms, 1),
                          "gb_per_s": round(nbytes / (ms * 1e-3) / 1e9, 1),
                          "gpu_launches": launches}))
        return 0

    # clocks and throttle reasons are sampled while all of the measurements below run
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = time_decode(engine, BATCH, CONTEXT, args.steps, args.warmup)
        value = BATCH * 1000.0 / ms
        kv_bytes_per_token = 2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * elt
        step_bytes = engine.model.weight_bytes() + BATCH * mean_ctx * kv_bytes_per_token
        achieved = step_bytes / (ms * 1e-3) / 1e9

        e2e = time_e2e(engine, BATCH, CONTEXT, args.steps, args.warmup)

        pre_ms = time_prefill(engine, PREFILL_TOKENS // CONTEXT, CONTEXT)
        pre_flops = model_flops_prefill(cfg, PREFILL_TOKENS // CONTEXT, CONTEXT)
        peak_flops = peaks["bf16_tflops"] * 1e12 if dtype == "bfloat16" else 80e12
        prefill = {"value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                   "ms": round(pre_ms, 4), "frac": round(pre_flops / (pre_ms * 1e-3) / peak_flops, 4)}

        time.sleep(0.12)
    clock_summary = clocks.summary()
    # the other batch sizes run without the clock sampler beside them: a step at batch 1 is
    # short enough for the sampler's process to show in it
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _ = time_decode(engine, b, CONTEXT, args.steps, args.warmup, seed=b)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)

    out = {
        "metric": "decode tok/s, GPT-2 124M, batch 8, context 1024", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / REFERENCE_DECODE_TOK_S, 1), "dtype": args.dtype,
        "data": "synthetic: random-init weights N(0,0.02), uniform random token ids",
        "config": {"model": "gpt2-124M", "n_layer": cfg.n_layers, "n_layer_model": 12,
                   "n_embd": cfg.d_model, "n_head": cfg.n_heads, "head_dim": cfg.head_dim,
                   "n_inner": cfg.d_mlp, "vocab_size": cfg.vocab_size,
                   "n_positions": cfg.max_seq_len, "tied_head": cfg.tie_embeddings,
                   "global_batch": BATCH, "seq_len": CONTEXT,
                   "decode_context_mean": round(mean_ctx, 1), "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights + cache read per step)",
                   "peaks": peaks["source"],
                   "baseline": "reference CPU decode 35.1 tok/s at batch 1 (README.md:25)"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": BATCH * 4, "d2h_bytes_per_step": BATCH * 4},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
