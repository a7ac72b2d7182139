#!/usr/bin/env python3
"""Headline measurement: GPT-2 124M, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--dtype bf16|fp32] [--impl reference]

A "step" is one decode step of a batch of 8 sequences near the model's full context.  The
line printed is one JSON object: ``value`` = decoded tokens per second on the device (CUDA
events around exactly K captured steps), ``e2e`` = the same through the Python entry point
``Engine.generate`` with host tokens in and out, plus

* ``prefill``: 2,048 tokens as 2 x 1024 in one step: median and best of the replayed step, the
  time of a step whose lengths were never seen before (inside a shape class that has a
  recording, and in a class seen for the very first time), flop fraction of the peak;
* ``roofline``: bytes a decode step has to read / its time, against the measured copy bandwidth;
* ``points``: decode tokens per second at batch 1, 8 and 64 and contexts 128, 512 and ~1014;
* ``fp32``: the headline step and the prefill in true 32-bit (no tensor cores);
* ``workloads``: GPT-2 medium (8 unequal prompts, 256 steps) and GPT-2 XL (64 prompts of 128
  tokens decoded to 1024) through ``Engine.generate``: time to the first token, decode and
  end-to-end tokens per second, bytes per step and their fraction of the copy bandwidth;
* ``clocks`` and ``gpu_launches``.

Every decode step reads all weights (247 MB in bf16) and the cache of the live requests,
far more than the 126 MB L2, so no L2 flush is needed between timed steps.  Model sizes come
from the package's presets (config files), none stands here.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = "gpt2"                      # preset names (nimbus_infer_rs_b200/config/presets/)
OTHER_MODELS = ("gpt2-medium", "gpt2-xl")
CONTEXT = 1024
BATCH = 8
PREFILL_TOKENS = 2048
REFERENCE_DECODE_TOK_S = 35.1      # the reference's published CPU figure (README.md:25), batch 1
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
FP32_LANES_PER_SM = 128            # FMA lanes of an SM: nominal fp32 peak = SMs x lanes x 2 x clock


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


def _timed_step(engine, entries):
    import torch
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    engine.step(entries)
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1)


def time_prefill(engine, n_seqs, length, reps=7):
    """One step of `n_seqs` prompts of `length` tokens, logits of each last token.  Returns
    milliseconds: median and best of `reps` replays of the recorded step (after two runs that
    warm up and record it), and the median over `reps` steps whose lengths were never seen
    before (a few tokens shorter each time: the step's shape class has a recording, its
    lengths are new)."""
    V = engine.spec.vocab_size

    def run(lengths, seed):
        slots = [engine.alloc_slot() for _ in lengths]
        prompts = [prompts_for(1, n, V, seed + i)[0] for i, n in enumerate(lengths)]
        ms = _timed_step(engine, [(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        for s in slots:
            engine.free_slot(s)
        return ms

    run([length // 2 + 3] * n_seqs, 99)                # another class: loads the kernels
    first_sight = run([length] * n_seqs, 100)          # plain launches: the class is new
    run([length] * n_seqs, 101)                        # recorded here
    replays = [run([length] * n_seqs, 102 + r) for r in range(reps)]
    fresh = [run([length - 1 - 2 * r - i for i in range(n_seqs)], 200 + r) for r in range(reps)]
    return {"median": statistics.median(replays), "best": min(replays),
            "fresh_lengths": statistics.median(fresh), "first_sight": first_sight}


def model_flops_prefill(cfg, n_seqs, length):
    d, m, L, V = cfg.d_model, cfg.d_mlp, cfg.n_layers, cfg.vocab_size
    hq, hk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    T = n_seqs * length
    linear = 2 * T * L * (d * (hq + 2 * hk) + hq * d + 2 * d * m)
    attn = n_seqs * L * 2 * 2 * cfg.n_heads * cfg.head_dim * (length * (length + 1) // 2)
    head = 2 * n_seqs * d * V
    return linear + attn + head


def kv_bytes_per_token(cfg, elt):
    return 2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * elt


def fp32_peak_tflops(clock_mhz):
    """Nominal: every SM retires `FP32_LANES_PER_SM` fused multiply-adds a clock."""
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    return sms * FP32_LANES_PER_SM * 2 * clock_mhz * 1e6 / 1e12


def run_workload(engine, cfg, prompt_lens, n_new, hbm_gbs, windows=()):
    """A request list through Engine.generate (greedy, host tokens in and out every step).
    Timed on the host clock, the device waited for at each stamp: the prompts' step up to the
    first tokens, then the decode steps.  `windows`: contexts at which the decode rate of the
    32 steps around (or before) them is reported as well."""
    import torch
    from nimbus_infer_rs_b200 import SamplingParams
    V = engine.spec.vocab_size
    prompts = [prompts_for(1, n, V, 900 + i)[0] for i, n in enumerate(prompt_lens)]
    lead = min(range(len(prompts)), key=lambda i: len(prompts[i]))   # lives longest
    stamps = {}

    def on_token(i, tok, step):
        if i == lead:
            torch.cuda.synchronize()
            stamps[step] = time.perf_counter()

    torch.cuda.synchronize()
    t_start = time.perf_counter()
    out = engine.generate(prompts, SamplingParams(max_new_tokens=n_new, temperature=0.0),
                          on_token=on_token, max_batch=len(prompts))
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    n_out = [len(o) for o in out]
    decoded = sum(n_out) - len(prompts)              # tokens that came from decode steps
    last = max(stamps)
    decode_s = stamps[last] - stamps[0]
    # bytes the decode steps had to read: every weight once a step, and the cache of each live
    # sequence (a sequence with n tokens out ran n - 1 decode steps)
    kvb = kv_bytes_per_token(cfg, 2)
    n_steps = max(n_out) - 1
    nbytes = n_steps * engine.model.weight_bytes()
    for plen, n in zip(prompt_lens, n_out):
        nbytes += kvb * sum(plen + t + 1 for t in range(n - 1))
    res = {"prompt_tokens": sum(prompt_lens), "prefill_ms": round((stamps[0] - t_start) * 1e3, 2),
           "decode_steps": n_steps, "decoded_tokens": decoded,
           "decode_tok_s": round(decoded / decode_s, 1),
           "e2e_tok_s": round(sum(n_out) / (t_end - t_start), 1),
           "decode_gb_per_step": round(nbytes / n_steps / 1e9, 3),
           "hbm_frac": round(nbytes / decode_s / 1e9 / hbm_gbs, 4)}
    for c in windows:
        hi = min(c - prompt_lens[lead], last)        # the step that brings the context to c
        lo = hi - 32
        if lo < 1:
            continue
        dt = stamps[hi] - stamps[lo]
        step_bytes = engine.model.weight_bytes() + len(prompts) * (c - 16) * kvb
        res[f"c{c}"] = {"tok_s": round(len(prompts) * 32 / dt, 1), "ms_per_step": round(dt / 32 * 1e3, 3),
                        "hbm_frac": round(step_bytes / (dt / 32) / 1e9 / hbm_gbs, 4)}
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--no-points", action="store_true", help="skip the other batch sizes and contexts")
    ap.add_argument("--no-fp32", action="store_true", help="skip the 32-bit figures")
    ap.add_argument("--no-workloads", action="store_true", help="skip the medium and XL workloads")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one phase only (for profiling); prints a reduced line")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of the decode step")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only decode: context the steps end at")
    ap.add_argument("--model", default=MODEL, choices=[MODEL, *OTHER_MODELS],
                    help="layer sizes (a preset); other than the default only with --only")
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
    from nimbus_infer_rs_b200.config import load_preset

    peaks = load_peaks()
    dtype = "bfloat16" if args.dtype == "bf16" else "float32"
    if args.model != MODEL and args.only == "all":
        print("--model other than gpt2 needs --only decode or --only prefill")
        return 2
    _, cfg, _ = load_preset(args.model)
    cache_tokens = max(64, args.batch if args.only == "decode" else 64) * CONTEXT + 64
    engine = Engine.random(args.model, seed=0, dtype=dtype, cache_tokens=cache_tokens)
    elt = 2 if dtype == "bfloat16" else 4

    if args.only == "prefill":
        pre = time_prefill(engine, PREFILL_TOKENS // CONTEXT, CONTEXT, reps=8)
        flops = model_flops_prefill(cfg, PREFILL_TOKENS // CONTEXT, CONTEXT)
        print(json.dumps({"only": "prefill", "model": args.model, "dtype": args.dtype,
                          "ms": round(pre["median"], 4), "ms_best": round(pre["best"], 4),
                          "fresh_lengths_ms": round(pre["fresh_lengths"], 4),
                          "first_sight_ms": round(pre["first_sight"], 4),
                          "tokens_per_s": round(PREFILL_TOKENS / (pre["median"] * 1e-3), 1),
                          "tflops": round(flops / (pre["median"] * 1e-3) / 1e12, 1)}))
        return 0
    if args.only == "decode":
        ms, launches, mean_ctx = time_decode(engine, args.batch, args.context, args.steps, args.warmup)
        nbytes = engine.model.weight_bytes() + args.batch * mean_ctx * kv_bytes_per_token(cfg, elt)
        print(json.dumps({"only": "decode", "model": args.model, "dtype": args.dtype,
                          "batch": args.batch, "context": args.context, "ms_per_step": round(ms, 4),
                          "tokens_per_s": round(args.batch * 1000.0 / ms, 1),
                          "gb_per_s": round(nbytes / (ms * 1e-3) / 1e9, 1),
                          "gpu_launches": launches}))
        return 0

    n_pre = PREFILL_TOKENS // CONTEXT
    pre_flops = model_flops_prefill(cfg, n_pre, CONTEXT)
    # clocks and throttle reasons are sampled while all of the measurements below run
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = time_decode(engine, BATCH, CONTEXT, args.steps, args.warmup)
        value = BATCH * 1000.0 / ms
        step_bytes = engine.model.weight_bytes() + BATCH * mean_ctx * kv_bytes_per_token(cfg, elt)
        achieved = step_bytes / (ms * 1e-3) / 1e9

        e2e = time_e2e(engine, BATCH, CONTEXT, args.steps, args.warmup)

        pre = time_prefill(engine, n_pre, CONTEXT)
        time.sleep(0.12)
    clock_summary = clocks.summary()
    fp32_peak = fp32_peak_tflops(clock_summary.get("sm_max_mhz") or 1965)
    peak_flops = peaks["bf16_tflops"] * 1e12 if dtype == "bfloat16" else fp32_peak * 1e12
    prefill = {"value": round(PREFILL_TOKENS / (pre["median"] * 1e-3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(pre["median"], 4),
               "frac": round(pre_flops / (pre["median"] * 1e-3) / peak_flops, 4),
               "ms_best": round(pre["best"], 4), "fresh_lengths_ms": round(pre["fresh_lengths"], 4),
               "first_sight_ms": round(pre["first_sight"], 4)}
    # the other batch sizes and contexts run without the clock sampler beside them: a step at
    # batch 1 is short enough for the sampler's process to show in it
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _ = time_decode(engine, b, CONTEXT, args.steps, args.warmup, seed=b)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
        for c in (128, 512):
            for b in (1, BATCH, 64):
                st = min(args.steps, c - args.warmup - 8)
                pms, _, _ = time_decode(engine, b, c, st, args.warmup, seed=b + c)
                points[f"decode_b{b}_c{c}"] = round(b * 1000.0 / pms, 1)

    fp32 = None
    if not args.no_fp32 and dtype == "bfloat16":
        del engine
        torch.cuda.empty_cache()
        e32 = Engine.random(MODEL, seed=0, dtype="float32", cache_tokens=16 * CONTEXT + 64)
        ms32, _, ctx32 = time_decode(e32, BATCH, CONTEXT, 16, 3)
        b32 = e32.model.weight_bytes() + BATCH * ctx32 * kv_bytes_per_token(cfg, 4)
        p32 = time_prefill(e32, n_pre, CONTEXT, reps=3)
        fp32 = {"decode_b8_tok_s": round(BATCH * 1000.0 / ms32, 1), "decode_ms_per_step": round(ms32, 4),
                "decode_hbm_frac": round(b32 / (ms32 * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                "prefill_ms": round(p32["median"], 3),
                "prefill_tok_s": round(PREFILL_TOKENS / (p32["median"] * 1e-3), 1),
                "prefill_frac": round(pre_flops / (p32["median"] * 1e-3) / (fp32_peak * 1e12), 4),
                "peak_tflops": round(fp32_peak, 1)}
        del e32
        engine = None

    workloads = {}
    if not args.no_workloads and dtype == "bfloat16":
        engine = None
        torch.cuda.empty_cache()
        # GPT-2 medium: 8 unequal prompts, 256 decode steps; a sequence that reaches the end of
        # the context stops earlier
        _, mcfg, _ = load_preset("gpt2-medium")
        em = Engine.random("gpt2-medium", seed=0, dtype="bfloat16", cache_tokens=8 * CONTEXT + 64)
        lens = [32, 160, 288, 416, 544, 672, 800, 1000]
        # (a run of another, larger shape class first: it loads the kernels and leaves the
        # allocator with blocks that are large enough; the timed run is then the first sight of
        # its own shape class, as a fresh request list is)
        run_workload(em, mcfg, [min(l + 40, 1016) for l in lens], 4, peaks["hbm_gbs"])
        workloads["medium"] = run_workload(em, mcfg, lens, 257, peaks["hbm_gbs"])
        del em
        torch.cuda.empty_cache()
        # GPT-2 XL: 64 prompts of 128 tokens, decoded to the end of the context
        _, xcfg, _ = load_preset("gpt2-xl")
        ex = Engine.random("gpt2-xl", seed=0, dtype="bfloat16", cache_tokens=64 * CONTEXT + 64)
        run_workload(ex, xcfg, [96] * 64, 4, peaks["hbm_gbs"])
        workloads["xl"] = run_workload(ex, xcfg, [128] * 64, CONTEXT - 128, peaks["hbm_gbs"],
                                       windows=(256, 512, 1024))
        del ex

    b1 = points.get("decode_b1")
    out = {
        "metric": "decode tok/s, GPT-2 124M, batch 8, context 1024", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(b1 / REFERENCE_DECODE_TOK_S, 1) if b1 else None, "dtype": args.dtype,
        "data": "synthetic: random-init weights N(0,0.02), uniform random token ids",
        "config": {"model": "gpt2-124M", "n_layer": cfg.n_layers, "n_layer_model": 12,
                   "n_embd": cfg.d_model, "n_head": cfg.n_heads, "head_dim": cfg.head_dim,
                   "n_inner": cfg.d_mlp, "vocab_size": cfg.vocab_size,
                   "n_positions": cfg.max_seq_len, "tied_head": cfg.tie_embeddings,
                   "global_batch": BATCH, "seq_len": CONTEXT,
                   "decode_context_mean": round(mean_ctx, 1), "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights + cache read per step)",
                   "peaks": peaks["source"] + "; fp32: nominal SMs x 128 FMA lanes x 2 x max clock",
                   "baseline": "vs_baseline = batch-1 decode / the reference's CPU batch-1 decode, "
                               "35.1 tok/s (README.md:25)",
                   "medium": "gpt2-medium L24 d1024 H16 m4096: 8 prompts of 32..1000 tokens, 256 steps",
                   "xl": "gpt2-xl L48 d1600 H25 m6400: 64 prompts of 128 tokens decoded to 1024"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": BATCH * 4, "d2h_bytes_per_step": BATCH * 4},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "fp32": fp32,
        "workloads": workloads,
        "clocks": clock_summary,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
