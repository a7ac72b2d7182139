"""Command line, in the manner of the reference's ``nimbus-rs`` (src/main.rs:19-59):

    python -m nimbus_infer_rs_b200 generate --model DIR --ids 1,2,3 [options]
    python -m nimbus_infer_rs_b200 bench    --model DIR [--prefill N] [--decode N] [--runs R]
    python -m nimbus_infer_rs_b200 logits   --model DIR --ids 1,2,3
    python -m nimbus_infer_rs_b200 inspect  --model DIR
    python -m nimbus_infer_rs_b200 random   --out DIR (--config CONFIG.json | --preset NAME) --seed S

Instead of ``--model DIR`` every command but ``random`` takes ``--random PRESET --seed-weights
S``: a model of a named size (``gpt2`` = the reference's defaults, src/config.rs:45-66;
``gpt2-medium``, ``gpt2-xl``, ``tiny-a``, ``tiny-b``) with seeded random weights, no file on disk.

Flag names, meanings and defaults follow the reference where it has them (``--model``,
``--ids``, ``--max-new-tokens`` 64, ``--temperature`` 0 = greedy, ``--top-k`` 0, ``--top-p``
1.0, ``--repetition-penalty`` 1.0, ``--seed``, ``--json``; ``--prefill`` 128, ``--decode`` 64,
``--runs`` 3).  Added: ``--dtype bfloat16|float32``, ``--stop ID,ID``, ``;`` between the id
lists of a batch, ``--batch``, ``--keep-stored-dtype`` / ``--cast-weights``.  There is no tokenizer, so ``--prompt TEXT`` is refused as the
reference refuses it for a checkpoint without one (src/engine.rs:245-251); ``--quant``
accepts only ``fp32``.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _parse_ids(text: str) -> list[list[int]]:
    """``1,2,3`` or several lists separated by ``;`` (src/main.rs:130-134 for one list)."""
    out = []
    for part in text.split(";"):
        part = part.strip()
        if not part:
            continue
        try:
            out.append([int(p.strip()) for p in part.split(",")])
        except ValueError:
            raise SystemExit(f"error: bad token id in {part!r}")
    if not out:
        raise SystemExit("error: pass --ids 1,2,3")
    return out


def _common(ap):
    ap.add_argument("--model", help="folder with config.json and the weight file")
    ap.add_argument("--random", metavar="PRESET",
                    help="instead of --model: a model of a named size with seeded random weights "
                         "(gpt2, gpt2-medium, gpt2-xl, tiny-a, tiny-b); nothing is read from disk")
    ap.add_argument("--seed-weights", type=int, default=0, help="seed of --random's weights")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--quant", default="fp32", help="only fp32 (no quantized weights here)")
    g = ap.add_mutually_exclusive_group()
    g.add_argument("--keep-stored-dtype", action="store_true",
                   help="bfloat16 runs: matrices stored in 32-bit stay so (and run on the fp32 "
                        "kernels) even when the file holds no bf16 matrix at all")
    g.add_argument("--cast-weights", action="store_true",
                   help="bfloat16 runs: round every matrix stored in 32-bit to bf16")


def _load(args, **kw):
    from . import Engine
    if args.quant not in ("fp32", "f32", "none"):
        raise SystemExit(f"error: quant mode {args.quant!r} is not built (expected fp32)")
    if (args.model is None) == (args.random is None):
        raise SystemExit("error: pass --model DIR or --random PRESET")
    if args.random is not None:
        return Engine.random(args.random, seed=args.seed_weights, dtype=args.dtype,
                             device=args.device, **kw)
    cast = True if args.cast_weights else (False if args.keep_stored_dtype else None)
    return Engine.load(args.model, dtype=args.dtype, device=args.device, cast_weights=cast, **kw)


def cmd_generate(args) -> int:
    from . import SamplingParams
    if args.prompt is not None:
        raise SystemExit("error: this checkpoint has no tokenizer; pass --ids instead")
    if args.ids is None:
        raise SystemExit("error: pass --prompt TEXT or --ids 1,2,3")
    prompts = _parse_ids(args.ids)
    engine = _load(args)
    params = SamplingParams(
        max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
        top_p=args.top_p, repetition_penalty=args.repetition_penalty, seed=args.seed,
        stop_tokens=[int(x) for x in args.stop.split(",")] if args.stop else [])
    on_token = None
    if args.stream:   # ids as they are produced (the reference streams text, src/main.rs:157-167)
        many = len(prompts) > 1

        def on_token(request, token, step):
            print(f"{request}:{token}" if many else token, end=" ", flush=True)
    t0 = time.perf_counter()
    out = engine.generate(prompts, params, on_token=on_token)
    dt = time.perf_counter() - t0
    if args.stream:
        print(flush=True)
    n = sum(len(o) for o in out)
    if args.json:
        if len(prompts) == 1:   # src/main.rs:176-182
            print(json.dumps({"prompt_tokens": len(prompts[0]), "generated_ids": out[0],
                              "text": str(out[0])}))
        else:
            print(json.dumps({"prompt_tokens": [len(p) for p in prompts], "generated_ids": out}))
    else:
        for o in out:
            print(o)
    print(f"[{n} tokens in {dt:.2f}s = {n / dt:.1f} tok/s]", file=sys.stderr)   # src/main.rs:186
    return 0


def cmd_logits(args) -> int:
    """The numerics probe of the reference (src/main.rs:285-312): the whole id list in one
    step, then argmax, first and last four logits and the sum of the last row."""
    import torch
    ids = _parse_ids(args.ids)[0]
    engine = _load(args, cache_tokens=max(64, len(ids)))
    slot = engine.alloc_slot()
    logits = engine.step([(slot, ids, [len(ids) - 1])])[0].cpu()
    engine.check_errors()
    engine.free_slot(slot)
    best = int(torch.argmax(logits))
    print(json.dumps({
        "argmax": best, "argmax_logit": round(float(logits[best]), 6),
        "head": [round(float(v), 6) for v in logits[:4]],
        "tail": [round(float(v), 6) for v in logits[-4:]],
        "sum": round(float(logits.double().sum()), 6)}))
    return 0


def cmd_inspect(args) -> int:
    print(json.dumps(_load(args).inspect()))
    return 0


def cmd_bench(args) -> int:
    """Prefill N tokens, then decode, timed as the reference times them (src/main.rs:191-269):
    synthetic prompt ids from the same hash, a warm-up, R runs; prefill includes the head of
    the last row; decode samples at temperature 1.0 from seed 1.  The best run is the one with
    the highest tokens per second (the reference's ``min`` keeps the slowest)."""
    import torch
    from . import SamplingParams
    from .sampling import BatchSampler, SequenceSampler
    engine = _load(args, cache_tokens=args.batch * (args.prefill + args.decode + 64))
    V = engine.spec.vocab_size
    prompt = [(i * 2654435761 + 12345) % (V - 8) + 8 for i in range(args.prefill)]  # :200-203
    prompts = [prompt] * args.batch
    engine.generate(prompts, SamplingParams(max_new_tokens=2))                        # :206
    best = {"prefill": 0.0, "decode": 0.0, "e2e": 0.0}
    last = []
    for _ in range(args.runs):
        params = SamplingParams(max_new_tokens=args.decode, seed=1)
        sampler = BatchSampler(params, engine.ops, engine.rt.device)
        seqs = [SequenceSampler(params, i) for i in range(args.batch)]
        slots = [engine.alloc_slot() for _ in prompts]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        logits = engine.step([(s, p, None) for s, p in zip(slots, prompts)])
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for step in range(args.decode):
            toks = sampler.sample(logits, seqs)
            if step == args.decode - 1:
                break
            logits = engine.step([(s, [t], None) for s, t in zip(slots, toks)])
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        for s in slots:
            engine.free_slot(s)
        last = seqs[0].generated
        best["prefill"] = max(best["prefill"], args.batch * args.prefill / (t1 - t0))
        best["decode"] = max(best["decode"], args.batch * args.decode / (t2 - t1))
        best["e2e"] = max(best["e2e"], args.batch * args.decode / (t2 - t0))
    info = engine.inspect()
    result = {
        "engine": "nimbus_infer_rs_b200", "quant": args.dtype, "model": info["name"],
        "params": info["n_params"], "batch": args.batch, "prefill_tokens": args.prefill,
        "decode_tokens": args.decode, "runs": args.runs,
        "prefill_tok_s": round(best["prefill"], 3), "decode_tok_s": round(best["decode"], 3),
        "e2e_tok_s": round(best["e2e"], 3), "weight_mb": info["weight_mb"],
        "kv_cache_mb": info["kv_cache_mb"], "first_generated_ids": last[:8]}
    text = json.dumps(result, indent=2)
    print(text)
    if args.json:
        with open(args.json, "w") as f:
            f.write(text)
    return 0


def cmd_random(args) -> int:
    from .config import load_json, load_preset, resolve_architecture
    from .weights import write_random_model
    import torch
    if (args.config is None) == (args.preset is None):
        raise SystemExit("error: pass --config CONFIG.json or --preset NAME")
    if args.preset is not None:
        arch, cfg, opts = load_preset(args.preset)
    else:
        obj = load_json(args.config)
        arch = resolve_architecture(obj)
        cfg, opts = arch.config_cls.from_json(obj), {}
    if args.std is not None:
        opts["std"] = args.std
    if args.bias_std is not None:
        opts["bias_std"] = args.bias_std
    d = write_random_model(args.out, cfg, args.seed, **opts,
                           dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(json.dumps({"wrote": str(d), "n_params": cfg.n_params(opts.get("bias_std", 0.0) > 0)}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nimbus_infer_rs_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate")
    _common(g)
    g.add_argument("--prompt")
    g.add_argument("--ids")
    g.add_argument("--max-new-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--stop", default="")
    g.add_argument("--stream", action="store_true", help="print token ids as they are produced")
    g.add_argument("--json", action="store_true")
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("bench")
    _common(b)
    b.add_argument("--prefill", type=int, default=128)
    b.add_argument("--decode", type=int, default=64)
    b.add_argument("--runs", type=int, default=3)
    b.add_argument("--batch", type=int, default=1)
    b.add_argument("--json", default=None, metavar="PATH")
    b.set_defaults(fn=cmd_bench)

    l = sub.add_parser("logits")
    _common(l)
    l.add_argument("--ids", required=True)
    l.set_defaults(fn=cmd_logits)

    i = sub.add_parser("inspect")
    _common(i)
    i.set_defaults(fn=cmd_inspect)

    r = sub.add_parser("random")
    r.add_argument("--out", required=True)
    r.add_argument("--config", help="a config.json to take the sizes from")
    r.add_argument("--preset", help="or a named size: gpt2, gpt2-medium, gpt2-xl, tiny-a, tiny-b")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=None, help="spread of the matrices (0.02)")
    r.add_argument("--bias-std", type=float, default=None,
                   help="spread of the linear biases (0: none are written)")
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_random)

    args = ap.parse_args(argv)
    try:
        return args.fn(args)
    except (ValueError, FileNotFoundError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
