"""The engine: a loaded model, its cache, the step function and the generation loop.

Reference analogue: ``Engine`` (src/engine.rs:44-48,71-239,255-293) with ``Model::
forward_hidden`` / ``logits_last`` (src/model.rs:271-325) as its step.  There one call runs
one sequence from the cache's single position; here ``step`` runs a batch of sequences, each
from its own cached length, and returns logits at the rows asked for.
"""
from __future__ import annotations

from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache import SequenceCache
from ..config.registry import get_architecture, load_config
from ..csrc import ops as ops_mod
from ..sampling import BatchSampler, SamplingParams, SequenceSampler
from ..weights.loader import find_weight_file, load_params
from ..weights.safetensors_io import SafeTensorsFile
from .batch import pack_step
from .context import StepContext
from .generate import plan_batches, run_batch, token_budget
from .model import PRECISIONS, Model, Runtime
from .step_graphs import StepGraphs, q_bound, row_padding


class Engine:
    def __init__(self, model: Model, config, *, cache_tokens: int | None = None,
                 n_slots: int | None = None):
        self.model = model
        self.spec = model.spec
        self.config = config
        self.rt = model.rt
        self.ops = ops_mod.backend()
        self.graph_safe = model.graph_safe()
        if cache_tokens is None:
            cache_tokens = 8 * self.spec.max_seq_len
        kv_req, st_req = model.storage_requests()
        for entry in range(len(model.run_order)):
            model.kv_source(entry)          # a bad cache_from fails here, not in a step
        self.cache = SequenceCache(kv_req, st_req, cache_tokens=cache_tokens,
                                   max_seq_len=self.spec.max_seq_len, dtype=self.rt.act_dtype,
                                   device=self.rt.device, n_slots=n_slots)
        # steps of a shape that comes again are replayed as CUDA graphs (``step_graphs = None``
        # keeps every step on plain launches)
        self.step_graphs = StepGraphs(self) if (
            self.graph_safe and self.rt.device.type == "cuda") else None
        # buffers and recorded steps of finished decode sessions, by batch size and sampling mode
        self.decode_states: dict = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def load(cls, model_dir: str | Path, dtype: str = "bfloat16", device: str = "cuda:0", *,
             cache_tokens: int | None = None, n_slots: int | None = None,
             cast_weights: bool | None = None) -> "Engine":
        """Load ``config.json`` and the weight file of ``model_dir``.  ``dtype``: ``bfloat16``
        (the serving precision) or ``float32`` (everything in true 32-bit).  ``cast_weights``
        (bfloat16 runs): ``True`` rounds matrices stored in 32-bit to bf16, ``False`` keeps
        them as stored, ``None`` rounds them only if the file holds no bf16 matrix at all."""
        if dtype not in PRECISIONS:
            raise ValueError(f"dtype must be one of {sorted(PRECISIONS)}, got {dtype!r}")
        arch, config = load_config(model_dir)
        rt = Runtime(torch.device(device), PRECISIONS[dtype])
        spec = arch.build_spec(config)
        model = Model(spec, rt)
        with SafeTensorsFile(find_weight_file(model_dir)) as f:
            plan = arch.weight_plan(config, spec, set(f.names()))
            params = load_params(model.param_specs(), plan, f, precision=rt.precision,
                                 device=rt.device, cast_weights=cast_weights)
        model.bind(params)
        return cls(model, config, cache_tokens=cache_tokens, n_slots=n_slots)

    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bfloat16", device: str = "cuda:0", *,
               cache_tokens: int | None = None, n_slots: int | None = None,
               **random_options) -> "Engine":
        """A model with seeded random weights, loaded through the same by-name plan as a
        weight file (nothing is written to disk).  ``config``: a typed configuration, a
        config.json object, or the name of a preset (``gpt2``, ``gpt2-medium``, ``gpt2-xl``,
        ``tiny-a``, ``tiny-b``), whose own spread of the random values applies unless
        ``random_options`` say otherwise."""
        from ..config.presets import load_preset
        from ..config.registry import resolve_architecture
        from ..weights.loader import TensorDict
        if dtype not in PRECISIONS:
            raise ValueError(f"dtype must be one of {sorted(PRECISIONS)}, got {dtype!r}")
        if isinstance(config, str):
            arch, config, preset_options = load_preset(config)
            random_options = {**preset_options, **random_options}
        elif isinstance(config, dict):
            arch = resolve_architecture(config)
            config = arch.config_cls.from_json(config)
        else:
            arch = get_architecture(config.architecture)
        if arch.random_tensors is None:
            raise ValueError(f"architecture {arch.name!r} has no random-weights mode")
        rt = Runtime(torch.device(device), PRECISIONS[dtype])
        spec = arch.build_spec(config)
        model = Model(spec, rt)
        source = TensorDict(arch.random_tensors(config, seed, **random_options))
        plan = arch.weight_plan(config, spec, set(source.names()))
        model.bind(load_params(model.param_specs(), plan, source, precision=rt.precision,
                               device=rt.device))
        return cls(model, config, cache_tokens=cache_tokens, n_slots=n_slots)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # ------------------------------------------------------------------ the step function
    def _check_entries(self, entries):
        if not entries:
            raise ValueError("a step needs at least one sequence")
        V = self.spec.vocab_size
        out = []
        for e in entries:
            slot, tokens = int(e[0]), e[1]
            want = e[2] if len(e) > 2 else None
            arr = np.asarray(tokens)
            if arr.ndim != 1 or arr.size == 0:
                raise ValueError(f"slot {slot}: a step needs at least one token per sequence")
            if not np.issubdtype(arr.dtype, np.integer):
                raise ValueError(f"slot {slot}: token ids must be integers")
            if arr.min() < 0 or arr.max() >= V:
                raise ValueError(f"slot {slot}: token id outside 0..{V - 1}")
            if want is None:
                want = [arr.size - 1]
            want = [int(w) for w in want]
            for w in want:
                if not 0 <= w < arr.size:
                    raise ValueError(f"slot {slot}: wanted place {w} is outside this step's "
                                     f"{arr.size} tokens")
            out.append((slot, arr.astype(np.int32), want))
        return out

    def step(self, entries: Sequence) -> torch.Tensor | None:
        """Run one step.  ``entries``: ``(slot, tokens, want)`` per sequence; ``tokens`` are the
        sequence's next tokens (its whole prompt, or one token, or any chunk), ``want`` the
        places among them whose logits are returned (default: the last).  Only these tokens
        are run, as one batch, against what earlier steps left in the cache.  Returns fp32
        logits ``[wanted, vocab]`` in the order of the entries and of ``want``, or ``None``
        when nothing is wanted.  Everything is checked on the host before the first launch."""
        entries = self._check_entries(entries)
        self.cache.reserve([(slot, len(toks)) for slot, toks, _ in entries])
        pos0 = [self.cache.lens[slot] for slot, _, _ in entries]
        # with recordings on, a step's rows are padded so that steps of nearly the same size
        # share one (padding rows change no result); the plain first run of a shape and its
        # replays use the same padded layout and bounds, so they agree bit for bit
        pad = row_padding(sum(len(t) for _, t, _ in entries)) if self.step_graphs else 1
        packed = pack_step(entries, pos0, pad_rows_to=pad)
        done, logits = self.step_graphs.run(packed) if self.step_graphs else (False, None)
        if not done:
            layout = packed.on_device(
                packed.copy_to(self.rt.device),
                max_kv_len=self.step_graphs.kv_bound(packed) if self.step_graphs else None,
                max_q_len=q_bound(packed.max_q_len) if self.step_graphs else None)
            ctx = StepContext(self.rt, self.ops, layout, self.model.position, self.cache)
            logits = self.model.forward(ctx)
        for slot, toks, _ in entries:
            self.cache.advance(slot, len(toks))
        return logits

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | None = None,
                 on_token: Callable[[int, int, int], None] | None = None,
                 max_batch: int | None = None) -> list[list[int]]:
        """Generate for every prompt (token ids); returns the new ids per prompt, the prompt
        not included.  ``on_token(request_index, token, step)`` is called per sampled token."""
        params = params or SamplingParams()
        params.validate()
        prompts = [list(map(int, p)) for p in prompts]
        for i, p in enumerate(prompts):
            if not p:  # src/engine.rs:261-263
                raise ValueError(f"prompt {i} is an empty token sequence")
        n_new = [token_budget(len(p), params.max_new_tokens, self.spec.max_seq_len) for p in prompts]
        free_pages = min(g.pool.n_free for g in self.cache.groups) if self.cache.groups \
            else self.cache.n_pages
        batches = plan_batches([len(p) for p in prompts], n_new,
                               max_batch=max_batch or self.cache.slots.n_free,
                               cache_pages=free_pages)
        sampler = BatchSampler(params, self.ops, self.rt.device)
        seq_samplers = {i: SequenceSampler(params, i) for i in range(len(prompts))}
        out: list[list[int]] = [[] for _ in prompts]
        for batch in batches:
            res = run_batch(self, prompts, batch, params, sampler, seq_samplers, on_token)
            for i, ids in res.items():
                out[i] = ids
            self.check_errors()
        return out

    def check_errors(self) -> None:
        """Raise if a kernel of a step that has finished gave up a wait (its results are not
        valid).  ``step`` hands out logits that are still being computed; whoever has waited
        for them (copied them to the host, read sampled tokens) calls this before using them.
        ``generate`` does so itself."""
        self.ops.raise_device_errors()

    # ------------------------------------------------------------------ reports
    def inspect(self) -> dict:
        """What the reference's ``inspect`` prints (src/main.rs:333-369), read off the model's
        description: the kinds of its parts, what its mixers keep per token, and the element
        types its weights are held in (a matrix held in float32 runs on the CUDA-core
        kernels, also in a bfloat16 run)."""
        spec = self.spec

        def kinds(specs):
            seen = []
            for ps in specs:
                if ps.kind not in seen:
                    seen.append(ps.kind)
            return seen[0] if len(seen) == 1 else seen

        def arg(specs, key):
            seen = []
            for ps in specs:
                v = ps.args.get(key)
                if v is not None and v not in seen:
                    seen.append(v)
            return None if not seen else (seen[0] if len(seen) == 1 else seen)

        mixers = [l.mixer for l in spec.layers]
        ffns = [l.ffn for l in spec.layers]
        kv_req, _ = self.model.storage_requests()
        reqs = []
        for r in kv_req.values():
            if r not in reqs:
                reqs.append(r)
        one = (lambda vals: None if not vals else (vals[0] if len(set(vals)) == 1 else vals))
        by_dtype: dict[str, int] = {}
        for t in self.model.params.values():
            if t is not None:
                key = str(t.dtype).replace("torch.", "")
                by_dtype[key] = by_dtype.get(key, 0) + t.numel() * t.element_size()
        return {
            "name": getattr(self.config, "name", "model"), "architecture": spec.architecture,
            "n_params": self.model.n_params(),
            "weight_mb": round(sum(by_dtype.values()) / 2 ** 20, 2),
            "weight_mb_by_dtype": {k: round(v / 2 ** 20, 2) for k, v in sorted(by_dtype.items())},
            "kv_cache_mb": round(self.cache.bytes() / 2 ** 20, 2),
            "vocab": spec.vocab_size, "layers": len(spec.layers),
            "heads": arg(mixers, "n_heads"), "kv_heads": one([r.n_kv_heads for r in reqs]),
            "d_model": spec.width, "head_dim": one([r.head_dim for r in reqs]),
            "max_seq_len": spec.max_seq_len, "norm": kinds([spec.final_norm]
                                                           + [l.norm_mixer for l in spec.layers]
                                                           + [l.norm_ffn for l in spec.layers]),
            "mixer": kinds(mixers), "ffn": kinds(ffns), "activation": arg(ffns, "activation"),
            "pos": spec.position.kind, "tie_head": spec.tie_head,
            "dtype": self.rt.precision, "cache_tokens": self.cache.cache_tokens,
        }
