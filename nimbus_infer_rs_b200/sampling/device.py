"""Token selection for a batch of logits on the device.

Greedy decoding, temperature sampling, top-k sampling and the repetition penalty run as
kernels; the random number of each draw comes from the sequence's own host generator so that
results do not depend on batching.  Top-p sampling is a kernel as well; it hands back the rows
whose cut lies beyond their thousand largest logits (and rows with a NaN), and those the float64
restatement of the reference's sampler settles on the host (sampling/host.py), with the number
that was already drawn.  The older way (the device picks each row's largest logits, the host
decides among them) is kept for logits on the host and for a top-k beyond the kernel's room.
"""
from __future__ import annotations

import numpy as np
import torch

from . import host as host_sampler
from .params import DEFAULT_SEED, SamplingParams
from .rng import Xoshiro256pp, sequence_seed


_POOL = None


def _pool():
    """Threads for the rows that the host's sampler takes whole (made on first use)."""
    global _POOL
    if _POOL is None:
        import os
        from concurrent.futures import ThreadPoolExecutor
        _POOL = ThreadPoolExecutor(max_workers=max(2, min(16, os.cpu_count() or 2)),
                                   thread_name_prefix="nimbus-sampler")
    return _POOL


class _Drawn:
    """A generator that hands out one number that was drawn before."""

    def __init__(self, value: float):
        self.value = value

    def next_f64(self) -> float:
        return self.value


class SequenceSampler:
    """Per-sequence sampling state: generator and generated history."""

    def __init__(self, params: SamplingParams, seq_index: int):
        seed = DEFAULT_SEED if params.seed is None else params.seed
        self.rng = Xoshiro256pp(sequence_seed(seed, seq_index))
        self.generated: list[int] = []


class BatchSampler:
    def __init__(self, params: SamplingParams, ops, device):
        params.validate()
        self.params = params
        self.ops = ops
        self.device = device

    def needs_host(self) -> bool:
        """True if no kernel of the backend selects tokens with these options (a top-k beyond
        the top-p kernel's room; a stand-in backend without the sampling kernels)."""
        p = self.params
        if p.greedy:
            return False
        if p.top_p < 1.0:
            return not (hasattr(self.ops, "sample_top_p") and p.top_k <= self.ops.top_p_max_k())
        return p.top_k > 0 and not hasattr(self.ops, "sample_top_k")

    #: candidates the device hands to the host's sampler when top-k / top-p is on
    N_CANDIDATES = 1024

    def _filtered(self, logits: torch.Tensor, seqs: list[SequenceSampler]) -> list[int]:
        """top-k / top-p sampling: the reference's float64 sampler on the host.  Both filters
        only keep the largest logits, so the device first picks each row's largest thousand
        (with the row's softmax denominator) and the host decides among them; a row whose cut
        does not fall among them, or that has a NaN, is brought over whole.  With a repetition
        penalty the logits of the generated tokens come along, wherever they rank."""
        p = self.params
        n, vocab = logits.shape
        fast = logits.is_cuda and hasattr(self.ops, "top_candidates")
        out: list[int | None] = [None] * n
        if fast:
            temp = max(float(np.float32(p.temperature)), 1e-6)
            keep = min(self.N_CANDIDATES, vocab)
            vals, idx, counts, stats = self.ops.top_candidates(logits, keep, temp)
            gen = [None] * n
            if p.repetition_penalty != 1.0:
                gen = [np.array(sorted({t for t in s.generated if 0 <= t < vocab}), dtype=np.int64)
                       for s in seqs]
                flat = np.concatenate([g + i * vocab for i, g in enumerate(gen)]) if n else gen
                gen_vals = logits.reshape(-1)[torch.from_numpy(flat).to(logits.device)].cpu().numpy() \
                    if len(flat) else np.zeros(0, np.float32)
                ends = np.cumsum([len(g) for g in gen])
            vals, idx = vals.cpu().numpy(), idx.cpu().numpy()
            counts, stats = counts.cpu().numpy(), stats.cpu().numpy()
            for i, s in enumerate(seqs):
                g_idx = g_vals = None
                if gen[i] is not None and len(gen[i]):
                    g_idx, g_vals = gen[i], gen_vals[ends[i] - len(gen[i]):ends[i]]
                out[i] = host_sampler.sample_from_candidates(
                    vals[i], idx[i], int(counts[i]), float(stats[i, 0]), float(stats[i, 1]), p,
                    s.rng, keep, vocab, g_idx, g_vals)
        todo = [i for i in range(n) if out[i] is None]
        if todo:
            # whole rows: one copy for all of them, then a thread per row (sorting 50,000 values
            # takes milliseconds, numpy lets go of the interpreter lock meanwhile, and every
            # sequence draws from its own generator)
            sel = logits.detach() if len(todo) == n else logits.detach()[
                torch.tensor(todo, device=logits.device)]
            rows = sel.to("cpu").numpy()

            def one(j):
                i = todo[j]
                return host_sampler.sample(rows[j], p, seqs[i].generated, seqs[i].rng)
            if len(todo) == 1:
                results = [one(0)]
            else:
                results = list(_pool().map(one, range(len(todo))))
            for j, i in enumerate(todo):
                out[i] = results[j]
        return out

    def sample(self, logits: torch.Tensor, seqs: list[SequenceSampler]) -> list[int]:
        """``logits`` fp32 [n, vocab] (may be modified), one row per entry of ``seqs``."""
        p = self.params
        n = logits.shape[0]
        assert n == len(seqs)
        if self.needs_host() or (not logits.is_cuda and not p.greedy and (p.top_k > 0 or p.top_p < 1.0)):
            out = self._filtered(logits, seqs)
        else:
            if p.repetition_penalty != 1.0 and any(s.generated for s in seqs):
                width = max(len(s.generated) for s in seqs)
                hist = np.full((n, width), -1, dtype=np.int32)
                lens = np.zeros(n, dtype=np.int32)
                for i, s in enumerate(seqs):
                    hist[i, :len(s.generated)] = s.generated
                    lens[i] = len(s.generated)
                self.ops.repetition_penalty(logits, torch.from_numpy(hist).to(self.device),
                                            torch.from_numpy(lens).to(self.device),
                                            float(p.repetition_penalty))
            ids = torch.empty(n, dtype=torch.int32, device=logits.device)
            if p.greedy:
                self.ops.argmax(logits, ids)
            else:
                us = [s.rng.next_f64() for s in seqs]
                u = torch.tensor(us, dtype=torch.float64).to(logits.device)
                if p.top_p < 1.0:
                    self.ops.sample_top_p(logits, p.top_k, float(np.float32(p.top_p)),
                                          float(p.temperature), u, ids)
                elif p.top_k > 0:
                    self.ops.sample_top_k(logits, p.top_k, float(p.temperature), u, ids)
                else:
                    self.ops.sample_temperature(logits, float(p.temperature), u, ids)
            out = ids.to("cpu").tolist()
            todo = [i for i, t in enumerate(out) if t < 0]
            if todo:
                # rows the kernel handed back (a NaN; a cut beyond the largest thousand logits):
                # the host decides on the whole row, with the number already drawn and the
                # penalty already applied; a thread per row
                sel = logits.detach() if len(todo) == n else logits.detach()[
                    torch.tensor(todo, device=logits.device)]
                rows = sel.to("cpu").numpy()
                plain = SamplingParams(temperature=p.temperature, top_k=p.top_k, top_p=p.top_p)

                def one(j):
                    return host_sampler.sample(rows[j], plain, [], _Drawn(us[todo[j]]))
                results = [one(0)] if len(todo) == 1 else list(_pool().map(one, range(len(todo))))
                for j, i in enumerate(todo):
                    out[i] = results[j]
        for s, t in zip(seqs, out):
            s.generated.append(int(t))
        return [int(t) for t in out]
