"""Token selection for a batch of logits on the device.

Greedy decoding, temperature sampling and the repetition penalty run as kernels; the random
number of each draw comes from the sequence's own host generator so that results do not
depend on batching.  With top-k or top-p filtering on, the batch's logits are brought to the
host and the float64 restatement of the reference's sampler decides (sampling/host.py).
"""
from __future__ import annotations

import numpy as np
import torch

from . import host as host_sampler
from .params import DEFAULT_SEED, SamplingParams
from .rng import Xoshiro256pp, sequence_seed


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
        p = self.params
        return (not p.greedy) and (p.top_k > 0 or p.top_p < 1.0)

    def sample(self, logits: torch.Tensor, seqs: list[SequenceSampler]) -> list[int]:
        """``logits`` fp32 [n, vocab] (may be modified), one row per entry of ``seqs``."""
        p = self.params
        n = logits.shape[0]
        assert n == len(seqs)
        if self.needs_host():
            rows = logits.detach().to("cpu").numpy()
            out = [host_sampler.sample(rows[i], p, s.generated, s.rng) for i, s in enumerate(seqs)]
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
                u = torch.tensor([s.rng.next_f64() for s in seqs], dtype=torch.float64)
                self.ops.sample_temperature(logits, float(p.temperature),
                                            u.to(logits.device), ids)
            out = ids.to("cpu").tolist()
        for s, t in zip(seqs, out):
            s.generated.append(int(t))
        return [int(t) for t in out]
