"""The generation loop above the step function.

Per sequence it is the reference's loop (src/engine.rs:255-293): the prompt in one step, then
sample → record → stop check → one more token.  ``n_new = min(max_new_tokens, max_seq_len -
prompt_len)``; a sampled stop token is kept in the output and ends the sequence; the last
sampled token is never run through the model.  Here a *batch* of prompts of unequal lengths
starts together; a sequence that ends leaves the batch and gives its slot back while the
others go on; and a list of requests longer than one batch may hold is run as several
batches one after another over the same cache.

The decisions (who is in which batch, who is still active, when a sequence ends) are plain
host code in this file and are tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Sequence

from ..cache.paged import PAGE, pages_for
from ..sampling.params import SamplingParams


def token_budget(prompt_len: int, max_new_tokens: int, max_seq_len: int) -> int:
    """src/engine.rs:265-266 (saturating)."""
    return min(max_new_tokens, max(0, max_seq_len - prompt_len))


def plan_batches(prompt_lens: Sequence[int], n_new: Sequence[int], *, max_batch: int,
                 cache_pages: int) -> list[list[int]]:
    """Cut the request list, in order, into batches that fit: at most ``max_batch`` sequences
    and at most ``cache_pages`` pages when every sequence has reached its final length (the
    last sampled token is not cached)."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    batches: list[list[int]] = []
    cur: list[int] = []
    cur_pages = 0
    for i, (p, n) in enumerate(zip(prompt_lens, n_new)):
        need = pages_for(p + max(0, n - 1))
        if need > cache_pages:
            raise ValueError(
                f"request {i} needs {need * PAGE} cached tokens, the cache holds {cache_pages * PAGE}")
        if cur and (len(cur) >= max_batch or cur_pages + need > cache_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


@dataclass
class SequenceProgress:
    """Where one sequence stands in its generation."""
    index: int                 # position in the request list
    prompt_len: int
    n_new: int                 # tokens it may generate
    stop_tokens: frozenset
    generated: list[int] = field(default_factory=list)
    finished: bool = False

    def __post_init__(self):
        if self.n_new == 0:
            self.finished = True

    def record(self, token: int) -> bool:
        """Take a sampled token; True if the sequence goes on (src/engine.rs:280-287)."""
        assert not self.finished
        self.generated.append(int(token))
        step = len(self.generated) - 1
        if token in self.stop_tokens or step == self.n_new - 1:
            self.finished = True
        return not self.finished


def run_batch(engine, prompts: list[list[int]], indices: list[int], params: SamplingParams,
              sampler, seq_samplers, on_token: Callable | None) -> dict[int, list[int]]:
    """One batch from prompts to its last token.  Returns generated ids per request index."""
    max_len = engine.spec.max_seq_len
    stops = frozenset(int(t) for t in params.stop_tokens)
    seqs = [SequenceProgress(i, len(prompts[i]),
                             token_budget(len(prompts[i]), params.max_new_tokens, max_len), stops)
            for i in indices]
    results = {s.index: s.generated for s in seqs}
    live = [s for s in seqs if not s.finished]
    if not live:
        return results
    slots = {s.index: engine.alloc_slot() for s in live}

    def take(seq_list, tokens):
        """Record one sampled token per sequence; returns those that go on, with their token."""
        nxt = []
        for s, tok in zip(seq_list, tokens):
            if on_token is not None:
                on_token(s.index, tok, len(s.generated))
            if s.record(tok):
                nxt.append((s, tok))
            else:
                engine.free_slot(slots.pop(s.index))
        return nxt

    session = None
    try:
        # the prompts, in one step; logits of each last token
        logits = engine.step([(slots[s.index], prompts[s.index], [s.prompt_len - 1]) for s in live])
        nxt = take(live, sampler.sample(logits, [seq_samplers[s.index] for s in live]))
        if nxt and not sampler.needs_host() and (
                params.repetition_penalty == 1.0 or hasattr(engine.ops, "history_append")):
            # token selection stays on the device: one captured step per token
            from .decode import DecodeSession
            members = [s for s, _ in nxt]
            session = DecodeSession(engine, [slots[s.index] for s in members],
                                    [tok for _, tok in nxt], params,
                                    [seq_samplers[s.index] for s in members])
            alive = list(range(len(members)))
            tokens = [tok for _, tok in nxt]
            while alive:
                session.step(tokens)       # host tokens in ...
                tokens = session.read_tokens()   # ... and out
                for i in alive:
                    seq_samplers[members[i].index].generated.append(tokens[i])
                going = {s.index for s, _ in take([members[i] for i in alive],
                                                  [tokens[i] for i in alive])}
                for i in alive:
                    if members[i].index not in going:
                        session.retire(i)
                alive = [i for i in alive if members[i].index in going]
        else:
            while nxt:
                live = [s for s, _ in nxt]
                logits = engine.step([(slots[s.index], [tok], [0]) for s, tok in nxt])
                nxt = take(live, sampler.sample(logits, [seq_samplers[s.index] for s in live]))
    finally:
        if session is not None:
            session.close()
        for slot in slots.values():
            engine.free_slot(slot)
    return results
