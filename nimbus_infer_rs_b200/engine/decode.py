"""Decoding a batch token by token without leaving the device.

A :class:`DecodeSession` holds a batch's decode state in fixed device buffers (the current
token, position and slot of every row) and runs one step at a time: the model on one token
per live sequence, token selection on the device, and the hand-over of the selected tokens
to the next step.  Because every buffer keeps its address and no kernel's launch shape
depends on the sequences' lengths, the whole step is captured once in a CUDA graph and then
replayed: a decode step of a small model is bound by launch latency, not by arithmetic.

It runs the same model, parts, cache and kernels as ``Engine.step``; the only additions are
the in-place token hand-over and the graph.  A sequence that ends becomes a padding row
(slot -1), which every kernel skips.
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache.paged import PAGE
from ..sampling.params import SamplingParams
from .batch import BatchLayout
from .context import StepContext


class DecodeSession:
    def __init__(self, engine, slots: list[int], first_tokens: list[int],
                 params: SamplingParams | None = None, seq_samplers=None, use_graph: bool = True):
        """``slots``: the live sequences (already prefilled); ``first_tokens``: the token each
        one runs next.  ``seq_samplers``: per-sequence sampling state (needed unless greedy)."""
        self.engine = engine
        self.params = params or SamplingParams(temperature=0.0)
        self.seq_samplers = seq_samplers
        self.n = len(slots)
        self.slots = list(slots)
        self.live = [True] * self.n
        dev = engine.rt.device
        self.use_graph = bool(use_graph) and dev.type == "cuda" and engine.graph_safe
        n = self.n
        host = np.zeros(3 * n, dtype=np.int32)
        host[:n] = first_tokens
        host[n:2 * n] = [engine.cache.lens[s] for s in slots]
        host[2 * n:] = slots
        # The device buffers and the recorded step are kept by the engine between batches of
        # the same size and sampling mode: a new batch fills the buffers again and replays the
        # graph it finds, instead of recording one of its own.
        self._key = (n, self.params.greedy,
                     float(self.params.temperature) if not self.params.greedy else 0.0,
                     int(self.params.top_k) if not self.params.greedy else 0,
                     float(self.params.top_p) if not self.params.greedy else 1.0,
                     float(self.params.repetition_penalty))
        kept = engine.decode_states.pop(self._key, None) if self.use_graph else None
        if kept is not None:
            self._buf, self.next_tokens, self.want_rows, self.cu_rows, self.u = kept["buffers"]
            self._buf.copy_(torch.from_numpy(host), non_blocking=False)
            self._graph, self._graph_launches, self.logits = kept["graph"], kept["launches"], kept["logits"]
            self.hist, self.hist_len = kept["history"]
            self._steps = 1 if self._graph is not None else 0
        else:
            self._buf = torch.from_numpy(host).to(dev)
            self.next_tokens = torch.zeros(n, dtype=torch.int32, device=dev)
            self.want_rows = torch.arange(n, dtype=torch.int32, device=dev)
            self.cu_rows = torch.arange(n + 1, dtype=torch.int32, device=dev)
            self.u = torch.zeros(n, dtype=torch.float64, device=dev)
            self.logits = None
            self._graph = None
            self._graph_launches = 0
            self._steps = 0
            self.hist = self.hist_len = None
            if self.params.repetition_penalty != 1.0:
                # what each sequence has generated, for the penalty: the token a row runs is
                # appended on the device at the start of every step
                self.hist = torch.zeros((n, engine.spec.max_seq_len), dtype=torch.int32, device=dev)
                self.hist_len = torch.zeros(n, dtype=torch.int32, device=dev)
        buf = self._buf
        self.tokens, self.row_pos, self.row_slot = buf[:n], buf[n:2 * n], buf[2 * n:]
        self._stage = None
        self._out_stage = None
        p = self.params
        on_device = p.greedy or (
            (p.top_p >= 1.0 or (hasattr(engine.ops, "sample_top_p")
                                and p.top_k <= engine.ops.top_p_max_k()))
            and (p.top_k == 0 or hasattr(engine.ops, "sample_top_k")))
        if not on_device or (p.repetition_penalty != 1.0 and not hasattr(engine.ops, "history_append")):
            raise ValueError("a decode session selects tokens with the sampling kernels only "
                             "(top-k within the top-p kernel's room)")
        if self.hist is not None:
            # tokens generated before this session, all but the one each row runs first
            self.hist_len.zero_()
            for i in range(n):
                before = list(seq_samplers[i].generated[:-1]) if seq_samplers is not None else []
                if before:
                    before = before[-self.hist.shape[1]:]
                    self.hist[i, :len(before)] = torch.tensor(before, dtype=torch.int32)
                    self.hist_len[i:i + 1].fill_(len(before))
        self.last_u: list[float] = []
        self._sampled = False      # a step of this session has selected tokens

    # ------------------------------------------------------------------ one step
    def _layout(self) -> BatchLayout:
        n = self.n
        eng = self.engine
        return BatchLayout(
            n_rows=n, n_tokens=n, n_seqs=n, n_want=n, tokens=self.tokens, row_pos=self.row_pos,
            row_slot=self.row_slot, want_rows=self.want_rows, cu_rows=self.cu_rows,
            seq_slot=self.row_slot, seq_pos0=self.row_pos, seq_lens=[1] * n,
            seq_pos0_host=[eng.cache.lens[s] for s in self.slots],
            seq_slots_host=list(self.slots), max_q_len=1, max_kv_len=eng.spec.max_seq_len,
            is_decode=True, want_all_rows=True)

    def _device_step(self) -> None:
        eng = self.engine
        ctx = StepContext(eng.rt, eng.ops, self._layout(), eng.model.position, eng.cache)
        if self.hist is not None:
            eng.ops.history_append(self.hist, self.hist_len, self.tokens, self.row_slot)
        self.logits = eng.model.forward(ctx)
        if self.hist is not None:
            eng.ops.repetition_penalty(self.logits, self.hist, self.hist_len,
                                       float(self.params.repetition_penalty))
        if self.params.greedy:
            eng.ops.argmax(self.logits, self.next_tokens)
        elif self.params.top_p < 1.0:
            eng.ops.sample_top_p(self.logits, self.params.top_k, float(np.float32(self.params.top_p)),
                                 float(self.params.temperature), self.u, self.next_tokens)
        elif self.params.top_k > 0:
            eng.ops.sample_top_k(self.logits, self.params.top_k, float(self.params.temperature),
                                 self.u, self.next_tokens)
        else:
            eng.ops.sample_temperature(self.logits, float(self.params.temperature), self.u,
                                       self.next_tokens)
        eng.ops.advance_decode(self.tokens, self.next_tokens, self.row_pos, self.row_slot)

    def step(self, tokens: list[int] | None = None) -> None:
        """Run the current token of every live sequence and select its next token (left on the
        device in ``next_tokens``; ``read_tokens`` brings them to the host).  ``tokens``: the
        token each row runs in this step, from the host (one per row of the session, any value
        for rows that have ended); without it the tokens selected by the previous step are
        used as they lie on the device."""
        eng = self.engine
        cache = eng.cache
        grow = [(s, 1) for s, alive in zip(self.slots, self.live) if alive]
        if not grow:
            return
        if tokens is None and self._sampled and not self.params.greedy and (
                self.params.top_k > 0 or self.params.top_p < 1.0):
            # the kernel may have handed a row back (a mark instead of a token on the device)
            raise ValueError("with top-k or top-p a step takes its tokens from the host: pass "
                             "what read_tokens() returned")
        if tokens is not None:
            if self._stage is None:
                # two pinned buffers taken in turn, each with an event that says its last copy
                # has left it: a step's tokens are never overwritten by the next step's while
                # their copy to the device may still be waiting in the stream
                cuda = eng.rt.device.type == "cuda"
                self._stage = [torch.empty(self.n, dtype=torch.int32, pin_memory=cuda) for _ in range(2)]
                self._stage_np = [t.numpy() for t in self._stage]      # the same pinned memory
                self._stage_done = [torch.cuda.Event() if cuda else None for _ in range(2)]
                self._stage_turn = 0
            i = self._stage_turn
            self._stage_turn ^= 1
            if self._stage_done[i] is not None:
                self._stage_done[i].synchronize()     # returns at once if never recorded or done
            self._stage_np[i][:] = tokens
            self.tokens.copy_(self._stage[i], non_blocking=True)
            if self._stage_done[i] is not None:
                self._stage_done[i].record()
        if any(cache.lens[s] % PAGE == 0 or cache.lens[s] + 1 > cache.max_seq_len for s, _ in grow):
            cache.reserve(grow)            # a new page somewhere, or an error to raise
        if not self.params.greedy:
            us = [self.seq_samplers[i].rng.next_f64() if alive else 0.0
                  for i, alive in enumerate(self.live)]
            self.u.copy_(torch.tensor(us, dtype=torch.float64), non_blocking=False)
            self.last_u = us
        if not self.use_graph or self._steps == 0:
            self._device_step()            # the first step runs plainly and warms the kernels
        else:
            if self._graph is None:
                self._capture()            # records the step; nothing runs yet
            launches = eng.ops.launches
            self._graph.replay()
            eng.ops.launches = launches + self._graph_launches
        self._steps += 1
        self._sampled = True
        for s, _ in grow:
            cache.advance(s, 1)

    def _capture(self) -> None:
        eng = self.engine
        before = eng.ops.launches
        from .step_graphs import no_collection
        graph = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(graph):
            self._device_step()
        self._graph_launches = eng.ops.launches - before
        eng.ops.launches = before
        self._graph = graph

    # ------------------------------------------------------------------ host side
    def read_tokens(self) -> list[int]:
        """The tokens selected by the last step, on the host (waits for the step): one copy
        into pinned memory on the step's stream, then a wait for that stream."""
        if self.next_tokens.device.type != "cuda":
            tokens = self.next_tokens.tolist()
        else:
            if self._out_stage is None:
                self._out_stage = torch.empty(self.n, dtype=torch.int32, pin_memory=True)
                self._out_np = self._out_stage.numpy()
            self._out_stage.copy_(self.next_tokens, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self.engine.ops.raise_device_errors()     # a kernel of the step gave up a wait
            tokens = self._out_np.tolist()
        if any(t < 0 for t, alive in zip(tokens, self.live) if alive):
            tokens = self._settle_on_host(tokens)
        return tokens

    def _settle_on_host(self, tokens: list[int]) -> list[int]:
        """Rows the sampling kernel handed back (a cut of top-p beyond the row's largest
        thousand logits; a NaN): the host's sampler decides on the whole row with the number
        that was drawn for this step.  The device keeps the mark in ``next_tokens``, so the
        next step must be given its tokens from the host."""
        from ..sampling import host as host_sampler
        from ..sampling.device import _Drawn, _pool
        todo = [i for i, t in enumerate(tokens) if t < 0 and self.live[i]]
        rows = self.logits.detach()[torch.tensor(todo, device=self.logits.device)].to("cpu").numpy()

        def one(j):
            return int(host_sampler.sample(rows[j], self.params, [], _Drawn(self.last_u[todo[j]])))
        results = [one(0)] if len(todo) == 1 else list(_pool().map(one, range(len(todo))))
        for j, i in enumerate(todo):
            tokens[i] = results[j]
        self.host_settled = getattr(self, "host_settled", 0) + 1
        return tokens

    def retire(self, index: int) -> None:
        """Sequence ``index`` of the session has ended: its row becomes padding."""
        if self.live[index]:
            self.live[index] = False
            self.row_slot[index:index + 1].fill_(-1)

    def close(self) -> None:
        """The batch is over: the buffers and the recorded step go back to the engine for the
        next batch of this size."""
        if self.use_graph and self._graph is not None and self._buf is not None:
            self.engine.decode_states[self._key] = {
                "buffers": (self._buf, self.next_tokens, self.want_rows, self.cu_rows, self.u),
                "graph": self._graph, "launches": self._graph_launches, "logits": self.logits,
                "history": (self.hist, self.hist_len),
                # scratch buffers of the kernel library that the graph points into
                "scratch": self.engine.ops.scratch_refs() if hasattr(self.engine.ops, "scratch_refs") else None}
            while len(self.engine.decode_states) > 8:
                self.engine.decode_states.pop(next(iter(self.engine.decode_states)))
        self._buf = None

    @property
    def n_live(self) -> int:
        return sum(self.live)
