"""Whole steps as CUDA graphs.

Every kernel of a step reads the batch (tokens, positions, slots, block tables) from device
memory, and no launch shape depends on anything but the step's *shape*: how many rows,
sequences and wanted places it has, its longest chunk, and (for one-token steps) the range
its longest sequence falls in.  Rows (beyond 64) and the longest chunk are rounded up to
multiples of 64 and 128, so that prompts of nearly the same lengths fall into one shape.  So
the launches of a step can be recorded once and replayed for every later step of the same
shape, whatever its tokens, slots and lengths: the host then issues one graph launch instead
of about a hundred kernel launches, and stays ahead of the GPU.  A shape is recorded when it comes for the second time (the first run is plain and has
warmed every kernel it needs); a bounded number of graphs is kept, the least recently used
one goes first.

Only models whose parts are all ``graph_safe`` take this path.  The results are those of the
plain launches: the same kernels run on the same data.
"""
from __future__ import annotations

import gc
import weakref
from collections import OrderedDict
from contextlib import contextmanager

import torch

from .batch import PackedStep
from .context import StepContext


def _kv_range(n: int, longest: int) -> int:
    """Upper end of the power-of-two range that ``n`` falls in (at most ``longest``)."""
    r = 64
    while r < n:
        r *= 2
    return min(r, longest)


ROW_BUCKET = 64      # steps of more rows than this are padded to a multiple of it
Q_BUCKET = 128       # a step's longest chunk counts as the next multiple of this


def row_padding(n_tokens: int) -> int:
    """What a step's row count is rounded up to, so that steps of nearly the same size share
    a recording: nothing for small steps (a decode step of a small batch), else a multiple of
    64.  Padding rows are skipped by every kernel and change no result."""
    return 1 if n_tokens <= ROW_BUCKET else ROW_BUCKET


def q_bound(max_q_len: int) -> int:
    """The chunk length that stands for ``max_q_len`` in the step's launches (grids over the
    rows of a sequence are sized by it; CTAs beyond a sequence's rows leave at once)."""
    return 1 if max_q_len <= 1 else -(-max_q_len // Q_BUCKET) * Q_BUCKET


@contextmanager
def no_collection():
    """No cyclic garbage collection inside: while a stream is being recorded, nothing may free
    CUDA graphs or device memory, and a collection could do just that to objects of an engine
    that is no longer used."""
    was_enabled = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        yield
    finally:
        if was_enabled:
            gc.enable()


class StepGraphs:
    def __init__(self, engine, capacity: int = 8, max_logit_bytes: int = 256 << 20):
        # the engine owns this object: a plain reference back would make a cycle, and the
        # engine's graphs would then be freed whenever the collector runs
        self.engine = weakref.proxy(engine)
        self.capacity = int(capacity)
        self.max_logit_bytes = int(max_logit_bytes)
        self._graphs: OrderedDict = OrderedDict()
        self._seen: dict = {}
        self.replays = 0
        self.captures = 0

    def kv_bound(self, p: PackedStep) -> int:
        """The length that stands for ``max_kv_len`` in the step's launches (how the keys are
        split among CTAs depends on it): the upper end of the range the longest sequence falls
        in, so that one recording serves the whole range.  The plain first run of a shape uses
        the same bound, so that it and the replays give identical results."""
        return _kv_range(p.max_kv_len, self.engine.spec.max_seq_len)

    def key(self, p: PackedStep):
        # whether every sequence starts at a page boundary decides which kernels append keys
        # and values, so it is part of the shape
        from ..cache.paged import PAGE
        aligned = all(q % PAGE == 0 for q in p.seq_pos0_host)
        return (p.n_rows, p.n_seqs, p.n_want, q_bound(p.max_q_len), p.is_decode, p.want_all_rows,
                self.kv_bound(p), aligned)

    def run(self, p: PackedStep):
        """Run the step by replay if its shape has a graph (recording one if it is due);
        returns ``(True, logits)``, or ``(False, None)`` if the caller has to launch it plainly."""
        eng = self.engine
        if self.capacity <= 0:
            return False, None          # recording is switched off
        if p.n_want * eng.spec.vocab_size * 4 > self.max_logit_bytes:
            return False, None          # the copy of the logits out of the graph would be large
        key = self.key(p)
        entry = self._graphs.get(key)
        if entry is None:
            n = self._seen.get(key, 0)
            if n == 0:
                if len(self._seen) > 4096:
                    self._seen.clear()
                self._seen[key] = 1
                return False, None
            entry = self._record(p, key)
        else:
            self._graphs.move_to_end(key)
            p.copy_to(eng.rt.device, into=entry["buf"])
        launches = eng.ops.launches
        entry["graph"].replay()
        eng.ops.launches = launches + entry["launches"]
        self.replays += 1
        out = entry["logits"]
        return True, (None if out is None else out.clone())

    def _record(self, p: PackedStep, key):
        eng = self.engine
        buf = torch.empty(p.buf.size, dtype=torch.int32, device=eng.rt.device)
        p.copy_to(eng.rt.device, into=buf)
        layout = p.on_device(buf, max_kv_len=self.kv_bound(p), max_q_len=q_bound(p.max_q_len))
        before = eng.ops.launches
        graph = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(graph):
            ctx = StepContext(eng.rt, eng.ops, layout, eng.model.position, eng.cache)
            logits = eng.model.forward(ctx)
        entry = {"graph": graph, "buf": buf, "logits": logits,
                 "launches": eng.ops.launches - before,
                 # scratch buffers of the kernel library that the graph points into
                 "scratch": eng.ops.scratch_refs() if hasattr(eng.ops, "scratch_refs") else None}
        eng.ops.launches = before
        self._graphs[key] = entry
        self.captures += 1
        while len(self._graphs) > self.capacity:
            self._graphs.popitem(last=False)
        return entry

    def clear(self) -> None:
        self._graphs.clear()
        self._seen.clear()
