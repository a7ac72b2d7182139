"""The packed layout of one step: the tokens of all its sequences as consecutive rows.

Row ``r`` carries a token, its absolute position in its sequence and its sequence's slot.
Padding rows (token -1, slot -1) may be appended; every kernel skips them, so padding
changes no result.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class BatchLayout:
    n_rows: int                 # rows including padding
    n_tokens: int               # rows that carry a token
    n_seqs: int
    n_want: int
    tokens: torch.Tensor        # int32 [n_rows]
    row_pos: torch.Tensor       # int32 [n_rows]
    row_slot: torch.Tensor      # int32 [n_rows]
    want_rows: torch.Tensor     # int32 [n_want]: rows whose logits are asked for
    cu_rows: torch.Tensor       # int32 [n_seqs + 1]: first row of each sequence
    seq_slot: torch.Tensor      # int32 [n_seqs]
    seq_pos0: torch.Tensor      # int32 [n_seqs]: tokens cached before this step
    seq_lens: list[int]         # host: tokens of each sequence in this step
    seq_pos0_host: list[int]
    seq_slots_host: list[int]
    max_q_len: int
    max_kv_len: int             # longest sequence after this step
    is_decode: bool             # one token per sequence
    want_all_rows: bool = False  # want_rows is 0, 1, ..., n_rows - 1


@dataclass
class PackedStep:
    """A step's layout on the host: one int32 buffer ``[tokens | row_pos | row_slot | cu_rows |
    seq_slot | seq_pos0 | want]`` and what the host knows about it."""
    buf: np.ndarray
    offs: list[int]
    n_rows: int
    n_tokens: int
    n_seqs: int
    n_want: int
    seq_lens: list[int]
    seq_pos0_host: list[int]
    seq_slots_host: list[int]
    max_q_len: int
    max_kv_len: int
    is_decode: bool
    want_all_rows: bool

    def on_device(self, dev: torch.Tensor, max_kv_len: int | None = None,
                  max_q_len: int | None = None) -> BatchLayout:
        """The layout over ``dev``, a device copy of ``buf``.  ``max_kv_len`` / ``max_q_len``:
        bounds to stand for the step's own longest sequence and longest chunk (launch shapes
        are sized by them; every kernel reads the true lengths from ``dev``)."""
        o = self.offs
        parts = [dev[o[i]:o[i + 1]] for i in range(7)]
        return BatchLayout(
            n_rows=self.n_rows, n_tokens=self.n_tokens, n_seqs=self.n_seqs, n_want=self.n_want,
            tokens=parts[0], row_pos=parts[1], row_slot=parts[2], cu_rows=parts[3],
            seq_slot=parts[4], seq_pos0=parts[5], want_rows=parts[6], seq_lens=self.seq_lens,
            seq_pos0_host=self.seq_pos0_host, seq_slots_host=self.seq_slots_host,
            max_q_len=self.max_q_len if max_q_len is None else max_q_len,
            max_kv_len=self.max_kv_len if max_kv_len is None else max_kv_len,
            is_decode=self.is_decode, want_all_rows=self.want_all_rows)

    def copy_to(self, device, into: torch.Tensor | None = None) -> torch.Tensor:
        """One host-to-device copy of the buffer (through pinned memory on a GPU); ``into``: a
        device buffer of the same size that is written instead of a new one."""
        host = torch.from_numpy(self.buf)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        if into is None:
            return host.to(device, non_blocking=True)
        into.copy_(host, non_blocking=True)
        return into


def pack_step(entries, pos0: list[int], pad_rows_to: int = 1) -> PackedStep:
    """``entries``: ``(slot, tokens, want)`` per sequence; ``pos0``: tokens already cached."""
    n_seqs = len(entries)
    lens = [len(e[1]) for e in entries]
    n_tokens = sum(lens)
    n_rows = -(-n_tokens // pad_rows_to) * pad_rows_to
    n_want = sum(len(e[2]) for e in entries)
    sizes = [n_rows, n_rows, n_rows, n_seqs + 1, n_seqs, n_seqs, n_want]
    offs = [0]
    for z in sizes:
        offs.append(offs[-1] + z)
    buf = np.empty(offs[-1], dtype=np.int32)
    tokens, row_pos, row_slot, cu_rows, seq_slot, seq_pos0, want = (
        buf[offs[i]:offs[i + 1]] for i in range(7))
    tokens[:] = -1
    row_pos[:] = 0
    row_slot[:] = -1
    r = 0
    w = 0
    for i, (slot, toks, wants) in enumerate(entries):
        t = lens[i]
        tokens[r:r + t] = toks
        row_pos[r:r + t] = np.arange(pos0[i], pos0[i] + t, dtype=np.int32)
        row_slot[r:r + t] = slot
        cu_rows[i] = r
        seq_slot[i] = slot
        seq_pos0[i] = pos0[i]
        for x in wants:
            want[w] = r + x
            w += 1
        r += t
    cu_rows[n_seqs] = r
    return PackedStep(
        buf=buf, offs=offs, n_rows=n_rows, n_tokens=n_tokens, n_seqs=n_seqs, n_want=n_want,
        seq_lens=lens, seq_pos0_host=list(pos0), seq_slots_host=[int(e[0]) for e in entries],
        max_q_len=max(lens) if lens else 0,
        max_kv_len=max((p + t for p, t in zip(pos0, lens)), default=0),
        is_decode=all(t == 1 for t in lens),
        want_all_rows=(n_want == n_rows and bool((want == np.arange(n_rows, dtype=np.int32)).all())))


def build_layout(entries, pos0: list[int], device, pad_rows_to: int = 1) -> BatchLayout:
    """Pack the step and bring it to the device: one host buffer, one copy."""
    packed = pack_step(entries, pos0, pad_rows_to)
    return packed.on_device(packed.copy_to(device))
