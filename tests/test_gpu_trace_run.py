"""bin/trace_run as a user runs it: a subprocess fed JSON lines, answering `done <step>`,
writing <step>.f32; the same requests replayed whole, token by token and in unequal batches
must give the plain implementation's logits."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_helpers import DTYPES, assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _replay(model_dir, dtype, out_dir, steps, max_tokens):
    proc = subprocess.Popen(
        [str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(max_tokens)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd="/")
    for st in steps:
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {st['step']}", line      # the next step comes only after this
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


def _read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, vocab))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_whole_decoded_and_batched(model_dirs, tmp_path, name, dtype):
    vocab = json.loads((model_dirs[name] / "config.json").read_text())["vocab_size"]
    lens = {"A": [70, 5, 33, 128], "B": [40, 1, 64, 17]}[name]
    reqs = {f"r{i}": random_tokens(vocab, n, seed=50 + i) for i, n in enumerate(lens)}
    refs = {k: plain_logits(model_dirs[name], v) for k, v in reqs.items()}

    # (1) each request alone and whole
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}],
              "end": [k]} for i, (k, v) in enumerate(reqs.items())]
    _replay(model_dirs[name], dtype, tmp_path / "whole", steps, max_tokens=128)
    for i, k in enumerate(reqs):
        assert_close(_read(tmp_path / "whole", i, vocab), refs[k], dtype, f"whole {k}")

    # (2) the last 32 tokens (or all but the first) one by one
    k, v = "r0", reqs["r0"]
    head = len(v) - 32
    steps = [{"step": 0, "entries": [{"id": k, "tokens": v[:head], "want": []}], "end": []}]
    steps += [{"step": 1 + j, "entries": [{"id": k, "tokens": [v[head + j]], "want": [0]}],
               "end": [k] if j == 31 else []} for j in range(32)]
    _replay(model_dirs[name], dtype, tmp_path / "dec", steps, max_tokens=128)
    assert not (tmp_path / "dec" / "0.f32").exists()             # nothing was wanted there
    got = torch.cat([_read(tmp_path / "dec", 1 + j, vocab) for j in range(32)])
    assert_close(got, refs[k][head:], dtype, "last 32 one by one")

    # (3) batches of unequal lengths: prompts (all but the last 4 tokens, at least 1) in one
    # step, then one token each; shorter requests end earlier.  Each batch in a process of its
    # own, then both one after the other in one process, on a cache that holds just one of them
    # at a time: the second batch gets the slots and pages the first gave back.
    def batch_steps(ids, first_step):
        plen = {k: max(1, len(reqs[k]) - 4) for k in ids}
        steps = [{"step": first_step, "entries": [{"id": k, "tokens": reqs[k][:plen[k]],
                                                   "want": [plen[k] - 1]} for k in ids], "end": []}]
        pos, live = dict(plen), list(ids)
        order = [list(ids)]
        while True:
            ending = [k for k in live if pos[k] >= len(reqs[k])]
            if ending:
                steps[-1]["end"] = ending
                live = [k for k in live if k not in ending]
            if not live:
                break
            steps.append({"step": first_step + len(steps), "entries": [
                {"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live], "end": []})
            order.append(list(live))
            for k in live:
                pos[k] += 1
        return steps, order, plen

    def check(out, first_step, order, plen, ids, what):
        got = {k: [] for k in ids}
        for si, members in enumerate(order):
            rows = _read(out, first_step + si, vocab)
            assert rows.shape[0] == len(members)
            for ri, k in enumerate(members):
                got[k].append(rows[ri:ri + 1])
        for k in ids:
            assert_close(torch.cat(got[k]), refs[k][plen[k] - 1:], dtype, f"{what} {k}")

    rounds = (["r0", "r1", "r2"], ["r3", "r1"])
    held = [sum(-(-len(reqs[k]) // 64) * 64 for k in ids) for ids in rounds]
    for rnd, ids in enumerate(rounds):
        steps, order, plen = batch_steps(ids, 0)
        _replay(model_dirs[name], dtype, tmp_path / f"batch{rnd}", steps, max_tokens=held[rnd])
        check(tmp_path / f"batch{rnd}", 0, order, plen, ids, f"batch {rnd}")
    all_steps, parts = [], []
    for ids in rounds:
        steps, order, plen = batch_steps(ids, len(all_steps))
        parts.append((len(all_steps), order, plen, ids))
        all_steps += steps
    _replay(model_dirs[name], dtype, tmp_path / "both", all_steps, max_tokens=max(held))
    for rnd, (first, order, plen, ids) in enumerate(parts):
        check(tmp_path / "both", first, order, plen, ids, f"one process, batch {rnd}")
