"""bin/trace_run's own logic (requests to slots, what is written when, what is given back),
run inside this process on the torch-CPU stand-in of the kernel library.  The program as a
user runs it, on the GPU, is in test_gpu_trace_run.py."""
import importlib.machinery
import importlib.util
import io
import json
import sys
from pathlib import Path

import numpy as np
import torch

import plain_gpt2 as P

ROOT = Path(__file__).resolve().parent.parent


def _main():
    loader = importlib.machinery.SourceFileLoader("trace_run_program", str(ROOT / "bin" / "trace_run"))
    spec = importlib.util.spec_from_loader(loader.name, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod.main


def _run(monkeypatch, capsys, argv, steps):
    monkeypatch.setattr(sys, "argv", ["trace_run", *argv, "--device", "cpu"])
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps) + "\n"))
    assert _main()() == 0
    return capsys.readouterr().out.split("\n")


def test_two_batches_on_a_cache_that_holds_one(model_dirs, cpu_backend, tmp_path, monkeypatch, capsys):
    """Unequal prompts in one step, then a token each; the shorter request ends earlier; the
    second batch fits only into what the first gave back (--max-tokens 128 = two pages)."""
    W = P.PlainWeights(model_dirs["A"])
    V = 512
    g = torch.Generator().manual_seed(4)
    a, b, c = (torch.randint(0, V, (n,), generator=g).tolist() for n in (9, 3, 60))
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:6], "want": [0, 5]},
                                {"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [a[6]], "want": [0]},
                                {"id": "b", "tokens": [b[2]], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [a[7]], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": [a[8]], "want": [0]}], "end": ["a"]},
        # the same names again are new requests; both need a page, and there are two
        {"step": 4, "entries": [{"id": "a", "tokens": c, "want": [59]},
                                {"id": "b", "tokens": b, "want": [2]}], "end": ["a", "b"]},
        {"step": 5, "entries": [], "end": []},
    ]
    out = tmp_path / "out"
    lines = _run(monkeypatch, capsys, ["--model", str(model_dirs["A"]), "--dtype", "float32",
                                       "--out", str(out), "--max-tokens", "128"], steps)
    assert [l for l in lines if l] == [f"done {i}" for i in range(6)]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "1.f32", "3.f32", "4.f32"]   # 2, 5: nothing wanted

    def read(step):
        return torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, V)).double()

    la, lb, lc = P.forward_logits(W, a), P.forward_logits(W, b), P.forward_logits(W, c)
    for got, want in ((read(0), la[[0, 5]]), (read(1), torch.stack([la[6], lb[2]])),
                      (read(3), la[[8]]), (read(4), torch.stack([lc[59], lb[2]]))):
        assert got.shape == want.shape
        assert float((got - want).abs().max()) <= 2e-5 * float(want.abs().max())


def test_a_preset_instead_of_a_folder(cpu_backend, tmp_path, monkeypatch, capsys):
    steps = [{"step": 7, "entries": [{"id": 1, "tokens": [5, 17, 3], "want": [2]}], "end": [1]}]
    lines = _run(monkeypatch, capsys, ["--random", "tiny-b", "--seed-weights", "3", "--dtype",
                                       "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"], steps)
    assert "done 7" in lines
    first = np.fromfile(tmp_path / "o" / "7.f32", dtype="<f4")
    _run(monkeypatch, capsys, ["--random", "tiny-b", "--seed-weights", "3", "--dtype", "float32",
                               "--out", str(tmp_path / "p"), "--max-tokens", "64"], steps)
    again = np.fromfile(tmp_path / "p" / "7.f32", dtype="<f4")
    assert first.shape == again.shape and np.array_equal(first, again) and np.isfinite(first).all()


def test_more_live_tokens_than_max_tokens_is_an_error_not_a_wrong_answer(cpu_backend, tmp_path,
                                                                          monkeypatch, capsys):
    import pytest

    from nimbus_infer_rs_b200.cache import CacheError
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]},
                                     {"id": "b", "tokens": [3], "want": [0]}], "end": []}]
    with pytest.raises(CacheError):
        _run(monkeypatch, capsys, ["--random", "tiny-b", "--dtype", "float32", "--out",
                                   str(tmp_path / "o"), "--max-tokens", "64"], steps)
    assert not (tmp_path / "o" / "0.f32").exists()
