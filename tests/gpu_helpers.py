"""Shared by the GPU tests: tolerances and small runners."""
from __future__ import annotations

import torch

import plain_gpt2 as P

# largest allowed |engine - plain| relative to the largest |plain logit| of the comparison
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
DTYPES = ["float32", "bfloat16"]


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    scale = float(ref.abs().max())
    err = (got - ref).abs()
    worst = float(err.max())
    if worst > TOL[dtype] * scale:
        idx = int(err.reshape(err.shape[0], -1).max(dim=1).values.argmax()) if err.dim() > 1 else 0
        raise AssertionError(f"{what}: max error {worst:.3e} > {TOL[dtype]:.0e} * {scale:.3e} "
                             f"(first dimension index of the worst row: {idx})")


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(model_dir, tokens) -> torch.Tensor:
    return P.forward_logits(P.PlainWeights(model_dir), tokens)


def assert_greedy_matches(got: list[int], W, prompt, dtype: str, stop_tokens=()) -> None:
    """Token-by-token against the plain implementation.  A difference is accepted only where
    the plain logits of the two candidates are closer than the tolerance (a near tie); the
    sequences part ways there, so the comparison ends."""
    ctx = list(prompt)
    for step, tok in enumerate(got):
        logits = P.forward_logits(W, ctx)[-1]
        want = int(torch.argmax(logits))
        if tok != want:
            gap = float(logits[want] - logits[tok])
            assert gap <= 2 * TOL[dtype] * float(logits.abs().max()), \
                f"step {step}: got {tok}, plain says {want} (logit gap {gap:.3e})"
            return
        ctx.append(tok)
        if tok in stop_tokens:
            assert step == len(got) - 1
