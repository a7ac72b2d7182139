"""Random-weights mode: write a model folder (config.json + model.safetensors) from a
configuration and a seed.

The reference's fixture was made this way by its sibling engine
(benchmarks/cross_engine.py:43-64: ``Engine.random(config, seed=42)``): matrices and
embeddings ~N(0, 0.02), norm weights 1, norm biases 0, no linear biases.  Here the standard
deviations are arguments so that tests can give biases and norm weights a spread too.

Values are drawn in fp32 from a seeded CPU generator, one tensor after another in a fixed
order, then rounded to the storage type.  Matrices and tables are stored in ``dtype``
(bfloat16 by default, the serving precision); vectors are stored in fp32.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.gpt2 import GPT2Config
from ..config.registry import get_architecture
from .safetensors_io import write_safetensors


def gpt2_tensors(cfg: GPT2Config, seed: int, *, std: float = 0.02, bias_std: float = 0.0,
                 gamma_jitter: float = 0.0, beta_std: float = 0.0,
                 dtype: torch.dtype = torch.bfloat16, scheme: str = "nimbus") -> dict:
    """Random GPT-2 tensors under the names of ``scheme``: ``"nimbus"`` (the reference's,
    src/engine.rs:110-225) or ``"checkpoint"`` (published GPT-2 files: fused ``c_attn``)."""
    if scheme not in ("nimbus", "checkpoint"):
        raise ValueError("scheme must be 'nimbus' or 'checkpoint'")
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    d, m, V, P = cfg.d_model, cfg.d_mlp, cfg.vocab_size, cfg.max_seq_len
    hq, hk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim

    def mat(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(dtype)

    def vec(n, s, mean=0.0):
        if s > 0:
            return torch.randn(n, generator=g, dtype=torch.float32) * s + mean
        return torch.full((n,), mean, dtype=torch.float32)

    out: dict[str, torch.Tensor] = {}
    ck = scheme == "checkpoint"
    out["wte.weight" if ck else "wte"] = mat(V, d)
    out["wpe.weight" if ck else "wpe"] = mat(P, d)
    for i in range(cfg.n_layers):
        p = f"h.{i}."
        n1, n2 = ("ln_1", "ln_2") if ck else ("norm1", "norm2")
        out[f"{p}{n1}.weight"] = vec(d, gamma_jitter, 1.0)
        out[f"{p}{n1}.bias"] = vec(d, beta_std)
        q, k, v = mat(d, hq), mat(d, hk), mat(d, hk)       # stored (in, out)
        if ck:
            out[f"{p}attn.c_attn.weight"] = torch.cat([q, k, v], dim=1).contiguous()
            if bias_std > 0:
                out[f"{p}attn.c_attn.bias"] = vec(hq + 2 * hk, bias_std)
            out[f"{p}attn.c_proj.weight"] = mat(hq, d)
            if bias_std > 0:
                out[f"{p}attn.c_proj.bias"] = vec(d, bias_std)
        else:
            out[f"{p}attn.q.weight"], out[f"{p}attn.k.weight"], out[f"{p}attn.v.weight"] = q, k, v
            if bias_std > 0:
                out[f"{p}attn.q.bias"] = vec(hq, bias_std)
                out[f"{p}attn.k.bias"] = vec(hk, bias_std)
                out[f"{p}attn.v.bias"] = vec(hk, bias_std)
            out[f"{p}attn.o.weight"] = mat(hq, d)
            if bias_std > 0:
                out[f"{p}attn.o.bias"] = vec(d, bias_std)
        out[f"{p}{n2}.weight"] = vec(d, gamma_jitter, 1.0)
        out[f"{p}{n2}.bias"] = vec(d, beta_std)
        fc, pj = ("mlp.c_fc", "mlp.c_proj") if ck else ("mlp.fc", "mlp.proj")
        out[f"{p}{fc}.weight"] = mat(d, m)
        if bias_std > 0:
            out[f"{p}{fc}.bias"] = vec(m, bias_std)
        out[f"{p}{pj}.weight"] = mat(m, d)
        if bias_std > 0:
            out[f"{p}{pj}.bias"] = vec(d, bias_std)
    nf = "ln_f" if ck else "norm_f"
    out[f"{nf}.weight"] = vec(d, gamma_jitter, 1.0)
    out[f"{nf}.bias"] = vec(d, beta_std)
    if not cfg.tie_embeddings:
        out["lm_head.weight"] = mat(V, d) if ck else mat(d, V)
    return out


def write_random_model(model_dir: str | Path, cfg, seed: int, **kw) -> Path:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir`` for any registered
    architecture's configuration."""
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    arch = get_architecture(cfg.architecture)
    if arch.random_tensors is None:
        raise ValueError(f"architecture {arch.name!r} has no random-weights mode")
    tensors = arch.random_tensors(cfg, seed, **kw)
    (d / "config.json").write_text(json.dumps(cfg.to_json(), indent=2) + "\n")
    write_safetensors(d / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return d
