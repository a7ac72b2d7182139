"""The tiny configurations the tests run on.  They differ in every size and option: head
counts and groups, widths that are no power of two, number of layers, vocabulary, the norms'
eps, the activation, tied or own head, score scaling, naming scheme and storage type."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from nimbus_infer_rs_b200.config import GPT2Config
from nimbus_infer_rs_b200.weights import write_random_model

# tiny A: written with checkpoint-style keys; n_inner left out (4 x width)
TINY_A = {
    "model_type": "gpt2", "vocab_size": 512, "n_positions": 128, "n_embd": 64, "n_layer": 2,
    "n_head": 4, "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
    "tie_word_embeddings": True,
}
# tiny B: explicit inner size, exact GELU, own head, per-layer score divisor
TINY_B = {
    "model_type": "gpt2", "vocab_size": 1000, "n_positions": 64, "n_embd": 96, "n_layer": 3,
    "n_head": 3, "n_inner": 320, "activation_function": "gelu", "layer_norm_epsilon": 1e-6,
    "tie_word_embeddings": False, "scale_attn_by_inverse_layer_idx": True,
}
# tiny C: the reference's own keys; grouped key/value heads, head size not width/heads,
# long context for far-key tests, no score scaling by head size
TINY_C = {
    "name": "tiny-c", "vocab_size": 777, "n_layers": 2, "n_heads": 6, "n_kv_heads": 2,
    "d_model": 80, "head_dim": 48, "d_mlp": 136, "max_seq_len": 448, "norm": "layernorm",
    "activation": "gelu", "pos_encoding": "learned", "tie_embeddings": True,
    "norm_eps": 3e-5, "scale_attn_by_head_dim": False,
}

RECIPES = {
    # name: (config json, seed, random-weight options)
    "A": (TINY_A, 11, dict(std=0.02, bias_std=0.01, gamma_jitter=0.02, scheme="checkpoint",
                           dtype=torch.bfloat16)),
    "B": (TINY_B, 22, dict(std=0.05, bias_std=0.02, scheme="nimbus", dtype=torch.bfloat16)),
    "C": (TINY_C, 33, dict(std=0.05, bias_std=0.02, gamma_jitter=0.05, beta_std=0.02,
                           scheme="nimbus", dtype=torch.float32)),
}


def make_model(root: Path, name: str) -> Path:
    cfg_json, seed, opts = RECIPES[name]
    cfg = GPT2Config.from_json(cfg_json)
    d = write_random_model(Path(root) / f"tiny_{name}", cfg, seed, **opts)
    # keep the config in the spelling under test
    (d / "config.json").write_text(json.dumps(cfg_json, indent=2))
    return d


def make_all(root: Path) -> dict[str, Path]:
    return {n: make_model(root, n) for n in RECIPES}
