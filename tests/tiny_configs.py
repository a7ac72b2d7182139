"""The tiny configurations the tests run on.  They differ in every size and option: head
counts and groups, widths that are no power of two, number of layers, vocabulary, the norms'
eps, the activation, tied or own head, score scaling, naming scheme and storage type."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from nimbus_infer_rs_b200.config import GPT2Config, preset_json, preset_random_options

# tiny A (checkpoint-style keys; n_inner left out: 4 x width) and tiny B (explicit inner size,
# exact GELU, own head, per-layer score divisor) are the package's presets of those names
TINY_A = preset_json("tiny-a")
TINY_B = preset_json("tiny-b")
# tiny C: the reference's own keys; grouped key/value heads, head size not width/heads,
# long context for far-key tests, no score scaling by head size
TINY_C = {
    "name": "tiny-c", "vocab_size": 777, "n_layers": 2, "n_heads": 6, "n_kv_heads": 2,
    "d_model": 80, "head_dim": 48, "d_mlp": 136, "max_seq_len": 448, "norm": "layernorm",
    "activation": "gelu", "pos_encoding": "learned", "tie_embeddings": True,
    "norm_eps": 3e-5, "scale_attn_by_head_dim": False,
}

# tiny D: heads of 64 (the tensor-core prefill attention), two key/value heads for four query
# heads, a context of several pages
TINY_D = {
    "model_type": "gpt2", "vocab_size": 300, "n_positions": 320, "n_embd": 256, "n_layer": 2,
    "n_head": 4, "n_kv_heads": 2, "n_inner": 384, "activation_function": "gelu_new",
    "layer_norm_epsilon": 2e-5, "tie_word_embeddings": True,
}

RECIPES = {
    # name: (config json, seed, random-weight options)
    "A": (TINY_A, 11, dict(preset_random_options("tiny-a"), scheme="checkpoint", dtype=torch.bfloat16)),
    "B": (TINY_B, 22, dict(preset_random_options("tiny-b"), scheme="nimbus", dtype=torch.bfloat16)),
    # C: matrices stored in 32-bit next to bf16 tables (a file that mixes element types: the
    # 32-bit tensors stay 32-bit in a bfloat16 run)
    "C": (TINY_C, 33, dict(std=0.05, bias_std=0.02, gamma_jitter=0.05, beta_std=0.02,
                           scheme="nimbus", dtype=torch.float32)),
    "D": (TINY_D, 44, dict(std=0.04, bias_std=0.02, gamma_jitter=0.03, beta_std=0.01,
                           scheme="checkpoint", dtype=torch.bfloat16)),
}
BF16_TABLES = {"C": ("wte", "wpe")}


def make_model(root: Path, name: str) -> Path:
    from nimbus_infer_rs_b200.models.gpt2 import random_tensors
    from nimbus_infer_rs_b200.weights import write_safetensors
    cfg_json, seed, opts = RECIPES[name]
    cfg = GPT2Config.from_json(cfg_json)
    d = Path(root) / f"tiny_{name}"
    d.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(cfg, seed, **opts)
    for t in BF16_TABLES.get(name, ()):
        tensors[t] = tensors[t].to(torch.bfloat16)
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt", "seed": str(seed)})
    # the config in the spelling under test
    (d / "config.json").write_text(json.dumps(cfg_json, indent=2))
    return d


def make_all(root: Path) -> dict[str, Path]:
    return {n: make_model(root, n) for n in RECIPES}
