"""A plain, slow GPT-2 written from the reference's formulas: whole sequences, no cache, one
function per part, CPU only.  It shares no code with the package: it has its own reader of
config.json and of the weight file.  Every function cites the reference lines it restates.

The reference itself (Rust) cannot be compiled or imported here (no Rust toolchain), so
this implementation rests on the formulas; tests/golden/ holds small outputs of it together
with the script that made them.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------- file reading
def read_safetensors(path) -> dict[str, torch.Tensor]:
    """src/safetensors.rs:42-98,113-146: u64 header length, JSON header, raw data; F32, F16
    and BF16 widened to fp32 -- here to float64 right away."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = data[a:b]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(np.float64)
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = torch.from_numpy(arr.reshape(info["shape"]).copy())
    return out


def read_config(model_dir) -> dict:
    """src/config.rs:45-133 (keys and defaults) with the checkpoint-style spellings as aliases.
    Returns a plain dict with the reference's field names."""
    obj = json.loads((Path(model_dir) / "config.json").read_text())

    def get(keys, default):
        for k in keys:
            if obj.get(k) is not None:
                return obj[k]
        return default

    c = {
        "vocab_size": get(["vocab_size"], 50257),
        "n_layers": get(["n_layers", "n_layer"], 12),
        "n_heads": get(["n_heads", "n_head"], 12),
        "d_model": get(["d_model", "n_embd"], 768),
        "max_seq_len": get(["max_seq_len", "n_positions"], 1024),
        "tie_embeddings": get(["tie_embeddings", "tie_word_embeddings"], True),
        "norm_eps": get(["norm_eps", "layer_norm_epsilon"], 1e-5),
        "scale_attn_by_head_dim": get(["scale_attn_by_head_dim", "scale_attn_weights"], True),
        "scale_attn_by_inverse_layer_idx": get(["scale_attn_by_inverse_layer_idx"], False),
    }
    c["d_mlp"] = get(["d_mlp", "n_inner"], 4 * c["d_model"])
    c["head_dim"] = get(["head_dim"], c["d_model"] // c["n_heads"])   # src/config.rs:154-156
    c["n_kv_heads"] = get(["n_kv_heads"], c["n_heads"])               # src/config.rs:158-160
    if obj.get("activation_function") is not None:
        c["gelu"] = "erf" if obj["activation_function"] == "gelu" else "tanh"
    else:
        a = obj.get("activation", "gelu")
        nimbus_style = any(k in obj for k in ("d_model", "n_layers", "n_heads", "d_mlp",
                                              "max_seq_len", "norm", "pos_encoding",
                                              "tie_embeddings", "norm_eps"))
        if a in ("gelu_erf", "gelu_exact"):
            c["gelu"] = "erf"
        elif a == "gelu" and not nimbus_style:
            c["gelu"] = "erf"
        else:
            c["gelu"] = "tanh"   # src/config.rs:104 with src/ops.rs:21-24
    return c


class PlainWeights:
    """Tensors under the reference's names (src/engine.rs:110-225), every linear weight as
    stored there: ``(in, out)``.  Checkpoint-style files are renamed and ``c_attn`` is split."""

    def __init__(self, model_dir):
        d = Path(model_dir)
        path = next(p for p in (d / "weights.safetensors", d / "model.safetensors") if p.exists())
        t = read_safetensors(path)
        cfg = read_config(model_dir)
        t = {k[len("transformer."):] if k.startswith("transformer.") else k: v
             for k, v in t.items()}
        if "wte.weight" in t:
            hq = cfg["n_heads"] * cfg["head_dim"]
            hk = cfg["n_kv_heads"] * cfg["head_dim"]
            r = {"wte": t["wte.weight"], "wpe": t["wpe.weight"],
                 "norm_f.weight": t["ln_f.weight"], "norm_f.bias": t["ln_f.bias"]}
            for i in range(cfg["n_layers"]):
                p = f"h.{i}."
                for a, b in (("ln_1", "norm1"), ("ln_2", "norm2")):
                    r[f"{p}{b}.weight"] = t[f"{p}{a}.weight"]
                    r[f"{p}{b}.bias"] = t[f"{p}{a}.bias"]
                w = t[f"{p}attn.c_attn.weight"]
                r[f"{p}attn.q.weight"], r[f"{p}attn.k.weight"], r[f"{p}attn.v.weight"] = \
                    w[:, :hq], w[:, hq:hq + hk], w[:, hq + hk:]
                if f"{p}attn.c_attn.bias" in t:
                    b = t[f"{p}attn.c_attn.bias"]
                    r[f"{p}attn.q.bias"], r[f"{p}attn.k.bias"], r[f"{p}attn.v.bias"] = \
                        b[:hq], b[hq:hq + hk], b[hq + hk:]
                for a, b in (("attn.c_proj", "attn.o"), ("mlp.c_fc", "mlp.fc"),
                             ("mlp.c_proj", "mlp.proj")):
                    r[f"{p}{b}.weight"] = t[f"{p}{a}.weight"]
                    if f"{p}{a}.bias" in t:
                        r[f"{p}{b}.bias"] = t[f"{p}{a}.bias"]
            if not cfg["tie_embeddings"]:
                r["lm_head.weight"] = t["lm_head.weight"].t()   # stored (vocab, width) there
            t = r
        self.t = t
        self.cfg = cfg

    def __getitem__(self, name):
        return self.t[name]

    def get(self, name):
        return self.t.get(name)


# --------------------------------------------------------------------------- the parts
def embed(tokens, wte, wpe, pos_offset=0):
    """src/model.rs:285-295: row of wte plus row of wpe at the absolute position."""
    idx = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(pos_offset, pos_offset + idx.numel())
    return wte[idx] + wpe[pos]


def layer_norm(x, weight, bias, eps):
    """src/ops.rs:32-40: mean; biased variance of (x - mean); 1/sqrt(var + eps)."""
    mean = x.sum(-1, keepdim=True) / x.shape[-1]
    var = ((x - mean) ** 2).sum(-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(var + eps)
    return (x - mean) * inv * weight + bias


def linear(x, w_in_out, bias):
    """src/model.rs:88-119 with src/engine.rs:93-101: y = x W (+ b), W stored (in, out)."""
    y = x @ w_in_out
    return y if bias is None else y + bias


def softmax_row(s):
    """src/ops.rs:6-18: subtract the maximum, exponentiate, divide by the sum if positive."""
    e = torch.exp(s - s.max())
    tot = e.sum()
    return e / tot if tot > 0 else e


def attention(h, W, i, cfg, layer_idx):
    """src/model.rs:359-433: q, k, v projections; per head and query row, scores over keys
    0..row with the scale of src/config.rs:162-168 (and the per-layer divisor), keys after
    the row masked with -1e9, softmax over all, weighted sum of the values; heads merged."""
    T = h.shape[0]
    H, Hk, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    p = f"h.{i}."
    q = linear(h, W[f"{p}attn.q.weight"], W.get(f"{p}attn.q.bias")).reshape(T, H, hd)
    k = linear(h, W[f"{p}attn.k.weight"], W.get(f"{p}attn.k.bias")).reshape(T, Hk, hd)
    v = linear(h, W[f"{p}attn.v.weight"], W.get(f"{p}attn.v.bias")).reshape(T, Hk, hd)
    scale = hd ** -0.5 if cfg["scale_attn_by_head_dim"] else 1.0
    if cfg["scale_attn_by_inverse_layer_idx"]:
        scale = scale / (layer_idx + 1)
    group = H // Hk
    out = torch.zeros(T, H, hd, dtype=h.dtype)
    for head in range(H):
        kv = head // group                      # src/model.rs:390
        for t in range(T):
            s = torch.full((T,), -1e9, dtype=h.dtype)
            s[:t + 1] = (k[:t + 1, kv] @ q[t, head]) * scale   # src/model.rs:403-409
            prob = softmax_row(s)
            out[t, head] = prob[:t + 1] @ v[:t + 1, kv]        # src/model.rs:411-419
    return out.reshape(T, H * hd)


def gelu_tanh(x):
    """src/ops.rs:21-24."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def gelu_erf(x):
    """The exact form, 0.5 x (1 + erf(x / sqrt 2)); not in the reference."""
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def mlp(h, W, i, cfg):
    """src/model.rs:462-473."""
    p = f"h.{i}."
    mid = linear(h, W[f"{p}mlp.fc.weight"], W.get(f"{p}mlp.fc.bias"))
    mid = gelu_erf(mid) if cfg["gelu"] == "erf" else gelu_tanh(mid)
    return linear(mid, W[f"{p}mlp.proj.weight"], W.get(f"{p}mlp.proj.bias"))


def block(x, W, i, cfg):
    """src/model.rs:297-300 with :345-357,:437-439 and :448-460,:485-487 (pre-norm)."""
    p = f"h.{i}."
    h = layer_norm(x, W[f"{p}norm1.weight"], W[f"{p}norm1.bias"], cfg["norm_eps"])
    a = attention(h, W, i, cfg, i)
    x = x + linear(a, W[f"{p}attn.o.weight"], W.get(f"{p}attn.o.bias"))
    h = layer_norm(x, W[f"{p}norm2.weight"], W[f"{p}norm2.bias"], cfg["norm_eps"])
    return x + mlp(h, W, i, cfg)


def forward_logits(W: PlainWeights, tokens, dtype=torch.float64) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, vocab] (src/model.rs:271-325; the
    reference takes the head of the last row only)."""
    cfg = W.cfg
    assert 0 < len(tokens) <= cfg["max_seq_len"]
    cast = (lambda t: None if t is None else t.to(dtype))
    Wd = _Cast(W, cast)
    x = embed(tokens, Wd["wte"], Wd["wpe"])
    for i in range(cfg["n_layers"]):
        x = block(x, Wd, i, cfg)
    x = layer_norm(x, Wd["norm_f.weight"], Wd["norm_f.bias"], cfg["norm_eps"])
    head = Wd["wte"].t() if cfg["tie_embeddings"] else Wd["lm_head.weight"]   # (in, out)
    return x @ head


class _Cast:
    def __init__(self, W, fn):
        self.W, self.fn, self.cache = W, fn, {}

    def __getitem__(self, name):
        if name not in self.cache:
            self.cache[name] = self.fn(self.W[name])
        return self.cache[name]

    def get(self, name):
        return self.fn(self.W.get(name)) if self.W.get(name) is not None else None


# --------------------------------------------------------------------------- generation
def greedy_generate(W: PlainWeights, prompt, n_new, stop_tokens=(), dtype=torch.float64):
    """src/engine.rs:255-293 without a cache: the whole context is re-run for every token
    (as tests/engine.rs:38-55 does); first index of the maximum (src/sampler.rs:172-180)."""
    ctx = list(prompt)
    n_new = min(n_new, max(0, W.cfg["max_seq_len"] - len(prompt)))
    out = []
    for step in range(n_new):
        logits = forward_logits(W, ctx, dtype)[-1]
        tok = int(torch.argmax(logits))
        out.append(tok)
        if tok in stop_tokens or step == n_new - 1:
            break
        ctx.append(tok)
    return out
