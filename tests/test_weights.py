import json

import pytest
import torch

import nimbus_infer_rs_b200  # noqa: F401
from nimbus_infer_rs_b200.config import GPT2Config, get_architecture
from nimbus_infer_rs_b200.engine.model import Model, Runtime
from nimbus_infer_rs_b200.models.gpt2 import random_tensors as gpt2_tensors
from nimbus_infer_rs_b200.weights import (SafeTensorsError, SafeTensorsFile, WeightError,
                                          find_weight_file, load_params, write_safetensors)
from tiny_configs import TINY_A, TINY_B, TINY_C


def _load(cfg_json, tensors, tmp_path, precision="bfloat16", cast=None):
    cfg = GPT2Config.from_json(cfg_json)
    arch = get_architecture("gpt2")
    spec = arch.build_spec(cfg)
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with SafeTensorsFile(find_weight_file(tmp_path)) as f:
        plan = arch.weight_plan(cfg, spec, set(f.names()))
        return load_params(model.param_specs(), plan, f, precision=precision, device="cpu",
                           cast_weights=cast), cfg


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "d": torch.randn(4).half()}
    write_safetensors(tmp_path / "x.safetensors", t, metadata={"k": "v"})
    with SafeTensorsFile(tmp_path / "x.safetensors") as f:
        assert f.names() == ["a", "b", "c", "d"] and f.metadata == {"k": "v"}
        for k, v in t.items():
            got = f.tensor(k)
            assert got.dtype == v.dtype and torch.equal(got, v)
        with pytest.raises(SafeTensorsError, match="missing tensor 'zz'"):
            f.tensor("zz")


def test_half_precision_bit_patterns_of_the_reference(tmp_path):
    """Bytes written by hand, not by this library's writer: the F16 patterns and the BF16 pair
    of the reference's own unit tests (src/safetensors.rs:196-222) come out as the same values."""
    f16 = [0x0000, 0x3C00, 0x4000, 0x7C00, 0x7E00, 0xFC00]
    bf16 = [0x3F80, 0x4000]                              # the top halves of 1.0f32 and 2.0f32
    hdr = json.dumps({"h": {"dtype": "F16", "shape": [6], "data_offsets": [0, 12]},
                      "w": {"dtype": "BF16", "shape": [2], "data_offsets": [12, 16]}}).encode()
    body = b"".join(v.to_bytes(2, "little") for v in f16 + bf16)
    p = tmp_path / "half.safetensors"
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + body)
    with SafeTensorsFile(p) as f:
        h = f.tensor("h").float()
        assert h[:3].tolist() == [0.0, 1.0, 2.0]
        assert h[3] == float("inf") and torch.isnan(h[4]) and h[5] == float("-inf")
        assert f.tensor("w").dtype == torch.bfloat16 and f.tensor("w").float().tolist() == [1.0, 2.0]


def test_safetensors_bad_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafeTensorsError, match="too small"):
        SafeTensorsFile(p)
    p.write_bytes((10 ** 6).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafeTensorsError, match="exceeds file size"):
        SafeTensorsFile(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafeTensorsError, match="size mismatch"):
        SafeTensorsFile(p)
    hdr = json.dumps({"t": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 4)
    with pytest.raises(SafeTensorsError, match="unsupported dtype"):
        SafeTensorsFile(p)


@pytest.mark.parametrize("cfg_json, scheme", [(TINY_A, "checkpoint"), (TINY_B, "nimbus"),
                                              (TINY_C, "nimbus")])
def test_loads_by_name_in_both_schemes(cfg_json, scheme, tmp_path):
    cfg = GPT2Config.from_json(cfg_json)
    tensors = gpt2_tensors(cfg, 5, bias_std=0.01, scheme=scheme)
    params, _ = _load(cfg_json, tensors, tmp_path)
    hq, hk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    w = params["layers.1.mixer.qkv.weight"]
    assert w.shape == (hq + 2 * hk, cfg.d_model) and w.dtype == torch.bfloat16
    # the fused matrix is [q; k; v], each transposed from its stored (in, out)
    if scheme == "nimbus":
        assert torch.equal(w[:hq], tensors["h.1.attn.q.weight"].t())
        assert torch.equal(w[hq + hk:], tensors["h.1.attn.v.weight"].t())
        assert torch.equal(params["layers.0.ffn.proj.weight"], tensors["h.0.mlp.proj.weight"].t())
    else:
        assert torch.equal(w, tensors["h.1.attn.c_attn.weight"].t())
    assert params["layers.0.mixer.qkv.bias"].dtype == torch.float32
    assert params["final_norm.weight"].dtype == torch.float32
    if cfg.tie_embeddings:
        assert "head.weight" not in params
    else:
        assert params["head.weight"].shape == (cfg.vocab_size, cfg.d_model)


def test_element_types_follow_the_rule(tmp_path):
    cfg = GPT2Config.from_json(TINY_B)
    t32 = gpt2_tensors(cfg, 5, dtype=torch.float32)
    p, _ = _load(TINY_B, t32, tmp_path, "bfloat16", cast=False)
    assert p["embedding.table"].dtype == torch.float32          # kept as stored on request
    p, _ = _load(TINY_B, t32, tmp_path, "bfloat16", cast=True)
    assert p["embedding.table"].dtype == torch.bfloat16
    # no bf16 matrix in the whole file = a full-precision checkpoint: a bfloat16 run rounds it
    p, _ = _load(TINY_B, t32, tmp_path, "bfloat16", cast=None)
    assert p["embedding.table"].dtype == torch.bfloat16
    assert p["layers.1.mixer.qkv.weight"].dtype == torch.bfloat16
    assert p["layers.1.norm_ffn.weight"].dtype == torch.float32  # vectors are always 32-bit
    # a file of bf16 matrices in which one tensor was kept in 32-bit: that one stays 32-bit
    mixed = dict(gpt2_tensors(cfg, 5, dtype=torch.bfloat16))
    mixed["h.1.mlp.fc.weight"] = t32["h.1.mlp.fc.weight"]
    p, _ = _load(TINY_B, mixed, tmp_path, "bfloat16", cast=None)
    assert p["layers.1.ffn.fc.weight"].dtype == torch.float32
    assert p["layers.0.ffn.fc.weight"].dtype == torch.bfloat16
    t16 = gpt2_tensors(cfg, 5, dtype=torch.bfloat16)
    p, _ = _load(TINY_B, t16, tmp_path, "bfloat16")
    assert p["layers.0.ffn.fc.weight"].dtype == torch.bfloat16  # kept in bfloat16
    p, _ = _load(TINY_B, t16, tmp_path, "float32")
    assert p["layers.0.ffn.fc.weight"].dtype == torch.float32
    assert torch.equal(p["layers.0.ffn.fc.weight"], t16["h.0.mlp.fc.weight"].t().float())


def test_missing_biases_are_fine_but_partial_qkv_bias_is_zero_filled(tmp_path):
    cfg = GPT2Config.from_json(TINY_B)
    t = gpt2_tensors(cfg, 5, bias_std=0.0)                      # no linear biases at all
    p, _ = _load(TINY_B, t, tmp_path)
    assert p["layers.0.mixer.qkv.bias"] is None and p["layers.0.ffn.fc.bias"] is None
    t["h.0.attn.k.bias"] = torch.ones(cfg.n_kv_heads * cfg.head_dim)
    p, _ = _load(TINY_B, t, tmp_path)
    b = p["layers.0.mixer.qkv.bias"]
    hq = cfg.n_heads * cfg.head_dim
    assert b[:hq].abs().sum() == 0 and torch.all(b[hq:2 * hq] == 1)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = GPT2Config.from_json(TINY_B)
    t = gpt2_tensors(cfg, 5, bias_std=0.01)
    del t["h.1.norm2.bias"]
    del t["h.2.attn.o.weight"]
    t["h.0.attn.rotary_inv_freq"] = torch.zeros(4)
    t["stray"] = torch.zeros(2, 2)
    t["wpe"] = torch.zeros(cfg.max_seq_len + 1, cfg.d_model)
    t["h.0.mlp.fc.weight"] = t["h.0.mlp.fc.weight"].t().contiguous()
    with pytest.raises(WeightError) as e:
        _load(TINY_B, t, tmp_path)
    err = e.value
    assert err.missing == ["h.1.norm2.bias", "h.2.attn.o.weight"]
    assert err.unexpected == ["h.0.attn.rotary_inv_freq", "stray"]
    assert len(err.wrong_shape) == 2
    text = str(err)
    assert "wpe is [65, 96], expected [64, 96]" in text
    assert "h.0.mlp.fc.weight is [320, 96], expected [96, 320]" in text
    assert "missing tensors (2)" in text and "unexpected tensors (2)" in text


def test_mask_buffers_and_tied_head_copy_are_not_weights(tmp_path):
    cfg = GPT2Config.from_json(TINY_A)
    t = gpt2_tensors(cfg, 5, scheme="checkpoint")
    t = {("transformer." + k): v for k, v in t.items()}
    t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)
    t["transformer.h.0.attn.masked_bias"] = torch.tensor(-1e4)
    t["lm_head.weight"] = t["transformer.wte.weight"].clone()
    p, _ = _load(TINY_A, t, tmp_path)
    assert p["embedding.table"].shape == (512, 64)


def test_no_weight_file(tmp_path):
    with pytest.raises(FileNotFoundError, match="no weights.safetensors or model.safetensors"):
        find_weight_file(tmp_path)


def test_random_mode_is_seeded(tmp_path):
    cfg = GPT2Config.from_json(TINY_A)
    a, b, c = gpt2_tensors(cfg, 7), gpt2_tensors(cfg, 7), gpt2_tensors(cfg, 8)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["wte"], c["wte"])
    assert a["wte"].dtype == torch.bfloat16 and a["h.0.norm1.weight"].dtype == torch.float32
