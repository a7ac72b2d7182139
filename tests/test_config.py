import json

import pytest

from nimbus_infer_rs_b200.config import (ACT_ERF, ACT_TANH, ConfigError, GPT2Config,
                                         get_architecture, load_config, resolve_architecture)
import nimbus_infer_rs_b200  # noqa: F401  (registers gpt2)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_defaults_are_the_references():
    c = GPT2Config.from_json({})            # src/config.rs:45-66
    assert (c.vocab_size, c.n_layers, c.n_heads, c.d_model, c.d_mlp, c.max_seq_len) == \
        (50257, 12, 12, 768, 3072, 1024)
    assert c.head_dim == 64 and c.n_kv_heads == 12 and c.tie_embeddings
    assert c.norm_eps == 1e-5 and c.activation == ACT_TANH and c.scale_attn_by_head_dim
    assert c.n_params(with_linear_biases=True) == 124439808   # docs/make_demo_svg.py:31


def test_null_keeps_default():
    c = GPT2Config.from_json({"head_dim": None, "n_kv_heads": None, "d_model": 128, "n_heads": 4})
    assert c.head_dim == 32 and c.n_kv_heads == 4 and c.d_mlp == 512


def test_both_spellings_give_the_same_fields():
    a = GPT2Config.from_json(TINY_A)
    assert (a.d_model, a.n_layers, a.n_heads, a.d_mlp, a.max_seq_len, a.vocab_size) == \
        (64, 2, 4, 256, 128, 512)
    assert a.activation == ACT_TANH and a.tie_embeddings and a.head_dim == 16
    b = GPT2Config.from_json(TINY_B)
    assert b.activation == ACT_ERF and not b.tie_embeddings and b.d_mlp == 320
    assert b.scale_attn_by_inverse_layer_idx and b.norm_eps == 1e-6
    assert b.attn_scale(2) == pytest.approx(32 ** -0.5 / 3)
    c = GPT2Config.from_json(TINY_C)
    assert c.head_dim == 48 and c.n_kv_heads == 2 and c.kv_group_size == 3
    assert c.activation == ACT_TANH            # the reference's "gelu" is the tanh form
    assert c.attn_scale(1) == 1.0


def test_activation_spellings():
    assert GPT2Config.from_json({"activation_function": "gelu"}).activation == ACT_ERF
    assert GPT2Config.from_json({"activation_function": "gelu_new"}).activation == ACT_TANH
    assert GPT2Config.from_json({"activation": "gelu", "d_model": 768}).activation == ACT_TANH
    assert GPT2Config.from_json({"activation": "gelu", "n_embd": 768}).activation == ACT_ERF
    assert GPT2Config.from_json({"activation": "gelu_erf", "d_model": 768}).activation == ACT_ERF
    with pytest.raises(ConfigError, match="unknown activation"):
        GPT2Config.from_json({"activation": "relu6"})


def test_round_trip_through_to_json():
    for src in (TINY_A, TINY_B, TINY_C):
        c = GPT2Config.from_json(src)
        assert GPT2Config.from_json(c.to_json()) == c
        assert resolve_architecture(c.to_json()).name == "gpt2"


@pytest.mark.parametrize("bad, match", [
    ({"n_heads": 12, "n_kv_heads": 5, "d_model": 768}, "divisible by n_kv_heads"),
    ({"n_heads": 5, "d_model": 768}, "divisible by n_heads"),
    ({"norm": "rmsnorm"}, "architecture not supported"),
    ({"pos_encoding": "rope"}, "architecture not supported"),
    ({"activation": "swiglu"}, "architecture not supported"),
    ({"vocab_size": 0}, "positive"),
    ({"n_layers": "twelve"}, "expected an integer"),
    ({"d_model": 12.5}, "expected an integer"),
    ({"tie_embeddings": "yes"}, "true/false"),
    ({"norm_eps": -1.0}, "positive"),
])
def test_rejections(bad, match):
    with pytest.raises(ConfigError, match=match):
        GPT2Config.from_json(bad)


def test_all_problems_are_named_at_once():
    with pytest.raises(ConfigError) as e:
        GPT2Config.from_json({"vocab_size": -3, "n_layers": "x"})
    assert "vocab_size" in str(e.value) and "n_layers" in str(e.value)


def test_registry_resolution(tmp_path):
    assert get_architecture("GPT2LMHeadModel").name == "gpt2"
    assert resolve_architecture({"architectures": ["GPT2LMHeadModel"]}).name == "gpt2"
    assert resolve_architecture({"model_type": "gpt2"}).name == "gpt2"
    assert resolve_architecture(TINY_C).name == "gpt2"      # by the three switches
    with pytest.raises(ConfigError, match="architecture not supported"):
        resolve_architecture({"model_type": "llama"})
    with pytest.raises(ConfigError, match="architecture not supported"):
        resolve_architecture({"norm": "rmsnorm", "activation": "swiglu", "pos_encoding": "rope"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "gpt2" and cfg.d_model == 96
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)


def test_spec_is_data_and_takes_its_numbers_from_config():
    arch = get_architecture("gpt2")
    cfg = GPT2Config.from_json(TINY_B)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and spec.run_order() == (0, 1, 2)
    assert spec.layers[2].mixer.args["scale"] == pytest.approx(32 ** -0.5 / 3)
    assert spec.layers[0].ffn.args == {"width": 96, "hidden": 320, "activation": ACT_ERF}
    assert spec.final_norm.args["eps"] == 1e-6 and not spec.tie_head


def test_presets_are_config_files_read_through_the_registry():
    from nimbus_infer_rs_b200.config import (load_preset, preset_json, preset_names,
                                             preset_random_options)
    assert set(preset_names()) >= {"gpt2", "gpt2-medium", "gpt2-xl", "tiny-a", "tiny-b"}
    arch, cfg, opts = load_preset("gpt2")
    assert arch.name == "gpt2" and opts == {"std": 0.02}
    # the reference's defaults are this size (src/config.rs:45-66, docs/make_demo_svg.py:31)
    assert cfg == GPT2Config.from_json({}).replace(name="gpt2")
    assert cfg.n_params(with_linear_biases=True) == 124_439_808
    assert load_preset("gpt2-medium")[1].n_params() == 354_823_168
    assert load_preset("GPT2-XL")[1].n_params() == 1_557_611_200
    _, b, opts = load_preset("tiny-b")
    assert (b.n_layers, b.d_model, b.n_heads, b.d_mlp, b.vocab_size) == (3, 96, 3, 320, 1000)
    assert not b.tie_embeddings and opts == {"std": 0.05, "bias_std": 0.02}
    assert "random_weights" not in preset_json("tiny-a") and preset_random_options("tiny-a")["gamma_jitter"] == 0.02
    for bad in ("gpt3", "../gpt2", ""):
        with pytest.raises(ConfigError, match="no preset named"):
            load_preset(bad)
