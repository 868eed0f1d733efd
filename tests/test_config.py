"""Configuration and registry (no GPU)."""
import json

import pytest

from beglin_b200.config import ConfigError, load_config
from helpers import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config():
    arch, cfg = load_config(TINY_B)
    assert arch.name == "Qwen2ForCausalLM"
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 3, 1)
    assert cfg.head_dim == 32 and cfg.intermediate_size == 200 and cfg.vocab_size == 384
    assert cfg.rope_theta == 1000000.0 and cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and spec.head_name == "lm_head.weight"
    assert all(l.mixer.window is None for l in spec.layers)


def test_head_dim_window_and_scaling_come_from_config():
    arch, cfg = load_config(TINY_C)
    assert cfg.head_dim == 48
    spec = arch.build_spec(cfg)
    assert [l.mixer.window for l in spec.layers] == [None, 24]
    scale = spec.layers[0].mixer.position.freq_scale
    assert len(scale) == 24 and scale[0] == 1.0 and abs(scale[-1] - 1 / 8.0) < 1e-12
    assert spec.head_name is None


def test_config_from_file(tmp_path):
    p = tmp_path / "config.json"
    p.write_text(json.dumps(TINY_A))
    arch, cfg = load_config(str(tmp_path))
    assert cfg.hidden_size == 64 and cfg.tie_word_embeddings is True
    arch2, cfg2 = load_config(str(p))
    assert cfg2 == cfg


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
                                 "num_key_value_heads", "rope_theta", "rms_norm_eps", "vocab_size"])
def test_missing_required_key(key):
    c = dict(TINY_A)
    del c[key]
    with pytest.raises(ConfigError, match=f"missing '{key}'"):
        load_config(c)


@pytest.mark.parametrize("key,bad", [("hidden_size", "64"), ("rope_theta", True), ("tie_word_embeddings", 1),
                                     ("model_type", 3), ("architectures", "Qwen2ForCausalLM"),
                                     ("num_hidden_layers", 2.5)])
def test_wrong_type_is_an_error(key, bad):
    c = dict(TINY_A)
    c[key] = bad
    with pytest.raises(ConfigError):
        load_config(c)


def test_unknown_architecture_lists_supported():
    c = dict(TINY_A, architectures=["MysteryForCausalLM"])
    with pytest.raises(ConfigError, match="supported: .*Qwen2ForCausalLM"):
        load_config(c)
    c = dict(TINY_A)
    del c["architectures"]
    arch, _ = load_config(c)               # falls back to model_type
    assert arch.name == "Qwen2ForCausalLM"
    c["model_type"] = "mystery"
    with pytest.raises(ConfigError):
        load_config(c)


def test_inconsistent_sizes():
    with pytest.raises(ConfigError, match="multiple"):
        load_config(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="divisible"):
        load_config(dict(TINY_A, hidden_size=66))
    with pytest.raises(ConfigError, match="hidden_act"):
        load_config(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="sliding_window"):
        load_config(dict(TINY_A, use_sliding_window=True))
    with pytest.raises(ConfigError, match="llama3"):
        load_config(dict(TINY_A, rope_scaling={"rope_type": "yarn", "factor": 2.0}))


def test_rope_scaling_null_is_none():
    _, cfg = load_config(dict(TINY_A, rope_scaling=None))
    assert cfg.rope_scaling is None


def test_bias_and_tying_follow_the_tensor_list():
    names = ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight"]
    c = dict(TINY_A)
    del c["tie_word_embeddings"]
    _, cfg = load_config(c, tensor_names=names)
    assert cfg.qkv_bias is False and cfg.tie_word_embeddings is True
    _, cfg = load_config(c, tensor_names=names + ["model.layers.0.self_attn.q_proj.bias", "lm_head.weight"])
    assert cfg.qkv_bias is True and cfg.tie_word_embeddings is False
    with pytest.raises(ConfigError, match="lm_head"):
        load_config(dict(TINY_A, tie_word_embeddings=False), tensor_names=names)
    # a folder that says "tied" but carries a head of its own: the tensor wins, as in the reference
    _, cfg = load_config(dict(TINY_A, tie_word_embeddings=True), tensor_names=names + ["lm_head.weight"])
    assert cfg.tie_word_embeddings is False


def test_json_roundtrip_of_typed_config():
    _, cfg = load_config(TINY_C)
    _, again = load_config(cfg.to_json_dict())
    assert again == cfg


def test_command_line_takes_the_configuration_from_qwen_hf_config(tmp_path, monkeypatch, capsys):
    """QWEN_HF_CONFIG names the config.json (qwen_infer.c:20121); a path that does not exist is reported with
    that path, before anything is loaded."""
    from beglin_b200 import cli
    monkeypatch.setenv("QWEN_BASE", str(tmp_path))
    monkeypatch.setenv("QWEN_HF_CONFIG", str(tmp_path / "elsewhere" / "cfg.json"))
    assert cli.main(["qwen_infer", "greedy", "4"]) == 1
    err = capsys.readouterr().err
    assert "FATAL" in err and "elsewhere/cfg.json" in err and "arch config" in err
    monkeypatch.delenv("QWEN_HF_CONFIG")
    assert cli.main(["qwen_infer", "greedy", "4"]) == 1
    assert str(tmp_path / "config.json") in capsys.readouterr().err
