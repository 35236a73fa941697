"""Configuration and registry."""

import json

import pytest

import shrike_b200.models  # noqa: F401
from shrike_b200.config import (
    ARCHITECTURES, ConfigError, LayerRun, load_config, parse_config,
)
from tests.tiny_configs import TINY, TINY_A, TINY_B, TINY_C


def test_package_import_is_light():
    import subprocess
    import sys

    code = "import sys, shrike_b200; assert 'torch' not in sys.modules; print(shrike_b200.SamplingParams().max_new_tokens)"
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(__import__('pathlib').Path(__file__).parents[1]))
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip() == "128"


def test_sizes_come_from_config_json():
    a, b = parse_config(TINY_A), parse_config(TINY_B)
    assert (a.hidden_size, a.vocab_size, a.num_layers) == (64, 256, 2)
    assert (b.hidden_size, b.vocab_size, b.num_layers) == (192, 384, 3)
    ma, mb = a.layers[0].mixer, b.layers[0].mixer
    assert (ma.num_heads, ma.num_kv_heads, ma.head_dim) == (4, 2, 16)
    assert (mb.num_heads, mb.num_kv_heads, mb.head_dim) == (6, 3, 32)  # head_dim derived: 192 // 6
    assert ma.scale == 16 ** -0.5 and mb.scale == 32 ** -0.5
    assert ma.position.theta == 10000.0 and mb.position.theta == 1e6
    assert a.layers[0].mixer_norm.eps == 1e-6 and b.final_norm.eps == 1e-5
    assert a.layers[1].feed_forward.intermediate == 128 and b.layers[2].feed_forward.intermediate == 320
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.eos_token_ids == [255] and b.eos_token_ids == [383]
    assert ma.qkv_bias and not ma.out_bias
    assert [r.layer for r in b.order] == [0, 1, 2] and [r.cache for r in b.order] == [0, 1, 2]


def test_window_layers():
    c = parse_config(TINY_C)
    assert [layer.mixer.window for layer in c.layers] == [None, 24, 24, 24]
    assert all(layer.mixer.window is None for layer in parse_config(TINY_A).layers)


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta"])
def test_missing_key_is_named(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        parse_config(raw)


def test_bad_values_are_refused():
    with pytest.raises(ConfigError, match="multiple"):
        parse_config(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="rope_scaling"):
        parse_config(dict(TINY_A, rope_scaling={"type": "yarn", "factor": 4}))
    with pytest.raises(ConfigError, match="hidden_act"):
        parse_config(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="dtype"):
        parse_config(dict(TINY_A, torch_dtype="float16"))
    with pytest.raises(ConfigError, match="positive integer"):
        parse_config(dict(TINY_A, hidden_size=-4))


def test_registry_dispatches_on_architecture():
    assert "Qwen2ForCausalLM" in ARCHITECTURES
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*Qwen2ForCausalLM"):
        parse_config(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        parse_config({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_dtype_names():
    assert parse_config(dict(TINY_A, torch_dtype="bfloat16")).dtype == "bfloat16"
    raw = {k: v for k, v in TINY_A.items() if k != "torch_dtype"}
    assert parse_config(raw).dtype == "bfloat16"  # the reference's default (qwen.py:49)
    assert parse_config(dict(raw, dtype="float32")).dtype == "float32"


def test_load_config_and_missing_file(tmp_path):
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(tmp_path).hidden_size == 192


def test_run_order_is_validated():
    config = parse_config(TINY_A)
    config.order = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(1, 1, writes_cache=False)]
    config.validate()
    config.order = [LayerRun(0, 0), LayerRun(1, 0)]
    with pytest.raises(ConfigError, match="both write cache 0"):
        config.validate()
    config.order = [LayerRun(0, 1, writes_cache=False)]
    with pytest.raises(ConfigError, match="before any run wrote"):
        config.validate()
    config.order = [LayerRun(5, 0)]
    with pytest.raises(ConfigError, match="names layer 5"):
        config.validate()


def test_tiny_configs_differ_everywhere():
    keys = ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta"]
    for key in keys:
        assert len({TINY[name][key] for name in "ABC"}) == 3, key
