"""Configuration and registry (no GPU)."""

import json

import pytest

from gllm_b200.config import (ARCHITECTURES, ConfigError, GeneratorParams, LlamaConfig, architecture_for,
                              load_config, register_architecture)
from gllm_b200.config.presets import load_preset, preset_names
from tiny_models import TINY, TINY_A, TINY_B, TINY_C


def test_every_size_comes_from_config_json():
    a, b = load_config(dict(TINY_A)), load_config(dict(TINY_B))
    assert isinstance(a, LlamaConfig)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 3, 1, 32)
    assert a.rope_scaling is None and b.rope_scaling.factor == 8.0
    assert b.rope_scaling.original_max_position_embeddings == 64
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.eos_token_ids == (255,) and b.eos_token_ids == (7,)   # list and int both accepted
    assert a.dtype == "float32" and b.dtype == "bfloat16"
    assert a.rms_norm_eps == 1e-5 and b.rms_norm_eps == 1e-6


def test_round_trip_through_config_json(tmp_path):
    for raw in TINY.values():
        cfg = load_config(dict(raw))
        p = tmp_path / "config.json"
        p.write_text(json.dumps(cfg.to_dict()))
        assert load_config(str(tmp_path)) == cfg
        assert load_config(str(p)) == cfg


def test_defaults_and_window():
    raw = dict(TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"], raw["rope_theta"]
    cfg = load_config(raw)
    assert cfg.head_dim == 16 and cfg.num_key_value_heads == 4 and cfg.rope_theta == 10000.0
    c = load_config(dict(TINY_C))
    assert c.sliding_window == 24 and c.layer_types[1] == "sliding_attention"
    only_window = dict(TINY_A, sliding_window=8)
    assert load_config(only_window).layer_types == ("sliding_attention",) * 2


def test_bias_keys_are_read_and_written_back(tmp_path):
    """``attention_bias`` / ``mlp_bias``: false where absent (every Llama 3.x checkpoint), carried through
    ``to_dict``, and the random-weights mode writes the bias tensors the keys ask for and no others."""
    from safetensors.torch import load_file

    from gllm_b200.weights import write_random_model

    assert not load_config(dict(TINY_A)).attention_bias and not load_config(dict(TINY_A)).mlp_bias
    c = load_config(dict(TINY_C))
    assert c.attention_bias and not c.mlp_bias
    assert load_config(c.to_dict()) == c
    names = set(load_file(write_random_model(str(tmp_path / "m"), c, seed=1) + "/model.safetensors"))
    assert "model.layers.0.self_attn.o_proj.bias" in names and "model.layers.2.self_attn.k_proj.bias" in names
    assert not any("mlp" in n and n.endswith(".bias") for n in names)


@pytest.mark.parametrize("change,match", [
    (dict(hidden_size=None), "hidden_size"),
    (dict(rms_norm_eps=None), "rms_norm_eps"),
    (dict(vocab_size=None), "vocab_size"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias="yes"), "attention_bias"),
    (dict(torch_dtype="float16"), "torch_dtype"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_scaling"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "low_freq_factor"),
    (dict(head_dim=15), "head_dim"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["sliding_attention", "full_attention"]), "sliding_window"),
    (dict(eos_token_id="x"), "eos_token_id"),
])
def test_bad_config_is_refused(change, match):
    raw = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            del raw[k]
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=match):
        load_config(raw)


def test_registry():
    assert architecture_for("LlamaForCausalLM").config_class is LlamaConfig
    with pytest.raises(KeyError, match="LlamaForCausalLM"):
        architecture_for("NoSuchModel")
    with pytest.raises(ConfigError, match="architectures"):
        load_config({"hidden_size": 8})
    marker = object()
    register_architecture("ToyForTest", LlamaConfig, lambda cfg: marker)
    try:
        cfg = load_config(dict(TINY_A, architectures=["ToyForTest"]))
        assert cfg.architecture == "ToyForTest"
        assert architecture_for("ToyForTest").build_spec(cfg) is marker
    finally:
        del ARCHITECTURES["ToyForTest"]


def test_spec_is_data():
    cfg = load_config(dict(TINY_C))
    spec = architecture_for(cfg.architecture).build_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.plan] == [0, 1, 2]
    assert spec.layers[1].mixer.params["window"] == 24 and spec.layers[0].mixer.params["window"] is None
    assert spec.layers[0].mixer.kind == "attention" and spec.layers[0].feed_forward.kind == "swiglu"
    assert spec.head_name is None and spec.ignorable_names == ("lm_head.weight",)
    assert architecture_for("LlamaForCausalLM").build_spec(load_config(dict(TINY_B))).head_name == "lm_head.weight"


def test_generator_params():
    p = GeneratorParams(block_size=16, max_batch_size=8, max_seq_len=4096)
    assert p.resolved_num_blocks() == 8 * 256 and p.max_blocks_per_request == 256
    assert GeneratorParams(16, 1, 100, model_dtype="fp32").model_dtype == "float32"
    with pytest.raises(ValueError):
        GeneratorParams(0, 1, 1)
    with pytest.raises(ValueError):
        GeneratorParams(16, 1, 16, model_dtype="int8")
    with pytest.raises(ValueError, match="kv_dtype"):
        GeneratorParams(16, 1, 16, model_dtype="bfloat16", kv_dtype="float32")


def test_presets_parse():
    assert "llama-3.2-1b" in preset_names()
    cfg = load_config(load_preset("llama-3.2-1b"))
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.vocab_size, cfg.head_dim) == (16, 2048, 128256, 64)
    assert cfg.rope_scaling.factor == 32.0 and cfg.tie_word_embeddings
    assert not load_config(load_preset("llama-3.1-8b")).tie_word_embeddings
