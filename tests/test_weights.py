"""Checkpoint reading and the random-weights mode (no GPU)."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from gllm_b200.config import load_config
from gllm_b200.models.decoder import DecoderModel, expected_tensors_of_spec
from gllm_b200.config.registry import architecture_for
from gllm_b200.weights import WeightError, open_checkpoint, write_random_model
from tiny_models import TINY_A, TINY_B, write_tiny


def _model(folder, dtype=torch.float32):
    cfg = load_config(folder)
    return DecoderModel(architecture_for(cfg.architecture).build_spec(cfg), dtype, "cpu")


def test_random_mode_writes_a_loadable_folder(tmp_path):
    folder = write_tiny("B", str(tmp_path / "m"))
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    raw = load_file(os.path.join(folder, "model.safetensors"))
    assert raw["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert raw["lm_head.weight"].shape == (384, 96)                      # untied head is drawn
    assert raw["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    w = raw["model.norm.weight"].float()
    assert 0.05 < (w - 1).abs().mean() < 0.2                             # 1 + N(0, 0.1)
    again = write_tiny("B", str(tmp_path / "m2"))
    raw2 = load_file(os.path.join(again, "model.safetensors"))
    assert all(torch.equal(raw[k], raw2[k]) for k in raw)                # same seed, same weights
    model = _model(folder, torch.bfloat16)
    model.load(open_checkpoint(folder))
    assert model.head is not model.embedding
    assert model.layers[0].mixer.w_qkv.shape == ((3 + 2) * 32, 96)
    assert model.layers[0].mixer.w_qkv.dtype == torch.bfloat16
    assert model.layers[0].mixer_norm.weight.dtype == torch.float32      # vectors stay 32-bit


def test_tied_head_and_dtype_policy(tmp_path):
    folder = write_tiny("A", str(tmp_path / "m"))                        # stored in float32
    raw = load_file(os.path.join(folder, "model.safetensors"))
    assert "lm_head.weight" not in raw and raw["model.embed_tokens.weight"].dtype == torch.float32
    m32 = _model(folder, torch.float32)
    m32.load(open_checkpoint(folder))
    assert m32.head is m32.embedding and m32.embedding.dtype == torch.float32
    assert torch.equal(m32.embedding, raw["model.embed_tokens.weight"])
    m16 = _model(folder, torch.bfloat16)
    m16.load(open_checkpoint(folder))
    assert m16.embedding.dtype == torch.bfloat16
    # a stored head beside tied embeddings is ignored, not an error
    raw["lm_head.weight"] = raw["model.embed_tokens.weight"].clone()
    save_file(raw, os.path.join(folder, "model.safetensors"))
    _model(folder).load(open_checkpoint(folder))


def test_one_error_lists_everything(tmp_path):
    folder = write_tiny("B", str(tmp_path / "m"))
    path = os.path.join(folder, "model.safetensors")
    raw = load_file(path)
    del raw["model.layers.1.mlp.up_proj.weight"]
    del raw["lm_head.weight"]
    raw["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
    raw["model.layers.0.rotary.inv_freq"] = torch.zeros(16)
    save_file(raw, path)
    with pytest.raises(WeightError) as err:
        _model(folder).load(open_checkpoint(folder))
    msg = str(err.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "lm_head.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.rotary.inv_freq" in msg
    assert "wrong shapes (1)" in msg and "found [96, 95], expected [96, 96]" in msg


def test_sharded_checkpoint_and_missing_folder(tmp_path):
    folder = write_tiny("A", str(tmp_path / "m"))
    path = os.path.join(folder, "model.safetensors")
    raw = load_file(path)
    names = sorted(raw)
    half = len(names) // 2
    save_file({k: raw[k] for k in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({k: raw[k] for k in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    os.remove(path)
    index = {"weight_map": {k: f"model-0000{1 if i < half else 2}-of-00002.safetensors" for i, k in enumerate(names)}}
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    m = _model(folder)
    m.load(open_checkpoint(folder))
    assert torch.equal(m.embedding, raw["model.embed_tokens.weight"])
    with pytest.raises(WeightError, match="does not exist"):
        open_checkpoint(str(tmp_path / "nope"))
    os.makedirs(tmp_path / "empty")
    with pytest.raises(WeightError, match="no .safetensors"):
        open_checkpoint(str(tmp_path / "empty"))


def test_expected_tensor_table_matches_the_reference_names():
    cfg = load_config(dict(TINY_A))
    exp = expected_tensors_of_spec(architecture_for(cfg.architecture).build_spec(cfg))
    assert exp["model.embed_tokens.weight"].shape == (256, 64)
    assert exp["model.layers.1.self_attn.v_proj.weight"].shape == (32, 64)
    assert exp["model.layers.0.mlp.down_proj.weight"].shape == (64, 128)
    assert exp["model.layers.0.post_attention_layernorm.weight"].role == "vector"
    assert "lm_head.weight" not in exp and len(exp) == 2 + 2 * 9
