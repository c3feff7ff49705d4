"""The tiny configurations the tests use, as raw config.json dicts, and helpers
that write them as model folders with random weights in a temporary place.

They differ in every size and option: layers, width, head counts and groups
(GQA, MQA, MHA), head size, feed-forward width, vocabulary (384 and the odd
311), rope base and scaling, eps, tied or untied head, stored dtype, norm
weights, and (C, D) a bounded window on one layer; D has the head size of 64
that the tensor-core attention kernels are tuned for.
"""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import load_file

TINY_A = dict(
    architectures=["LlamaForCausalLM"], hidden_size=64, head_dim=16, intermediate_size=128, hidden_act="silu",
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, eos_token_id=[255],
    torch_dtype="float32", rope_theta=10000.0, vocab_size=256, tie_word_embeddings=True,
)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=96, head_dim=32, intermediate_size=160, hidden_act="silu",
    num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, rms_norm_eps=1e-6, eos_token_id=7,
    torch_dtype="bfloat16", rope_theta=500000.0, vocab_size=384, tie_word_embeddings=False,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
)
TINY_C = dict(
    architectures=["LlamaForCausalLM"], hidden_size=72, head_dim=16, intermediate_size=104, hidden_act="silu",
    num_hidden_layers=3, num_attention_heads=5, num_key_value_heads=5, rms_norm_eps=3e-5, eos_token_id=[1, 2],
    torch_dtype="bfloat16", rope_theta=30000.0, vocab_size=311, tie_word_embeddings=True,
    sliding_window=24, layer_types=["full_attention", "sliding_attention", "full_attention"], attention_bias=True,
)
TINY_D = dict(
    architectures=["LlamaForCausalLM"], hidden_size=128, head_dim=64, intermediate_size=200, hidden_act="silu",
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, rms_norm_eps=1e-5, eos_token_id=[0],
    torch_dtype="bfloat16", rope_theta=10000.0, vocab_size=500, tie_word_embeddings=True,
    sliding_window=40, layer_types=["sliding_attention", "full_attention"], mlp_bias=True,
)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
# how each one's random weights are drawn
DRAW = {
    "A": dict(seed=11, std=0.05, norm_jitter=0.0, std_overrides={"q_proj": 0.3, "k_proj": 0.3}),
    "B": dict(seed=12, std=0.04, norm_jitter=0.1, std_overrides={"q_proj": 0.25, "k_proj": 0.25}),
    "C": dict(seed=13, std=0.05, norm_jitter=0.05, std_overrides={"q_proj": 0.3, "k_proj": 0.3}),
    "D": dict(seed=14, std=0.04, norm_jitter=0.05, std_overrides={"q_proj": 0.2, "k_proj": 0.2}),
}


def write_tiny(name: str, folder: str, sharp: bool = True) -> str:
    """Write tiny model ``name`` into ``folder`` through the engine's
    random-weights mode and return the folder.

    ``sharp`` draws the query and key projections six times wider than the
    rest, so scores are large and attention settles on few keys: a key that is
    missed, doubled or read from a wrong page then moves the logits by far more
    than float32 rounding.  bfloat16 cannot resolve scores that large (its
    rounding of q and k alone moves such logits by over ten percent), so
    bfloat16 runs draw those projections only three times wider.
    """
    from gllm_b200.config import load_config
    from gllm_b200.weights import write_random_model

    cfg = load_config(dict(TINY[name]))
    draw = dict(DRAW[name])
    if not sharp:
        draw["std_overrides"] = {k: v / 2 for k, v in draw["std_overrides"].items()}
    return write_random_model(folder, cfg, **draw)


def read_raw(folder: str, round_to_bf16: bool = False):
    """(config.json dict, {name: tensor}) as stored; with ``round_to_bf16`` the
    matrices are rounded to bf16 values (norm weights stay as stored), which is
    what a bfloat16 run of the engine holds."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = load_file(os.path.join(folder, "model.safetensors"))
    if round_to_bf16:
        weights = {
            k: (v.to(torch.bfloat16).to(torch.float32) if v.dim() >= 2 else v.to(torch.float32))
            for k, v in weights.items()
        }
    return cfg, weights
