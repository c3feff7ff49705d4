"""``LlamaForCausalLM`` as a ModelSpec: pre-norm RMSNorm decoder, grouped-query
attention with (llama3-scaled) rotary positions, SwiGLU feed-forward, tied or
untied head.  The only architecture the reference runs (gllm/model/model.py).

Tensor names are those the reference reads (gllm/model/model.py:105,115,
gllm/model/transformer.py:21,31, gllm/model/layers/attention.py:55-61,
gllm/model/layers/mlp.py:21-25).  The reference always multiplies by the
embedding table for the head (gllm/model/model.py:232-239); here
``tie_word_embeddings: false`` reads ``lm_head.weight``.
"""

from __future__ import annotations

from dataclasses import asdict

from gllm_b200.config.llama_config import LlamaConfig
from gllm_b200.config.registry import register_architecture
from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rope = PartSpec(
        "rotary",
        dict(
            head_dim=cfg.head_dim,
            rotary_dim=cfg.head_dim,
            theta=cfg.rope_theta,
            scaling=None if cfg.rope_scaling is None else asdict(cfg.rope_scaling),
            interleaved=False,
        ),
    )
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        sliding = bool(cfg.layer_types) and cfg.layer_types[i] == "sliding_attention"
        mixer = PartSpec(
            "attention",
            dict(
                hidden_size=cfg.hidden_size,
                num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim,
                position=rope,
                window=cfg.sliding_window if sliding else None,
                bias=cfg.attention_bias,
                output_bias=cfg.attention_bias,
            ),
            {
                **{n: f"{p}.self_attn.{n}_proj.weight" for n in "qkvo"},
                **({f"{n}_bias": f"{p}.self_attn.{n}_proj.bias" for n in "qkvo"} if cfg.attention_bias else {}),
            },
        )
        ffn = PartSpec(
            "swiglu",
            dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, bias=cfg.mlp_bias),
            {
                **{n: f"{p}.mlp.{n}_proj.weight" for n in ("gate", "up", "down")},
                **({f"{n}_bias": f"{p}.mlp.{n}_proj.bias" for n in ("gate", "up", "down")} if cfg.mlp_bias else {}),
            },
        )
        norm = dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps)
        layers.append(
            LayerSpec("prenorm", dict(
                mixer_norm=PartSpec("rmsnorm", norm, {"weight": f"{p}.input_layernorm.weight"}),
                mixer=mixer,
                feed_forward_norm=PartSpec("rmsnorm", norm, {"weight": f"{p}.post_attention_layernorm.weight"}),
                feed_forward=ffn,
            ))
        )
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=tuple(layers),
        plan=tuple(PlanEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps), {"weight": "model.norm.weight"}),
        embedding_name="model.embed_tokens.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        eos_token_ids=cfg.eos_token_ids,
        ignorable_names=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec)
