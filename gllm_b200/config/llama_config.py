"""``LlamaForCausalLM``'s own config.json keys as a typed configuration.

The reference reads nine of them (gllm/model/model.py:63-76) and ignores
``rope_scaling``, ``vocab_size``, ``tie_word_embeddings`` and ``architectures``.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any

from gllm_b200.config.model_config import DTYPE_NAMES, ConfigError, ModelConfig, as_eos, require


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json with ``rope_type: "llama3"``.

    The reference ignores this key (gllm/model/model.py:117-128 builds the
    table from ``rope_theta`` alone), so long-context Llama 3.x checkpoints
    would get unscaled frequencies there.  The four numbers have their
    published meaning: frequencies whose wavelength is longer than
    ``original_max_position_embeddings / low_freq_factor`` are divided by
    ``factor``, those shorter than ``original / high_freq_factor`` are kept,
    and the band between is interpolated.
    """

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """``LlamaForCausalLM``: pre-norm RMSNorm decoder, grouped-query attention
    with rotary positions, SwiGLU feed-forward, tied or untied head."""

    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    hidden_act: str = "silu"
    rms_norm_eps: float = 0.0
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    tie_word_embeddings: bool = False
    max_position_embeddings: int | None = None
    bos_token_id: int | None = None
    # Optional, absent from Llama 3.x checkpoints: a bounded attention window
    # and which layers use it ("full_attention" | "sliding_attention").
    sliding_window: int | None = None
    layer_types: tuple[str, ...] = field(default_factory=tuple)
    # Biases on the four attention projections / on the three feed-forward projections.  False in every
    # Llama 3.x checkpoint and not read by the reference (gllm/model/layers/attention.py:139-142,
    # gllm/model/layers/mlp.py:44-47 multiply by the weights only).
    attention_bias: bool = False
    mlp_bias: bool = False

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        hidden = int(require(d, "hidden_size"))
        heads = int(require(d, "num_attention_heads"))
        kv_heads = int(d.get("num_key_value_heads", heads))
        layers = int(require(d, "num_hidden_layers"))
        if heads <= 0 or kv_heads <= 0 or layers <= 0 or hidden <= 0:
            raise ConfigError("hidden_size, head counts and num_hidden_layers must be positive")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // heads
        head_dim = int(head_dim)
        if heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})"
            )
        if head_dim % 2:
            raise ConfigError("head_dim must be even (rotary positions pair its two halves)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            # gllm/model/layers/mlp.py:38-41 accepts only silu as well.
            raise ConfigError(f"hidden_act {act!r} is not supported (only 'silu')")
        for bias_key in ("attention_bias", "mlp_bias"):
            if not isinstance(d.get(bias_key, False), bool):
                raise ConfigError(f"{bias_key} must be true or false")
        dtype_name = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype_name not in DTYPE_NAMES:
            raise ConfigError(f"torch_dtype {dtype_name!r} is not one of {sorted(DTYPE_NAMES)}")
        scaling = d.get("rope_scaling")
        rope_scaling = None
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind in (None, "default"):
                rope_scaling = None
            elif kind == "llama3":
                try:
                    rope_scaling = RopeScaling(
                        rope_type="llama3",
                        factor=float(scaling["factor"]),
                        low_freq_factor=float(scaling["low_freq_factor"]),
                        high_freq_factor=float(scaling["high_freq_factor"]),
                        original_max_position_embeddings=int(scaling["original_max_position_embeddings"]),
                    )
                except KeyError as e:
                    raise ConfigError(f"rope_scaling lacks key {e.args[0]!r}") from None
                if rope_scaling.high_freq_factor <= rope_scaling.low_freq_factor:
                    raise ConfigError("rope_scaling.high_freq_factor must exceed low_freq_factor")
                if rope_scaling.factor <= 0:
                    raise ConfigError("rope_scaling.factor must be positive")
            else:
                raise ConfigError(f"rope_scaling type {kind!r} is not supported (only 'llama3')")
        window = d.get("sliding_window")
        layer_types = tuple(d.get("layer_types") or ())
        if layer_types:
            if len(layer_types) != layers:
                raise ConfigError("layer_types must name every layer")
            bad = sorted(set(layer_types) - {"full_attention", "sliding_attention"})
            if bad:
                raise ConfigError(f"unknown layer_types {bad}")
            if "sliding_attention" in layer_types and not window:
                raise ConfigError("layer_types names sliding_attention but sliding_window is absent")
        elif window:
            layer_types = ("sliding_attention",) * layers
        if window is not None and int(window) <= 0:
            raise ConfigError("sliding_window must be positive")
        eps = float(require(d, "rms_norm_eps"))
        if not eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        vocab = int(require(d, "vocab_size"))
        max_pos = d.get("max_position_embeddings")
        return cls(
            architecture=str(archs[0]),
            vocab_size=vocab,
            hidden_size=hidden,
            dtype=DTYPE_NAMES[dtype_name],
            eos_token_ids=as_eos(d.get("eos_token_id")),
            intermediate_size=int(require(d, "intermediate_size")),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            hidden_act=act,
            rms_norm_eps=eps,
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=rope_scaling,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=None if max_pos is None else int(max_pos),
            bos_token_id=d.get("bos_token_id"),
            sliding_window=None if window is None else int(window),
            layer_types=layer_types,
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
        )

    def to_dict(self) -> dict[str, Any]:
        """The config.json that ``from_dict`` reads back to an equal object."""
        d: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else asdict(self.rope_scaling),
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.dtype,
            "eos_token_id": list(self.eos_token_ids),
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
        }
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
            d["layer_types"] = list(self.layer_types)
        return d
