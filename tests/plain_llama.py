"""A plain, slow implementation of the Llama decoder for the tests to compare
the engine with: whole sequences, no cache, no batching, one function for each
part.  It shares no code with ``gllm_b200`` (it reads the raw config.json dict
and the raw tensors) and every function cites the reference formula it restates
(paths are inside TheEpicDolphin/gllm).

Two things the reference does not have are written from their published
meaning, not from the reference: llama3 frequency scaling (the reference
ignores ``rope_scaling``, gllm/model/model.py:117-128) and an untied output head
(the reference always multiplies by the embedding table,
gllm/model/model.py:232-239).  A bounded attention window, which Llama 3.x does
not use, follows the usual meaning: a token at position p sees positions
p - window + 1 .. p.

Where the reference computes in the model dtype (norm statistics, softmax, the
cos/sin table) this file computes in the dtype it is called with (float32 or
float64): it is the exact-arithmetic meaning of the formulas, which the engine's
fp32 path must match to rounding.

``plain_forward(..., stored=torch.bfloat16)`` is the same arithmetic with every activation that a bfloat16
model keeps between two operations rounded to bfloat16 where it is kept: the outputs of the norms, of the
q/k/v projections, of the rotation, of the attention, and SiLU(gate) * up.  The residual stream, the
statistics, the softmax and the logits stay in the dtype of the call.  It is what a bfloat16 engine
computes up to the order of its sums, so a bfloat16 run can be held to a much closer bound than against
the exact arithmetic.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ positions
def plain_inverse_frequencies(cfg: dict) -> torch.Tensor:
    """theta_m = rope_theta ** (-2m / D), m = 0 .. D/2-1  (gllm/model/model.py:121-122),
    then the llama3 rule on each frequency.  float64."""
    d = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    theta = float(cfg.get("rope_theta", 10000.0))
    m = torch.arange(d // 2, dtype=torch.float64)
    freq = theta ** (-2.0 * m / d)
    scaling = cfg.get("rope_scaling")
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / freq
        smooth = (orig / wavelen - low) / (high - low)
        mid = (1.0 - smooth) * freq / factor + smooth * freq
        freq = torch.where(wavelen < orig / high, freq, torch.where(wavelen > orig / low, freq / factor, mid))
    return freq


def plain_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [T, heads, D]: split each head in its two halves x1 | x2 and return
    [x1*cos - x2*sin | x1*sin + x2*cos]  (gllm/model/layers/attention.py:91-118),
    angle[p, m] = p * theta_m  (gllm/model/model.py:124).  The frequencies are
    rounded to float32 once (as the engine holds them), the angle is formed in
    float32, and sine and cosine are taken in x's dtype."""
    d = x.shape[-1]
    ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(x.dtype)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


# ----------------------------------------------------------------------- norm
def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x*x) + eps) * w  (gllm/model/layers/norm.py:20-22)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------ attention
def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_positions: torch.Tensor,
                    k_positions: torch.Tensor, window: int | None = None,
                    scale: float | None = None) -> torch.Tensor:
    """q [Tq, Hq, D], k, v [T, Hkv, D] -> [Tq, Hq, D].
    Kv head of query head h is h // (Hq/Hkv): the expand/reshape of
    gllm/ops/attention/reference_attention.py:19-30.  Scores QK^T / D**0.5 (:40),
    -inf where the key lies after the query (the triu bias of
    gllm/llm/llm.py:272-274), softmax over keys (:45), times V (:48)."""
    tq, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    k = k.repeat_interleave(g, dim=1)
    v = v.repeat_interleave(g, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k)
    scores = scores * scale if scale is not None else scores / d ** 0.5
    qp, kp = q_positions[:, None], k_positions[None, :]
    hidden = kp > qp
    if window:
        hidden = hidden | (kp <= qp - window)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v)


def _kept(x: torch.Tensor, stored) -> torch.Tensor:
    """x as it reads back after being kept in ``stored`` (None: kept as it is)."""
    return x if stored is None else x.to(stored).to(x.dtype)


def _proj(x, w, name):
    """x W^T, plus the bias ``<name>.bias`` where the checkpoint has one (``attention_bias`` / ``mlp_bias`` in
    config.json; the reference's projections have none, gllm/model/layers/linear.py:20)."""
    y = x @ w[f"{name}.weight"].T
    return y + w[f"{name}.bias"] if f"{name}.bias" in w else y


def plain_attention_layer(x, w, prefix, cfg, positions, inv_freq, window, kv_from=None, stored=None):
    """q/k/v projections without bias (gllm/model/layers/attention.py:139-142),
    heads split along the feature axis (:145-148), rotation of q and k (:151),
    attention, output projection (:181-182).  Returns (out, (k, v)); with
    ``kv_from`` the layer attends over another layer's rotated keys and values."""
    hq, hkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    d = cfg.get("head_dim") or cfg["hidden_size"] // hq
    t = x.shape[0]
    q = _kept(_proj(x, w, f"{prefix}.q_proj"), stored).view(t, hq, d)
    q = _kept(plain_rope(q, positions, inv_freq), stored)
    if kv_from is None:
        k = _kept(_proj(x, w, f"{prefix}.k_proj"), stored).view(t, hkv, d)
        v = _kept(_proj(x, w, f"{prefix}.v_proj"), stored).view(t, hkv, d)
        k = _kept(plain_rope(k, positions, inv_freq), stored)
    else:
        k, v = kv_from
    o = _kept(plain_attention(q, k, v, positions, positions, window), stored)
    return _proj(o.reshape(t, hq * d), w, f"{prefix}.o_proj"), (k, v)


# --------------------------------------------------------------- feed-forward
def plain_mlp(x, w, prefix, stored=None):
    """down(silu(gate(x)) * up(x))  (gllm/model/layers/mlp.py:44-47)."""
    g = _proj(x, w, f"{prefix}.gate_proj")
    u = _proj(x, w, f"{prefix}.up_proj")
    return _proj(_kept(g * torch.sigmoid(g) * u, stored), w, f"{prefix}.down_proj")


# ---------------------------------------------------------------------- model
def plain_forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, plan=None, rows=None,
                  stored=None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence (with ``rows``: only at those positions, [len(rows), V];
    the sequence is still run whole).

    x = E[tokens]  (gllm/model/model.py:175-182); per layer
    x = x + attn(norm_in(x)); x = x + mlp(norm_post(x))  (the deferred adds of
    gllm/model/transformer.py:58-78 written out); logits = norm_f(x) E^T
    (gllm/model/model.py:228-239) or norm_f(x) W_head^T when the head is untied.

    ``plan``: list of (layer, reads_cache_of) in running order; default each
    layer once in order.  ``stored``: the dtype activations are kept in between operations (see the
    head of this file); None keeps them in ``dtype``.
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    inv_freq = plain_inverse_frequencies(cfg)
    eps = cfg["rms_norm_eps"]
    n_layers = cfg["num_hidden_layers"]
    layer_types = cfg.get("layer_types") or (
        ["sliding_attention"] * n_layers if cfg.get("sliding_window") else ["full_attention"] * n_layers
    )
    x = w["model.embed_tokens.weight"][tokens]
    plan = plan if plan is not None else [(i, None) for i in range(n_layers)]
    kv_of_entry = []
    for layer, reads in plan:
        p = f"model.layers.{layer}"
        window = cfg.get("sliding_window") if layer_types[layer] == "sliding_attention" else None
        h = _kept(plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], eps), stored)
        a, kv = plain_attention_layer(h, w, f"{p}.self_attn", cfg, positions, inv_freq, window,
                                      kv_from=None if reads is None else kv_of_entry[reads], stored=stored)
        kv_of_entry.append(kv)
        x = x + a
        h = _kept(plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], eps), stored)
        x = x + plain_mlp(h, w, f"{p}.mlp", stored=stored)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = _kept(plain_rmsnorm(x, w["model.norm.weight"], eps), stored)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


# -------------------------------------------------------------------- sampler
def plain_sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """The distribution the reference samples from, for one row
    (gllm/sample/sampler.py:67-88): divide by temperature (:77); keep the top_k
    highest (0 = whole vocabulary, :35-45); softmax over them, cumulative sum in
    descending order, keep entries whose cumulative sum is <= top_p and always
    the first (:56-63); softmax again over what is left (:85).
    Returns (probs [V] float64, number of candidates)."""
    z = logits.to(torch.float64) / temperature
    v = z.numel()
    k = v if top_k == 0 else min(top_k, v)
    vals, ids = torch.topk(z, k, sorted=True)
    p = torch.softmax(vals, dim=-1)
    keep = torch.cumsum(p, dim=-1) <= top_p
    keep[0] = True
    vals = vals.masked_fill(~keep, float("-inf"))
    p = torch.softmax(vals, dim=-1)
    out = torch.zeros(v, dtype=torch.float64)
    out[ids] = p
    return out, int(keep.sum())


def plain_top_logprobs(logits: torch.Tensor, num: int):
    """log_softmax of the raw logits (no temperature, whole vocabulary) at the
    ``num`` highest tokens in descending order (gllm/sample/sampler.py:90-106)."""
    lp = torch.log_softmax(logits.to(torch.float64), dim=-1)
    vals, ids = torch.topk(lp, num, sorted=True)
    return vals, ids
