"""The plain implementation itself (no GPU): against the outputs of the
reference's own model code on the tiny models A and B (tests/golden, made by
tests/golden/make_golden.py), and its parts against known values.

A is anchored whole, token by token from the reference's cache, and for requests
that arrive beside decoding neighbours.  B is anchored in everything but the two
things the reference lacks: the llama3 scaling rule (the reference ran with a
table of angles made from the plain frequencies) and the choice of an untied head
matrix; those two are held by the property tests below."""

import json
import math
import os

import pytest
import torch
from safetensors.torch import load_file

from plain_llama import (plain_attention, plain_forward, plain_inverse_frequencies, plain_rmsnorm, plain_rope,
                         plain_sampling_distribution, plain_top_logprobs)
from tiny_models import TINY_A, TINY_B, read_raw, write_tiny

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_equals_the_reference_model_code(tmp_path):
    golden = load_file(os.path.join(GOLDEN, "tiny_a_reference.safetensors"))
    with open(os.path.join(GOLDEN, "tiny_a_reference.json")) as f:
        meta = json.load(f)
    folder = write_tiny("A", str(tmp_path / "m"))
    cfg, weights = read_raw(folder)
    for i, prompt in enumerate(meta["prompts"]):
        want = golden[f"logits_{i}"]
        got32 = plain_forward(cfg, weights, prompt, torch.float32)
        got64 = plain_forward(cfg, weights, prompt, torch.float64)
        assert got32.shape == want.shape
        assert float((got32 - want).abs().max()) < 5e-6
        assert float((got64 - want.double()).abs().max()) < 5e-6
        # greedy continuation, token by token, as the reference generated it
        tokens = list(prompt)
        for t in meta["greedy"][i]:
            assert int(plain_forward(cfg, weights, tokens, torch.float64)[-1].argmax()) == t
            tokens.append(t)


def _golden(name):
    with open(os.path.join(GOLDEN, f"{name}.json")) as f:
        meta = json.load(f)
    return load_file(os.path.join(GOLDEN, f"{name}.safetensors")), meta


def test_plain_equals_the_reference_decoding_token_by_token_and_mixed_arrival(tmp_path):
    golden, meta = _golden("tiny_a_reference")
    cfg, weights = read_raw(write_tiny("A", str(tmp_path / "m")))
    prompts, conts = meta["prompts"], meta["continuations"]
    # the reference decoded the continuation of prompt 2 one token at a time from its cache
    whole = plain_forward(cfg, weights, prompts[2] + conts[2], torch.float32)
    want = golden["decode_2"]
    assert want.shape[0] == len(conts[2])
    assert float((whole[len(prompts[2]):] - want).abs().max()) < 5e-6
    # arrivals: request i joins at step i with its whole prompt, then brings its fixed tokens one by one
    fed = [0, 0, 0]
    for s, active in enumerate(meta["mixed_schedule"]):
        for i in active:
            n_prompt = len(prompts[i])
            seq = prompts[i] + conts[i][:fed[i]]
            logits = plain_forward(cfg, weights, seq, torch.float32)
            want = golden[f"mixed_{s}_{i}"]
            got = logits if fed[i] == 0 else logits[-1:]
            assert got.shape == want.shape and (fed[i] > 0 or got.shape[0] == n_prompt)
            assert float((got - want).abs().max()) < 5e-6, (s, i)
            fed[i] += 1


def test_plain_equals_the_reference_on_tiny_b_with_its_table_and_head_put_in(tmp_path):
    golden, meta = _golden("tiny_b_reference")
    cfg, weights = read_raw(write_tiny("B", str(tmp_path / "m")))
    assert cfg["rope_scaling"]["rope_type"] == "llama3" and not cfg["tie_word_embeddings"]
    for i, prompt in enumerate(meta["prompts"]):
        got = plain_forward(cfg, weights, prompt, torch.float32)
        want = golden[f"logits_{i}"]
        assert got.shape == want.shape
        assert float((got - want).abs().max()) < 1e-5, i
    seq = meta["prompts"][3] + meta["continuation"]
    got = plain_forward(cfg, weights, seq, torch.float32)[len(meta["prompts"][3]):]
    assert float((got - golden["decode_3"]).abs().max()) < 1e-5
    assert float(golden["decode_3"].abs().max()) > 0.1              # the comparison is not of zeros


def test_llama3_rule_is_continuous_monotone_and_has_the_stated_limits():
    """The rule's published meaning, checked as properties over a dense sweep of
    wavelengths instead of the few frequencies a head size gives: short waves
    untouched, long waves slowed by ``factor``, a straight blend in between
    that meets both ends, and a larger factor never speeds a frequency up."""
    for factor, low, high, orig in ((8.0, 1.0, 4.0, 64.0), (32.0, 1.0, 4.0, 8192.0)):
        d = 4096
        cfg = dict(head_dim=d, hidden_size=d, num_attention_heads=1, rope_theta=500000.0,
                   rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=low, high_freq_factor=high,
                                     original_max_position_embeddings=orig))
        f = plain_inverse_frequencies(cfg)
        base = plain_inverse_frequencies({k: v for k, v in cfg.items() if k != "rope_scaling"})
        wl = 2 * math.pi / base
        ratio = f / base
        assert torch.equal(ratio[wl < orig / high], torch.ones_like(ratio[wl < orig / high]))
        torch.testing.assert_close(ratio[wl > orig / low], torch.full_like(ratio[wl > orig / low], 1 / factor))
        assert (ratio[1:] <= ratio[:-1] + 1e-12).all()                # longer waves are slowed at least as much
        assert float((ratio[1:] - ratio[:-1]).abs().max()) < 0.01     # no jump at either edge of the blend
        mid = (wl >= orig / high) & (wl <= orig / low)
        smooth = (orig / wl[mid] - low) / (high - low)                # 1 at the short edge, 0 at the long edge
        torch.testing.assert_close(ratio[mid], (1 - smooth) / factor + smooth)


def test_llama3_frequencies_hit_all_three_branches():
    f = plain_inverse_frequencies(dict(TINY_B))
    base = 500000.0 ** (-2.0 * torch.arange(16, dtype=torch.float64) / 32)
    # original 64: wavelengths < 16 kept, > 64 divided by 8, between interpolated
    wl = 2 * math.pi / base
    kept, divided = wl < 16, wl > 64
    assert kept.any() and divided.any() and (~kept & ~divided).any()
    assert torch.equal(f[kept], base[kept])
    torch.testing.assert_close(f[divided], base[divided] / 8)
    mid = ~kept & ~divided
    assert ((f[mid] < base[mid]) & (f[mid] > base[mid] / 8)).all()
    assert torch.equal(plain_inverse_frequencies(dict(TINY_A)), 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16))


def test_rope_is_a_rotation_of_the_two_halves():
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    inv = torch.tensor([1.0, 0.5, 0.25, 0.125], dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 3, 7])
    y = plain_rope(x, pos, inv)
    assert torch.equal(y[0], x[0])                                            # position 0: identity
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))
    a = 7 * 0.5
    torch.testing.assert_close(y[4, 1, 1], x[4, 1, 1] * math.cos(a) - x[4, 1, 5] * math.sin(a))
    torch.testing.assert_close(y[4, 1, 5], x[4, 1, 1] * math.sin(a) + x[4, 1, 5] * math.cos(a))


def test_rmsnorm_and_attention_values():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    torch.testing.assert_close(plain_rmsnorm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0),
                               torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]], dtype=torch.float64))
    q = torch.zeros(3, 2, 4, dtype=torch.float64)
    k = torch.zeros(3, 1, 4, dtype=torch.float64)
    v = torch.arange(12, dtype=torch.float64).view(3, 1, 4)
    pos = torch.arange(3)
    o = plain_attention(q, k, v, pos, pos)                                   # uniform scores: causal running mean
    torch.testing.assert_close(o[2, 0], v[:, 0].mean(0))
    torch.testing.assert_close(o[0, 1], v[0, 0])
    o = plain_attention(q, k, v, pos, pos, window=2)
    torch.testing.assert_close(o[2, 0], v[1:, 0].mean(0))                    # position 2 sees 1 and 2 only


def test_untied_head_and_plan(tmp_path):
    folder = write_tiny("B", str(tmp_path / "m"))
    cfg, w = read_raw(folder)
    toks = [1, 2, 3, 4, 5]
    base = plain_forward(cfg, w, toks)
    w2 = dict(w)
    w2["lm_head.weight"] = w["lm_head.weight"] * 2
    torch.testing.assert_close(plain_forward(cfg, w2, toks), base * 2)
    twice = plain_forward(cfg, w, toks, plan=[(0, None), (1, None), (1, None), (2, None)])
    assert float((twice - base).abs().max()) > 1e-3
    shared = plain_forward(cfg, w, toks, plan=[(0, None), (1, None), (2, 1)])
    assert float((shared - base).abs().max()) > 1e-4


def test_activations_kept_in_bfloat16(tmp_path):
    """``stored``: keeping activations in the dtype of the call changes nothing; keeping them in bfloat16 moves
    the logits by bfloat16 rounding (a part in a hundred at most here), not by more."""
    folder = write_tiny("A", str(tmp_path / "m"))
    cfg, w = read_raw(folder, round_to_bf16=True)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg["vocab_size"], (40,), generator=g).tolist()
    exact = plain_forward(cfg, w, toks)
    assert torch.equal(plain_forward(cfg, w, toks, stored=torch.float64), exact)
    kept = plain_forward(cfg, w, toks, stored=torch.bfloat16)
    err = float((kept - exact).abs().max()) / float(exact.abs().max())
    assert 1e-5 < err < 2e-2, err


def test_sampler_distribution_rules():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 3.0])
    p, n = plain_sampling_distribution(logits, 1.0, 0, 1.0)
    torch.testing.assert_close(p, torch.softmax(logits.double(), -1))
    assert n == 5
    p, n = plain_sampling_distribution(logits, 1.0, 2, 1.0)
    assert n == 2 and p[4] > p[0] > 0 and float(p[1] + p[2] + p[3]) == 0
    # softmax = .636 .234 .086 ...: cumulative .636, .870: top_p .8 keeps only the first (the crossing one is dropped)
    p, n = plain_sampling_distribution(logits, 1.0, 0, 0.8)
    assert n == 1 and float(p[4]) == 1.0
    p, n = plain_sampling_distribution(logits, 1.0, 0, 0.9)
    assert n == 2
    p, n = plain_sampling_distribution(logits, 1.0, 0, 0.01)
    assert n == 1                                                             # the first is always kept
    vals, ids = plain_top_logprobs(logits, 2)
    assert ids.tolist() == [4, 0]
    torch.testing.assert_close(vals, torch.log_softmax(logits.double(), -1)[[4, 0]])
