"""Replays the same requests through ``bin/trace_run`` whole, with the last 32
tokens one by one, in portions of changing size, and mixed with other requests
over a pool so small that pages are used again, in float32 and in bfloat16, and
compares every logit with the plain implementation."""

import pytest
import torch

from plain_llama import plain_forward
from replay_helpers import (BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN, FP32_TOL, LENGTHS, compare, mixed_steps, replay, rounded,
                            run_steps, sequences, single_request_steps)
from tiny_models import read_raw, write_tiny

pytestmark = pytest.mark.gpu

# tokens per cache page: A and B with the small pages their own configurations name, C and D with 16
PAGE = {"A": 4, "B": 8, "C": 16, "D": 16}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_all_cuts(name, dtype, tmp_path):
    folder = write_tiny(name, str(tmp_path / "model"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    vocab = cfg["vocab_size"]
    seqs = sequences(vocab, seed=5)
    # float32 against the exact arithmetic; bfloat16 against the same arithmetic with the activations kept in
    # bfloat16, which a bfloat16 run follows five times closer than the exact one
    stored = None if dtype == "float32" else torch.bfloat16
    plain = {k: plain_forward(cfg, weights, v, torch.float64, stored=stored) for k, v in seqs.items()}
    tol = (FP32_TOL, None) if dtype == "float32" else (BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN)

    steps, index = single_request_steps(seqs)
    results = replay(folder, dtype, steps, str(tmp_path / "out1"), max_tokens=rounded(max(LENGTHS.values())), vocab=vocab,
                     block_size=PAGE[name])
    compare(results, index, plain, *tol)

    # 4 live requests at most, 448 tokens: less than the requests' total, so pages are used again
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    results = replay(folder, dtype, steps, str(tmp_path / "out2"), max_tokens=448, vocab=vocab, block_size=PAGE[name])
    compare(results, index, plain, *tol)


def test_trace_run_refuses_a_page_that_does_not_fit_the_rounding(tmp_path):
    folder = write_tiny("A", str(tmp_path / "model"))
    with pytest.raises(RuntimeError):
        replay(folder, "float32", [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}], "end": []}],
               str(tmp_path / "out"), max_tokens=64, vocab=256, block_size=24)


@pytest.mark.parametrize("dtype,name", [("float32", "B"), ("bfloat16", "D")])
def test_decoding_across_the_sequence_bucket_of_the_decode_graph(dtype, name, tmp_path):
    """Decode steps are captured per sequence bucket (1,024 tokens, then doubling).  One request
    decodes from 1,010 cached tokens to 1,040: the steps before position 1,024 replay one graph, the
    steps after it another, and the logits on both sides are those of the plain implementation."""
    from gllm_b200.engine.replay import build_runner

    folder = write_tiny(name, str(tmp_path / "model"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    g = torch.Generator().manual_seed(21)
    toks = torch.randint(0, cfg["vocab_size"], (1040,), generator=g).tolist()
    plain = {"x": plain_forward(cfg, weights, toks, torch.float64, stored=None if dtype == "float32" else torch.bfloat16)}
    _, runner = build_runner(folder, dtype, max_tokens=2048, block_size=PAGE[name])
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:1010], "want": [1009]}], "end": []}]
    index = [(0, 0, "x", 1009)]
    for i, p in enumerate(range(1010, 1040)):
        steps.append({"step": i + 1, "entries": [{"id": "r", "tokens": [toks[p]], "want": [0]}], "end": []})
        index.append((i + 1, 0, "x", p))
    results = run_steps(runner, steps)
    tol = (FP32_TOL, None) if dtype == "float32" else (BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN)
    compare(results, index, plain, *tol)
    keys = [k for k in runner._graphs if k[0] == "decode"]
    assert {k[2] for k in keys} == {1024, 2048}, keys
    assert runner.graph_replays >= 20


@pytest.mark.parametrize("pair_gemm", [False, True])
def test_replay_through_the_stream_decode_kernel(tmp_path, monkeypatch, pair_gemm):
    """The single tokens of tiny D (head size 64, one kv head, a window of 40 on one layer, pages of
    16) through the persistent TMA decode kernel, which steps this small would not pick by themselves:
    the tail decoded token by token, and the mixed steps with pages used again.  The second time every
    product that is not cut along K also runs on pairs of CTAs, as in large mixed steps."""
    monkeypatch.setenv("GLLM_B200_STREAM_MIN_ITEMS", "1")
    if pair_gemm:
        monkeypatch.setenv("GLLM_B200_PAIR_MIN_TOKENS", "1")
    folder = write_tiny("D", str(tmp_path / "model"), sharp=False)
    cfg, weights = read_raw(folder, round_to_bf16=True)
    vocab = cfg["vocab_size"]
    seqs = sequences(vocab, seed=5)
    plain = {k: plain_forward(cfg, weights, v, torch.float64, stored=torch.bfloat16) for k, v in seqs.items()}
    steps, index = single_request_steps(seqs)
    results = replay(folder, "bfloat16", steps, str(tmp_path / "out1"), max_tokens=rounded(max(LENGTHS.values())),
                     vocab=vocab)
    compare(results, index, plain, BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN)
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    results = replay(folder, "bfloat16", steps, str(tmp_path / "out2"), max_tokens=448, vocab=vocab)
    compare(results, index, plain, BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN)
