"""The engine at the full layer sizes of Llama 3.2 1B (hidden 2048, 32/8 heads of 64, feed-forward 8192,
vocabulary 128256, llama3 rope scaling, tied head) with two layers and random weights, against the plain
implementation: whole, in portions with decoding, in float32 and in bfloat16.  These are the sizes the
tensor-core kernels are tuned for (every fast path runs: tcgen05 products in both orientations, the gated
epilogue, unsummed splits, tensor-core attention, CUDA-graph decode steps)."""

import os

import pytest
import torch

from plain_llama import plain_forward
from replay_helpers import (BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN, BF16_TOL_MAX, BF16_TOL_MEAN, compare, mixed_steps, run_steps, sequences,
                            single_request_steps)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full_width_model(tmp_path_factory):
    from gllm_b200.config import load_config
    from gllm_b200.config.presets import load_preset
    from gllm_b200.weights import write_random_model
    from tiny_models import read_raw

    raw = load_preset("llama-3.2-1b")
    raw["num_hidden_layers"] = 2
    folder = str(tmp_path_factory.mktemp("full_width") / "model")
    write_random_model(folder, load_config(raw), seed=5, std=0.02, std_overrides={"q_proj": 0.05, "k_proj": 0.05})
    cfg, weights = read_raw(folder)                 # stored in bfloat16: both runs see the same values
    weights = {k: v.float() for k, v in weights.items()}
    g = torch.Generator().manual_seed(6)
    tokens = torch.randint(0, cfg["vocab_size"], (200,), generator=g).tolist()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    want = plain_forward(cfg, weights, tokens, torch.float32)
    return folder, cfg, tokens, want, weights


@pytest.fixture(scope="module")
def full_width_sequences(full_width_model):
    """Five sequences of 33 to 210 tokens and the plain implementation's logits at every position."""
    folder, cfg, _, _, weights = full_width_model
    seqs = sequences(cfg["vocab_size"], seed=8)
    plain = {k: plain_forward(cfg, weights, v, torch.float32) for k, v in seqs.items()}
    kept = {k: plain_forward(cfg, weights, v, torch.float32, stored=torch.bfloat16) for k, v in seqs.items()}
    return seqs, plain, kept


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_every_cut_against_the_plain_implementation(full_width_model, full_width_sequences, dtype):
    """At the layer sizes the tensor-core kernels are tuned for, every position's logits of every
    request: whole; most of it in one step and the last 32 tokens one by one; in portions of changing
    size down to two tokens; and mixed, up to four live requests over a pool of 448 tokens for 1,108
    tokens of requests, so that pages are used again."""
    from gllm_b200.engine.replay import build_runner

    folder, cfg, _, _, _ = full_width_model
    seqs, plain, kept = full_width_sequences
    # the plain side is float32 here (float64 over this vocabulary takes minutes on the CPU); the bfloat16 run
    # is held to the plain implementation that keeps its activations in bfloat16
    tol = (5e-4, None) if dtype == "float32" else (BF16_KEPT_TOL_MAX, BF16_KEPT_TOL_MEAN)
    plain = plain if dtype == "float32" else kept
    _, runner = build_runner(folder, dtype, max_tokens=448)
    steps, index = single_request_steps(seqs)
    compare(run_steps(runner, steps), index, plain, *tol)
    assert runner.cache.num_free_pages() == runner.cache.num_blocks
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    compare(run_steps(runner, steps), index, plain, *tol)
    assert runner.cache.groups[0].allocator.total_reused > 0
    assert runner.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_layers(full_width_model, dtype):
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.engine.step import StepEntry

    folder, cfg, tokens, want, _ = full_width_model
    _, runner = build_runner(folder, dtype, max_tokens=512)
    scale = float(want.abs().max())
    # the plain side is float32 here (float64 over this vocabulary takes minutes on the CPU)
    bound = (5e-4 if dtype == "float32" else 5e-2) * scale
    rows = [0, 1, 63, 64, 127, 199]
    got = runner.run([StepEntry("whole", tokens, rows)]).float().cpu()
    assert float((got - want[rows]).abs().max()) <= bound
    runner.finish("whole")
    p = 0
    for n in [130, 2, 1, 1, 1, 65]:
        got = runner.run([StepEntry("cut", tokens[p:p + n], [n - 1])]).float().cpu()
        assert float((got[0] - want[p + n - 1]).abs().max()) <= bound, p
        p += n
    assert dtype == "float32" or runner.graph_replays > 0


def test_full_width_crowd_against_the_plain_implementation(full_width_model):
    """40 requests with 1,000 cached tokens each decode one token in the same step in which a 41st
    request's portion of 300 tokens is prefilled (the persistent decode kernel, the tcgen05 prefill
    kernel, products of 340 tokens on one CTA and on pairs of CTAs per tile, unsummed splits); in the
    next step they decode beside a portion of 120 tokens (a step of 160 tokens: the products' range
    of 129 to 255 tokens).  Four of the forty and the late request are compared with the plain
    implementation run on their whole sequences, the others with bounds of sanity."""
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.engine.step import StepEntry

    folder, cfg, _, want, weights = full_width_model
    _, runner = build_runner(folder, "bfloat16", max_tokens=41 * 1024, max_live=41)
    g = torch.Generator().manual_seed(7)
    vocab = cfg["vocab_size"]
    prompts = [torch.randint(0, vocab, (1000,), generator=g).tolist() for _ in range(40)]
    nexts = [torch.randint(0, vocab, (2,), generator=g).tolist() for _ in range(40)]
    late = torch.randint(0, vocab, (420,), generator=g).tolist()
    sampled = [0, 13, 27, 39]
    plain = {i: plain_forward(cfg, weights, prompts[i] + nexts[i], torch.float32, rows=[1000, 1001]) for i in sampled}
    plain["late"] = plain_forward(cfg, weights, late, torch.float32, rows=[299, 419])
    for first in range(0, 40, 4):                        # four prompts a step
        runner.run([StepEntry(f"r{i}", prompts[i], []) for i in range(first, first + 4)])
    scale = float(want.abs().max())
    for step, (lo, hi) in enumerate([(0, 300), (300, 420)]):
        entries = [StepEntry("late", late[lo:hi], [hi - lo - 1])]
        entries += [StepEntry(f"r{i}", [nexts[i][step]], [0]) for i in range(40)]
        got = runner.run(entries).float().cpu()
        pairs = [("late", got[0])] + [(i, got[1 + i]) for i in sampled]
        for key, row in pairs:
            err = (row - plain[key][step]).abs()
            assert float(err.max()) <= BF16_TOL_MAX * scale and float(err.mean()) <= BF16_TOL_MEAN * scale, (
                step, key, float(err.max()), float(err.mean()))
        # the 36 others are sane too: finite, and no two requests share a row
        assert bool(got.isfinite().all()) and len({int(r.argmax()) for r in got}) > 20
