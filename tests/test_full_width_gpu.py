"""The engine at the full layer sizes of Llama 3.2 1B (hidden 2048, 32/8 heads of 64, feed-forward 8192,
vocabulary 128256, llama3 rope scaling, tied head) with two layers and random weights, against the plain
implementation: whole, in portions with decoding, in float32 and in bfloat16.  These are the sizes the
tensor-core kernels are tuned for (every fast path runs: tcgen05 products in both orientations, the gated
epilogue, unsummed splits, tensor-core attention, CUDA-graph decode steps)."""

import json
import os

import pytest
import torch

from plain_llama import plain_forward

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
    g = torch.Generator().manual_seed(6)
    tokens = torch.randint(0, cfg["vocab_size"], (200,), generator=g).tolist()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    want = plain_forward(cfg, weights, tokens, torch.float32)
    return folder, cfg, tokens, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_layers(full_width_model, dtype):
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.engine.step import StepEntry

    folder, cfg, tokens, want = full_width_model
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


def test_full_width_crowd_gives_each_request_the_logits_it_gets_alone(full_width_model):
    """40 requests with 1,000 cached tokens each decode one token in the same step in which a 41st
    request's portion of 300 tokens is prefilled (the persistent decode kernel, the tcgen05 prefill
    kernel, products of 340 tokens on one CTA and on pairs of CTAs per tile, unsummed splits).  Each
    sampled request's logits are those it gets when it runs alone, to bfloat16 rounding."""
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.engine.step import StepEntry

    folder, cfg, _, want = full_width_model
    _, runner = build_runner(folder, "bfloat16", max_tokens=41 * 1024, max_live=41)
    g = torch.Generator().manual_seed(7)
    vocab = cfg["vocab_size"]
    prompts = [torch.randint(0, vocab, (1000,), generator=g).tolist() for _ in range(40)]
    nexts = torch.randint(0, vocab, (40,), generator=g).tolist()
    late = torch.randint(0, vocab, (300,), generator=g).tolist()
    sampled = [0, 13, 27, 39]
    alone = {}
    for i in sampled:
        runner.run([StepEntry("alone", prompts[i], [])])
        alone[i] = runner.run([StepEntry("alone", [nexts[i]], [0])]).float().cpu()[0]
        runner.finish("alone")
    alone["late"] = runner.run([StepEntry("alone", late, [299])]).float().cpu()[0]
    runner.finish("alone")
    for first in range(0, 40, 4):                        # four prompts a step
        runner.run([StepEntry(f"r{i}", prompts[i], []) for i in range(first, first + 4)])
    entries = [StepEntry("late", late, [299])] + [StepEntry(f"r{i}", [nexts[i]], [0]) for i in range(40)]
    got = runner.run(entries).float().cpu()
    scale = float(want.abs().max())
    pairs = [("late", got[0])] + [(i, got[1 + i]) for i in sampled]
    for key, row in pairs:
        err = (row - alone[key]).abs()
        assert float(err.max()) <= 5e-2 * scale and float(err.mean()) <= 5e-3 * scale, (key, float(err.max()))
    # the 36 others are sane too: finite, and no two requests share a row
    assert bool(got.isfinite().all()) and len({int(r.argmax()) for r in got}) > 20
