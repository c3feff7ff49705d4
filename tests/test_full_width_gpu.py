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
