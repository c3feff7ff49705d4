"""Each part of a layer alone against its plain restatement, and a model whose plan names a
layer twice and lets one entry read another's cache."""

import math
import os
from types import SimpleNamespace

import pytest
import torch

from plain_llama import (plain_attention_layer, plain_forward, plain_inverse_frequencies, plain_mlp, plain_rmsnorm)
from tiny_models import TINY_B, TINY_D, read_raw, write_tiny

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


def getter(weights, dtype):
    def get(name, role="matrix"):
        t = weights[name]
        t = t.to(torch.float32) if role == "vector" else t.to(dtype)
        return t.cuda().contiguous()

    return get


def context_for(part_requirements, token_lists, dtype, block_size=8):
    """A cache manager and a step runner (without a model) that lay batches out for a part."""
    from gllm_b200.cache import CacheManager
    from gllm_b200.engine.step import StepRunner

    cache = CacheManager(part_requirements, block_size, 64, 4, 64 * block_size, dtype, "cuda")
    runner = StepRunner(SimpleNamespace(device=torch.device("cuda:0"), dtype=dtype), cache, 1024, cuda_graphs=False)
    return cache, runner


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from gllm_b200.parts import NORMS, build_part
    from gllm_b200.models.spec import PartSpec

    g = torch.Generator().manual_seed(0)
    w = {"n.weight": 1 + 0.1 * torch.randn(96, generator=g)}
    norm = build_part(NORMS, PartSpec("rmsnorm", dict(size=96, eps=1e-6), {"weight": "n.weight"}))
    assert list(norm.expected_tensors()) == ["n.weight"]
    norm.load(getter(w, dtype), dtype, "cuda")
    resid = torch.randn(11, 96, generator=g).cuda()
    branch = torch.randn(11, 96, generator=g).to(dtype).cuda()
    want_resid = resid.double() + branch.double()
    want = plain_rmsnorm(want_resid, w["n.weight"].double().cuda(), 1e-6)
    got = norm.forward(branch, resid, dtype)
    torch.testing.assert_close(resid.double(), want_resid, rtol=1e-6, atol=1e-6)       # the stream moved on, in fp32
    torch.testing.assert_close(got.double(), want, **tol(dtype))


def test_rotary_part_frequencies():
    from gllm_b200.parts import POSITION_ENCODINGS, build_part
    from gllm_b200.models.spec import PartSpec

    rope = build_part(POSITION_ENCODINGS, PartSpec("rotary", dict(
        head_dim=32, theta=TINY_B["rope_theta"], scaling=TINY_B["rope_scaling"])))
    rope.load(None, torch.float32, "cuda")
    inv_freq, rotary_dim, interleaved = rope.rotary()
    want = plain_inverse_frequencies(dict(TINY_B)).to(torch.float32)
    assert rotary_dim == 32 and not interleaved and torch.equal(inv_freq.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from gllm_b200.parts import FEED_FORWARDS, build_part
    from gllm_b200.models.spec import PartSpec

    g = torch.Generator().manual_seed(1)
    w = {f"m.{n}_proj.weight": (torch.randn(s, generator=g) * 0.1).to(dtype).float()
         for n, s in (("gate", (160, 96)), ("up", (160, 96)), ("down", (96, 160)))}
    ffn = build_part(FEED_FORWARDS, PartSpec("swiglu", dict(hidden_size=96, intermediate_size=160),
                                             {n: f"m.{n}_proj.weight" for n in ("gate", "up", "down")}))
    assert {e.shape for e in ffn.expected_tensors().values()} == {(160, 96), (96, 160)}
    ffn.load(getter(w, dtype), dtype, "cuda")
    x = torch.randn(9, 96, generator=g).to(dtype)
    from gllm_b200 import ops

    got = ops.as_tensor(ffn.forward(x.cuda(), None))
    want = plain_mlp(x.double(), {k: v.double() for k, v in w.items()}, "m")
    torch.testing.assert_close(got.double().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_in_portions(dtype, window):
    """The attention part alone: a sequence fed in portions of 23, 2, 1, 1 and 30 tokens beside another
    request equals the whole-sequence plain attention layer."""
    from gllm_b200 import ops
    from gllm_b200.engine.step import StepEntry
    from gllm_b200.parts import MIXERS, build_part
    from gllm_b200.models.spec import PartSpec

    g = torch.Generator().manual_seed(2)
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=32, hidden_size=96, rope_theta=10000.0)
    shapes = {"q": (128, 96), "k": (64, 96), "v": (64, 96), "o": (96, 128)}
    # float32: wide q and k projections, so attention settles on few keys and a wrong key shows;
    # bfloat16 cannot resolve scores that large, so its projections are narrower
    qk_std = 0.3 if dtype == torch.float32 else 0.1
    w = {f"a.{n}_proj.weight": (torch.randn(s, generator=g) * (qk_std if n in "qk" else 0.1)).to(dtype).float()
         for n, s in shapes.items()}
    spec = PartSpec("attention", dict(hidden_size=96, num_heads=4, num_kv_heads=2, head_dim=32, window=window,
                                      position=PartSpec("rotary", dict(head_dim=32, theta=10000.0))),
                    {n: f"a.{n}_proj.weight" for n in shapes})
    attn = build_part(MIXERS, spec)
    attn.load(getter(w, dtype), dtype, "cuda")
    req = attn.kv_requirement()
    assert (req.tensors, req.window) == (((2, 32), (2, 32)), window) and attn.state_requirement() is None
    cache, runner = context_for([(req, None, None)], None, dtype)
    caches = cache.mixer_caches()
    xs = {"a": torch.randn(57, 96, generator=g).to(dtype), "b": torch.randn(31, 96, generator=g).to(dtype)}
    inv_freq = plain_inverse_frequencies(cfg)
    want = {k: plain_attention_layer(x.double(), {n: t.double() for n, t in w.items()}, "a", cfg,
                                     torch.arange(x.shape[0]), inv_freq, window)[0] for k, x in xs.items()}
    cuts = {"a": [23, 2, 1, 1, 30], "b": [5, 1, 20, 4, 1]}
    pos = {"a": 0, "b": 0}
    for step in range(5):
        entries, rows = [], []
        for k in ("b", "a"):
            n = cuts[k][step]
            entries.append(StepEntry(k, [0] * n, []))
            rows.append((k, pos[k], n))
        _, ctx, _ = runner.build(entries)
        # the step function puts portions before single tokens: recover each request's rows from cu_q order
        order = sorted(range(2), key=lambda i: (rows[i][2] == 1, i))
        x = torch.cat([xs[rows[i][0]][rows[i][1]:rows[i][1] + rows[i][2]] for i in order]).cuda()
        got = ops.as_tensor(attn.forward(x, ctx, caches[0])).double().cpu()
        off = 0
        for i in order:
            k, p, n = rows[i]
            torch.testing.assert_close(got[off:off + n], want[k][p:p + n], **tol(dtype))
            off += n
            cache.commit(k, n)
            pos[k] += n
        ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_plan_runs_a_layer_twice_and_shares_a_cache(dtype, tmp_path):
    """The order of layers is data: entry 2 runs layer 1 again (with a cache of its own), entry 4 runs
    layer 0 over the cache of entry 1 (stores nothing).  Whole, then portions with decoding."""
    from gllm_b200.cache import CacheManager
    from gllm_b200.config import ARCHITECTURES, LlamaConfig, register_architecture
    from gllm_b200.engine.step import StepEntry, StepRunner
    from gllm_b200.models.llama import build_llama_spec
    from gllm_b200.models.loading import load_model
    from gllm_b200.models.spec import PlanEntry
    from dataclasses import replace
    import json

    plan = [(0, None), (1, None), (1, None), (2, None), (0, 1)]

    def build_spec(cfg):
        spec = build_llama_spec(cfg)
        return replace(spec, plan=tuple(PlanEntry(layer, reads) for layer, reads in plan))

    register_architecture("PlannedLlamaForTest", LlamaConfig, build_spec)
    try:
        folder = write_tiny("B", str(tmp_path / "m"), sharp=(dtype == "float32"))
        with open(os.path.join(folder, "config.json")) as f:
            raw = json.load(f)
        raw["architectures"] = ["PlannedLlamaForTest"]
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(raw, f)
        cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
        config, model = load_model(folder, dtype, "cuda:0")
        reqs = model.cache_requirements()
        assert len(reqs) == 5 and reqs[4][2] == 1
        cache = CacheManager(reqs, 8, 40, 2, 320, model.dtype, "cuda:0")
        assert len(cache.groups) == 1 and cache.groups[0].pool.shape[0] == 4      # four caches for five entries
        runner = StepRunner(model, cache, 512)
        g = torch.Generator().manual_seed(3)
        toks = torch.randint(0, 384, (90,), generator=g).tolist()
        want = plain_forward(cfg, weights, toks, torch.float64, plan=plan)
        scale = max(1.0, float(want.abs().max()))
        bound = 2e-4 * scale if dtype == "float32" else 5e-2 * scale
        got = runner.run([StepEntry("whole", toks, list(range(90)))]).double().cpu()
        assert float((got - want).abs().max()) <= bound
        runner.finish("whole")
        p = 0
        for n in [40, 2, 17, 1, 1, 1, 28]:
            got = runner.run([StepEntry("cut", toks[p:p + n], list(range(n)))]).double().cpu()
            assert float((got - want[p:p + n]).abs().max()) <= bound, p
            p += n
    finally:
        del ARCHITECTURES["PlannedLlamaForTest"]
