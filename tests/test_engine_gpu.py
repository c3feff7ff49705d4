"""Generation through the Python entry point and the command line, against the
plain implementation: greedy tokens, long decoding, the first tokens of a
sequence, chunked prefill with preemption, sampling options and the async path."""

import asyncio
import json
import os
import subprocess
import sys
import threading

import pytest
import torch

from plain_llama import plain_forward
from tiny_models import read_raw, write_tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_greedy_check(cfg, weights, prompt, produced, slack):
    """Every produced token is the plain implementation's argmax given the
    tokens before it, or within ``slack`` (of the largest logit) of it."""
    tokens = list(prompt)
    for t in produced:
        logits = plain_forward(cfg, weights, tokens, torch.float64)[-1]
        best = int(logits.argmax())
        if t != best:
            assert float(logits[best] - logits[t]) <= slack * float(logits.abs().max()), (len(tokens), t, best)
        tokens.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(name, dtype, tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny(name, str(tmp_path / "m"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (1, 7, 16, 23, 40)]
    # few pages, small portions: chunked prefill, continuous batching and preemption all happen
    params = GeneratorParams(block_size=8, max_batch_size=3, max_seq_len=64, num_blocks=10, model_dtype=dtype,
                             max_num_batched_tokens=24, prefill_chunk=8)
    engine = LLMEngine(folder, params, device="cuda:0")
    reqs = [GenerationRequest(prompt_token_ids=p, max_new_tokens=12, temperature=0.0, ignore_eos=True) for p in prompts]
    results = engine.generate(reqs)
    slack = 1e-5 if dtype == "float32" else 0.05
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12 and r.finish_reason == "length"
        plain_greedy_check(cfg, weights, p, r.token_ids, slack)
    assert engine.counters["preemptions"] >= 1
    engine.cache.check_invariants()
    assert engine.cache.num_free_pages() == 10 and not engine.scheduler.has_work
    # the same requests one by one give the same tokens (float32: exactly)
    if dtype == "float32":
        for req, r in zip(reqs, results):
            assert engine.generate([req])[0].token_ids == r.token_ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_prefill_portions_replay_a_graph(dtype, tmp_path):
    """A prompt of 150 tokens fed in portions of 32: the first full portion is run and captured, the
    next three replay the graph over a growing context; the tokens are the plain implementation's."""
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny("D", str(tmp_path / "m"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    g = torch.Generator().manual_seed(14)
    prompt = torch.randint(0, cfg["vocab_size"], (150,), generator=g).tolist()
    params = GeneratorParams(block_size=16, max_batch_size=2, max_seq_len=256, model_dtype=dtype, prefill_chunk=32)
    engine = LLMEngine(folder, params, device="cuda:0")
    before = engine.runner.graph_replays
    out = engine.generate([GenerationRequest(prompt_token_ids=prompt, max_new_tokens=8, temperature=0.0,
                                             ignore_eos=True)])[0]
    assert any(k[0] == "prefill" and k[1] == 32 for k in engine.runner._graphs)
    assert engine.runner.graph_replays - before >= 3
    plain_greedy_check(cfg, weights, prompt, out.token_ids, 1e-5 if dtype == "float32" else 0.05)
    # a second prompt of another length reuses the graph from its first portion on
    prompt2 = torch.randint(0, cfg["vocab_size"], (70,), generator=g).tolist()
    out2 = engine.generate([GenerationRequest(prompt_token_ids=prompt2, max_new_tokens=4, temperature=0.0,
                                              ignore_eos=True)])[0]
    plain_greedy_check(cfg, weights, prompt2, out2.token_ids, 1e-5 if dtype == "float32" else 0.05)


def test_many_decoded_tokens_beside_full_prefill_portions(tmp_path, monkeypatch):
    """40 requests with prompts of 1,040 tokens, admitted under a budget of 2,048 tokens a step: while
    the last ones are prefilled in portions of 512, more than 32 others decode, so one step runs the
    prefill attention kernel, the persistent decode kernel (which holds every SM), its merge and the
    products on pairs of CTAs, each scheduled before the one ahead of it is done.  Every request's
    tokens are the plain implementation's."""
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine
    from gllm_b200.config import load_config
    from gllm_b200.ops import attention_bf16, gemm_bf16
    from gllm_b200.weights import write_random_model

    raw = dict(architectures=["LlamaForCausalLM"], hidden_size=512, head_dim=64, intermediate_size=1024,
               hidden_act="silu", num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
               rms_norm_eps=1e-5, eos_token_id=[0], torch_dtype="bfloat16", rope_theta=10000.0, vocab_size=1000,
               tie_word_embeddings=False)
    folder = write_random_model(str(tmp_path / "m"), load_config(raw), seed=21, std=0.03, norm_jitter=0.05,
                                std_overrides={"q_proj": 0.06, "k_proj": 0.06})
    cfg, weights = read_raw(folder, round_to_bf16=True)
    calls = []
    monkeypatch.setattr(gemm_bf16, "_PAIR_FORCED", True)    # a model this narrow would keep to the one-CTA kernel
    real_pair, real_decode = gemm_bf16.linear_pair, attention_bf16.decode_attention
    monkeypatch.setattr(gemm_bf16, "linear_pair",
                        lambda x, *a, **k: (calls.append(("pair", x.shape[0])), real_pair(x, *a, **k))[1])
    monkeypatch.setattr(attention_bf16, "decode_attention",
                        lambda q, *a, **k: (calls.append(("decode", q.shape[0])), real_decode(q, *a, **k))[1])
    g = torch.Generator().manual_seed(15)
    prompts = [torch.randint(1, cfg["vocab_size"], (1040,), generator=g).tolist() for _ in range(2)]
    params = GeneratorParams(block_size=16, max_batch_size=40, max_seq_len=1280, model_dtype="bfloat16",
                             max_num_batched_tokens=2048, prefill_chunk=512)
    engine = LLMEngine(folder, params, device="cuda:0")
    outs = engine.generate([GenerationRequest(prompt_token_ids=prompts[i % 2], max_new_tokens=32, temperature=0.0,
                                              ignore_eos=True) for i in range(40)])
    assert all(len(o.token_ids) == 32 for o in outs)
    wide = [i for i, c in enumerate(calls) if c[0] == "decode" and c[1] >= 33]      # 33 x 9 spans: the stream kernel
    assert wide and any(c[0] == "pair" and c[1] >= 129 + 33 for c in calls[wide[0]:wide[0] + 2])
    for i in (0, 1, 20, 21, 38, 39):
        plain_greedy_check(cfg, weights, prompts[i % 2], outs[i].token_ids[:2], 0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_random_crowd_over_a_small_pool(dtype, tmp_path):
    """48 requests of random lengths, greedy and sampled, over 40 pages and 6 slots: admissions wait,
    requests are preempted and computed again, decode steps replay graphs between mixed steps.  Every
    request gets its tokens, no page is lost, and the greedy ones are the plain implementation's."""
    import random

    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny("D", str(tmp_path / "m"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    rnd = random.Random(3)
    g = torch.Generator().manual_seed(3)
    reqs = []
    for i in range(48):
        n = rnd.choice([1, 2, 5, 17, 31, 64, 100, 150])
        greedy = i % 3 != 2
        reqs.append(GenerationRequest(
            prompt_token_ids=torch.randint(1, cfg["vocab_size"], (n,), generator=g).tolist(),
            max_new_tokens=rnd.choice([1, 2, 9, 30]), temperature=0.0 if greedy else 0.9, top_k=20, top_p=0.9, seed=i,
            ignore_eos=True))
    params = GeneratorParams(block_size=16, max_batch_size=6, max_seq_len=192, model_dtype=dtype, num_blocks=40,
                             max_num_batched_tokens=96, prefill_chunk=32)
    engine = LLMEngine(folder, params, device="cuda:0")
    outs = engine.generate(reqs)
    assert [len(o.token_ids) for o in outs] == [r.max_new_tokens for r in reqs]
    engine.cache.check_invariants()
    assert engine.cache.num_free_pages() == 40 and engine.counters["preemptions"] >= 1
    assert engine.runner.graph_replays > 0
    checked = 0
    for r, o in zip(reqs, outs):
        if r.temperature == 0.0 and checked < 10 and len(r.prompt_token_ids) + r.max_new_tokens <= 120:
            plain_greedy_check(cfg, weights, r.prompt_token_ids, o.token_ids[:6], 1e-5 if dtype == "float32" else 0.05)
            checked += 1
    assert checked == 10


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompts_run_as_graphs_of_few_tokens(dtype, tmp_path):
    """Lone prompts of 2 .. 100 tokens are padded to 16, 32, 64 or 128 tokens by a null portion and
    replayed as graphs: every bucket's edge and its neighbours give the plain implementation's tokens."""
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny("D", str(tmp_path / "m"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    params = GeneratorParams(block_size=16, max_batch_size=2, max_seq_len=256, model_dtype=dtype, prefill_chunk=128)
    engine = LLMEngine(folder, params, device="cuda:0")
    g = torch.Generator().manual_seed(16)
    for n in (2, 3, 14, 15, 16, 17, 30, 31, 32, 33, 62, 63, 64, 65, 100, 128):
        prompt = torch.randint(1, cfg["vocab_size"], (n,), generator=g).tolist()
        out = engine.generate([GenerationRequest(prompt_token_ids=prompt, max_new_tokens=2, temperature=0.0,
                                                 ignore_eos=True)])[0]
        plain_greedy_check(cfg, weights, prompt, out.token_ids, 1e-5 if dtype == "float32" else 0.05)
    buckets = {k[1] for k in engine.runner._graphs if k[0] == "prefill"}
    assert buckets == {16, 32, 64, 128}


def test_long_decoding_and_first_tokens(tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny("C", str(tmp_path / "m"))
    cfg, weights = read_raw(folder)
    engine = LLMEngine(folder, GeneratorParams(block_size=16, max_batch_size=2, max_seq_len=400, model_dtype="float32"),
                       device="cuda:0")
    # a one-token prompt: the very first positions of a sequence, then 300 decoded tokens across 19 pages
    # and far past the 24-token window of layer 1
    res = engine.generate([GenerationRequest(prompt_token_ids=[5], max_new_tokens=300, temperature=0.0, ignore_eos=True)])[0]
    assert len(res.token_ids) == 300
    tokens = [5] + res.token_ids
    logits = plain_forward(cfg, weights, tokens[:-1], torch.float64)
    for i in list(range(0, 20)) + list(range(20, 300, 7)) + [299]:
        best = int(logits[i].argmax())
        if tokens[i + 1] != best:
            assert float(logits[i, best] - logits[i, tokens[i + 1]]) < 1e-5 * float(logits[i].abs().max()), i


def test_stop_tokens_logprobs_and_sampling_options(tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny("B", str(tmp_path / "m"))
    cfg, weights = read_raw(folder)
    engine = LLMEngine(folder, GeneratorParams(block_size=16, max_batch_size=4, max_seq_len=64, model_dtype="float32"),
                       device="cuda:0")
    prompt = [9, 8, 7, 6, 5]
    free_run = engine.generate([GenerationRequest(prompt_token_ids=prompt, max_new_tokens=8, temperature=0.0,
                                                  ignore_eos=True, max_num_logprobs=3)])[0]
    assert len(free_run.logprobs) == 8 and free_run.logprobs[0].candidate_token_ids[0] == free_run.token_ids[0]
    want = torch.log_softmax(plain_forward(cfg, weights, prompt, torch.float64)[-1], -1)
    assert abs(free_run.logprobs[0].logprobs[0] - float(want.max())) < 1e-4
    assert abs(free_run.token_logprobs[0] - float(want.max())) < 1e-4
    # the third token as a stop token: generation ends there and keeps it (gllm/engine/llm_engine.py:124-127)
    stop = free_run.token_ids[2]
    if stop not in free_run.token_ids[:2]:
        r = engine.generate([GenerationRequest(prompt_token_ids=prompt, max_new_tokens=8, temperature=0.0,
                                               ignore_eos=True, stop_token_ids=[stop])])[0]
        assert r.token_ids == free_run.token_ids[:3] and r.finish_reason == "stop"
    # eos from config.json (7) stops unless ignored; sampled runs are reproducible by seed and differ across seeds
    a = engine.generate([GenerationRequest(prompt_token_ids=prompt, max_new_tokens=20, temperature=1.0, top_k=0,
                                           top_p=1.0, seed=s, ignore_eos=True) for s in (1, 1, 2)])
    assert a[0].token_ids == a[1].token_ids and a[0].token_ids != a[2].token_ids
    assert a[0].text == " ".join(map(str, a[0].token_ids))
    with pytest.raises(ValueError, match="only supports"):
        engine.generate([GenerationRequest(prompt_token_ids=list(range(64)), max_new_tokens=1)])
    with pytest.raises(ValueError, match="vocabulary"):
        engine.generate([GenerationRequest(prompt_token_ids=[400], max_new_tokens=1)])
    with pytest.raises(RuntimeError, match="tokenizer"):
        engine.generate([GenerationRequest(prompt="hello", max_new_tokens=1)])


def test_enqueue_request_and_run(tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    folder = write_tiny("A", str(tmp_path / "m"))
    engine = LLMEngine(folder, GeneratorParams(block_size=4, max_batch_size=2, max_seq_len=32, model_dtype="float32"),
                       device="cuda:0")
    reqs = [GenerationRequest(prompt_token_ids=[1 + i, 2, 3], max_new_tokens=5, temperature=0.0, ignore_eos=True)
            for i in range(5)]
    expected = [r.token_ids for r in engine.generate(reqs)]

    async def client():
        not_running = await asyncio.gather(engine.enqueue_request(reqs[0]), return_exceptions=True)
        assert isinstance(not_running[0], RuntimeError)
        thread = threading.Thread(target=engine.run, daemon=True)
        thread.start()
        while not engine.alive:
            await asyncio.sleep(0.01)
        bad = GenerationRequest(prompt_token_ids=list(range(40)), max_new_tokens=1)
        results = await asyncio.gather(*[engine.enqueue_request(r) for r in reqs], engine.enqueue_request(bad),
                                       return_exceptions=True)
        engine.stop()
        thread.join(timeout=10)
        return results

    results = asyncio.run(client())
    assert isinstance(results[-1], ValueError)                       # delivered on its own future
    assert [r.token_ids for r in results[:-1]] == expected           # more requests than slots: they wait, none is refused


def test_command_line(tmp_path):
    folder = str(tmp_path / "m")
    cfg_path = str(tmp_path / "cfg.json")
    from tiny_models import TINY_B

    with open(cfg_path, "w") as f:
        json.dump(TINY_B, f)
    env = dict(os.environ, PYTHONPATH=ROOT)
    subprocess.run([sys.executable, "-m", "gllm_b200", "make-random", "--config", cfg_path, "--out", folder, "--seed", "3"],
                   check=True, env=env, cwd=ROOT)
    out = subprocess.run(
        [sys.executable, "-m", "gllm_b200", "generate", "--model", folder, "--prompt-ids", "5 17 3", "--prompt-ids",
         "9,9,9,1", "--max-new-tokens", "4", "--temperature", "0", "--ignore-eos", "--max-seq-len", "64",
         "--max-batch-size", "2", "--model-dtype", "float32"],
        check=True, env=env, cwd=ROOT, capture_output=True, text=True,
    )
    lines = [json.loads(line) for line in out.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(line["token_ids"]) == 4 for line in lines)
    cfg, weights = read_raw(folder)
    plain_greedy_check(cfg, weights, [5, 17, 3], lines[0]["token_ids"], 1e-5)
