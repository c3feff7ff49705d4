"""The reference arm of bench.py: TheEpicDolphin/gllm's own engine, unmodified,
timed on the same random Llama 3.2 1B folder and the same workload as this
repository's arm.

The reference's ``gllm/`` tree lies under ``baseline/_ref/gllm`` as its checkout
has it (``pip install --target baseline/_ref`` installs no module, because the
tree has no ``__init__.py`` and ``setup.py`` uses ``find_packages()``; the tree is
copied instead).  Nothing of it is changed or rebound: the model it "downloads"
(gllm/model/model.py:49-83) is found in hub cache folders of the layout
``models--<org>--<name>/{refs/main, snapshots/<revision>/<file>}`` that this module
prepares in a temporary place (``HF_HOME`` for config.json, the engine's
``local_cache_dir`` for tokenizer.json and model.safetensors) with
``HF_HUB_OFFLINE=1``.  The tokenizer is a word-level vocabulary in which the text
"5 17 3" is the ids [5, 17, 3], so prompts are given token ids.

What is timed is what the reference's own harness times
(benchmarks/utils.py:45-59): the wall clock of one ``engine.generate()`` between
two ``torch.cuda.synchronize()``.  One decode step is the difference of two such
calls that generate ``1 + W + K`` and ``1 + W`` tokens, divided by K: both hold
the same prefill and the same W first steps.  The reference's generate() waits
for the sampled tokens of every step on the host, so its device time and its
end-to-end time are one number.
"""

from __future__ import annotations

import contextlib
import json
import os
import shutil
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")
REPO_ID = "gllm-b200/llama-3.2-1b-random"
REVISION = "0" * 40


def _hub_cache_file(cache_dir: str, filename: str) -> str:
    """Path of ``filename`` of REPO_ID inside a hub cache rooted at ``cache_dir``
    (the refs and snapshot folders are made on the way)."""
    repo = os.path.join(cache_dir, "models--" + REPO_ID.replace("/", "--"))
    os.makedirs(os.path.join(repo, "refs"), exist_ok=True)
    with open(os.path.join(repo, "refs", "main"), "w") as f:
        f.write(REVISION)
    snap = os.path.join(repo, "snapshots", REVISION)
    os.makedirs(snap, exist_ok=True)
    return os.path.join(snap, filename)


def prepare_hub(tmp: str, raw_config: dict, seed: int = 0, std: float = 0.02) -> str:
    """Write the random model as three hub caches under ``tmp`` and return the
    engine's ``local_cache_dir``.  The weights are the ones this repository's
    arm draws (same configuration, seed and deviation)."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    from gllm_b200.config import load_config
    from gllm_b200.weights import write_random_model

    cfg = load_config(dict(raw_config))
    folder = write_random_model(os.path.join(tmp, "folder"), cfg, seed=seed, std=std)
    local_cache = os.path.join(tmp, "gllm_cache")
    hub = os.path.join(tmp, "hf_home", "hub")
    os.replace(os.path.join(folder, "model.safetensors"),
               _hub_cache_file(os.path.join(local_cache, "models"), "model.safetensors"))
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    eos = config.get("eos_token_id")
    config["eos_token_id"] = eos if isinstance(eos, list) else [eos]     # the reference reads a list only
    with open(_hub_cache_file(hub, "config.json"), "w") as f:
        json.dump(config, f)
    tok = Tokenizer(WordLevel({str(i): i for i in range(cfg.vocab_size)}, unk_token="0"))
    tok.pre_tokenizer = WhitespaceSplit()
    tok.save(_hub_cache_file(os.path.join(local_cache, "tokenizers"), "tokenizer.json"))
    return local_cache


def set_offline_env(tmp: str) -> None:
    """Must run before ``huggingface_hub`` is imported: it reads these once."""
    if "huggingface_hub" in sys.modules:
        raise RuntimeError("huggingface_hub was imported before the offline cache was set up")
    os.environ["HF_HOME"] = os.path.join(tmp, "hf_home")
    os.environ.pop("HF_HUB_CACHE", None)
    os.environ.pop("HUGGINGFACE_HUB_CACHE", None)
    os.environ["HF_HUB_OFFLINE"] = "1"


def _prompts(batch: int, tokens: int, vocab: int, seed: int) -> list[str]:
    import torch

    g = torch.Generator().manual_seed(seed)
    # ids below the special tokens, so that no prompt holds the end-of-sequence id
    return [" ".join(map(str, torch.randint(0, vocab - 256, (tokens,), generator=g).tolist())) for _ in range(batch)]


def timed_generate(engine, prompts: list[str], new_tokens: int) -> float:
    """Milliseconds of one stock ``generate()`` call, timed as
    benchmarks/utils.py:45-59 does; greedy by the reference's own means
    (``top_k=1``: its sampler has no other greedy mode)."""
    import torch
    from gllm.engine.llm_engine_base import GenerationRequest

    reqs = [GenerationRequest(prompt=p, max_new_tokens=new_tokens, stop_tokens=[], temperature=1.0, top_k=1, top_p=1.0)
            for p in prompts]
    sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)
    sync()
    t0 = time.perf_counter()
    with contextlib.redirect_stdout(sys.stderr):          # the engine prints a line per request
        results = engine.generate(reqs)
    sync()
    ms = (time.perf_counter() - t0) * 1000
    short = [len(r.token_ids) for r in results if len(r.token_ids) != new_tokens]
    if short:
        raise RuntimeError(f"a request ended early ({short} of {new_tokens} tokens): the timing does not hold")
    return ms


def make_engine(local_cache: str, max_batch_size: int, max_seq_len: int, block_size: int, device: str = "cuda"):
    from gllm.config.generator_params import GeneratorParams
    from gllm.engine.llm_engine import LLMEngine

    params = GeneratorParams(block_size=block_size, max_batch_size=max_batch_size, max_seq_len=max_seq_len)
    return LLMEngine(hf_model=REPO_ID, gen_params=params, device=device, local_cache_dir=local_cache)


def decode_ms_per_step(engine, batch, context, vocab, warmup, steps, reps, blocks_left):
    """Median over ``reps`` pairs of generate() calls of
    (t(1+warmup+steps tokens) - t(1+warmup tokens)) / steps, and the median
    time of the short call.  Every call takes fresh pages (the reference never
    hands a released page out again: gllm/model/kv_cache/paged_kv_cache.py:88-104
    pops from an OrderedDict without a key once the never-used pages are gone),
    so the number of calls is bounded by ``blocks_left``."""
    per_call = batch * (1 + (context + warmup + steps + 1) // engine.llm.gen_params.block_size)
    diffs, shorts = [], []
    for rep in range(reps):
        if blocks_left[0] < 2 * per_call:
            break
        prompts = _prompts(batch, context, vocab, seed=100 + rep)
        t_short = timed_generate(engine, prompts, 1 + warmup)
        t_long = timed_generate(engine, prompts, 1 + warmup + steps)
        blocks_left[0] -= 2 * per_call
        diffs.append((t_long - t_short) / steps)
        shorts.append(t_short)
    if not diffs:
        raise RuntimeError("the reference's page pool is too small for one pair of calls of this length")
    diffs.sort()
    shorts.sort()
    return diffs[len(diffs) // 2], shorts[len(shorts) // 2], len(diffs)


def run(args, peaks: dict, raw_config: dict, sampler_cls, sizes: dict, bench_config, settle: int = 0) -> dict:
    if not os.path.isdir(os.path.join(REF_ROOT, "gllm", "engine")):
        return {"impl": "reference", "unavailable": "the reference's gllm/ tree is not under baseline/_ref"}
    tmp = tempfile.mkdtemp(prefix="gllm_ref_bench_")
    try:
        set_offline_env(tmp)
        local_cache = prepare_hub(tmp, raw_config)
        sys.path.insert(0, REF_ROOT)
        import torch

        context, max_seq_len = sizes["context"], sizes["max_seq_len"]
        block_size, prefill_tokens = sizes["block_size"], sizes["prefill_tokens"]
        vocab = raw_config["vocab_size"]
        reps = 3
        # steps that are not timed after the prefill: this repository's arm lets the clocks settle first
        warm = args.warmup + settle
        # one engine sized like this repository's arm (64 requests of 4,096 tokens) serves batch 1 and 8
        engine = make_engine(local_cache, 64, max_seq_len, block_size)
        blocks_left = [64 * max_seq_len // block_size - 1]
        with contextlib.redirect_stdout(sys.stderr):
            timed_generate(engine, _prompts(1, 64, vocab, 1), 4)           # first-call costs (cuBLAS handles)
        blocks_left[0] -= 8
        # prefill: one request of 2,048 tokens, one generated token
        pf = []
        for rep in range(args.warmup_prefill + 5):
            ms = timed_generate(engine, _prompts(1, prefill_tokens, vocab, 200 + rep), 1)
            blocks_left[0] -= 1 + prefill_tokens // block_size
            if rep >= args.warmup_prefill:
                pf.append(ms)
        pf.sort()
        prefill_ms = pf[len(pf) // 2]
        points, points_ms = {}, {}
        b1_ms, _, _ = decode_ms_per_step(engine, 1, context, vocab, warm, args.steps, reps, blocks_left)
        points["decode_b1"], points_ms["decode_b1"] = round(1000.0 / b1_ms, 1), round(b1_ms, 4)
        clock = sampler_cls(0)
        clock.start()
        batch = 8
        dev_ms, t_short, n_pairs = decode_ms_per_step(engine, batch, context, vocab, warm, args.steps, reps,
                                                      blocks_left)
        clocks = clock.stop()
        del engine
        torch.cuda.empty_cache()
        # batch 64 fills more than half of the pages of an engine made for 64 requests: one call per engine
        try:
            times = {}
            for new_tokens in (1 + warm, 1 + warm + args.steps):
                engine = make_engine(local_cache, 64, max_seq_len, block_size)
                times[new_tokens] = timed_generate(engine, _prompts(64, context, vocab, 300), new_tokens)
                del engine
                torch.cuda.empty_cache()
            b64_ms = (times[1 + warm + args.steps] - times[1 + warm]) / args.steps
            points["decode_b64"], points_ms["decode_b64"] = round(64 * 1000.0 / b64_ms, 1), round(b64_ms, 4)
        except Exception as e:      # noqa: BLE001 - the headline does not depend on this point
            points["decode_b64"], points_ms["decode_b64"] = None, f"{type(e).__name__}: {e}"[:200]
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    wbytes = 2 * (raw_config["vocab_size"] * raw_config["hidden_size"] + raw_config["num_hidden_layers"] * (
        raw_config["hidden_size"] * (raw_config["num_attention_heads"] + 2 * raw_config["num_key_value_heads"])
        * raw_config["head_dim"] + raw_config["num_attention_heads"] * raw_config["head_dim"] * raw_config["hidden_size"]
        + 3 * raw_config["hidden_size"] * raw_config["intermediate_size"]))
    kv_per_token = 2 * 2 * raw_config["num_hidden_layers"] * raw_config["num_key_value_heads"] * raw_config["head_dim"]
    step_bytes = wbytes + batch * (context + warm + args.steps // 2) * kv_per_token
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9
    value = batch * 1000.0 / dev_ms
    return {
        "impl": "reference",
        "metric": "decode tok/s at batch 8 (Llama 3.2 1B sizes, random bf16 weights, 2,048 cached tokens)",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random N(0,0.02) weights (seed 0)",
        "config": bench_config(raw_config, batch, peaks, "greedy (top_k=1), inside the step"),
        "timing": (f"stock LLMEngine.generate(), wall clock between synchronizes; ms_per_step = median of {n_pairs} "
                   f"x (t({1 + warm + args.steps} tokens) - t({1 + warm} tokens)) / {args.steps}; "
                   "the reference has no llama3 frequency scaling (plain rope_theta)"),
        "e2e": {
            "value": round(value, 1),
            "unit": "tokens/s",
            # per step the reference reads back the sampled ids (int64), one block count per request
            # (.item()) and three isnan flags; token ids go up as kernel arguments, not as copies
            "h2d_bytes_per_step": 0,
            "d2h_bytes_per_step": batch * 8 + batch * 4 + 3,
        },
        "gpu_launches": 0,
        "clocks": clocks,
        "prefill": {
            "value": round(prefill_tokens * 1000.0 / prefill_ms, 1),
            "tokens": prefill_tokens,
            "ms": round(prefill_ms, 4),
            "frac": round(args.prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
            "b8_prefill_and_warmup_steps_ms": round(t_short, 2),
        },
        "roofline": {
            "bound": "hbm",
            "achieved": round(achieved, 1),
            "peak": peaks["hbm_gbs"],
            "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4),
        },
        "points": points,
        "points_ms_per_step": points_ms,
    }
