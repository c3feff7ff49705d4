"""Command line: ``python -m gllm_b200 <command>``.

The reference has no command line of its own beyond its benchmark script,
whose options are ``--model --batch-size --context-len --gen-len --device
--trace-file`` (benchmarks/benchmark_engine.py:8-16); ``benchmark`` keeps those
names and meanings (without ``--cpu-offloading``, which has no counterpart).
``generate`` exposes the request's fields under their own names
(gllm/engine/llm_engine_base.py:9-16) and the GeneratorParams fields
(gllm/config/generator_params.py:4-12).
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _add_generator_params(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-batch-size", type=int, default=8)
    ap.add_argument("--max-seq-len", type=int, default=4096)
    ap.add_argument("--model-dtype", choices=["bfloat16", "float32"], default=None)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--device", default="cuda")


def _params(args):
    from gllm_b200.config.generator_params import GeneratorParams

    return GeneratorParams(
        block_size=args.block_size, max_batch_size=args.max_batch_size, max_seq_len=args.max_seq_len,
        model_dtype=args.model_dtype, num_blocks=args.num_blocks,
        max_num_batched_tokens=args.max_num_batched_tokens, prefill_chunk=args.prefill_chunk,
    )


def cmd_generate(args) -> int:
    from gllm_b200 import GenerationRequest, LLMEngine

    engine = LLMEngine(args.model, _params(args), device=args.device)
    prompts = []
    for ids in args.prompt_ids or []:
        prompts.append(dict(prompt_token_ids=[int(t) for t in ids.replace(",", " ").split()]))
    for text in args.prompt or []:
        prompts.append(dict(prompt=text))
    if not prompts:
        print("give --prompt or --prompt-ids", file=sys.stderr)
        return 2
    reqs = [
        GenerationRequest(
            max_new_tokens=args.max_new_tokens, stop_tokens=args.stop_tokens or [], temperature=args.temperature,
            top_k=args.top_k, top_p=args.top_p, max_num_logprobs=args.max_num_logprobs, seed=args.seed,
            ignore_eos=args.ignore_eos, **p,
        )
        for p in prompts
    ]
    for res in engine.generate(reqs):
        print(json.dumps({"token_ids": res.token_ids, "text": res.text, "finish_reason": res.finish_reason,
                          "logprobs": [list(map(list, lp)) for lp in res.logprobs] if res.logprobs else None}))
    return 0


def cmd_make_random(args) -> int:
    from gllm_b200.config import load_config
    from gllm_b200.config.presets import load_preset
    from gllm_b200.weights import write_random_model

    if args.config:
        with open(args.config) as f:
            raw = json.load(f)
    else:
        raw = load_preset(args.preset)
    if args.num_layers is not None:
        raw["num_hidden_layers"] = args.num_layers
    if args.dtype:
        raw["torch_dtype"] = args.dtype
    write_random_model(args.out, load_config(raw), seed=args.seed, std=args.std, norm_jitter=args.norm_jitter)
    print(args.out)
    return 0


def cmd_benchmark(args) -> int:
    import torch

    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    params = GeneratorParams(block_size=args.block_size, max_batch_size=args.batch_size,
                             max_seq_len=args.context_len + args.gen_len + 1, model_dtype=args.model_dtype)
    engine = LLMEngine(args.model, params, device=args.device)
    g = torch.Generator().manual_seed(0)
    vocab = engine.config.vocab_size
    reqs = [
        GenerationRequest(prompt_token_ids=torch.randint(0, vocab, (args.context_len,), generator=g).tolist(),
                          max_new_tokens=args.gen_len, temperature=1.0, top_k=50, top_p=0.95, ignore_eos=True, seed=i)
        for i in range(args.batch_size)
    ]
    torch.cuda.reset_peak_memory_stats()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    if args.trace_file:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            engine.generate(reqs)
        prof.export_chrome_trace(args.trace_file)
    else:
        engine.generate(reqs)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1000
    peak = torch.cuda.max_memory_allocated() / 2**20
    print(f"[B={args.batch_size} C={args.context_len} G={args.gen_len}] duration: {ms:.6f} ms  peak memory: {peak:.0f} MiB")
    return 0


def cmd_replay(args) -> int:
    from gllm_b200.engine.replay import main as replay_main

    return replay_main(args.rest)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gllm_b200")
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from prompts with a model folder")
    g.add_argument("--model", required=True)
    g.add_argument("--prompt", action="append")
    g.add_argument("--prompt-ids", action="append", help="token ids separated by spaces or commas")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--stop-tokens", nargs="*")
    g.add_argument("--temperature", type=float, default=0.7)
    g.add_argument("--top-k", type=int, default=40)
    g.add_argument("--top-p", type=float, default=0.9)
    g.add_argument("--max-num-logprobs", type=int, default=0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--ignore-eos", action="store_true")
    _add_generator_params(g)
    g.set_defaults(fn=cmd_generate)

    m = sub.add_parser("make-random", help="write a model folder with random weights")
    m.add_argument("--out", required=True)
    src = m.add_mutually_exclusive_group(required=True)
    src.add_argument("--config", help="a config.json")
    src.add_argument("--preset", help="a named config.json shipped with the package")
    m.add_argument("--seed", type=int, default=0)
    m.add_argument("--std", type=float, default=0.02)
    m.add_argument("--norm-jitter", type=float, default=0.0)
    m.add_argument("--num-layers", type=int, default=None)
    m.add_argument("--dtype", choices=["bfloat16", "float32"], default=None)
    m.set_defaults(fn=cmd_make_random)

    b = sub.add_parser("benchmark", help="time one generate() call (the reference's benchmark_engine.py)")
    b.add_argument("--model", required=True)
    b.add_argument("--batch-size", required=True, type=int)
    b.add_argument("--context-len", required=True, type=int)
    b.add_argument("--gen-len", required=True, type=int)
    b.add_argument("--device", default="cuda")
    b.add_argument("--trace-file", default=None)
    b.add_argument("--block-size", type=int, default=32)
    b.add_argument("--model-dtype", choices=["bfloat16", "float32"], default=None)
    b.set_defaults(fn=cmd_benchmark)

    r = sub.add_parser("replay", help="trace replay (same as bin/trace_run)")
    r.add_argument("rest", nargs=argparse.REMAINDER)
    r.set_defaults(fn=cmd_replay)

    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
