"""The body of ``bin/trace_run`` (see its header for the protocol)."""

from __future__ import annotations

import argparse
import json
import os
import sys

REPLAY_PAGE_TOKENS = 16      # default tokens per cache page; divides the 64-token rounding of --max-tokens
MAX_LIVE_REQUESTS = 4


def check_block_size(block_size: int) -> int:
    """``--max-tokens`` counts every request rounded up to 64 tokens (to the page, for larger pages):
    the pool of ``max_tokens // block_size`` pages holds that exactly when the page divides 64 or is a
    multiple of it."""
    if block_size <= 0 or (64 % block_size and block_size % 64):
        raise ValueError(f"--block-size {block_size}: a page must divide 64 tokens or be a multiple of 64")
    return block_size


def build_runner(model_dir: str, dtype: str, max_tokens: int, block_size: int = REPLAY_PAGE_TOKENS,
                 max_live: int = MAX_LIVE_REQUESTS, device: str = "cuda:0"):
    import torch

    from gllm_b200.cache.manager import CacheManager
    from gllm_b200.engine.step import StepRunner
    from gllm_b200.models.loading import load_model

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs on a GPU only")
    check_block_size(block_size)
    config, model = load_model(model_dir, dtype, device)
    num_blocks = max(1, max_tokens // block_size)
    cache = CacheManager(
        model.cache_requirements(),
        block_size=block_size,
        num_blocks=num_blocks,
        max_batch_size=max_live,
        max_seq_len=num_blocks * block_size,
        dtype=model.dtype,
        device=device,
    )
    runner = StepRunner(model, cache, max_tokens_per_step=num_blocks * block_size)
    return config, runner


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids step by step and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", required=True, type=int,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=REPLAY_PAGE_TOKENS,
                    help="tokens per cache page (default 16); divides 64 or is a multiple of it")
    args = ap.parse_args(argv)
    try:
        check_block_size(args.block_size)
    except ValueError as e:
        ap.error(str(e))

    from gllm_b200.engine.step import StepEntry

    os.makedirs(args.out, exist_ok=True)
    _, runner = build_runner(args.model, args.dtype, args.max_tokens, block_size=args.block_size)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [
            StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
            for e in step.get("entries", [])
        ]
        if entries:
            logits = runner.run(entries)
            if logits.shape[0]:
                host = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step['step']}.f32.tmp")
                with open(tmp, "wb") as f:
                    f.write(host.tobytes())
                os.replace(tmp, os.path.join(args.out, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            runner.finish(rid)
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
