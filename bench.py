#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second at the
Llama 3.2 1B sizes with random bf16 weights (batch 8, 2,048 cached tokens per
request, max_seq_len 4096, block_size 16), plus a 2,048-token prefill, decode
at batch 1 and 64, the end-to-end figure through ``LLMEngine`` and the decode
step's roofline fraction.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step of the whole batch (forward + greedy sampling).
``value`` is timed on the device with CUDA events around K steps; ``e2e`` is
wall-clock around K ``LLMEngine.step()`` calls, each of which copies the step's
metadata from pinned host memory and reads the sampled tokens back.  The model
(2.47 GB of weights) is larger than the 126 MB L2, so every step streams its
inputs from HBM; no explicit L2 flush is used.  The prefill is one step of 2,048 prompt
tokens, timed on the device (the host's share of the step overlaps a spin kernel).
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            peaks = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if k in raw:
                    peaks[k] = float(raw[k])
            peaks["source"] = "measured"
            return peaks
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {
            "sm_mhz": sm[len(sm) // 2] if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def make_model_folder(tmp: str, num_layers: int | None) -> str:
    from gllm_b200.config import load_config
    from gllm_b200.weights import write_random_model

    raw = raw_model_config(num_layers)
    folder = os.path.join(tmp, "llama-3.2-1b-random")
    write_random_model(folder, load_config(raw), seed=0, std=0.02)
    return folder


def weight_bytes(engine) -> int:
    """Bytes of every weight a decode step reads once (the embedding table only
    through the tied head, or the untied head)."""
    total = 0
    seen = set()
    model = engine.model
    tensors = [model.head]
    for block in model.layers:
        tensors += [block.mixer.w_qkv, block.mixer.w_o, block.feed_forward.w_gate_up, block.feed_forward.w_down,
                    block.mixer_norm.weight, block.feed_forward_norm.weight]
    tensors.append(model.final_norm.weight)
    for t in tensors:
        if t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    return total


def prefill_flops(cfg, t: int) -> float:
    """Flops of one whole prompt of ``t`` tokens with logits at the last row."""
    h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    hq, hkv, layers, v = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.num_hidden_layers, cfg.vocab_size
    per_token = layers * (h * (hq + 2 * hkv) * d + hq * d * h + 3 * h * i)
    gemm = 2.0 * t * per_token
    attn = layers * 4.0 * d * hq * t * (t + 1) / 2
    head = 2.0 * h * v
    return gemm + attn + head


def fill_engine(engine, batch: int, context: int, seed: int = 0):
    """Admit ``batch`` requests of ``context`` random prompt tokens and run steps
    until every one of them is decoding."""
    import torch

    from gllm_b200 import GenerationRequest

    g = torch.Generator().manual_seed(seed)
    vocab = engine.config.vocab_size
    states = []
    for b in range(batch):
        req = GenerationRequest(
            prompt_token_ids=torch.randint(0, vocab, (context,), generator=g).tolist(),
            max_new_tokens=engine.max_seq_len - context, temperature=0.0, ignore_eos=True,
        )
        states.append(engine.submit(req))
    while any(s.num_computed < len(s.prompt_token_ids) for s in states):
        engine.step()
    return states


def drain(engine, states):
    for s in states:
        engine.abort(s.id)


# Untimed decode steps between a repetition's prefill and its warm-up steps: the prefill of the batch
# (16k tokens at batch 8) runs the GPU into its power cap, and the decode steps after it run at the
# lowered clock for a while (measured in groups of 20 steps after the prefill: 0.917, 0.914, 0.905, 0.897 ms
# a step, then 0.893 from the eightieth step on); a decode benchmark measures the state decoding settles in.
SETTLE_STEPS = 96


def time_decode(engine, batch: int, context: int, steps: int, warmup: int, reps: int = 5):
    """``reps`` repetitions of: fill the engine with ``batch`` requests of ``context`` cached tokens,
    ``SETTLE_STEPS`` + ``warmup`` untimed steps, then ``steps`` timed ones.  Device time (CUDA events) and wall time (host clock, a
    synchronize on both sides) are taken around the SAME loop of ``LLMEngine.step()`` calls, each of which
    copies the step's metadata from pinned host memory and reads the sampled tokens of the step before it.
    Returns the medians: (device ms per step, wall ms per step, launches per step, h2d, d2h)."""
    import torch

    from gllm_b200 import ops

    dev, wall = [], []
    launches = h2d = d2h = 0
    for _ in range(reps):
        states = fill_engine(engine, batch, context)
        for _ in range(SETTLE_STEPS + warmup):
            engine.step()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ops.launch_count
        t0 = time.perf_counter()
        start.record()
        for _ in range(steps):
            engine.step()
        end.record()
        torch.cuda.synchronize()
        wall.append((time.perf_counter() - t0) * 1000 / steps)
        dev.append(start.elapsed_time(end) / steps)
        launches = (ops.launch_count - launches0) / steps
        h2d = engine.runner.last_h2d_bytes
        d2h = engine.runner.sampled.numel() * 4 + 4      # the sampled-token snapshot and the status word
        drain(engine, states)
    dev.sort()
    wall.sort()
    return dev[len(dev) // 2], wall[len(wall) // 2], launches, h2d, d2h


def time_prefill(engine, tokens: int, repeats: int, warmup: int):
    """One request of ``tokens`` prompt tokens and one generated token, ``repeats`` times.  Returns the
    medians (device ms, end-to-end ms).  Device: events around the step, behind a spin kernel of about a
    millisecond so that the host's share of the step (schedule, metadata, launch) is over when the start
    event fires; it holds the copy of the metadata.  End to end: the host clock from ``submit`` to the
    sampled token in host memory, no spin kernel."""
    import torch

    from gllm_b200 import GenerationRequest

    g = torch.Generator().manual_seed(1)
    vocab = engine.config.vocab_size

    def request():
        return GenerationRequest(prompt_token_ids=torch.randint(0, vocab, (tokens,), generator=g).tolist(),
                                 max_new_tokens=1, temperature=0.0, ignore_eos=True)

    dev, e2e = [], []
    for it in range(warmup + repeats):
        req = request()
        torch.cuda.synchronize()
        st = engine.submit(req)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(3_000_000)
        start.record()
        engine.step()
        end.record()
        torch.cuda.synchronize()
        engine.step()          # greedy steps are pipelined: this call reads the timed step's token
        assert st.is_finished, "the prefill step did not finish the one-token request"
        if it >= warmup:
            dev.append(start.elapsed_time(end))
    for it in range(warmup + repeats):
        req = request()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        st = engine.submit(req)
        while not st.is_finished:
            engine.step()
        ms = (time.perf_counter() - t0) * 1000
        if it >= warmup:
            e2e.append(ms)
    dev.sort()
    e2e.sort()
    return dev[len(dev) // 2], e2e[len(e2e) // 2]


BENCH_SIZES = dict(context=2048, max_seq_len=4096, block_size=16, prefill_tokens=2048, full_layers=16)


def bench_config(raw: dict, batch: int, peaks: dict, sampling: str) -> dict:
    """The flat ``config`` record both arms print."""
    return {
        "model": "llama-3.2-1b sizes",
        "layers": raw["num_hidden_layers"],
        "layers_of_full_model": BENCH_SIZES["full_layers"],
        "hidden": raw["hidden_size"],
        "heads": raw["num_attention_heads"],
        "kv_heads": raw["num_key_value_heads"],
        "head_dim": raw["head_dim"],
        "intermediate": raw["intermediate_size"],
        "vocab": raw["vocab_size"],
        "global_batch": batch,
        "seq_len": BENCH_SIZES["context"],
        "max_seq_len": BENCH_SIZES["max_seq_len"],
        "block_size": BENCH_SIZES["block_size"],
        "prefill_tokens": BENCH_SIZES["prefill_tokens"],
        "parallelism": "single GPU",
        "l2": "inputs larger than L2 (2.47 GB of weights per step)",
        "sampling": sampling,
        "peaks": peaks["source"],
        "repetitions": "median of 5",
        "settle_steps": SETTLE_STEPS,
    }


def raw_model_config(num_layers: int | None) -> dict:
    from gllm_b200.config.presets import load_preset

    raw = load_preset("llama-3.2-1b")
    if num_layers is not None:
        raw["num_hidden_layers"] = num_layers
    return raw


def run_ours(args) -> dict:
    import torch

    from gllm_b200 import GeneratorParams, LLMEngine

    peaks = load_peaks()
    context, max_seq_len = BENCH_SIZES["context"], BENCH_SIZES["max_seq_len"]
    block_size, prefill_tokens = BENCH_SIZES["block_size"], BENCH_SIZES["prefill_tokens"]
    layers = args.layers or BENCH_SIZES["full_layers"]
    tmp = tempfile.mkdtemp(prefix="gllm_b200_bench_")
    try:
        folder = make_model_folder(tmp, layers if layers != BENCH_SIZES["full_layers"] else None)
        params = GeneratorParams(block_size=block_size, max_batch_size=64, max_seq_len=max_seq_len,
                                 model_dtype="bfloat16", max_num_batched_tokens=8192, prefill_chunk=2048)
        engine = LLMEngine(folder, params, device="cuda:0")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    cfg = engine.config
    wbytes = weight_bytes(engine)
    kv_per_token = engine.cache.bytes_per_token()
    steps = args.steps
    reps = 5

    def step_bytes(b):
        return wbytes + b * (context + SETTLE_STEPS + args.warmup + steps // 2) * kv_per_token

    points, points_ms, rooflines, e2e_points = {}, {}, {}, {}
    for b in (1, 64):
        dev_ms, wall_ms, _, _, _ = time_decode(engine, b, context, steps, args.warmup, reps)
        points[f"decode_b{b}"] = round(b * 1000.0 / dev_ms, 1)
        points_ms[f"decode_b{b}"] = round(dev_ms, 4)
        e2e_points[f"decode_b{b}"] = round(b * 1000.0 / wall_ms, 1)
        rooflines[f"decode_b{b}"] = round(step_bytes(b) / (dev_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)

    prefill_ms, prefill_e2e_ms = time_prefill(engine, prefill_tokens, repeats=5, warmup=max(3, args.warmup))
    pf_flops = prefill_flops(cfg, prefill_tokens)

    sampler = ClockSampler(0)
    sampler.start()
    batch = 8
    dev_ms, wall_ms, launches, h2d, d2h = time_decode(engine, batch, context, steps, args.warmup, reps)
    clocks = sampler.stop()

    achieved = step_bytes(batch) / (dev_ms * 1e-3) / 1e9
    value = batch * 1000.0 / dev_ms
    rooflines["decode_b8"] = round(achieved / peaks["hbm_gbs"], 4)
    points_ms["decode_b8"] = round(dev_ms, 4)
    e2e_points["decode_b8"] = round(batch * 1000.0 / wall_ms, 1)
    record = {
        "metric": "decode tok/s at batch 8 (Llama 3.2 1B sizes, random bf16 weights, 2,048 cached tokens)",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random N(0,0.02) weights (seed 0)",
        "config": bench_config(cfg.to_dict(), batch, peaks, "greedy, inside the step"),
        "e2e": {
            "value": round(batch * 1000.0 / wall_ms, 1),
            "unit": "tokens/s",
            "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h),
        },
        "gpu_launches": int(round(launches * steps)),
        "clocks": clocks,
        "prefill": {
            "value": round(prefill_tokens * 1000.0 / prefill_ms, 1),
            "tokens": prefill_tokens,
            "ms": round(prefill_ms, 4),
            "frac": round(pf_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
            "e2e_ms": round(prefill_e2e_ms, 4),
            "e2e_value": round(prefill_tokens * 1000.0 / prefill_e2e_ms, 1),
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
        "points_e2e": e2e_points,
        "points_roofline_frac": rooflines,
    }
    return record


SCENARIOS = {
    # BASELINE.json configs[3]: 64 requests at once, prompts uniform in 128..2,048 tokens, 256 generated tokens each
    "llama-3.2-3b": dict(kind="mixed", requests=64, prompt=(128, 2048), new_tokens=256, max_batch=64, max_seq_len=4096,
                         pool_fraction=1.0),
    # BASELINE.json configs[4]: 128 requests arriving four at a time, prompts 512..8,192 tokens, 512 generated tokens;
    # the pool holds a third of what they could grow to, so requests are preempted and recomputed
    "llama-3.1-8b": dict(kind="staggered", requests=128, prompt=(512, 8192), new_tokens=512, max_batch=128,
                         max_seq_len=8704, pool_fraction=1.0 / 3, arrivals_per_step=4),
}


def run_scenario(args) -> dict:
    """A whole-engine run (scheduler on) at another model size: never the headline, a line of its own."""
    import torch

    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine
    from gllm_b200.config import load_config
    from gllm_b200.config.presets import load_preset
    from gllm_b200.weights import write_random_model

    sc = SCENARIOS[args.preset]
    raw = load_preset(args.preset)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    block_size = 16
    worst_pages = sc["max_batch"] * -(-sc["max_seq_len"] // block_size)
    num_blocks = max(-(-sc["max_seq_len"] // block_size) + 1, int(worst_pages * sc["pool_fraction"]))
    tmp = tempfile.mkdtemp(prefix="gllm_b200_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, args.preset), load_config(raw), seed=0, std=0.02)
        params = GeneratorParams(block_size=block_size, max_batch_size=sc["max_batch"], max_seq_len=sc["max_seq_len"],
                                 model_dtype="bfloat16", num_blocks=num_blocks, max_num_batched_tokens=8192,
                                 prefill_chunk=2048)
        engine = LLMEngine(folder, params, device="cuda:0")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    g = torch.Generator().manual_seed(3)
    vocab = engine.config.vocab_size
    lo, hi = sc["prompt"]
    lengths = torch.randint(lo, hi + 1, (sc["requests"],), generator=g).tolist()
    requests = [GenerationRequest(prompt_token_ids=torch.randint(0, vocab, (n,), generator=g).tolist(),
                                  max_new_tokens=sc["new_tokens"], temperature=0.0, ignore_eos=True) for n in lengths]
    # warm-up: compile and capture what a short run needs
    engine.generate([GenerationRequest(prompt_token_ids=list(range(1, 40)), max_new_tokens=4, temperature=0.0,
                                       ignore_eos=True)])
    for key in engine.counters:
        engine.counters[key] = 0
    sampler = ClockSampler(0)
    sampler.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    states = []
    pending = list(requests)
    per_step = sc.get("arrivals_per_step", len(pending))
    while pending or any(not s.is_finished for s in states):
        for _ in range(min(per_step, len(pending))):
            states.append(engine.submit(pending.pop(0)))
        engine.step()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    generated = sum(len(s.generated_token_ids) for s in states)
    assert generated == sc["requests"] * sc["new_tokens"], "a request ended early"
    return {
        "metric": f"generated tok/s, whole engine ({sc['kind']} arrival, {args.preset} sizes, random bf16 weights)",
        "value": round(generated / wall, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "higher_is_better": True,
        "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random N(0,0.02) weights (seed 0)",
        "config": {
            "model": f"{args.preset} sizes", "layers": raw["num_hidden_layers"], "layers_of_full_model": full_layers,
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "requests": sc["requests"], "prompt_min": lo, "prompt_max": hi, "new_tokens": sc["new_tokens"],
            "max_batch_size": sc["max_batch"], "max_seq_len": sc["max_seq_len"], "block_size": block_size,
            "pool_pages": num_blocks, "arrival": sc["kind"],
        },
        "wall_s": round(wall, 3),
        "prompt_tokens": int(sum(lengths)),
        "prefill_tokens_run": int(engine.counters["prefill_tokens"]),
        "decode_tokens_run": int(engine.counters["decode_tokens"]),
        "steps": int(engine.counters["steps"]),
        "preemptions": int(engine.scheduler.num_preemptions),
        "clocks": clocks,
    }


def run_reference(args) -> dict:
    sys.path.insert(0, ROOT)
    from baseline import reference_arm
    from gllm_b200.config import load_config

    raw = raw_model_config(args.layers)
    args.prefill_flops = prefill_flops(load_config(dict(raw)), BENCH_SIZES["prefill_tokens"])
    args.warmup_prefill = 3
    peaks = load_peaks()
    try:
        return reference_arm.run(args, peaks, raw, ClockSampler, BENCH_SIZES, bench_config, settle=SETTLE_STEPS)
    except Exception as e:      # noqa: BLE001 - the arm reports why it has no number instead of failing the run
        import traceback

        traceback.print_exc()
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the full model (named in config)")
    ap.add_argument("--kernel", default=None, help="time one kernel alone (see gllm_b200/kernel_bench.py)")
    ap.add_argument("--shape", default="", help="with --kernel: overrides such as batch=8,context=2048")
    ap.add_argument("--preset", default=None, choices=sorted(SCENARIOS),
                    help="a whole-engine scenario at another model size (a line of its own, not the headline)")
    args = ap.parse_args()
    if args.kernel:
        from gllm_b200 import kernel_bench

        overrides = {k: int(v) for k, v in (kv.split("=") for kv in args.shape.split(",") if kv)}
        print(json.dumps(kernel_bench.run(args.kernel, load_peaks(), overrides)))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this engine does not run on {args.gpus} GPUs")
        return 2
    if args.preset:
        print(json.dumps(run_scenario(args)))
        return 0
    args.warmup = max(3, args.warmup)
    # a repetition's context grows from `context + warmup` to `context + warmup + steps` tokens
    args.steps = max(1, min(args.steps, BENCH_SIZES["max_seq_len"] - BENCH_SIZES["context"] - SETTLE_STEPS - args.warmup - 2))
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
