"""Single-kernel workloads: each builds synthetic inputs, runs one kernel of the
engine a few times with an L2 flush between runs, and reports its time beside
the bytes or flops it has to move.  ``python bench.py --kernel NAME`` runs one;
the same command under ``ncu`` gives the profiles kept under ``profiles/``."""

from __future__ import annotations

import math

import torch


def _flush_l2(buf):
    buf.zero_()


def _time(fn, iters: int, flush) -> float:
    """Median device time of ``fn`` in microseconds."""
    times = []
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    for _ in range(iters):
        _flush_l2(flush)
        # keep the GPU busy while the host queues the launches, so the events bracket device time only
        torch.cuda._sleep(400_000)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    times.sort()
    return times[len(times) // 2]


def _paged_cache(batch, context, hkv, d, block_size, extra_tokens=0, sequential=0):
    """A pool holding ``batch`` requests of ``context`` tokens on scattered pages
    (``sequential``: each request's pages lie one after another instead)."""
    pages_per_req = -(-(context + extra_tokens) // block_size)
    num_pages = batch * pages_per_req + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    pool = torch.randn((num_pages, 2, hkv, block_size, d), generator=g, device="cuda", dtype=torch.float32)
    pool = pool.to(torch.bfloat16)
    perm = torch.randperm(num_pages - 1, generator=g, device="cuda").to(torch.int32)
    if sequential:
        perm = torch.arange(num_pages - 1, device="cuda", dtype=torch.int32)
    table = perm[: batch * pages_per_req].view(batch, pages_per_req).contiguous()
    return pool, table


def attention_decode(batch=64, context=2048, hq=32, hkv=8, d=64, block_size=16, iters=5, peaks=None, sequential=0,
                     stream=1):
    from gllm_b200.ops import attention_bf16

    pool, table = _paged_cache(batch, context, hkv, d, block_size, sequential=sequential)
    qkv = torch.randn(batch, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16)
    positions = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
    rows = torch.arange(batch, dtype=torch.int32, device="cuda")
    out = torch.empty(batch, hq * d, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    class _WS:
        def __init__(self):
            self.b = {}

        def get(self, name, n, dt):
            if name not in self.b:
                self.b[name] = torch.empty(n, dtype=dt, device="cuda")
            return self.b[name]

    ws = _WS()
    fn = lambda: attention_bf16.decode_attention(qkv, qkv.shape[1], pool, table, positions, rows, hq,
                                                 1.0 / math.sqrt(d), 0, context, ws, out,
                                                 kernel="stream" if stream else "split")
    us = _time(fn, iters, flush)
    nbytes = batch * context * 2 * hkv * d * 2
    gbs = nbytes / us / 1e3
    return {"kernel": "attention_decode (stream + merge)" if stream else "attention_decode (split + merge)", "us": round(us, 2), "bytes": nbytes,
            "achieved_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4),
            "shape": dict(batch=batch, context=context, heads=hq, kv_heads=hkv, head_dim=d, block_size=block_size)}


def attention_prefill(tokens=2048, context=0, hq=32, hkv=8, d=64, block_size=16, iters=5, peaks=None, tmem=1):
    from gllm_b200.ops import attention_bf16

    pool, table = _paged_cache(1, context + tokens, hkv, d, block_size)
    qkv = torch.randn(tokens, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    ctx = torch.tensor([context], dtype=torch.int32, device="cuda")
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(tokens, hq * d, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    kernel = attention_bf16.prefill_attention_tmem if tmem else attention_bf16.prefill_attention
    fn = lambda: kernel(qkv, qkv.shape[1], pool, table, cu, ctx, slots, 1, tokens, hq, 1.0 / math.sqrt(d), 0, out)
    us = _time(fn, iters, flush)
    flops = 4.0 * d * hq * (tokens * context + tokens * (tokens + 1) / 2)
    tf = flops / us / 1e6
    return {"kernel": "attention_prefill (tcgen05)" if tmem else "attention_prefill (mma.sync)", "us": round(us, 2), "flops": flops, "achieved_tflops": round(tf, 1),
            "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
            "shape": dict(tokens=tokens, context=context, heads=hq, kv_heads=hkv, head_dim=d, block_size=block_size)}


def linear(m=8, n=16384, k=2048, iters=5, peaks=None, out_fp32=False, gated=0, split=0, acc=0):
    """x [m, k] times a [n, k] weight.  ``gated``: the weight is a gate/up stack (n = 2 x features) and
    the epilogue writes SiLU(gate) * up.  ``split``: a product cut along K leaves its splits unsummed,
    as the decode step's products do (their consumers add them).  ``acc``: the product adds itself into
    an fp32 matrix (the residual stream), as the products that end a branch do for up to 64 tokens."""
    from gllm_b200 import ops

    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.float32 if out_fp32 else torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    resid = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    if gated:
        fn = lambda: ops.linear_gated(x, w)
    elif acc:
        fn = lambda: ops.linear(x, w, split_ok=True, add_into=resid)
    elif split:
        fn = lambda: ops.linear(x, w, split_ok=True)
    else:
        fn = lambda: ops.linear(x, w, out_dtype=out.dtype, out=out)
    us = _time(fn, iters, flush)
    nbytes = (m * k + n * k) * 2 + out.numel() * out.element_size()
    flops = 2.0 * m * n * k
    gbs, tf = nbytes / us / 1e3, flops / us / 1e6
    name = "linear (gated epilogue)" if gated else ("linear (adds into the residual)" if acc else
                                                     ("linear (unsummed splits)" if split else "linear"))
    return {"kernel": name, "us": round(us, 2), "achieved_gbs": round(gbs, 1), "achieved_tflops": round(tf, 1),
            "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4), "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
            "shape": dict(m=m, n=n, k=k)}


def linear_f32(m=2048, n=8192, k=2048, iters=5, peaks=None):
    """The true 32-bit product (FFMA, no tensor-core mode) of the float32 path."""
    from gllm_b200 import ops

    x = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda") * 0.02
    out = torch.empty(m, n, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.linear(x, w, out=out), iters, flush)
    nbytes = (m * k + n * k + m * n) * 4
    flops = 2.0 * m * n * k
    return {"kernel": "linear_f32 (FFMA)", "us": round(us, 2), "achieved_tflops": round(flops / us / 1e6, 1),
            "achieved_gbs": round(nbytes / us / 1e3, 1), "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4),
            "shape": dict(m=m, n=n, k=k)}


def decode_step(batch=8, context=2048, layers=2, iters=3, peaks=None):
    """Whole decode steps of a model with the Llama 3.2 1B layer sizes and ``layers`` layers, every kernel
    launched on its own (no CUDA graph), so that a profiler lists them one by one."""
    import os
    import shutil
    import tempfile

    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine
    from gllm_b200.config import load_config
    from gllm_b200.config.presets import load_preset
    from gllm_b200.weights import write_random_model

    raw = load_preset("llama-3.2-1b")
    raw["num_hidden_layers"] = layers
    tmp = tempfile.mkdtemp(prefix="gllm_b200_kernel_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, "model"), load_config(raw), seed=0, std=0.02)
        params = GeneratorParams(block_size=16, max_batch_size=max(batch, 8), max_seq_len=4096, model_dtype="bfloat16",
                                 cuda_graphs=False)
        engine = LLMEngine(folder, params, device="cuda:0")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    g = torch.Generator().manual_seed(0)
    vocab = engine.config.vocab_size
    states = [engine.submit(GenerationRequest(prompt_token_ids=torch.randint(0, vocab, (context,), generator=g).tolist(),
                                              max_new_tokens=64, temperature=0.0, ignore_eos=True)) for _ in range(batch)]
    while any(s.num_computed < len(s.prompt_token_ids) for s in states):
        engine.step()
    for _ in range(3):
        engine.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        engine.step()
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / iters
    return {"kernel": "decode_step (no graph)", "us": round(us, 2), "shape": dict(batch=batch, context=context, layers=layers)}


def add_rmsnorm(rows=8, hidden=2048, splits=8, iters=5, peaks=None):
    """resid += (sum of ``splits`` fp32 partial products, 0: a summed bf16 branch), then RMSNorm: the
    kernel between two products of a layer."""
    from gllm_b200 import ops

    resid = torch.randn(rows, hidden, device="cuda")
    weight = torch.ones(hidden, device="cuda")
    parts = torch.randn(max(splits, 1), rows, hidden, device="cuda")
    branch = ops.SplitSum(parts, torch.bfloat16) if splits else parts[0].to(torch.bfloat16)
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.add_rmsnorm(branch, resid, weight, 1e-5, torch.bfloat16, out=out), iters, flush)
    nbytes = rows * hidden * ((4 * splits if splits else 2) + 4 + 4 + 2) + hidden * 4
    gbs = nbytes / us / 1e3
    return {"kernel": "add_rmsnorm", "us": round(us, 2), "bytes": nbytes, "achieved_gbs": round(gbs, 1),
            "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4), "shape": dict(rows=rows, hidden=hidden, splits=splits)}


def argmax(rows=8, vocab=128256, iters=5, peaks=None):
    from gllm_b200 import ops

    logits = torch.randn(rows, vocab, device="cuda")
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.argmax(logits, out=out), iters, flush)
    nbytes = rows * vocab * 4
    gbs = nbytes / us / 1e3
    return {"kernel": "argmax", "us": round(us, 2), "bytes": nbytes, "achieved_gbs": round(gbs, 1),
            "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4), "shape": dict(rows=rows, vocab=vocab)}


KERNELS = {
    "attention_decode": attention_decode,
    "attention_prefill": attention_prefill,
    "linear": linear,
    "linear_f32": linear_f32,
    "decode_step": decode_step,
    "add_rmsnorm": add_rmsnorm,
    "argmax": argmax,
}


def run(name: str, peaks: dict, overrides: dict) -> dict:
    if name not in KERNELS:
        raise SystemExit(f"unknown kernel {name!r}; known: {sorted(KERNELS)}")
    return KERNELS[name](peaks=peaks, **overrides)
