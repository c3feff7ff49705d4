"""Drives ``bin/trace_run`` as a child process the way a user would and reads
the logits it writes."""

from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model_dir: str, dtype: str, steps: list[dict], out_dir: str, max_tokens: int, vocab: int,
           timeout: float = 900.0, block_size: int | None = None) -> dict[int, np.ndarray]:
    """Feed ``steps`` one at a time (the next only after ``done <step>``) and
    return {step: logits [wanted, vocab]}."""
    os.makedirs(out_dir, exist_ok=True)
    proc = subprocess.Popen(
        [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens)] + (["--block-size", str(block_size)] if block_size else []),
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1,
    )
    try:
        for step in steps:
            try:
                proc.stdin.write(json.dumps(step) + "\n")
                proc.stdin.flush()
            except BrokenPipeError:
                raise RuntimeError(f"trace_run ended before step {step['step']}; exit {proc.wait()}") from None
            line = proc.stdout.readline()
            if line.strip() != f"done {step['step']}":
                rest = proc.stdout.read()
                raise RuntimeError(f"trace_run answered {line!r} to step {step['step']}; exit {proc.poll()}; {rest}")
        proc.stdin.close()
        code = proc.wait(timeout=timeout)
    finally:
        if proc.poll() is None:
            proc.kill()
    if code != 0:
        raise RuntimeError(f"trace_run exited with {code}")
    out = {}
    for step in steps:
        wanted = sum(len(e.get("want", [])) for e in step["entries"])
        path = os.path.join(out_dir, f"{step['step']}.f32")
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, (step["step"], data.size, wanted, vocab)
            out[step["step"]] = data.reshape(wanted, vocab)
        else:
            assert not os.path.exists(path)
    return out


def rounded(n: int, to: int = 64) -> int:
    return -(-n // to) * to


def run_steps(runner, steps: list[dict]) -> dict[int, np.ndarray]:
    """The same steps through a step runner of this process (``engine.replay.build_runner``), as
    ``bin/trace_run`` runs them; {step: logits [wanted, vocab]}."""
    from gllm_b200.engine.step import StepEntry

    out = {}
    for step in steps:
        entries = [StepEntry(e["id"], list(e["tokens"]), list(e.get("want", []))) for e in step["entries"]]
        logits = runner.run(entries)
        if logits.shape[0]:
            out[step["step"]] = logits.float().cpu().numpy()
        for rid in step.get("end", []):
            runner.finish(rid)
    return out


LENGTHS = {"a": 150, "b": 97, "c": 64, "d": 33, "e": 210}
# |engine - plain| <= tol * max(1, max|plain|); bf16 also bounds the mean error
FP32_TOL = 2e-4
BF16_TOL_MAX = 5e-2
BF16_TOL_MEAN = 1e-2
# a bfloat16 run against the plain implementation that keeps its activations in bfloat16 where a bfloat16
# model keeps them (plain_forward(..., stored=torch.bfloat16)): what is left is the order of the sums, the
# bfloat16 probabilities of the tensor-core attention and the bfloat16 outputs of some products
BF16_KEPT_TOL_MAX = 2e-2
BF16_KEPT_TOL_MEAN = 2e-3


def sequences(vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return {k: torch.randint(0, vocab, (n,), generator=g).tolist() for k, n in LENGTHS.items()}


def single_request_steps(seqs, first_step=0):
    """Modes 1-3 one request after another: whole; most of it in one step and
    the last 32 tokens one by one; portions of changing size down to two."""
    steps, index = [], []
    s = first_step

    def add(entries, end=()):
        nonlocal s
        row = 0
        for rid, key, start, n in entries:
            for i in range(n):
                index.append((s, row, key, start + i))
                row += 1
        steps.append({
            "step": s,
            "entries": [{"id": rid, "tokens": seqs[key][start:start + n], "want": list(range(n))}
                        for rid, key, start, n in entries],
            "end": list(end),
        })
        s += 1

    for key, toks in seqs.items():
        n = len(toks)
        add([(f"{key}-whole", key, 0, n)], end=[f"{key}-whole"])
        head = max(1, n - 32)
        add([(f"{key}-tail", key, 0, head)])
        for p in range(head, n):
            add([(f"{key}-tail", key, p, 1)], end=[f"{key}-tail"] if p == n - 1 else [])
        sizes = [7, 2, 5, 3, 2, 16, 17, 2, 31, 1, 2, 9]
        p, i = 0, 0
        while p < n:
            c = min(sizes[i % len(sizes)], n - p)
            add([(f"{key}-cut", key, p, c)], end=[f"{key}-cut"] if p + c == n else [])
            p += c
            i += 1
    return steps, index


def mixed_steps(seqs, max_tokens, seed):
    """Mode 4: up to four live requests, portions of some beside decoded tokens
    of others, requests ending from the middle of the list, some left out of a
    step; admission keeps the live requests' rounded-up lengths within
    ``max_tokens`` so the pool is full often and freed pages are handed out again."""
    rnd = random.Random(seed)
    pending = list(seqs) + [k + "'" for k in seqs]          # every sequence twice
    key_of = lambda rid: rid.rstrip("'")
    pos, live, steps, index = {}, [], [], []
    s = 0
    while pending or live:
        while pending and len(live) < 4:
            need = rounded(len(seqs[key_of(pending[0])]))
            held = sum(rounded(len(seqs[key_of(r)])) for r in live)
            if held + need > max_tokens:
                break
            rid = pending.pop(0)
            live.append(rid)
            pos[rid] = 0
        entries, row = [], 0
        for rid in live:
            if len(live) > 1 and rnd.random() < 0.25:
                continue                                    # left out of this step
            toks = seqs[key_of(rid)]
            remaining = len(toks) - pos[rid]
            n = 1 if (pos[rid] > 0 and rnd.random() < 0.5) else rnd.choice([2, 3, 5, 8, 13, 21, 40])
            n = min(n, remaining)
            entries.append((rid, pos[rid], n))
        if not entries:
            continue
        ended = []
        step = {"step": s, "entries": [], "end": ended}
        for rid, start, n in entries:
            toks = seqs[key_of(rid)]
            step["entries"].append({"id": rid, "tokens": toks[start:start + n], "want": list(range(n))})
            for i in range(n):
                index.append((s, row, key_of(rid), start + i))
                row += 1
            pos[rid] += n
            if pos[rid] == len(toks):
                ended.append(rid)
                live.remove(rid)
        steps.append(step)
        s += 1
    return steps, index


def compare(results, index, plain, tol_max, tol_mean=None):
    worst, total, count = 0.0, 0.0, 0
    scale = max(1.0, max(float(p.abs().max()) for p in plain.values()))
    for step, row, key, position in index:
        got = results[step][row]
        want = plain[key][position].numpy()
        err = np.abs(got.astype(np.float64) - want)
        e = float(err.max())
        if e > tol_max * scale:
            raise AssertionError(
                f"first wrong token: step {step}, row {row}, request {key}, position {position}: "
                f"error {e:.3e} > {tol_max * scale:.3e}"
            )
        worst = max(worst, e)
        total += float(err.mean())
        count += 1
    print(f"compare: worst {worst / scale:.2e}, mean {total / count / scale:.2e} of the scale {scale:.3g} "
          f"(bounds {tol_max:.1e}, {tol_mean if tol_mean is not None else float('nan'):.1e})")
    if tol_mean is not None:
        assert total / count <= tol_mean * scale, f"mean error {total / count:.3e}"
    return worst


