"""Replays the same requests through ``bin/trace_run`` whole, with the last 32
tokens one by one, in portions of changing size, and mixed with other requests
over a pool so small that pages are used again, in float32 and in bfloat16, and
compares every logit with the plain implementation."""

import random

import numpy as np
import pytest
import torch

from plain_llama import plain_forward
from replay_helpers import replay, rounded
from tiny_models import TINY, read_raw, write_tiny

pytestmark = pytest.mark.gpu

LENGTHS = {"a": 150, "b": 97, "c": 64, "d": 33, "e": 210}
# |engine - plain| <= tol * max(1, max|plain|); bf16 also bounds the mean error
FP32_TOL = 2e-4
BF16_TOL_MAX = 5e-2
BF16_TOL_MEAN = 1e-2


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
    if tol_mean is not None:
        assert total / count <= tol_mean * scale, f"mean error {total / count:.3e}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_all_cuts(name, dtype, tmp_path):
    folder = write_tiny(name, str(tmp_path / "model"), sharp=(dtype == "float32"))
    cfg, weights = read_raw(folder, round_to_bf16=(dtype == "bfloat16"))
    vocab = cfg["vocab_size"]
    seqs = sequences(vocab, seed=5)
    plain = {k: plain_forward(cfg, weights, v, torch.float64) for k, v in seqs.items()}
    tol = (FP32_TOL, None) if dtype == "float32" else (BF16_TOL_MAX, BF16_TOL_MEAN)

    steps, index = single_request_steps(seqs)
    results = replay(folder, dtype, steps, str(tmp_path / "out1"), max_tokens=rounded(max(LENGTHS.values())), vocab=vocab)
    compare(results, index, plain, *tol)

    # 4 live requests at most, 448 tokens: less than the requests' total, so pages are used again
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    results = replay(folder, dtype, steps, str(tmp_path / "out2"), max_tokens=448, vocab=vocab)
    compare(results, index, plain, *tol)


@pytest.mark.parametrize("pair_gemm", [False, True])
def test_replay_through_the_stream_decode_kernel(tmp_path, monkeypatch, pair_gemm):
    """The single tokens of tiny D (head size 64, one kv head, a window of 40 on one layer, pages of
    16) through the persistent TMA decode kernel, which steps this small would not pick by themselves:
    the tail decoded token by token, and the mixed steps with pages used again.  The second time every
    product that is not cut along K also runs on pairs of CTAs, as in large mixed steps."""
    monkeypatch.setenv("GLLM_B200_STREAM_MIN_ITEMS", "1")
    if pair_gemm:
        monkeypatch.setenv("GLLM_B200_PAIR_MIN_TOKENS", "1")
    folder = write_tiny("D", str(tmp_path / "model"), sharp=False)
    cfg, weights = read_raw(folder, round_to_bf16=True)
    vocab = cfg["vocab_size"]
    seqs = sequences(vocab, seed=5)
    plain = {k: plain_forward(cfg, weights, v, torch.float64) for k, v in seqs.items()}
    steps, index = single_request_steps(seqs)
    results = replay(folder, "bfloat16", steps, str(tmp_path / "out1"), max_tokens=rounded(max(LENGTHS.values())),
                     vocab=vocab)
    compare(results, index, plain, BF16_TOL_MAX, BF16_TOL_MEAN)
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    results = replay(folder, "bfloat16", steps, str(tmp_path / "out2"), max_tokens=448, vocab=vocab)
    compare(results, index, plain, BF16_TOL_MAX, BF16_TOL_MEAN)
