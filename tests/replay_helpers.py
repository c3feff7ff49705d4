"""Drives ``bin/trace_run`` as a child process the way a user would and reads
the logits it writes."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model_dir: str, dtype: str, steps: list[dict], out_dir: str, max_tokens: int, vocab: int,
           timeout: float = 900.0) -> dict[int, np.ndarray]:
    """Feed ``steps`` one at a time (the next only after ``done <step>``) and
    return {step: logits [wanted, vocab]}."""
    os.makedirs(out_dir, exist_ok=True)
    proc = subprocess.Popen(
        [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1,
    )
    try:
        for step in steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
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
