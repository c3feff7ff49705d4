"""Compiles the CUDA sources under ``gllm_b200/csrc`` for sm_100a and loads them.

Each kernel module is one ``.cu`` file built by ``nvcc`` into a shared library
with ``extern "C"`` entry points and loaded through ``ctypes``.  A module is
compiled the first time something asks for it, so a run compiles only what
its model and dtype need.  Libraries are kept beside the sources in
``csrc/_build`` (named by a hash of source and flags); when that folder cannot
be written they go to a per-user folder under the system's temporary folder.
There is no fallback: if a module cannot be built or loaded, the call fails.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC_DIR = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--shared",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]

# module name -> source file (each includes only headers under csrc/)
MODULES = {
    "elementwise": "elementwise.cu",
    "gemm_fp32": "gemm_fp32.cu",
    "attention_simt": "attention_simt.cu",
    "sampling": "sampling.cu",
    "gemm_bf16": "gemm_bf16.cu",
    "gemm_bf16_pair": "gemm_bf16_pair.cu",
    "attention_bf16": "attention_bf16.cu",
    "attention_prefill_bf16": "attention_prefill_bf16.cu",
    "attention_prefill_tmem": "attention_prefill_tmem.cu",
    "attention_decode_tma": "attention_decode_tma.cu",
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class ExtensionError(RuntimeError):
    """A CUDA module could not be compiled or loaded."""


def _flags() -> list[str]:
    """NVCC_FLAGS plus what ``GLLM_B200_NVCC_EXTRA`` adds (for instance ``-DNAME=value`` of a tuning
    constant a source file exposes); the library's name follows the flags."""
    extra = os.environ.get("GLLM_B200_NVCC_EXTRA", "").split()
    return NVCC_FLAGS + extra


def _nvcc() -> str:
    cand = os.environ.get("GLLM_B200_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(cand):
        raise ExtensionError("nvcc not found (looked on PATH and at /usr/local/cuda/bin/nvcc)")
    return cand


def _headers() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cuh")) + sorted(CSRC_DIR.glob("*.h"))


def _digest(source: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_flags()).encode())
    for p in [source] + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:12]


def _build_dirs() -> list[Path]:
    dirs = [CSRC_DIR / "_build"]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(Path(tempfile.gettempdir()) / f"gllm_b200_build_{uid}")
    return dirs


def _writable_dir() -> Path:
    for d in _build_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}_{threading.get_ident()}"       # modules are built in parallel
            probe.write_bytes(b"")
            try:
                probe.unlink()
            except FileNotFoundError:
                pass
            return d
        except OSError:
            continue
    raise ExtensionError("no writable folder for compiled kernels")


def library_path(module: str) -> Path | None:
    """Path of the already built library of ``module``, or None."""
    source = CSRC_DIR / MODULES[module]
    name = f"gllm_{module}.{_digest(source)}.so"
    for d in _build_dirs():
        if (d / name).is_file():
            return d / name
    return None


def compile_module(module: str, verbose: bool = True) -> Path:
    """Build ``module`` if no library with the current hash exists."""
    if module not in MODULES:
        raise ExtensionError(f"unknown kernel module {module!r}")
    source = CSRC_DIR / MODULES[module]
    if not source.is_file():
        raise ExtensionError(f"kernel source {source} is missing")
    found = library_path(module)
    if found is not None:
        return found
    out_dir = _writable_dir()
    out = out_dir / f"gllm_{module}.{_digest(source)}.so"
    tmp_out = out_dir / f".{out.name}.{os.getpid()}.tmp"
    cmd = [_nvcc(), *_flags(), "-I", str(CSRC_DIR), "-o", str(tmp_out), str(source)]
    t0 = time.time()
    if verbose:
        print(f"[gllm_b200] compiling {source.name} for sm_100a ...", file=sys.stderr, flush=True)
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(
                    f"[gllm_b200] still compiling {source.name} ({time.time() - t0:.0f} s)",
                    file=sys.stderr,
                    flush=True,
                )

    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    try:
        output, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            tmp_out.unlink()
        except OSError:
            pass
        raise ExtensionError(f"nvcc failed on {source.name} (exit {proc.returncode}):\n{output}")
    os.replace(tmp_out, out)
    # libraries of older versions of this module's source are of no use any more
    for old in out_dir.glob(f"gllm_{module}.*.so"):
        if old != out and not os.environ.get("GLLM_B200_NVCC_EXTRA"):
            try:
                old.unlink()
            except OSError:
                pass
    if verbose:
        print(f"[gllm_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_module(module: str) -> ctypes.CDLL:
    """The loaded library of ``module``; compiles it on first use."""
    lib = _loaded.get(module)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(module)
        if lib is not None:
            return lib
        path = compile_module(module)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise ExtensionError(f"cannot load {path}: {e}") from e
        _loaded[module] = lib
        return lib


def build_all(verbose: bool = True) -> dict[str, Path]:
    """Compile every module whose source exists (in parallel)."""
    return compile_modules([m for m in MODULES if (CSRC_DIR / MODULES[m]).is_file()], verbose=verbose)


def compile_modules(names, verbose: bool = True) -> dict[str, Path]:
    """Compile the named modules that are not built yet, side by side (a first call that needs six
    modules then waits for the slowest of them, not for their sum)."""
    results: dict[str, Path] = {}
    errors: list[str] = []

    def _one(name):
        try:
            results[name] = compile_module(name, verbose=verbose)
        except ExtensionError as e:  # collected, raised together below
            errors.append(str(e))

    threads = [threading.Thread(target=_one, args=(m,)) for m in dict.fromkeys(names)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise ExtensionError("\n\n".join(errors))
    return results
