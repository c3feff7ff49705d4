"""Python entry points of the CUDA kernels.

Every function takes CUDA tensors, checks what the kernel assumes (device,
dtype, contiguity, sizes it accepts) and launches on the current stream.
There is no CPU path and no PyTorch fallback: a tensor that is not on a CUDA
device, or a kernel module that cannot be built, raises.

Naming: ``*_f32`` / ``*_bf16`` symbols are the two instantiations of a kernel
for the activation and weight-matrix type.  The residual stream, norm weights,
rotary frequencies, softmax statistics and logits are fp32 in both.
"""

from __future__ import annotations

import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from gllm_b200.ops.build import ExtensionError, build_all, load_module

__all__ = [
    "ExtensionError",
    "build_all",
    "embedding",
    "scale_softcap",
    "scatter_int32",
    "add_rmsnorm",
    "silu_mul",
    "rope_store",
    "linear",
    "paged_attention",
    "status_word",
    "check_status",
    "sample",
    "argmax",
    "SplitSum",
    "ADDED",
    "as_tensor",
    "linear_gated",
    "interleave_gate_up",
    "add_bias",
    "rmsnorm_heads",
]

P = c_void_p
_SIGNATURES = {
    "elementwise": {
        "gllm_embedding_{t}": [P, P, P, P, P, c_int, c_int, c_int, c_float, P, P],
        "gllm_scale_softcap_f32": [P, c_int64, c_float, c_float, P],
        "gllm_scatter_i32": [P, c_int64, P, P, c_int, P, P],
        "gllm_add_bias_{t}": [P, c_int64, P, c_int, c_int, P],
        "gllm_rmsnorm_heads_{t}": [P, c_int64, P, c_int, c_int, c_int, c_int, c_float, c_int, P],
        "gllm_add_rmsnorm_{t}": [P, P, c_int, c_int64, P, P, P, P, c_int, c_int, c_float, c_int, P],
        "gllm_sum_parts_{t}": [P, c_int, c_int64, P, c_int64, P],
        "gllm_silu_mul_{t}": [P, P, c_int, c_int, c_int, P],
        "gllm_rope_store_{t}": [P, P, c_int, c_int64, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, P, P],
    },
    "gemm_fp32": {
        "gllm_gemm_f32": [P, P, P, c_int, c_int, c_int, c_int64, c_int64, c_int64, P],
    },
    "sampling": {
        "gllm_sample": [P, c_int64, c_int, c_int, P, P, P, P, P, P, c_int, P, P, P, P, P, P, P],
        "gllm_argmax": [P, c_int64, c_int, c_int, P, P, P],
    },
    "attention_simt": {
        "gllm_attention_simt_{t}": [P, c_int64, P, c_int64, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_float, c_int, P, P],
    },
}

_functions: dict[str, object] = {}


def _fn(module: str, name: str):
    f = _functions.get(name)
    if f is not None:
        return f
    lib = load_module(module)
    for pattern, argtypes in _SIGNATURES[module].items():
        for t in ("f32", "bf16"):
            sym = pattern.format(t=t)
            if sym in _functions:
                continue
            try:
                func = getattr(lib, sym)
            except AttributeError:
                continue
            func.argtypes = argtypes
            func.restype = c_int
            _functions[sym] = func
    try:
        return _functions[name]
    except KeyError:
        raise ExtensionError(f"kernel module {module!r} exports no symbol {name!r}") from None


def _error_string(code: int) -> str:
    try:
        return torch.cuda.cudart().cudaGetErrorString(torch.cuda.cudart().cudaError(code))
    except Exception:
        return f"cudaError {code}"


def modules_for(dtype: torch.dtype, head_dims=(), sampling: bool = False) -> list[str]:
    """The kernel modules a model of this compute dtype with mixers of these head sizes will load."""
    if dtype == torch.float32:
        names = ["elementwise", "gemm_fp32", "attention_simt"]
    else:
        names = ["elementwise", "gemm_bf16", "gemm_bf16_pair", "attention_bf16", "attention_prefill_bf16"]
        if any(d in (64, 128) for d in head_dims):
            names += ["attention_prefill_tmem", "attention_decode_tma"]
        if any(d not in (32, 64, 128) for d in head_dims):
            names.append("attention_simt")
    if sampling:
        names.append("sampling")
    return names


def prepare(dtype: torch.dtype, head_dims=(), sampling: bool = False) -> None:
    """Compile (side by side) whatever of ``modules_for`` is not built yet."""
    from gllm_b200.ops.build import compile_modules

    compile_modules(modules_for(dtype, head_dims, sampling))


# number of kernel launches made through this module (benchmarks read it)
launch_count = 0


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise RuntimeError(f"{what}: launch failed: {_error_string(code)} (code {code})")


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise TypeError(f"kernels take float32 or bfloat16 activations, not {dtype}")


def _cuda(t: torch.Tensor, name: str, dtype: torch.dtype | None = None, contiguous: bool = True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this engine has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (every kernel is launched on it).  The raw getter costs a
    fraction of a microsecond; building a ``torch.cuda.Stream`` object for every launch cost 15 us."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------- status
_status: dict[int, torch.Tensor] = {}

STATUS_BITS = {
    1: "a token id outside the vocabulary",
    2: "a cache page id outside the pool",
    4: "a bounded wait inside a kernel ran out",
}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """The device's int32 status word that kernels OR error bits into."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Read the status word (a device sync) and raise if a kernel set a bit."""
    t = status_word(device)
    value = int(t.item())
    if value:
        t.zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit] or [f"status {value}"]
        raise RuntimeError("a kernel reported: " + "; ".join(reasons))


# ------------------------------------------------------------ unsummed splits
class SplitSum:
    """The result of a product that was cut along K and whose ``splits`` fp32
    partial results ``parts [splits, rows, cols]`` were left unsummed: the
    kernel that consumes it (``add_rmsnorm``, ``rope_store``) adds them in
    ascending order, which saves a reduction pass.  ``parts`` lives in one of
    two scratch buffers that the products take in turn: it survives the next
    product and is overwritten by the one after.  Consume a SplitSum (or call
    ``as_tensor`` on it) before two more products have run; reading it later
    raises."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype, generation: int | None = None):
        self.parts = parts
        self.dtype = dtype
        # the count of scratch-taking products on the device when this one ran (None: the parts are
        # the caller's own memory)
        self.generation = generation

    def check_alive(self) -> None:
        if self.generation is None:
            return
        from gllm_b200.ops import gemm_bf16

        now = gemm_bf16.scratch_generation(self.parts.device)
        if now - self.generation > 1:
            raise RuntimeError(
                f"an unsummed product was read after {now - self.generation} further products: its partial sums "
                "have been overwritten (sum it with ops.as_tensor before running two more products)")

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def device(self):
        return self.parts.device

    def tensor(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """The summed result as an ordinary tensor of ``dtype`` (into ``out``, contiguous, when given)."""
        self.check_alive()
        if out is None:
            out = torch.empty(tuple(self.shape), dtype=self.dtype, device=self.parts.device)
        f = _fn("elementwise", f"gllm_sum_parts_{_suffix(self.dtype)}")
        _check(f(self.parts.data_ptr(), self.parts.shape[0], self.parts.stride(0), out.data_ptr(), out.numel(),
                 _stream()), "sum_parts")
        return out


class _Added:
    """What a product returns when it has added its result into the matrix it was given
    (``linear(..., add_into=...)``): there is nothing left to add."""

    def __repr__(self):
        return "ops.ADDED"


ADDED = _Added()


def as_tensor(x):
    """``x`` itself, or the summed tensor of a SplitSum."""
    return x.tensor() if isinstance(x, SplitSum) else x


def _parts_args(x):
    if isinstance(x, SplitSum):
        x.check_alive()
        return x.parts.data_ptr(), x.parts.shape[0], x.parts.stride(0)
    return None, 0, 0


# ---------------------------------------------------------------- embedding
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None,
              sampled: torch.Tensor | None = None, token_row: torch.Tensor | None = None,
              scale: float = 1.0) -> torch.Tensor:
    """fp32 residual rows ``table[tokens] * scale`` (gllm/model/model.py:175-182; the reference has
    no multiplier).

    With ``sampled`` and ``token_row``: a negative token id stands for
    ``sampled[token_row[i]]``, the token the previous step's argmax left on the
    device for that request, so a decode step can be queued before the host
    has seen the previous step's tokens."""
    _cuda(tokens, "tokens", torch.int32)
    if sampled is not None:
        _cuda(sampled, "sampled", torch.int32)
        _cuda(token_row, "token_row", torch.int32)
    _cuda(table, "table")
    n, (vocab, hidden) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    else:
        _cuda(out, "out", torch.float32)
    f = _fn("elementwise", f"gllm_embedding_{_suffix(table.dtype)}")
    _check(f(tokens.data_ptr(), _ptr(sampled), _ptr(token_row) if sampled is not None else None, table.data_ptr(),
             out.data_ptr(), n, hidden, vocab, float(scale), status_word(table.device).data_ptr(), _stream()),
           "embedding")
    return out


def scatter_int32(dst: torch.Tensor, index: torch.Tensor, values: torch.Tensor) -> None:
    """``dst.view(-1)[index[i]] = values[i]`` for int32 tensors (indices are distinct); an index
    outside ``dst`` sets a status bit and is skipped."""
    _cuda(dst, "dst", torch.int32)
    _cuda(index, "index", torch.int32)
    _cuda(values, "values", torch.int32)
    if index.numel() != values.numel():
        raise ValueError("index and values differ in length")
    f = _fn("elementwise", "gllm_scatter_i32")
    _check(f(dst.data_ptr(), dst.numel(), index.data_ptr(), values.data_ptr(), index.numel(),
             status_word(dst.device).data_ptr(), _stream()), "scatter_int32")


def scale_softcap(logits: torch.Tensor, scale: float = 1.0, cap: float | None = None) -> torch.Tensor:
    """In place on fp32 ``logits``: multiply by ``scale``, then with ``cap``: ``cap * tanh(x / cap)``."""
    _cuda(logits, "logits", torch.float32)
    f = _fn("elementwise", "gllm_scale_softcap_f32")
    _check(f(logits.data_ptr(), logits.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return logits


# ------------------------------------------------- bias, norm of every head
def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x[r] += bias`` in place (``bias`` fp32, one value per column): the bias of a projection.  The
    reference's projections have none (gllm/model/layers/linear.py:20)."""
    _cuda(x, "x", contiguous=False)
    _cuda(bias, "bias", torch.float32)
    if x.dim() != 2 or x.stride(1) != 1 or bias.numel() != x.shape[1]:
        raise ValueError("add_bias takes rows of contiguous columns and one bias value per column")
    f = _fn("elementwise", f"gllm_add_bias_{_suffix(x.dtype)}")
    _check(f(x.data_ptr(), x.stride(0), bias.data_ptr(), x.shape[0], x.shape[1], _stream()), "add_bias")
    return x


def rmsnorm_heads(x: torch.Tensor, weight: torch.Tensor, eps: float, first_head: int, num_heads: int, head_dim: int,
                  unit_offset: bool = False) -> torch.Tensor:
    """RMSNorm of each of ``num_heads`` heads of ``head_dim`` columns, from head ``first_head`` on, of every row
    of ``x``, in place, with one weight of ``head_dim`` values for all of them; statistics in fp32.  (A norm of
    the queries and keys before their rotation; the reference has none.)"""
    _cuda(x, "x", contiguous=False)
    _cuda(weight, "weight", torch.float32)
    if x.dim() != 2 or x.stride(1) != 1 or (first_head + num_heads) * head_dim > x.shape[1]:
        raise ValueError("the heads do not lie inside the rows of x")
    if weight.numel() != head_dim or head_dim > 256:
        raise ValueError("rmsnorm_heads takes one weight value per column of a head, for heads of up to 256 columns")
    f = _fn("elementwise", f"gllm_rmsnorm_heads_{_suffix(x.dtype)}")
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), x.shape[0], int(first_head), int(num_heads), int(head_dim),
             float(eps), int(unit_offset), _stream()), "rmsnorm_heads")
    return x


# ------------------------------------------------------------- add + RMSNorm
def add_rmsnorm(
    branch: torch.Tensor | None,
    resid: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    out_dtype: torch.dtype,
    rows: torch.Tensor | None = None,
    unit_offset: bool = False,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``resid += branch`` (fp32, in place) then RMSNorm of the sum.

    With ``rows`` only those rows are normed and ``resid`` is left untouched.
    """
    _cuda(resid, "resid", torch.float32)
    _cuda(weight, "weight", torch.float32)
    hidden = resid.shape[-1]
    if weight.numel() != hidden:
        raise ValueError(f"norm weight has {weight.numel()} elements, rows have {hidden}")
    parts_ptr, n_parts, part_stride = _parts_args(branch)
    if isinstance(branch, SplitSum):
        if tuple(branch.shape) != tuple(resid.shape) or branch.dtype != out_dtype:
            raise ValueError("branch and resid differ in shape or dtype")
        branch = None
    elif branch is not None:
        _cuda(branch, "branch", out_dtype)
        if branch.shape != resid.shape:
            raise ValueError("branch and resid differ in shape")
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
        n_rows = rows.numel()
    else:
        n_rows = resid.numel() // hidden
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=out_dtype, device=resid.device)
    else:
        _cuda(out, "out", out_dtype)
    f = _fn("elementwise", f"gllm_add_rmsnorm_{_suffix(out_dtype)}")
    _check(f(_ptr(branch), parts_ptr, n_parts, part_stride, resid.data_ptr(), weight.data_ptr(), out.data_ptr(),
             _ptr(rows), n_rows, hidden, float(eps), int(unit_offset), _stream()), "add_rmsnorm")
    return out


# ------------------------------------------------------------------ SiLU·up
GATED_BLOCK = 64


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` of ``[n, 2*inter]``.  ``block`` 0: gate columns first, up columns after;
    ``block`` b: b gate columns alternate with the b up columns of the same features."""
    _cuda(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise ValueError("gate_up must have an even number of columns")
    inter = two_i // 2
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("elementwise", f"gllm_silu_mul_{_suffix(gate_up.dtype)}")
    _check(f(gate_up.data_ptr(), out.data_ptr(), n, inter, int(block), _stream()), "silu_mul")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = GATED_BLOCK) -> torch.Tensor:
    """Stack ``gate`` and ``up`` ``[inter, hidden]`` so that ``block`` gate rows alternate with the
    ``block`` up rows of the same features (``inter`` must be a multiple of ``block``)."""
    inter, hidden = gate.shape
    if inter % block:
        raise ValueError("intermediate size must be a multiple of the block")
    stacked = torch.stack([gate.view(inter // block, block, hidden), up.view(inter // block, block, hidden)], dim=1)
    return stacked.reshape(2 * inter, hidden).contiguous()


def linear_gated(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` for a weight stacked by ``interleave_gate_up``: one kernel
    with the activation in the product's epilogue where the tensor-core kernel takes the operands,
    the product and ``silu_mul`` otherwise."""
    _cuda(x, "x")
    _cuda(weight, "weight", x.dtype)
    if x.dtype == torch.bfloat16:
        from gllm_b200.ops import gemm_bf16

        fused = gemm_bf16.linear_gated(x, weight)
        if fused is not None:
            return fused
    return silu_mul(linear(x, weight), block=GATED_BLOCK)


# --------------------------------------------------- rotary + cache store
def rope_store(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    inv_freq: torch.Tensor | None,
    slot_mapping: torch.Tensor | None,
    cache_layer: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    interleaved: bool = False,
) -> torch.Tensor:
    """Rotate q and k of ``qkv`` in place and store k, v into the cache;
    returns ``qkv`` (a SplitSum is summed into a new tensor first, in the same
    kernel).

    ``cache_layer`` is ``[pages, 2, kv_heads, block_size, head_dim]``.
    """
    parts_ptr, n_parts, part_stride = _parts_args(qkv)
    if isinstance(qkv, SplitSum):
        qkv = torch.empty(tuple(qkv.shape), dtype=qkv.dtype, device=qkv.device)
    _cuda(qkv, "qkv")
    _cuda(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv width does not equal (heads + 2*kv_heads) * head_dim")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise ValueError("inv_freq must hold rotary_dim/2 frequencies")
    block_size = num_pages = 0
    if slot_mapping is not None:
        _cuda(slot_mapping, "slot_mapping", torch.int32)
        _cuda(cache_layer, "cache_layer", qkv.dtype)
        num_pages, two, hkv, block_size, d = cache_layer.shape
        if two != 2 or hkv != num_kv_heads or d != head_dim:
            raise ValueError("cache layer shape does not match the mixer's heads")
    f = _fn("elementwise", f"gllm_rope_store_{_suffix(qkv.dtype)}")
    _check(f(qkv.data_ptr(), parts_ptr, n_parts, part_stride, positions.data_ptr(), _ptr(inv_freq),
             _ptr(slot_mapping), _ptr(cache_layer) if slot_mapping is not None else None, n, num_heads,
             num_kv_heads, head_dim, rotary_dim, int(interleaved), block_size, num_pages,
             status_word(qkv.device).data_ptr(), _stream()), "rope_store")
    return qkv


# ------------------------------------------------------------------- linear
# Products of few tokens that end a branch add themselves into the residual stream
# (GLLM_B200_FUSE_ADD=0: they leave their result to the norm kernel after them).
ACCUMULATE_IN_PRODUCT = os.environ.get("GLLM_B200_FUSE_ADD", "1") != "0"


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None, split_ok: bool = False, add_into: torch.Tensor | None = None,
           bias: torch.Tensor | None = None):
    """``x @ weight.T`` with ``weight`` stored ``[out, in]``
    (gllm/model/layers/linear.py:20).  fp32 inputs run the FFMA kernel (no
    tensor-core mode); bf16 inputs run the tensor-core kernels with fp32
    accumulation.  With ``split_ok`` the result may be a SplitSum (for callers
    that hand it to ``add_rmsnorm`` or ``rope_store``).  With ``add_into``
    (fp32 ``[m, n]``, the residual stream) the product may add itself there
    and return ``ADDED``; when it returns anything else, nothing was added.  With ``bias`` (fp32, one
    value per output column) the result is an ordinary tensor with the bias added."""
    if bias is not None:
        return add_bias(linear(x, weight, out_dtype=out_dtype, out=out), bias)
    _cuda(x, "x")
    _cuda(weight, "weight", x.dtype)
    m, k = x.shape
    n, k2 = weight.shape
    if k != k2:
        raise ValueError(f"x has {k} columns, weight has {k2}")
    out_dtype = out_dtype or x.dtype
    if add_into is not None and x.dtype == torch.bfloat16 and out is None and ACCUMULATE_IN_PRODUCT:
        from gllm_b200.ops import gemm_bf16

        if gemm_bf16.linear_accumulate(x, weight, add_into):
            return ADDED
    if x.dtype == torch.bfloat16 and split_ok and out is None:
        from gllm_b200.ops import gemm_bf16

        split = gemm_bf16.linear_split(x, weight, out_dtype)
        if split is not None:
            return split
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    else:
        _cuda(out, "out", out_dtype)
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise TypeError("the fp32 product writes fp32")
        f = _fn("gemm_fp32", "gllm_gemm_f32")
        _check(f(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, k, k, n, _stream()), "gemm_f32")
        return out
    from gllm_b200.ops import gemm_bf16

    return gemm_bf16.linear_bf16(x, weight, out)


# ---------------------------------------------------------------- attention
def paged_attention_simt(
    q: torch.Tensor,
    q_stride: int,
    cache_layer: torch.Tensor,
    block_table: torch.Tensor,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    num_heads: int,
    scale: float,
    window: int,
    out: torch.Tensor,
) -> torch.Tensor:
    num_pages, _, hkv, block_size, d = cache_layer.shape
    n = positions.numel()
    f = _fn("attention_simt", f"gllm_attention_simt_{_suffix(q.dtype)}")
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], cache_layer.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), positions.data_ptr(), token_row.data_ptr(), n, num_heads, hkv, d, block_size,
             num_pages, float(scale), int(window), status_word(q.device).data_ptr(), _stream()), "attention_simt")
    return out


def paged_attention(
    qkv: torch.Tensor,
    cache_layer: torch.Tensor,
    block_table: torch.Tensor,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    num_heads: int,
    scale: float,
    window: int | None = None,
    batch=None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Causal attention of every token of the batch over its request's cache.

    ``qkv`` is ``[n, (heads + 2*kv_heads) * head_dim]`` with rotated queries in
    its first ``heads * head_dim`` columns; the keys and values of the batch's
    own tokens are already in ``cache_layer``.  ``token_row[i]`` is the row of
    ``block_table`` that token ``i``'s request uses.  ``batch`` optionally
    carries per-request metadata that the tensor-core kernels need.
    """
    _cuda(qkv, "qkv")
    _cuda(cache_layer, "cache_layer", qkv.dtype)
    _cuda(block_table, "block_table", torch.int32, contiguous=False)
    _cuda(positions, "positions", torch.int32)
    _cuda(token_row, "token_row", torch.int32)
    num_pages, two, hkv, block_size, d = cache_layer.shape
    if two != 2:
        raise ValueError("cache layer must be [pages, 2, kv_heads, block_size, head_dim]")
    if d % 16 or d > 256:
        raise ValueError(f"head_dim {d} is not supported: it must be a multiple of 16 up to 256")
    if num_heads % hkv:
        raise ValueError("the number of query heads must be a multiple of the number of kv heads")
    n = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * hkv) * d:
        raise ValueError("qkv width does not equal (heads + 2*kv_heads) * head_dim")
    if block_table.stride(1) != 1:
        raise ValueError("block_table rows must be contiguous")
    if out is None:
        out = torch.empty((n, num_heads * d), dtype=qkv.dtype, device=qkv.device)
    win = int(window) if window else 0
    if qkv.dtype == torch.bfloat16:
        from gllm_b200.ops import attention_bf16

        if attention_bf16.supports(d, block_size) and batch is not None:
            return attention_bf16.paged_attention_bf16(qkv, cache_layer, block_table, positions, token_row,
                                                       num_heads, scale, win, batch, out)
    return paged_attention_simt(qkv, qkv.shape[1], cache_layer, block_table, positions, token_row, num_heads,
                                scale, win, out)


# ----------------------------------------------------------------- sampling
MAX_LOGPROBS = 32


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None,
           scatter_index: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of every row (lowest index on ties), int32.
    With ``scatter_index`` row ``r``'s result is written to ``out[scatter_index[r]]``."""
    _cuda(logits, "logits", torch.float32, contiguous=False)
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise ValueError("logit rows must be contiguous")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if scatter_index is not None:
        _cuda(scatter_index, "scatter_index", torch.int32)
        if scatter_index.numel() < rows:
            raise ValueError("scatter_index needs one entry per row")
    f = _fn("sampling", "gllm_argmax")
    _check(f(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), _ptr(scatter_index), _stream()),
           "argmax")
    return out


def sample(
    logits: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    seed: torch.Tensor,
    counter: torch.Tensor,
    num_logprobs: torch.Tensor | None = None,
    max_logprobs: int = 0,
    return_probs: bool = False,
):
    """One token per row from fp32 ``logits [rows, vocab]``.

    Per row: ``temperature`` (0 = greedy), ``top_k`` (0 = whole vocabulary,
    1 = greedy), ``top_p``, ``seed`` (int64) and ``counter`` (int32) of the
    counter-based generator.  Returns a dict with ``tokens`` int32,
    ``logprobs`` (of the sampled tokens), ``num_candidates``, and when
    ``max_logprobs`` > 0 ``top_logprobs`` / ``top_ids`` ``[rows, max_logprobs]``
    of which the first ``min(num_logprobs[row], num_candidates[row])`` are valid;
    with ``return_probs`` also the distribution drawn from, ``[rows, vocab]``.
    """
    _cuda(logits, "logits", torch.float32, contiguous=False)
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise ValueError("logit rows must be contiguous")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("seed", seed, torch.int64),
                        ("counter", counter, torch.int32)):
        _cuda(t, name, dt)
        if t.numel() != rows:
            raise ValueError(f"{name} must have one entry per row")
    if max_logprobs > MAX_LOGPROBS:
        raise ValueError(f"at most {MAX_LOGPROBS} log-probabilities per token are supported")
    dev = logits.device
    out = {
        "tokens": torch.empty(rows, dtype=torch.int32, device=dev),
        "logprobs": torch.empty(rows, dtype=torch.float32, device=dev),
        "num_candidates": torch.empty(rows, dtype=torch.int32, device=dev),
    }
    top_lp = top_id = None
    if max_logprobs > 0:
        _cuda(num_logprobs, "num_logprobs", torch.int32)
        top_lp = torch.zeros((rows, max_logprobs), dtype=torch.float32, device=dev)
        top_id = torch.full((rows, max_logprobs), -1, dtype=torch.int32, device=dev)
        out["top_logprobs"], out["top_ids"] = top_lp, top_id
    probs = torch.empty((rows, vocab), dtype=torch.float32, device=dev) if return_probs else None
    if probs is not None:
        out["probs"] = probs
    f = _fn("sampling", "gllm_sample")
    _check(f(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(), top_k.data_ptr(),
             top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(),
             _ptr(num_logprobs) if max_logprobs > 0 else None, max_logprobs, out["tokens"].data_ptr(),
             out["logprobs"].data_ptr(), out["num_candidates"].data_ptr(), _ptr(top_lp), _ptr(top_id),
             _ptr(probs), _stream()), "sample")
    return out
