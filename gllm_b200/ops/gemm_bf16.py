"""bf16 matrix products ``x @ W.T`` with fp32 accumulation.

The engine's own kernel (``csrc/gemm_bf16.cu``: tcgen05.mma, accumulator in
tensor memory, operands by TMA) runs every product whose rows are 16-byte
aligned and whose inner size is a multiple of 8; decode steps (M <= 64) run it
with the weight as the 128-row operand and split along K.  Anything else (odd
inner sizes) goes to the library product (cuBLAS through ``torch.matmul``),
which is what the reference uses for every projection
(gllm/model/layers/linear.py:20).
"""

from __future__ import annotations

import os
from ctypes import c_int, c_int64, c_void_p

import torch

from gllm_b200.ops.build import load_module

P = c_void_p
FEW_TOKENS = 64

_umma = None
_scratch: dict[int, dict[str, torch.Tensor]] = {}


def _umma_fns():
    global _umma
    if _umma is None:
        lib = load_module("gemm_bf16")
        f = lib.gllm_gemm_bf16
        f.argtypes = [P, P, P, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, P, P, c_int, P, P]
        f.restype = c_int
        lib.gllm_gemm_bf16_splits.argtypes = [c_int, c_int, c_int]
        lib.gllm_gemm_bf16_splits.restype = c_int
        lib.gllm_gemm_bf16_tiles.argtypes = [c_int, c_int]
        lib.gllm_gemm_bf16_tiles.restype = c_int
        g = lib.gllm_gemm_bf16_gated
        g.argtypes = [P, P, P, c_int, c_int, c_int, c_int64, c_int64, c_int64, P, P]
        g.restype = c_int
        _umma = (f, lib.gllm_gemm_bf16_splits, lib.gllm_gemm_bf16_tiles, g)
    return _umma


_accumulate = None


def _accumulate_fn():
    global _accumulate
    if _accumulate is None:
        lib = load_module("gemm_bf16")
        acc = lib.gllm_gemm_bf16_accumulate
        acc.argtypes = [P, P, P, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, P, P]
        acc.restype = c_int
        _accumulate = acc
    return _accumulate


def _device_scratch(device: torch.device, partial_floats: int, tickets: int):
    """Per-device scratch of the split-K reduction: fp32 partial tiles (two
    buffers used in turn, so an unsummed result survives the next product) and
    the ticket counters (zeroed once; the kernel leaves them at zero)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _scratch.setdefault(idx, {"turn": 0, "retired": [], "generation": 0})
    s["generation"] += 1

    def grow(name, numel, make):
        # a buffer that is outgrown stays allocated: a captured graph may hold its address, and memory
        # given back to the allocator would be handed to somebody else while the graph still writes it
        if name in s:
            s["retired"].append(s[name])
        s[name] = make(numel)

    if "tickets" not in s or s["tickets"].numel() < tickets:
        grow("tickets", max(tickets, 4096), lambda n: torch.zeros(n, dtype=torch.int32, device=device))
    s["turn"] ^= 1
    name = f"partial{s['turn']}"
    if name not in s or s[name].numel() < partial_floats:
        # one item of 128 x 256 per SM (the most a product is cut into) fits without growing
        sms = torch.cuda.get_device_properties(idx).multi_processor_count
        grow(name, max(partial_floats, sms * 128 * 256), lambda n: torch.empty(n, dtype=torch.float32, device=device))
    return s[name], s["tickets"]


def scratch_generation(device: torch.device) -> int:
    """How many products have taken a scratch buffer on ``device`` so far.  An unsummed result
    (``ops.SplitSum``) lives in the buffer of the product that made it, which the product after the
    next one overwrites: a SplitSum remembers the generation it was made in and refuses to be read
    once two more products have run."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return _scratch.get(idx, {}).get("generation", 0)


_pair = None
# From this many tokens on, products that are not cut along K run on pairs of CTAs (cta_group::2) where
# a pair has enough to do (below).  GLLM_B200_PAIR_MIN_TOKENS overrides the threshold and drops the
# second condition: tests use 1 to run small steps through the kernel.
PAIR_MIN_TOKENS = int(os.environ.get("GLLM_B200_PAIR_MIN_TOKENS", 129))
_PAIR_FORCED = "GLLM_B200_PAIR_MIN_TOKENS" in os.environ
PAIR_MIN_BLOCKS = 64
_sm_pairs = {}


def pair_kernel_pays(x: torch.Tensor, n: int) -> bool:
    """The cluster's start and its two barriers cost about 2 us more than the one-CTA kernel's start:
    that is won back once a pair multiplies 64 blocks of 64 along K or more (measured at 2,048 tokens:
    the o-projection, 32 blocks per pair, is 2 us slower on pairs; qkv, 64, the same; down, 128, and
    gate/up, 224, quicker)."""
    m, k = x.shape
    if m < PAIR_MIN_TOKENS:
        return False
    if _PAIR_FORCED:
        return True
    dev = x.device.index or 0
    if dev not in _sm_pairs:
        _sm_pairs[dev] = max(1, torch.cuda.get_device_properties(dev).multi_processor_count // 2)
    items = -(-m // 256) * -(-n // 256)
    per_pair = -(-items // min(items, _sm_pairs[dev]))
    return per_pair * -(-k // 64) >= PAIR_MIN_BLOCKS


def _pair_fn():
    global _pair
    if _pair is None:
        lib = load_module("gemm_bf16_pair")
        f = lib.gllm_gemm_bf16_pair
        f.argtypes = [P, P, P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, P, P]
        f.restype = c_int
        _pair = f
    return _pair


def linear_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False) -> torch.Tensor:
    """``out = x @ weight.T`` (or its gated form, see ``linear_gated``) by the kernel in which two CTAs
    of a cluster share every 256x256 tile.  Any number of tokens is right; few are slow."""
    from gllm_b200 import ops

    m, k = x.shape
    code = _pair_fn()(x.data_ptr(), weight.data_ptr(), out.data_ptr(), int(out.dtype == torch.float32), int(gated), m,
                      weight.shape[0], k, x.stride(0), weight.stride(0), out.stride(0),
                      ops.status_word(x.device).data_ptr(), ops._stream())
    ops._check(code, "gemm_bf16_pair")
    return out


def tensor_core_kernel_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    k = x.shape[1]
    return (k % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    from gllm_b200 import ops

    f, splits_of, tiles_of = _umma_fns()[:3]
    m, k = x.shape
    n = weight.shape[0]
    splits = splits_of(m, n, k)
    if splits == 1 and pair_kernel_pays(x, n):
        return linear_pair(x, weight, out)
    partial, tickets = _device_scratch(x.device, splits * m * n if splits > 1 else 0, tiles_of(m, n))
    if splits > 1 and out.is_contiguous():
        # a second small kernel sums the splits: far quicker than the last CTA of a tile summing them
        code = f(x.data_ptr(), weight.data_ptr(), None, int(out.dtype == torch.float32), m, n, k, x.stride(0),
                 weight.stride(0), n, splits, partial.data_ptr(), tickets.data_ptr(), 0,
                 ops.status_word(x.device).data_ptr(), ops._stream())
        ops._check(code, "gemm_bf16")
        return ops.SplitSum(partial[: splits * m * n].view(splits, m, n), out.dtype,
                            scratch_generation(x.device)).tensor(out)
    code = f(x.data_ptr(), weight.data_ptr(), out.data_ptr(), int(out.dtype == torch.float32), m, n, k,
             x.stride(0), weight.stride(0), out.stride(0), splits, partial.data_ptr(), tickets.data_ptr(), 1,
             ops.status_word(x.device).data_ptr(), ops._stream())
    ops._check(code, "gemm_bf16")
    return out


def linear_split(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype):
    """The product as a SplitSum when the kernel would cut it along K; None
    when it would not (or does not take these operands)."""
    from gllm_b200 import ops

    if not tensor_core_kernel_takes(x, weight):
        return None
    f, splits_of, tiles_of = _umma_fns()[:3]
    m, k = x.shape
    n = weight.shape[0]
    splits = splits_of(m, n, k)
    if splits <= 1:
        return None
    partial, tickets = _device_scratch(x.device, splits * m * n, 0)
    code = f(x.data_ptr(), weight.data_ptr(), None, int(out_dtype == torch.float32), m, n, k, x.stride(0),
             weight.stride(0), n, splits, partial.data_ptr(), tickets.data_ptr(), 0,
             ops.status_word(x.device).data_ptr(), ops._stream())
    ops._check(code, "gemm_bf16")
    return ops.SplitSum(partial[: splits * m * n].view(splits, m, n), out_dtype, scratch_generation(x.device))


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    if tensor_core_kernel_takes(x, weight):
        return linear_tcgen05(x, weight, out)
    if out.dtype == torch.bfloat16:
        torch.matmul(x, weight.t(), out=out)
    else:
        # fp32 logits from bf16 operands: accumulate and write in fp32
        out.copy_(torch.mm(x, weight.t(), out_dtype=torch.float32))
    return out


def linear_gated(x: torch.Tensor, weight: torch.Tensor):
    """``silu(gate) * up`` of a weight stacked in blocks of 64 gate / 64 up rows, fused into the
    product's epilogue; None when the kernel does not take these operands."""
    from gllm_b200 import ops

    n, k = weight.shape
    if not tensor_core_kernel_takes(x, weight) or n % 128:
        return None
    m = x.shape[0]
    out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
    if pair_kernel_pays(x, n):
        return linear_pair(x, weight, out, gated=True)
    g = _umma_fns()[3]
    code = g(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), weight.stride(0), out.stride(0),
             ops.status_word(x.device).data_ptr(), ops._stream())
    ops._check(code, "gemm_bf16_gated")
    return out


# ---- a product that adds itself into the residual stream
def linear_accumulate(x: torch.Tensor, weight: torch.Tensor, acc: torch.Tensor) -> bool:
    """``acc += x @ weight.T`` (``acc`` fp32 ``[m, n]``) inside the product's epilogue, for up to 64
    tokens; False when the kernel does not take the operands (nothing was launched)."""
    from gllm_b200 import ops

    m, k = x.shape
    n = weight.shape[0]
    if (m > FEW_TOKENS or not tensor_core_kernel_takes(x, weight) or acc.dtype != torch.float32
            or tuple(acc.shape) != (m, n) or acc.stride(1) != 1):
        return False
    splits = _umma_fns()[1](m, n, k)
    code = _accumulate_fn()(x.data_ptr(), weight.data_ptr(), acc.data_ptr(), m, n, k, x.stride(0), weight.stride(0),
                            acc.stride(0), splits, ops.status_word(x.device).data_ptr(), ops._stream())
    ops._check(code, "gemm_bf16_accumulate")
    return True
