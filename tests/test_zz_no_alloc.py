"""The decode attention entry point for callers that cannot allocate device memory
(gllm_b200/csrc/attention_decode_noalloc.h), called through its exported C symbol and
compared with the ordinary entry point, which takes its scratch from the caller, and
with a plain float64 attention over the same pages (a fault both entry points share
would pass the first comparison).

Such callers (a plugin inside a runtime that owns all device memory, code between the
fixing of a memory budget and the end of the process, a loop that cannot afford an
allocation's device-wide synchronisation) have no place to get scratch from, so the library
carries it in its own device image.  This file is collected last on purpose: a run that
stops at the first failure has then already run every other test."""

import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

P = c_void_p
MAX_FLOATS = 4 * 1024 * 1024


def _library():
    from gllm_b200.ops.build import load_module

    lib = load_module("attention_bf16")
    noalloc = lib.gllm_attention_decode_bf16_noalloc
    noalloc.argtypes = [P, c_int64, P, c_int64, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_float, c_int, P, P]
    noalloc.restype = c_int
    ordinary = lib.gllm_attention_decode_bf16
    ordinary.argtypes = [P, c_int64, P, c_int64, P, P, c_int, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_float, c_int, P, P]
    ordinary.restype = c_int
    chunk = lib.gllm_attention_decode_chunk
    chunk.argtypes = [c_int]
    chunk.restype = c_int
    return noalloc, ordinary, chunk


def _case(seed, batch, context, hq, hkv, d, block_size):
    g = torch.Generator().manual_seed(seed)
    pages_per_request = -(-context // block_size)
    num_pages = batch * pages_per_request + 2
    pool = torch.randn(num_pages, 2, hkv, block_size, d, generator=g).to(torch.bfloat16).cuda()
    table = torch.randperm(num_pages, generator=g)[: batch * pages_per_request].to(torch.int32)
    table = table.view(batch, pages_per_request).contiguous().cuda()
    q = torch.randn(batch, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16).cuda()
    positions = torch.randint(context // 2, context, (batch,), generator=g).to(torch.int32).cuda()
    rows = torch.arange(batch, dtype=torch.int32).cuda()
    return pool, table, q, positions, rows


def _plain(pool, table, q, positions, hq, hkv, d, scale):
    """Plain attention of each query over keys 0 .. its position, gathered page by page."""
    pool, table, q = pool.double().cpu(), table.cpu().long(), q.double().cpu()
    out = []
    for b in range(q.shape[0]):
        n = int(positions[b]) + 1
        k = pool[table[b], 0].permute(0, 2, 1, 3).reshape(-1, hkv, d)[:n]      # [tokens, hkv, d]
        v = pool[table[b], 1].permute(0, 2, 1, 3).reshape(-1, hkv, d)[:n]
        k = k.repeat_interleave(hq // hkv, 1)
        v = v.repeat_interleave(hq // hkv, 1)
        scores = torch.einsum("hd,khd->hk", q[b, : hq * d].view(hq, d), k) * scale
        out.append(torch.einsum("hk,khd->hd", scores.softmax(-1), v).reshape(hq * d))
    return torch.stack(out)


def test_no_alloc_entry_point_equals_the_ordinary_one_twice_in_a_row():
    noalloc, ordinary, chunk_of = _library()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different sizes: the second finds the first one's leftovers in the scratch
    for seed, (batch, context, hq, hkv, d, bs) in enumerate([(6, 700, 32, 8, 64, 16), (3, 300, 12, 2, 128, 32)]):
        pool, table, q, positions, rows = _case(seed, batch, context, hq, hkv, d, bs)
        chunks = -(-context // chunk_of(d))
        scale = 1.0 / math.sqrt(d)
        want = torch.full((batch, hq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        got = torch.full_like(want, float("nan"))
        part_o = torch.empty(batch * hq * chunks * d, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(batch * hq * chunks * 2, dtype=torch.float32, device="cuda")
        code = ordinary(q.data_ptr(), q.shape[1], want.data_ptr(), want.shape[1], pool.data_ptr(), table.data_ptr(),
                        table.shape[1], positions.data_ptr(), rows.data_ptr(), batch, part_o.data_ptr(),
                        part_ml.data_ptr(), hq, pool.shape[2], d, bs, pool.shape[0], chunks, scale, 0,
                        status.data_ptr(), stream)
        assert code == 0
        code = noalloc(q.data_ptr(), q.shape[1], got.data_ptr(), got.shape[1], pool.data_ptr(), table.data_ptr(),
                       table.shape[1], positions.data_ptr(), rows.data_ptr(), batch, hq, pool.shape[2], d, bs,
                       pool.shape[0], chunks, scale, 0, status.data_ptr(), stream)
        assert code == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert not got.float().isnan().any()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)            # the same kernels: in fact bit for bit
        plain = _plain(pool, table, q, positions, hq, pool.shape[2], d, scale)
        torch.testing.assert_close(got.double().cpu(), plain, rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    noalloc, _, chunk_of = _library()
    pool, table, q, positions, rows = _case(5, 2, 64, 4, 2, 64, 16)
    out = torch.zeros(2, 4 * 64, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    too_many_chunks = MAX_FLOATS // (2 * 4 * (64 + 2)) + 1
    code = noalloc(q.data_ptr(), q.shape[1], out.data_ptr(), out.shape[1], pool.data_ptr(), table.data_ptr(),
                   table.shape[1], positions.data_ptr(), rows.data_ptr(), 2, 4, 2, 64, 16, pool.shape[0],
                   too_many_chunks, 0.125, 0, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == 1                             # cudaErrorInvalidValue: nothing was launched
    # sizes whose product wraps around 64 bits must not slip under the limit
    for nq, heads, chunks, hd in [(65535, 1024, 2 ** 31 - 1, 128), (2 ** 31 - 1, 2 ** 31 - 2, 2 ** 31 - 1, 64),
                                  (2, 4, 1, 2 ** 30), (2, 2 ** 31 - 2, 2 ** 31 - 1, 128)]:
        code = noalloc(q.data_ptr(), q.shape[1], out.data_ptr(), out.shape[1], pool.data_ptr(), table.data_ptr(),
                       table.shape[1], positions.data_ptr(), rows.data_ptr(), nq, heads, 2, hd, 16, pool.shape[0],
                       chunks, 0.125, 0, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert code == 1, (nq, heads, chunks, hd)
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0
