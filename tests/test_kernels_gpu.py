"""Each kernel alone against a plain PyTorch fp32/fp64 restatement of the same
operation, at sizes other than the tiny models' and the 1B model's."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.fixture(scope="module")
def ops():
    from gllm_b200 import ops as _ops

    return _ops


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(389, 72, generator=g).to(dtype).cuda()
    tokens = torch.randint(0, 389, (57,), generator=g).int().cuda()
    out = ops.embedding(tokens, table)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out, table[tokens.long()].float(), rtol=0, atol=0)
    ops.check_status()
    bad = tokens.clone()
    bad[3] = 389
    ops.embedding(bad, table)
    with pytest.raises(RuntimeError, match="token id"):
        ops.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 96, 2048, 2880])
def test_add_rmsnorm(ops, dtype, hidden):
    g = torch.Generator().manual_seed(1)
    n = 19
    resid = torch.randn(n, hidden, generator=g).cuda()
    branch = torch.randn(n, hidden, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).cuda()
    eps = 3e-5
    x = resid.double() + branch.double()
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
    r = resid.clone()
    got = ops.add_rmsnorm(branch, r, w, eps, dtype)
    torch.testing.assert_close(r.double(), x, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(got.double(), want, **tol(dtype))
    # rows: gather, residual untouched, no branch
    rows = torch.tensor([4, 0, 18], dtype=torch.int32).cuda()
    r2 = resid.clone()
    got = ops.add_rmsnorm(None, r2, w, eps, dtype, rows=rows)
    x2 = resid.double()[rows.long()]
    want2 = x2 / torch.sqrt((x2 * x2).mean(-1, keepdim=True) + eps) * w.double()
    torch.testing.assert_close(got.double(), want2, **tol(dtype))
    torch.testing.assert_close(r2, resid, rtol=0, atol=0)
    # unit offset: y = x_hat * (1 + w)
    got = ops.add_rmsnorm(None, resid.clone(), w - 1, eps, dtype, unit_offset=True)
    x3 = resid.double()
    want3 = x3 / torch.sqrt((x3 * x3).mean(-1, keepdim=True) + eps) * w.double()
    torch.testing.assert_close(got.double(), want3, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    g = torch.Generator().manual_seed(2)
    gu = (3 * torch.randn(13, 2 * 104, generator=g)).to(dtype).cuda()
    got = ops.silu_mul(gu)
    a, b = gu[:, :104].double(), gu[:, 104:].double()
    torch.testing.assert_close(got.double(), a * torch.sigmoid(a) * b, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("hq,hkv,d,rot", [(5, 5, 16, 16), (6, 2, 48, 32), (8, 1, 128, 128)])
def test_rope_store(ops, dtype, interleaved, hq, hkv, d, rot):
    g = torch.Generator().manual_seed(3)
    n, bs, pages = 23, 8, 9
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).to(dtype).cuda()
    positions = torch.randint(0, 5000, (n,), generator=g).int().cuda()
    inv_freq = (10000.0 ** (-torch.arange(rot // 2).double() * 2 / rot)).float().cuda()
    slots = torch.randperm(pages * bs, generator=g)[:n].int()
    slots[5] = -1
    slots = slots.cuda()
    cache = torch.full((pages, 2, hkv, bs, d), float("nan")).to(dtype).cuda()
    before = qkv.clone()
    ops.rope_store(qkv, positions, inv_freq, slots, cache, hq, hkv, d, rot, interleaved)
    ops.check_status()
    x = before.double().view(n, hq + 2 * hkv, d)
    ang = (positions.float()[:, None] * inv_freq[None]).double()
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    want = x.clone()
    rot_part = x[:, : hq + hkv, :rot]
    if interleaved:
        x1, x2 = rot_part[..., 0::2], rot_part[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], -1).flatten(-2)
    else:
        x1, x2 = rot_part[..., : rot // 2], rot_part[..., rot // 2:]
        o = torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], -1)
    want[:, : hq + hkv, :rot] = o
    got = qkv.double().view(n, hq + 2 * hkv, d)
    torch.testing.assert_close(got, want, **tol(dtype))
    # the cache holds exactly what the activations hold, and nothing else was touched
    seen = torch.zeros(pages, bs, dtype=torch.bool)
    for t in range(n):
        sl = int(slots[t])
        if sl < 0:
            continue
        p, off = divmod(sl, bs)
        seen[p, off] = True
        assert torch.equal(cache[p, 0, :, off], qkv.view(n, -1, d)[t, hq:hq + hkv])
        assert torch.equal(cache[p, 1, :, off], qkv.view(n, -1, d)[t, hq + hkv:])
    untouched = cache.float().isnan().all(dim=(1, 2, 4)).cpu()
    assert torch.equal(untouched, ~seen)


@pytest.mark.parametrize("m,n,k", [(1, 311, 72), (7, 96, 160), (65, 130, 100), (200, 384, 96), (33, 1000, 515),
                                   (129, 260, 2048), (300, 1001, 520), (257, 128, 4)])
def test_gemm_f32(ops, m, n, k):
    g = torch.Generator().manual_seed(4)
    a = torch.randn(m, k, generator=g).cuda()
    b = torch.randn(n, k, generator=g).cuda()
    got = ops.linear(a, b)
    want = a.double() @ b.double().T
    # fp32 accumulation over k terms of unit scale: the rounding error grows with k (1e-4 up to k = 512)
    torch.testing.assert_close(got.double(), want, rtol=1e-5, atol=1e-4 * max(1.0, k / 512))
    # a row's result does not depend on the rest of the batch: bitwise
    alone = ops.linear(a[m // 2:m // 2 + 1].contiguous(), b)
    assert torch.equal(alone[0], got[m // 2])


def _paged_case(g, dtype, lens, hq, hkv, d, bs, q_counts):
    """Requests with ``lens`` cached tokens; the last ``q_counts`` of each are
    the batch's queries.  Pages are scattered through a NaN-poisoned pool."""
    total_pages = sum(-(-n // bs) for n in lens) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    pool = torch.full((total_pages, 2, hkv, bs, d), float("nan")).to(dtype)
    max_blocks = max(-(-n // bs) for n in lens) + 1
    table = torch.full((len(lens) + 2, max_blocks), -1, dtype=torch.int32)
    ks, vs, qs, pos, rows = [], [], [], [], []
    for r, (n, nq) in enumerate(zip(lens, q_counts)):
        k = torch.randn(n, hkv, d, generator=g).to(dtype)
        v = torch.randn(n, hkv, d, generator=g).to(dtype)
        q = torch.randn(nq, hq, d, generator=g).to(dtype)
        # make attention peaky so that a single missed key shows: one far key per query head
        k[0] *= 3
        k[n // 2] *= 3
        row = r + 1
        for b in range(-(-n // bs)):
            page = perm.pop()
            table[row, b] = page
            chunk = slice(b * bs, min(n, (b + 1) * bs))
            m = chunk.stop - chunk.start
            pool[page, 0, :, :m] = k[chunk].transpose(0, 1)
            pool[page, 1, :, :m] = v[chunk].transpose(0, 1)
        ks.append(k); vs.append(v); qs.append(q)
        pos += list(range(n - nq, n))
        rows += [row] * nq
    return pool, table, ks, vs, qs, torch.tensor(pos, dtype=torch.int32), torch.tensor(rows, dtype=torch.int32)


def _plain_attn(q, k, v, qpos, window, scale):
    hq, hkv = q.shape[1], k.shape[1]
    k = k.double().repeat_interleave(hq // hkv, 1)
    v = v.double().repeat_interleave(hq // hkv, 1)
    s = torch.einsum("qhd,khd->hqk", q.double(), k) * scale
    kp = torch.arange(k.shape[0])[None, :]
    hide = kp > qpos[:, None]
    if window:
        hide = hide | (kp <= qpos[:, None] - window)
    s = s.masked_fill(hide[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", s.softmax(-1), v)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,bs,window", [
    (4, 2, 16, 4, None), (3, 1, 32, 8, None), (5, 5, 48, 16, 24), (8, 2, 64, 16, None), (6, 3, 128, 32, 100),
    (2, 1, 256, 16, None),
])
def test_attention_simt(ops, dtype, hq, hkv, d, bs, window):
    g = torch.Generator().manual_seed(5)
    lens, q_counts = [1, 37, 130, 300, 64], [1, 37, 1, 45, 2]
    pool, table, ks, vs, qs, pos, rows = _paged_case(g, dtype, lens, hq, hkv, d, bs, q_counts)
    n = pos.numel()
    qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=dtype)
    qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
    scale = 1.0 / math.sqrt(d)
    out = ops.paged_attention(qkv.cuda(), pool.cuda(), table.cuda(), pos.cuda(), rows.cuda(), hq, scale, window=window)
    ops.check_status()
    off = 0
    for r, nq in enumerate(q_counts):
        qpos = pos[off:off + nq].long()
        want = _plain_attn(qs[r], ks[r], vs[r], qpos, window, scale)
        got = out[off:off + nq].double().cpu().view(nq, hq, d)
        assert not got.isnan().any()
        torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else tol(dtype)))
        off += nq


@pytest.mark.parametrize("hq,hkv,d,bs,window", [
    (4, 2, 32, 4, None), (3, 1, 32, 8, None), (5, 5, 32, 16, 24), (32, 8, 64, 16, None), (6, 3, 128, 32, 100),
    (16, 1, 64, 16, None), (12, 2, 128, 16, 300), (7, 7, 64, 8, None), (40, 2, 64, 16, None),
    (9, 3, 64, 32, 200), (32, 8, 128, 16, None),
])
@pytest.mark.parametrize("kernel", ["split", "stream"])
def test_attention_decode_split_kv(ops, hq, hkv, d, bs, window, kernel):
    """One query token per request over caches of 1 .. 1500 tokens: several chunks of keys (128 or 256 by head size), a chunk
    that holds a single key, windows that start inside a chunk; the far keys carry the weight.  Both
    kernels: one CTA per chunk, and the persistent TMA stream (head sizes 64 and 128, pages of 8 and more)."""
    from gllm_b200.ops import attention_bf16

    if kernel == "stream" and (d not in (64, 128) or bs not in (16, 32) or hkv > 8 or hq // hkv > 16):
        pytest.skip("the stream kernel takes head sizes 64 and 128, pages of 16 and 32, up to 8 kv heads")

    g = torch.Generator().manual_seed(6)
    lens = [1, 37, 128, 129, 300, 1500, 64, 256, 257]
    pool, table, ks, vs, qs, pos, rows = _paged_case(g, torch.bfloat16, lens, hq, hkv, d, bs, [1] * len(lens))
    n = pos.numel()
    qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
    qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
    scale = 1.0 / math.sqrt(d)
    assert attention_bf16.supports(d, bs)
    out = torch.full((n, hq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    attention_bf16.decode_attention(qkv.cuda(), qkv.shape[1], pool.cuda(), table.cuda(), pos.cuda(), rows.cuda(), hq,
                                    scale, window or 0, max(lens), None, out, kernel=kernel)
    ops.check_status()
    for r in range(n):
        want = _plain_attn(qs[r], ks[r], vs[r], pos[r:r + 1].long(), window, scale)
        got = out[r].double().cpu().view(1, hq, d)
        assert not got.isnan().any()
        torch.testing.assert_close(got, want, **tol(torch.bfloat16))


@pytest.mark.parametrize("kernel", ["split", "stream"])
def test_attention_decode_long_context(ops, kernel):
    """Three requests of 20,000, 4,097 and 130 cached tokens in one call (dozens of chunks, spans the
    stream kernel walks through several times per CTA, a window on top), far keys carrying the weight."""
    from gllm_b200.ops import attention_bf16

    g = torch.Generator().manual_seed(16)
    hq, hkv, d, bs = 8, 2, 64, 16
    lens = [20000, 4097, 130]
    for window in (None, 5000):
        pool, table, ks, vs, qs, pos, rows = _paged_case(g, torch.bfloat16, lens, hq, hkv, d, bs, [1] * len(lens))
        n = pos.numel()
        qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
        qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
        scale = 1.0 / math.sqrt(d)
        out = torch.full((n, hq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        attention_bf16.decode_attention(qkv.cuda(), qkv.shape[1], pool.cuda(), table.cuda(), pos.cuda(), rows.cuda(),
                                        hq, scale, window or 0, max(lens), None, out, kernel=kernel)
        ops.check_status()
        for r in range(n):
            want = _plain_attn(qs[r], ks[r], vs[r], pos[r:r + 1].long(), window, scale)
            got = out[r].double().cpu().view(1, hq, d)
            assert not got.isnan().any()
            torch.testing.assert_close(got, want, **tol(torch.bfloat16))


def test_attention_mixed_batch_uses_both_kernels(ops):
    """Portions first, single tokens after, as the step function lays a batch out."""
    from types import SimpleNamespace

    g = torch.Generator().manual_seed(7)
    hq, hkv, d, bs = 8, 2, 64, 16
    lens, q_counts = [200, 90, 400, 33], [50, 2, 1, 1]
    pool, table, ks, vs, qs, pos, rows = _paged_case(g, torch.bfloat16, lens, hq, hkv, d, bs, q_counts)
    n = pos.numel()
    qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
    qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
    from gllm_b200.engine.step import Workspace

    batch = SimpleNamespace(
        num_prefill_tokens=52, num_prefill_requests=2, max_seq_len=400, max_q_len=50,
        workspace=Workspace(torch.device("cuda")),
        cu_q=torch.tensor([0, 50, 52, 53, 54], dtype=torch.int32).cuda(),
        context_lens=torch.tensor([150, 88, 399, 32], dtype=torch.int32).cuda(),
        state_slots=torch.tensor([1, 2, 3, 4], dtype=torch.int32).cuda(),
    )
    scale = 1.0 / math.sqrt(d)
    out = ops.paged_attention(qkv.cuda(), pool.cuda(), table.cuda(), pos.cuda(), rows.cuda(), hq, scale, batch=batch)
    ops.check_status()
    off = 0
    for r, nq in enumerate(q_counts):
        want = _plain_attn(qs[r], ks[r], vs[r], pos[off:off + nq].long(), None, scale)
        torch.testing.assert_close(out[off:off + nq].double().cpu().view(nq, hq, d), want, **tol(torch.bfloat16))
        off += nq


@pytest.mark.parametrize("hq,hkv,d,bs,window", [
    (4, 1, 64, 16, None), (3, 1, 32, 8, None), (32, 8, 64, 16, None), (6, 3, 128, 32, 100), (8, 8, 64, 4, 70),
    (16, 2, 128, 16, None), (5, 5, 32, 16, 24), (64, 1, 64, 16, None),
])
@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05"])
def test_attention_prefill_tensor_cores(ops, hq, hkv, d, bs, window, kernel):
    """Portions of prompts over a cache: a whole prompt, a portion after 250 cached tokens, two-token
    portions, portions that end inside a page and inside a key tile; the far keys carry the weight.
    Both tensor-core kernels: mma.sync (64-key tiles) and tcgen05 with tensor memory (128-key tiles)."""
    from gllm_b200.ops import attention_bf16

    if kernel == "tcgen05" and (d not in (64, 128) or bs < 8):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128 and pages of at least 8 tokens")

    g = torch.Generator().manual_seed(8)
    lens, q_counts = [130, 300, 2, 64, 67, 451], [130, 50, 2, 2, 65, 200]
    pool, table, ks, vs, qs, pos, rows = _paged_case(g, torch.bfloat16, lens, hq, hkv, d, bs, q_counts)
    # the cache's spare last page (finite), as the cache manager provides it; every other unused slot is NaN
    pool = torch.cat([pool, torch.zeros(1, *pool.shape[1:], dtype=pool.dtype)], 0)
    n = pos.numel()
    qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
    qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
    scale = 1.0 / math.sqrt(d)
    assert attention_bf16.prefill_supports(d, bs)
    cu = torch.tensor([0] + list(torch.tensor(q_counts).cumsum(0)), dtype=torch.int32).cuda()
    ctx = torch.tensor([a - b for a, b in zip(lens, q_counts)], dtype=torch.int32).cuda()
    slots = torch.arange(1, len(lens) + 1, dtype=torch.int32).cuda()
    out = torch.full((n, hq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    run = attention_bf16.prefill_attention if kernel == "mma_sync" else attention_bf16.prefill_attention_tmem
    qd, pd = qkv.cuda(), pool.cuda()
    if kernel == "tcgen05":
        assert attention_bf16.prefill_tmem_supports(d, bs, qd, pd)
    run(qd, qkv.shape[1], pd, table.cuda(), cu, ctx, slots, len(lens), max(q_counts), hq, scale, window or 0, out)
    ops.check_status()
    off = 0
    for r, nq in enumerate(q_counts):
        want = _plain_attn(qs[r], ks[r], vs[r], pos[off:off + nq].long(), window, scale)
        got = out[off:off + nq].double().cpu().view(nq, hq, d)
        assert not got.isnan().any(), r
        torch.testing.assert_close(got, want, **tol(torch.bfloat16))
        off += nq


@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05"])
@pytest.mark.parametrize("d", [64, 128])
def test_attention_prefill_long_context(ops, kernel, d):
    """Portions late in long requests: 700 tokens after 9,000 cached ones (dozens of key tiles before
    the diagonal, with and without a window) beside a whole prompt of 1,100 tokens."""
    from gllm_b200.ops import attention_bf16

    g = torch.Generator().manual_seed(17)
    hq, hkv, bs = 8, 2, 16
    lens, q_counts = [9700, 1100], [700, 1100]
    for window in (None, 3000):
        pool, table, ks, vs, qs, pos, rows = _paged_case(g, torch.bfloat16, lens, hq, hkv, d, bs, q_counts)
        pool = torch.cat([pool, torch.zeros(1, *pool.shape[1:], dtype=pool.dtype)], 0)
        n = pos.numel()
        qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
        qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
        scale = 1.0 / math.sqrt(d)
        cu = torch.tensor([0] + list(torch.tensor(q_counts).cumsum(0)), dtype=torch.int32).cuda()
        ctx = torch.tensor([a - b for a, b in zip(lens, q_counts)], dtype=torch.int32).cuda()
        slots = torch.arange(1, len(lens) + 1, dtype=torch.int32).cuda()
        out = torch.full((n, hq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        run = attention_bf16.prefill_attention if kernel == "mma_sync" else attention_bf16.prefill_attention_tmem
        run(qkv.cuda(), qkv.shape[1], pool.cuda(), table.cuda(), cu, ctx, slots, len(lens), max(q_counts), hq, scale,
            window or 0, out)
        ops.check_status()
        off = 0
        for r, nq in enumerate(q_counts):
            want = _plain_attn(qs[r], ks[r], vs[r], pos[off:off + nq].long(), window, scale)
            got = out[off:off + nq].double().cpu().view(nq, hq, d)
            assert not got.isnan().any(), r
            torch.testing.assert_close(got, want, **tol(torch.bfloat16))
            off += nq


@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("trend", ["rising", "falling"])
def test_attention_prefill_scores_with_a_trend(ops, kernel, d, trend):
    """Scores that rise by about 8 nats from one tile of 128 keys to the next: every row's maximum outgrows
    the reference it was exponentiated against in tile after tile (the tcgen05 kernel takes such a tile a
    second time and rescales its output, which random scores never ask of it after a row's first tile).
    Falling scores: the first keys keep all the weight and later tiles add almost nothing.  The first request
    is long enough (12 key tiles) for the tcgen05 kernel to split its last rows' key tiles between two CTAs,
    whose reference maxima then differ by dozens of nats when they are merged."""
    from gllm_b200.ops import attention_bf16

    g = torch.Generator().manual_seed(23)
    hq, hkv, bs = 8, 2, 16
    lens, q_counts = [1500, 900], [1500, 300]
    pool, table, ks, vs, qs, pos, rows = _paged_case(g, torch.bfloat16, lens, hq, hkv, d, bs, q_counts)
    u = torch.randn(d, generator=g)
    u = u / u.norm()
    scale = 1.0 / math.sqrt(d)
    for r, n in enumerate(lens):
        ramp = torch.arange(n, dtype=torch.float32) * (0.06 / scale)          # +7.7 nats per 128 keys
        if trend == "falling":
            ramp = ramp.flip(0)
        ks[r] = (torch.randn(n, hkv, d, generator=g) * 0.5 + ramp[:, None, None] * u).to(torch.bfloat16)
        qs[r] = (torch.randn(q_counts[r], hq, d, generator=g) * 0.5 + u).to(torch.bfloat16)
        for b in range(-(-n // bs)):
            chunk = slice(b * bs, min(n, (b + 1) * bs))
            pool[table[r + 1, b], 0, :, : chunk.stop - chunk.start] = ks[r][chunk].transpose(0, 1)
    pool = torch.cat([pool, torch.zeros(1, *pool.shape[1:], dtype=pool.dtype)], 0)
    n = pos.numel()
    qkv = torch.zeros(n, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
    qkv[:, : hq * d] = torch.cat(qs).reshape(n, hq * d)
    cu = torch.tensor([0] + list(torch.tensor(q_counts).cumsum(0)), dtype=torch.int32).cuda()
    ctx = torch.tensor([a - b for a, b in zip(lens, q_counts)], dtype=torch.int32).cuda()
    slots = torch.arange(1, len(lens) + 1, dtype=torch.int32).cuda()
    out = torch.full((n, hq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    run = attention_bf16.prefill_attention if kernel == "mma_sync" else attention_bf16.prefill_attention_tmem
    run(qkv.cuda(), qkv.shape[1], pool.cuda(), table.cuda(), cu, ctx, slots, len(lens), max(q_counts), hq, scale, 0, out)
    ops.check_status()
    off = 0
    for r, nq in enumerate(q_counts):
        want = _plain_attn(qs[r], ks[r], vs[r], pos[off:off + nq].long(), None, scale)
        got = out[off:off + nq].double().cpu().view(nq, hq, d)
        assert not got.isnan().any(), r
        torch.testing.assert_close(got, want, **tol(torch.bfloat16))
        off += nq


@pytest.mark.parametrize("m,n,k", [(1, 311, 72), (8, 3072, 2048), (7, 96, 160), (13, 2048, 8192), (33, 1000, 520),
                                   (64, 16384, 2048), (50, 130, 104), (3, 128256, 256), (65, 520, 200),
                                   (128, 256, 64), (300, 777, 1000), (2048, 3072, 2048), (1000, 16384, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_tensor_memory(ops, m, n, k, out_dtype):
    """The tcgen05 product in both orientations: few tokens (the weight is the 128-row operand, split
    along K with the last-ticket reduction: 3072x2048, 2048x8192) and many tokens; tails in M, N and K;
    twice in a row (the tickets return to zero)."""
    from gllm_b200.ops import gemm_bf16

    g = torch.Generator().manual_seed(9)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    assert gemm_bf16.tensor_core_kernel_takes(x, w)
    want = x.double() @ w.double().T
    for _ in range(2):
        got = ops.linear(x, w, out_dtype=out_dtype)
        ops.check_status()
        assert got.dtype == out_dtype
        if out_dtype == torch.float32:
            torch.testing.assert_close(got.double(), want, rtol=1e-4, atol=1e-4)
        else:
            torch.testing.assert_close(got.double(), want, rtol=1e-2, atol=1e-2)
    # a token's result does not depend on the rest of the batch: bitwise among batches of up to 16
    # tokens (one kernel variant, one cut of K), to rounding beyond
    alone = ops.linear(x[m // 2:m // 2 + 1].contiguous(), w, out_dtype=out_dtype)
    if m <= 16:
        assert torch.equal(alone[0], got[m // 2])
    else:
        torch.testing.assert_close(alone[0].double(), got[m // 2].double(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("m,n,k", [(1, 130, 72), (129, 256, 64), (257, 777, 1000), (300, 3072, 2048), (2112, 2048, 2048)])
def test_gemm_bf16_pair_of_ctas(ops, m, n, k):
    """The product on pairs of CTAs (cta_group::2), called directly: tails in M, N and K (a pair's
    second CTA may have no token row at all), both output types, twice in a row; then behind a
    kernel that holds the GPU and a small one (so that it is scheduled early, its CTAs starting one
    after the other as SMs come free), which must not change a bit."""
    from gllm_b200.ops import gemm_bf16

    g = torch.Generator().manual_seed(29)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    want = x.double() @ w.double().T
    for out_dtype, tol_ in ((torch.float32, 1e-4), (torch.bfloat16, 1e-2)):
        for _ in range(2):
            got = gemm_bf16.linear_pair(x, w, torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda"))
            ops.check_status()
            torch.testing.assert_close(got.double(), want, rtol=tol_, atol=tol_)
    first = gemm_bf16.linear_pair(x, w, torch.empty((m, n), dtype=torch.bfloat16, device="cuda"))
    big_x = torch.randn(4096, 2048, generator=g).to(torch.bfloat16).cuda()
    big_w = torch.randn(8192, 2048, generator=g).to(torch.bfloat16).cuda()
    resid = torch.zeros(8, 2048).cuda()
    for _ in range(3):
        ops.linear(big_x, big_w)
        ops.add_rmsnorm(None, resid, torch.ones(2048).cuda(), 1e-5, torch.bfloat16)
        again = gemm_bf16.linear_pair(x, w, torch.empty((m, n), dtype=torch.bfloat16, device="cuda"))
        assert torch.equal(first, again)
    ops.check_status()


@pytest.mark.parametrize("m,inter,k", [(130, 192, 96), (513, 1024, 2048)])
def test_gemm_bf16_pair_gated(ops, m, inter, k):
    from gllm_b200.ops import gemm_bf16

    g = torch.Generator().manual_seed(30)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    wg = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    wu = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    got = gemm_bf16.linear_pair(x, ops.interleave_gate_up(wg, wu),
                                torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda"), gated=True)
    ops.check_status()
    a, b = x.double() @ wg.double().T, x.double() @ wu.double().T
    torch.testing.assert_close(got.double(), a * torch.sigmoid(a) * b, rtol=2e-2, atol=2e-2)


def test_gemm_scratch_that_is_outgrown_stays_allocated(ops):
    """A captured graph holds the address of the split-K scratch it was captured with: when a later,
    larger product makes the scratch grow, the old buffer must not go back to the allocator (the next
    tensor would get its memory while the graph still writes partial sums there)."""
    from gllm_b200.ops import gemm_bf16

    dev = torch.device("cuda:0")
    before = {gemm_bf16._device_scratch(dev, 16, 16)[0].data_ptr() for _ in range(2)}     # both turns
    need = max(gemm_bf16._scratch[0][f"partial{t}"].numel() for t in (0, 1)) + 1
    after = {gemm_bf16._device_scratch(dev, need, 16)[0].data_ptr() for _ in range(2)}
    assert not (before & after)
    kept = {t.data_ptr() for t in gemm_bf16._scratch[0]["retired"]}
    assert before <= kept


def test_gemm_bf16_odd_inner_size_goes_to_the_library(ops):
    g = torch.Generator().manual_seed(10)
    x = torch.randn(5, 100, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(37, 100, generator=g).to(torch.bfloat16).cuda()
    got = ops.linear(x, w)
    torch.testing.assert_close(got.double(), x.double() @ w.double().T, rtol=2e-2, atol=2e-2)


def test_unsummed_splits_are_summed_by_their_consumers(ops):
    """A product cut along K may hand its fp32 partial results to add_rmsnorm or rope_store.  The
    residual stream, the rotated rows and the cache come out exactly as for the summed product; the
    normalised rows may differ by one bf16 step where the sum of squares, added in another order,
    moves the scale by one fp32 step."""

    def same_up_to_one_step(p, q):
        p, q = p.float(), q.float()
        return bool(((p - q).abs() <= p.abs() * 2.0 ** -7).all()) and float((p != q).float().mean()) < 0.02
    g = torch.Generator().manual_seed(11)
    m, k = 8, 2048
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2048, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    summed = ops.linear(x, w)
    split = ops.linear(x, w, split_ok=True)
    assert isinstance(split, ops.SplitSum) and split.parts.shape[0] > 1 and tuple(split.shape) == (m, 2048)
    assert torch.equal(split.tensor(), summed)
    resid = torch.randn(m, 2048, generator=g).cuda()
    wn = torch.ones(2048).cuda()
    r1, r2 = resid.clone(), resid.clone()
    a = ops.add_rmsnorm(summed, r1, wn, 1e-5, torch.bfloat16)
    split = ops.linear(x, w, split_ok=True)
    b = ops.add_rmsnorm(split, r2, wn, 1e-5, torch.bfloat16)
    assert torch.equal(r1, r2) and same_up_to_one_step(a, b)
    want = r1.double() * torch.rsqrt(r1.double().pow(2).mean(-1, keepdim=True) + 1e-5)
    torch.testing.assert_close(b.double(), want, rtol=2.0 ** -8, atol=1e-6)
    rows = torch.tensor([5, 1], dtype=torch.int32).cuda()
    split = ops.linear(x, w, split_ok=True)
    assert same_up_to_one_step(ops.add_rmsnorm(split, resid.clone(), wn, 1e-5, torch.bfloat16, rows=rows),
                               ops.add_rmsnorm(summed, resid.clone(), wn, 1e-5, torch.bfloat16, rows=rows))
    # rotary + store: 24 query heads and 4 kv heads of 64 make a width of 2048
    hq, hkv, d, bs = 24, 4, 64, 16
    positions = torch.arange(100, 100 + m, dtype=torch.int32).cuda()
    inv_freq = (10000.0 ** (-torch.arange(d // 2).double() * 2 / d)).float().cuda()
    slots = torch.arange(m, dtype=torch.int32).cuda()
    c1 = torch.zeros(2, 2, hkv, bs, d, dtype=torch.bfloat16).cuda()
    c2 = torch.zeros_like(c1)
    q1 = ops.rope_store(summed.clone(), positions, inv_freq, slots, c1, hq, hkv, d, d)
    q2 = ops.rope_store(ops.linear(x, w, split_ok=True), positions, inv_freq, slots, c2, hq, hkv, d, d)
    assert torch.equal(q1, q2) and torch.equal(c1, c2)


@pytest.mark.parametrize("m", [1, 8, 33, 64, 65, 300])
@pytest.mark.parametrize("inter,k", [(128, 64), (192, 96), (8192, 2048)])
def test_gemm_gated_epilogue(ops, m, inter, k):
    """silu(x Wg^T) * (x Wu^T) in the product's epilogue, both orientations, against the plain formula;
    and the unfused route (product, then silu_mul over the same block layout) gives the same."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    wg = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    wu = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).cuda()
    w = ops.interleave_gate_up(wg, wu)
    assert w.shape == (2 * inter, k) and torch.equal(w[:64], wg[:64]) and torch.equal(w[64:128], wu[:64])
    got = ops.linear_gated(x, w)
    ops.check_status()
    a, b = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = a * torch.sigmoid(a) * b
    assert got.shape == (m, inter) and got.dtype == torch.bfloat16
    torch.testing.assert_close(got.double(), want, rtol=2e-2, atol=2e-2)
    unfused = ops.silu_mul(ops.linear(x, w), block=64)
    torch.testing.assert_close(unfused.double(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m", [1, 3, 16, 40, 64])
@pytest.mark.parametrize("n,k", [(2048, 8192), (200, 136), (2048, 2048)])
def test_gemm_that_adds_itself_into_the_residual(ops, m, n, k):
    g = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    acc = torch.randn(m, n, generator=g).cuda()
    want = acc.double().cpu() + x.double().cpu() @ w.double().cpu().T
    result = ops.linear(x, w, split_ok=True, add_into=acc)
    assert result is ops.ADDED
    ops.check_status()
    assert float((acc.double().cpu() - want).abs().max()) <= 1e-2 * float(want.abs().max())
    # more than 64 tokens: nothing is added, the product comes back
    x2 = torch.randn(65, k, generator=g).to(torch.bfloat16).cuda()
    acc2 = torch.zeros(65, n).cuda()
    out = ops.linear(x2, w, split_ok=True, add_into=acc2)
    assert out is not ops.ADDED and float(acc2.abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_bias_and_norm_of_every_head(ops, dtype):
    """``add_bias`` on a strided view, and ``rmsnorm_heads`` on some of the heads of each row (head sizes that
    are no multiple of 32 among them), against their formulas in float64."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(37, 200, generator=g).to(dtype)
    bias = torch.randn(120, generator=g)
    xd = x.cuda()
    view = xd[:, 40:160]
    ops.add_bias(view, bias.cuda())
    want = x.double()
    want[:, 40:160] += bias.double()
    torch.testing.assert_close(xd.double().cpu(), want.to(dtype).double(), **tol(dtype))
    for d, heads, first, n, unit in [(64, 5, 0, 3, False), (48, 6, 2, 4, True), (16, 9, 8, 1, False), (256, 2, 1, 1, False)]:
        y = torch.randn(11, heads * d, generator=g).to(dtype)
        wgt = torch.randn(d, generator=g)
        yd = y.cuda()
        ops.rmsnorm_heads(yd, wgt.cuda(), 1e-5, first, n, d, unit_offset=unit)
        z = y.double().view(11, heads, d).clone()
        part = z[:, first:first + n]
        z[:, first:first + n] = part / torch.sqrt((part * part).mean(-1, keepdim=True) + 1e-5) * ((1.0 + wgt.double()) if unit else wgt.double())
        torch.testing.assert_close(yd.double().cpu().view(11, heads, d), z.to(dtype).double(), **tol(dtype))
