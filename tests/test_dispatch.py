"""Decisions the host takes before a launch, checked without a GPU: the step size a lone prompt
portion is padded to for its graph, and which products go to the kernel on pairs of CTAs."""

from types import SimpleNamespace


def bucket_of(n, graph_tokens=(2048,), max_tokens=8192, max_seq_len=4096):
    from gllm_b200.engine.step import StepRunner

    fake = SimpleNamespace(prefill_graph_tokens=graph_tokens, max_tokens=max_tokens,
                           cache=SimpleNamespace(max_seq_len=max_seq_len))
    return StepRunner._prefill_bucket(fake, n)


def test_prefill_buckets():
    # a bucket holds the portion exactly, or leaves room for a null portion of at least two tokens
    assert [bucket_of(n) for n in (2, 14, 15, 16, 17, 30, 31, 32)] == [16, 16, 32, 16, 32, 32, 64, 32]
    assert [bucket_of(n) for n in (62, 63, 64, 65, 126, 127, 128, 129)] == [64, 128, 64, 128, 128, 256, 128, 256]
    assert [bucket_of(n) for n in (1022, 1023, 1024, 1025, 2046, 2047, 2048)] == [1024, 1280, 1024, 1280, 2048, 2304, 2048]
    assert bucket_of(2049) == 0                                   # longer than the longest graphed portion
    for n in range(2, 2049):
        b = bucket_of(n)
        assert b == n or b >= n + 2, n
        assert b <= 2304 and (b in (16, 32, 64) or b % 128 == 0), (n, b)
    # the null portion is a sequence of its own and has to fit a block-table row; a step has a size limit
    assert bucket_of(100, max_seq_len=16) == 0
    assert bucket_of(300, graph_tokens=(512,), max_tokens=320) == 0
    assert bucket_of(320, graph_tokens=(512,), max_tokens=320) == 0   # 384 would exceed the step
    assert bucket_of(512, graph_tokens=(512,), max_tokens=512) == 512


def test_products_on_pairs_of_ctas(monkeypatch):
    from gllm_b200.ops import gemm_bf16

    monkeypatch.setattr(gemm_bf16, "_PAIR_FORCED", False)
    monkeypatch.setattr(gemm_bf16, "PAIR_MIN_TOKENS", 129)
    monkeypatch.setitem(gemm_bf16._sm_pairs, 0, 74)
    pays = lambda m, n, k: gemm_bf16.pair_kernel_pays(SimpleNamespace(shape=(m, k), device=SimpleNamespace(index=0)), n)
    assert not pays(128, 16384, 2048)                 # too few tokens for a tile of 256
    assert pays(2048, 16384, 2048) and pays(2048, 3072, 2048) and pays(2048, 2048, 8192)
    assert not pays(2048, 2048, 2048)                 # 64 tiles on 74 pairs, 32 blocks of K each
    assert pays(8192, 2048, 2048)                     # four tiles a pair
    assert not pays(300, 3072, 2048) and pays(300, 16384, 2048)
