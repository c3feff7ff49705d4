"""The sampling kernels against the plain restatement of the reference sampler."""

import pytest
import torch

from plain_llama import plain_sampling_distribution, plain_top_logprobs

pytestmark = pytest.mark.gpu


def _args(rows, temperature, top_k, top_p, seeds=None, counters=None, nlp=None):
    dev = "cuda"
    full = lambda v, dt: torch.full((rows,), v, dtype=dt, device=dev)
    return dict(
        temperature=full(temperature, torch.float32), top_k=full(top_k, torch.int32), top_p=full(top_p, torch.float32),
        seed=torch.arange(rows, dtype=torch.int64, device=dev) if seeds is None else seeds,
        counter=full(0, torch.int32) if counters is None else counters,
        num_logprobs=None if nlp is None else full(nlp, torch.int32),
    )


@pytest.mark.parametrize("vocab", [311, 4099, 128256])
def test_argmax_and_greedy(vocab):
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(9, vocab, generator=g).cuda()
    logits[3, 17] = logits[3, vocab - 1] = 50.0                 # a tie: the lowest index wins
    want = logits.argmax(-1)
    want[3] = 17
    assert torch.equal(ops.argmax(logits).long(), want)
    for t, k in ((0.0, 40), (0.8, 1)):
        out = ops.sample(logits, **_args(9, t, k, 0.9))
        assert torch.equal(out["tokens"].long(), want)
        assert out["num_candidates"].tolist() == [1] * 9
    lp = torch.log_softmax(logits.double(), -1).gather(1, want[:, None])[:, 0]
    torch.testing.assert_close(out["logprobs"].double(), lp, rtol=1e-4, atol=1e-4)
    # rows of a wider buffer (row stride > vocab)
    wide = torch.zeros(9, vocab + 5, device="cuda")
    wide[:, :vocab] = logits
    assert torch.equal(ops.argmax(wide[:, :vocab]).long(), want)


@pytest.mark.parametrize("temperature,top_k,top_p", [
    (1.0, 0, 1.0), (0.7, 40, 0.9), (1.0, 50, 0.95), (1.3, 0, 0.8), (0.5, 5, 1.0), (1.0, 2000, 0.5), (2.0, 7, 0.3),
])
@pytest.mark.parametrize("vocab", [384, 5003])
def test_distribution_equals_the_reference_rules(temperature, top_k, top_p, vocab):
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(1)
    logits = (2.5 * torch.randn(6, vocab, generator=g)).cuda()
    out = ops.sample(logits, **_args(6, temperature, top_k, top_p), return_probs=True)
    for r in range(6):
        want, n = plain_sampling_distribution(logits[r].cpu(), temperature, top_k, top_p)
        got = out["probs"][r].double().cpu()
        if int(out["num_candidates"][r]) != n:
            # two cases are no fault: a cumulative probability within rounding of top_p, and equal
            # logits on both sides of the cut (the kernel keeps or drops equal values together)
            z = logits[r].double().cpu() / temperature
            k = vocab if top_k == 0 else min(top_k, vocab)
            top = torch.topk(z, min(k + 1, vocab)).values
            p = torch.softmax(top[:k], -1).cumsum(-1)
            tie = n < top.numel() and float(top[n - 1]) == float(top[n])
            assert tie or float((p - top_p).abs().min()) < 1e-5, (r, int(out["num_candidates"][r]), n)
            continue
        torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-7)
        assert int(out["tokens"][r]) in torch.nonzero(want).flatten().tolist()


def test_draws_follow_the_distribution_and_depend_only_on_seed_and_counter():
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(2)
    vocab, rows = 97, 20000
    row = (1.5 * torch.randn(vocab, generator=g))
    logits = row[None].expand(rows, vocab).contiguous().cuda()
    args = _args(rows, 0.9, 12, 0.85, counters=torch.arange(rows, dtype=torch.int32, device="cuda"),
                 seeds=torch.full((rows,), 1234, dtype=torch.int64, device="cuda"))
    out = ops.sample(logits, **args)
    want, n = plain_sampling_distribution(row, 0.9, 12, 0.85)
    counts = torch.bincount(out["tokens"].long().cpu(), minlength=vocab).double()
    assert float(counts[want == 0].sum()) == 0                   # nothing outside the kept set
    expected = want * rows
    kept = want > 0
    chi2 = float((((counts - expected) ** 2)[kept] / expected[kept]).sum())
    assert chi2 < 3 * int(kept.sum()) + 20, chi2                 # loose bound on a chi-square with n-1 degrees
    # same (seed, counter) -> same token, whatever the row or the batch
    again = ops.sample(logits[:100].flip(0).contiguous(), **{k: (v[:100].flip(0).contiguous() if v is not None else None)
                                                            for k, v in args.items()})
    assert torch.equal(again["tokens"].flip(0), out["tokens"][:100])
    other = dict(args)
    other["seed"] = args["seed"] + 1
    assert not torch.equal(ops.sample(logits, **other)["tokens"], out["tokens"])


def test_top_logprobs():
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(3)
    logits = (3 * torch.randn(5, 1000, generator=g)).cuda()
    out = ops.sample(logits, **_args(5, 1.0, 8, 1.0, nlp=5), max_logprobs=5)
    for r in range(5):
        vals, ids = plain_top_logprobs(logits[r].cpu(), 5)
        assert out["top_ids"][r].tolist() == ids.tolist()
        torch.testing.assert_close(out["top_logprobs"][r].double().cpu(), vals, rtol=1e-4, atol=1e-4)
    # fewer candidates than asked for: min(max_num_logprobs, num_candidates) entries, the rest stays -1
    out = ops.sample(logits, **_args(5, 1.0, 3, 1.0, nlp=5), max_logprobs=5)
    assert out["num_candidates"].tolist() == [3] * 5
    assert (out["top_ids"][:, 3:] == -1).all() and (out["top_ids"][:, :3] >= 0).all()


def test_equal_logits_are_kept_or_dropped_together():
    from gllm_b200 import ops

    logits = torch.full((1, 64), -20.0)
    logits[0, [3, 9, 11, 30]] = torch.tensor([4.0, 2.0, 2.0, 1.0])       # the 2nd and 3rd highest tie
    out = ops.sample(logits.cuda(), **_args(1, 1.0, 2, 1.0), return_probs=True)
    assert int(out["num_candidates"][0]) == 3                            # top_k = 2 keeps both of the tied values
    # softmax .78 .105 .105 .04: top_p .9 is crossed inside the tie, so both tied values go
    out = ops.sample(logits.cuda(), **_args(1, 1.0, 0, 0.9), return_probs=True)
    assert int(out["num_candidates"][0]) == 1 and float(out["probs"][0, 3]) == 1.0
