"""A toy feed-forward with routing and a toy position encoding that is not rotary, both defined here,
are registered, built from a checkpoint and stepped (whole, in portions, decoded as CUDA graphs)
without a change to the package: parts are chosen layer by layer from the registries, and the
attention mixer takes whatever position encoding its spec names.  Neither toy is anybody's model."""

import pytest
import torch

from plain_llama import plain_mlp, plain_rmsnorm

pytestmark = pytest.mark.gpu

EXPERTS = 3
MAX_POS = 96


def register_toys():
    from gllm_b200 import ops
    from gllm_b200.config import register_architecture
    from gllm_b200.config.model_config import ModelConfig
    from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry
    from gllm_b200.parts import (FeedForward, PositionEncoding, TensorExpectation, register_feed_forward,
                                 register_position_encoding)
    from dataclasses import dataclass

    @register_feed_forward("toy_top1")
    class Top1Experts(FeedForward):
        """Every token goes through the one expert (a plain product, no activation) that its router
        logit (fp32) is largest for, scaled by the sigmoid of that logit."""

        def __init__(self, names, hidden_size, num_experts):
            super().__init__(names)
            self.hidden_size, self.num_experts = hidden_size, num_experts
            self.router, self.experts = None, None

        def expected_tensors(self):
            h = self.hidden_size
            exp = {self.names["router"]: TensorExpectation((self.num_experts, h), "vector")}
            for e in range(self.num_experts):
                exp[self.names["expert"].format(e)] = TensorExpectation((h, h))
            return exp

        def load(self, get, dtype, device):
            self.router = get(self.names["router"], "vector")                 # fp32 whatever the compute dtype
            self.experts = [get(self.names["expert"].format(e), "matrix") for e in range(self.num_experts)]

        def forward(self, x, ctx):
            logits = x.float() @ self.router.T                                # [n, E] fp32
            best = logits.argmax(-1)
            gate = torch.sigmoid(logits.gather(1, best[:, None]))             # [n, 1]
            out = torch.zeros(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            for e, w in enumerate(self.experts):                              # dense and branch-free: fine in a graph
                out += (best == e)[:, None] * ops.linear(x, w).float()
            return (out * gate).to(x.dtype)

    @register_position_encoding("toy_offset_table")
    class OffsetTable(PositionEncoding):
        """A table row per position, added to every query and key head."""

        def __init__(self, names, head_dim, max_positions):
            super().__init__(names)
            self.head_dim, self.max_positions, self.table = head_dim, max_positions, None

        def expected_tensors(self):
            return {self.names["table"]: TensorExpectation((self.max_positions, self.head_dim))}

        def load(self, get, dtype, device):
            self.table = get(self.names["table"], "matrix")

        def apply(self, qkv, ctx, num_heads, num_kv_heads, head_dim):
            rows = self.table[ctx.positions.long().clamp_(0, self.max_positions - 1)]
            qk = qkv[:, : (num_heads + num_kv_heads) * head_dim].view(qkv.shape[0], num_heads + num_kv_heads, head_dim)
            qk += rows[:, None, :]

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        num_heads: int = 0
        num_kv_heads: int = 0
        head_dim: int = 0
        intermediate_size: int = 0
        eps: float = 1e-5

        @classmethod
        def from_dict(cls, d):
            return cls(architecture=d["architectures"][0], vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
                       dtype=d["torch_dtype"], eos_token_ids=(), num_heads=d["num_heads"],
                       num_kv_heads=d["num_kv_heads"], head_dim=d["head_dim"],
                       intermediate_size=d["intermediate_size"], eps=d["eps"])

        def to_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        torch_dtype=self.dtype, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                        head_dim=self.head_dim, intermediate_size=self.intermediate_size, eps=self.eps)

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(size=h, eps=cfg.eps), {"weight": name})
        attn = lambda p: PartSpec(
            "attention",
            dict(hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                 position=PartSpec("toy_offset_table", dict(head_dim=cfg.head_dim, max_positions=MAX_POS),
                                   {"table": f"{p}.pos.weight"})),
            {n: f"{p}.attn.{n}.weight" for n in "qkvo"})
        routed = PartSpec("toy_top1", dict(hidden_size=h, num_experts=EXPERTS),
                          {"router": "layers.0.router.weight", "expert": "layers.0.expert{}.weight"})
        dense = PartSpec("swiglu", dict(hidden_size=h, intermediate_size=cfg.intermediate_size),
                         {n: f"layers.1.mlp.{n}_proj.weight" for n in ("gate", "up", "down")})
        layers = (   # different feed-forwards in different layers of one model
            LayerSpec("prenorm", dict(mixer=attn("layers.0"), feed_forward=routed, mixer_norm=norm("layers.0.n1.weight"),
                                      feed_forward_norm=norm("layers.0.n2.weight"))),
            LayerSpec("prenorm", dict(mixer=attn("layers.1"), feed_forward=dense, mixer_norm=norm("layers.1.n1.weight"),
                                      feed_forward_norm=norm("layers.1.n2.weight"))),
        )
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size, layers=layers, plan=(PlanEntry(0), PlanEntry(1)),
                         final_norm=norm("norm.weight"), embedding_name="embed.weight", head_name="head.weight")

    register_architecture("ToyPartsLM", ToyConfig, build_spec)


def plain_forward(cfg, w, tokens):
    """Whole sequence in float64: softmax(QK^T / sqrt(d) + causal mask) V with the table rows added to
    q and k, the routed feed-forward, the dense one.  Returns the logits and, per position, the relative
    gap between the two best router logits."""
    w = {k: v.double() for k, v in w.items()}
    x = w["embed.weight"][torch.tensor(tokens)]
    t = x.shape[0]
    hq, hkv, d = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    causal = torch.full((t, t), float("-inf")).triu(1).double()
    for layer in (0, 1):
        p = f"layers.{layer}"
        h = plain_rmsnorm(x, w[f"{p}.n1.weight"], cfg["eps"])
        q = (h @ w[f"{p}.attn.q.weight"].T).view(t, hq, d) + w[f"{p}.pos.weight"][:t, None, :]
        k = (h @ w[f"{p}.attn.k.weight"].T).view(t, hkv, d) + w[f"{p}.pos.weight"][:t, None, :]
        v = (h @ w[f"{p}.attn.v.weight"].T).view(t, hkv, d)
        k, v = k.repeat_interleave(hq // hkv, 1), v.repeat_interleave(hq // hkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / d ** 0.5 + causal
        a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(t, hq * d)
        x = x + a @ w[f"{p}.attn.o.weight"].T
        h = plain_rmsnorm(x, w[f"{p}.n2.weight"], cfg["eps"])
        if layer == 0:
            logits = h @ w["layers.0.router.weight"].T
            top2 = logits.topk(2, -1).values
            margin = (top2[:, 0] - top2[:, 1]) / top2[:, 0].abs().clamp_min(1e-6)       # per position
            best = logits.argmax(-1)
            y = torch.stack([h[i] @ w[f"layers.0.expert{int(best[i])}.weight"].T for i in range(t)])
            x = x + y * torch.sigmoid(logits.gather(1, best[:, None]))
        else:
            x = x + plain_mlp(h, w, f"{p}.mlp")
    return plain_rmsnorm(x, w["norm.weight"], cfg["eps"]) @ w["head.weight"].T, margin


def clear_cut_tokens(cfg, w, n, gen, gap=0.1):
    """n random tokens, redrawn position by position until the router's choice at that position is
    clear (the model is causal, so earlier positions do not move): routing is a hard choice, and a
    near tie would go either way in reduced precision."""
    toks = []
    for i in range(n):
        for _ in range(200):
            cand = toks + [int(torch.randint(0, cfg["vocab_size"], (1,), generator=gen))]
            if float(plain_forward(cfg, w, cand)[1][i]) > gap:
                break
        else:
            raise AssertionError("no token with a clear routing found")
        toks = cand
    return toks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_position_table(dtype, tmp_path):
    from safetensors.torch import load_file

    from gllm_b200.cache import CacheManager
    from gllm_b200.config import ARCHITECTURES, load_config
    from gllm_b200.engine.step import StepEntry, StepRunner
    from gllm_b200.models.loading import load_model
    from gllm_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS
    from gllm_b200.weights import write_random_model

    register_toys()
    try:
        raw = dict(architectures=["ToyPartsLM"], vocab_size=200, hidden_size=64, torch_dtype="bfloat16", num_heads=4,
                   num_kv_heads=2, head_dim=16, intermediate_size=96, eps=1e-5)
        folder = write_random_model(str(tmp_path / "toy"), load_config(raw), seed=33, std=0.08, norm_jitter=0.05,
                                    std_overrides={"router": 1.0, "pos": 0.5})
        weights = {k: v.float() for k, v in load_file(f"{folder}/model.safetensors").items()}
        if dtype == "bfloat16":   # what a bfloat16 run holds: matrices rounded, norm and router weights as stored
            weights = {k: (v if v.dim() == 1 or "router" in k else v.to(torch.bfloat16).float()) for k, v in weights.items()}
        assert weights["layers.0.router.weight"].shape == (EXPERTS, 64) and "layers.1.pos.weight" in weights
        config, model = load_model(folder, dtype, "cuda:0")
        cache = CacheManager(model.cache_requirements(), 16, 24, 3, MAX_POS, model.dtype, "cuda:0")
        runner = StepRunner(model, cache, 128)
        g = torch.Generator().manual_seed(8)
        seqs = {k: clear_cut_tokens(raw, weights, n, g) for k, n in (("a", 60), ("b", 37))}
        want = {k: plain_forward(raw, weights, v)[0] for k, v in seqs.items()}
        scale = max(1.0, max(float(x.abs().max()) for x in want.values()))
        bound = 2e-4 * scale if dtype == "float32" else 5e-2 * scale
        cuts = {"a": [25, 2, 30, 1, 1, 1], "b": [5, 29, 1, 1, 1]}
        pos = {"a": 0, "b": 0}
        for step in range(6):
            entries, meta = [], []
            for k in ("a", "b"):
                if step < len(cuts[k]):
                    n = cuts[k][step]
                    entries.append(StepEntry(k, seqs[k][pos[k]:pos[k] + n], list(range(n))))
                    meta.append((k, pos[k], n))
                    pos[k] += n
            got = runner.run(entries).double().cpu()
            off = 0
            for k, p, n in meta:
                assert float((got[off:off + n] - want[k][p:p + n]).abs().max()) <= bound, (step, k)
                off += n
        assert runner.graph_replays > 0
    finally:
        del ARCHITECTURES["ToyPartsLM"]
        del FEED_FORWARDS["toy_top1"]
        del POSITION_ENCODINGS["toy_offset_table"]
