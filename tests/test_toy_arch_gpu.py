"""What a new architecture may need beyond new parts, registered from here without a change to
the package: a block with ONE shared norm and parallel branches (another set of part names than
the pre-norm block's), a mixer that caches one latent vector per token instead of keys and values
(its own page layout, its own cache group beside the attention layer's), and a model with an
embedding multiplier, a logit scale and a soft cap on the logits.  Every cut of the replay tests
(whole, token by token, changing portions, mixed over a pool so small that pages are used again)
against a plain float64 restatement, in float32 and in bfloat16."""

from dataclasses import dataclass

import pytest
import torch

from plain_llama import plain_attention_layer, plain_inverse_frequencies, plain_mlp, plain_rmsnorm
from replay_helpers import (BF16_TOL_MAX, BF16_TOL_MEAN, FP32_TOL, compare, mixed_steps, run_steps, sequences,
                            single_request_steps)

pytestmark = pytest.mark.gpu

LATENT = 24
EMBEDDING_SCALE, LOGIT_SCALE, LOGIT_CAP = 1.7, 0.6, 3.0


def register_toy():
    from gllm_b200 import ops
    from gllm_b200.config import register_architecture
    from gllm_b200.config.model_config import ModelConfig
    from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry
    from gllm_b200.parts import (Block, KVPageRequirement, Mixer, TensorExpectation, register_block, register_mixer)

    @register_mixer("toy_latent")
    class LatentMeanMixer(Mixer):
        """c_t = W_c x_t is cached, one vector of ``latent`` numbers per token; y_t = W_o mean(c_0 .. c_t).
        Everything that varies between steps is read from device memory, so decode steps and portions
        may be captured."""

        graph_safe_portions = True

        def __init__(self, names, hidden_size, latent):
            super().__init__(names)
            self.hidden_size, self.latent = hidden_size, latent
            self.w_c = self.w_o = None

        def kv_requirement(self):
            return KVPageRequirement(((1, self.latent),))

        def expected_tensors(self):
            return {self.names["c"]: TensorExpectation((self.latent, self.hidden_size)),
                    self.names["o"]: TensorExpectation((self.hidden_size, self.latent))}

        def load(self, get, dtype, device):
            self.w_c, self.w_o = get(self.names["c"], "matrix"), get(self.names["o"], "matrix")

        def forward(self, x, ctx, cache):
            view = ctx.groups[cache.group]
            pages = cache.tensor(0)                                   # [pages, 1, block_size, latent]
            bs = view.block_size
            c = ops.as_tensor(ops.linear(x, self.w_c))
            slots = view.slot_mapping.long()
            pages[slots // bs, 0, slots % bs] = c
            tables = view.block_table[ctx.token_row.long()].clamp(min=0).long()          # [n, blocks]
            cached = pages[tables, 0].reshape(x.shape[0], -1, self.latent).float()         # [n, tokens, latent]
            seen = torch.arange(cached.shape[1], device=x.device)[None, :] <= ctx.positions[:, None]
            mean = (cached * seen[:, :, None]).sum(1) / (ctx.positions[:, None].float() + 1.0)
            return ops.linear(mean.to(x.dtype), self.w_o)

    @register_block("toy_parallel")
    class ParallelBlock(Block):
        """x += mixer(norm(x)) + feed_forward(norm(x)) with one norm for both branches."""

        graph_safe_portions = True
        part_kinds = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def forward(self, branch, resid, ctx, cache):
            x = self.norm.forward(branch, resid, ctx.dtype)
            mixed = ops.as_tensor(self.mixer.forward(x, ctx, cache))
            return mixed + ops.as_tensor(self.feed_forward.forward(x, ctx)), resid

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        intermediate_size: int = 0
        num_heads: int = 0
        head_dim: int = 0
        eps: float = 1e-5

        @classmethod
        def from_dict(cls, d):
            return cls(architecture=d["architectures"][0], vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
                       dtype=d["torch_dtype"], eos_token_ids=(), intermediate_size=d["intermediate_size"],
                       num_heads=d["num_heads"], head_dim=d["head_dim"], eps=d["eps"])

        def to_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        torch_dtype=self.dtype, intermediate_size=self.intermediate_size, num_heads=self.num_heads,
                        head_dim=self.head_dim, eps=self.eps)

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(size=h, eps=cfg.eps), {"weight": name})
        ffn = lambda p: PartSpec("swiglu", dict(hidden_size=h, intermediate_size=cfg.intermediate_size),
                                 {n: f"{p}.mlp.{n}_proj.weight" for n in ("gate", "up", "down")})
        latent = PartSpec("toy_latent", dict(hidden_size=h, latent=LATENT),
                          {"c": "layers.0.latent.c.weight", "o": "layers.0.latent.o.weight"})
        attn = PartSpec("attention", dict(hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=1,
                                          head_dim=cfg.head_dim,
                                          position=PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=10000.0))),
                        {n: f"layers.1.self_attn.{n}_proj.weight" for n in "qkvo"})
        layers = (
            LayerSpec("toy_parallel", dict(norm=norm("layers.0.n.weight"), mixer=latent, feed_forward=ffn("layers.0"))),
            LayerSpec("prenorm", dict(mixer_norm=norm("layers.1.n1.weight"), mixer=attn,
                                      feed_forward_norm=norm("layers.1.n2.weight"), feed_forward=ffn("layers.1"))),
        )
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size, layers=layers,
                         plan=(PlanEntry(0), PlanEntry(1)), final_norm=norm("norm.weight"),
                         embedding_name="embed.weight", head_name="head.weight",
                         embedding_scale=EMBEDDING_SCALE, logit_scale=LOGIT_SCALE, logit_softcap=LOGIT_CAP)

    register_architecture("ToyLatentLM", ToyConfig, build_spec)


def unregister_toy():
    from gllm_b200.config import ARCHITECTURES
    from gllm_b200.parts import BLOCKS, MIXERS

    ARCHITECTURES.pop("ToyLatentLM", None)
    MIXERS.pop("toy_latent", None)
    BLOCKS.pop("toy_parallel", None)


def plain_toy_forward(cfg, w, tokens):
    """Whole sequence, float64, no cache."""
    w = {k: v.double() for k, v in w.items()}
    x = w["embed.weight"][torch.tensor(tokens)] * EMBEDDING_SCALE
    t = x.shape[0]
    h = plain_rmsnorm(x, w["layers.0.n.weight"], cfg["eps"])
    c = h @ w["layers.0.latent.c.weight"].T
    mean = c.cumsum(0) / torch.arange(1, t + 1, dtype=torch.float64)[:, None]
    x = x + mean @ w["layers.0.latent.o.weight"].T + plain_mlp(h, w, "layers.0.mlp")
    att_cfg = dict(num_attention_heads=cfg["num_heads"], num_key_value_heads=1, head_dim=cfg["head_dim"],
                   hidden_size=cfg["hidden_size"], rope_theta=10000.0)
    h = plain_rmsnorm(x, w["layers.1.n1.weight"], cfg["eps"])
    x = x + plain_attention_layer(h, w, "layers.1.self_attn", att_cfg, torch.arange(t),
                                  plain_inverse_frequencies(att_cfg), None)[0]
    h = plain_rmsnorm(x, w["layers.1.n2.weight"], cfg["eps"])
    x = x + plain_mlp(h, w, "layers.1.mlp")
    logits = plain_rmsnorm(x, w["norm.weight"], cfg["eps"]) @ w["head.weight"].T * LOGIT_SCALE
    return LOGIT_CAP * torch.tanh(logits / LOGIT_CAP)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parallel_block_latent_cache_and_scaled_head(dtype, tmp_path):
    from safetensors.torch import load_file

    from gllm_b200.config import load_config
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.weights import write_random_model

    register_toy()
    try:
        raw = dict(architectures=["ToyLatentLM"], vocab_size=300, hidden_size=80, torch_dtype="bfloat16",
                   intermediate_size=112, num_heads=2, head_dim=32, eps=1e-5)
        folder = write_random_model(str(tmp_path / "toy"), load_config(raw), seed=31, std=0.08, norm_jitter=0.05)
        weights = {k: v.float() for k, v in load_file(f"{folder}/model.safetensors").items()}
        _, runner = build_runner(folder, dtype, max_tokens=448, block_size=8)
        cache = runner.cache
        assert len(cache.groups) == 2                                  # latent pages and key/value pages
        assert [g.requirement.elements_per_token for g in cache.groups] == [LATENT, 2 * 32]
        assert cache.groups[0].pool.shape == (1, 448 // 8 + 1, 8 * LATENT)
        item = 4 if dtype == "float32" else 2
        assert cache.bytes_per_token() == (LATENT + 64) * item
        seqs = sequences(300, seed=3)
        plain = {k: plain_toy_forward(raw, weights, v) for k, v in seqs.items()}
        assert float(max(p.abs().max() for p in plain.values())) < LOGIT_CAP
        tol = (FP32_TOL, None) if dtype == "float32" else (BF16_TOL_MAX, BF16_TOL_MEAN)
        steps, index = single_request_steps(seqs)
        compare(run_steps(runner, steps), index, plain, *tol)
        steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
        compare(run_steps(runner, steps), index, plain, *tol)
        assert all(g.allocator.total_reused > 0 for g in cache.groups)
        assert runner.graph_replays > 0
        cache.check_invariants()
    finally:
        unregister_toy()


def test_a_block_gets_exactly_the_parts_it_declares():
    from gllm_b200.models.decoder import _build_layer
    from gllm_b200.models.spec import LayerSpec, PartSpec

    norm = PartSpec("rmsnorm", dict(size=8, eps=1e-5), {"weight": "n"})
    with pytest.raises(ValueError, match="lacks"):
        _build_layer(LayerSpec("prenorm", dict(mixer_norm=norm)))
    with pytest.raises(KeyError, match="no block of kind"):
        _build_layer(LayerSpec("no_such_block", {}))


def test_an_unsummed_product_read_too_late_raises():
    """A block that holds a mixer's unsummed result across two more products is told so."""
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(1)
    x = (torch.randn(8, 2048, generator=g) * 0.1).to(torch.bfloat16).cuda()
    w = (torch.randn(2048, 2048, generator=g) * 0.02).to(torch.bfloat16).cuda()
    first = ops.linear(x, w, split_ok=True)
    assert isinstance(first, ops.SplitSum)
    kept = first.tensor().float()
    second = ops.linear(x, w, split_ok=True)
    torch.testing.assert_close(first.tensor().float(), kept)          # survives the next product
    ops.as_tensor(second)
    ops.linear(x, w, split_ok=True)
    with pytest.raises(RuntimeError, match="overwritten"):
        first.tensor()


# ------------------------------------------------------------------------------------------------
# Attention with biased projections and a norm of every query and key head before the rotation: options of the
# built-in attention part that Llama does not use, through a toy architecture registered from here.
QK_EPS = 1e-6


def register_biased():
    from gllm_b200.config import register_architecture
    from gllm_b200.config.model_config import ModelConfig
    from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

    @dataclass(frozen=True)
    class BiasedConfig(ModelConfig):
        intermediate_size: int = 0
        num_heads: int = 0
        num_kv_heads: int = 0
        head_dim: int = 0
        num_layers: int = 0
        eps: float = 1e-5

        @classmethod
        def from_dict(cls, d):
            return cls(architecture=d["architectures"][0], vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
                       dtype=d["torch_dtype"], eos_token_ids=(), intermediate_size=d["intermediate_size"],
                       num_heads=d["num_heads"], num_kv_heads=d["num_kv_heads"], head_dim=d["head_dim"],
                       num_layers=d["num_layers"], eps=d["eps"])

        def to_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        torch_dtype=self.dtype, intermediate_size=self.intermediate_size, num_heads=self.num_heads,
                        num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, num_layers=self.num_layers, eps=self.eps)

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(size=h, eps=cfg.eps), {"weight": name})

        def layer(i):
            p = f"layers.{i}"
            names = {n: f"{p}.attn.{n}.weight" for n in "qkvo"}
            names.update({f"{n}_bias": f"{p}.attn.{n}.bias" for n in "qkvo"})
            names.update({"q_norm": f"{p}.attn.q_norm.weight", "k_norm": f"{p}.attn.k_norm.weight"})
            attn = PartSpec("attention", dict(hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
                                              head_dim=cfg.head_dim, bias=True, output_bias=True, qk_norm_eps=QK_EPS,
                                              position=PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=10000.0))),
                            names)
            ffn = PartSpec("swiglu", dict(hidden_size=h, intermediate_size=cfg.intermediate_size),
                           {n: f"{p}.mlp.{n}_proj.weight" for n in ("gate", "up", "down")})
            return LayerSpec("prenorm", dict(mixer_norm=norm(f"{p}.n1.weight"), mixer=attn,
                                             feed_forward_norm=norm(f"{p}.n2.weight"), feed_forward=ffn))

        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size, layers=tuple(layer(i) for i in range(cfg.num_layers)),
                         plan=tuple(PlanEntry(i) for i in range(cfg.num_layers)), final_norm=norm("norm.weight"),
                         embedding_name="embed.weight", head_name="head.weight")

    register_architecture("ToyBiasedLM", BiasedConfig, build_spec)


def plain_biased_forward(cfg, w, tokens):
    """Whole sequence, float64, no cache: q = norm_head(W_q x + b_q), k likewise, v = W_v x + b_v, rotation,
    attention, W_o a + b_o."""
    from plain_llama import plain_attention, plain_rope

    w = {k: v.double() for k, v in w.items()}
    x = w["embed.weight"][torch.tensor(tokens)]
    t = x.shape[0]
    hq, hkv, d = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    pos = torch.arange(t)
    inv_freq = plain_inverse_frequencies(dict(head_dim=d, rope_theta=10000.0, hidden_size=cfg["hidden_size"],
                                              num_attention_heads=hq))
    head_norm = lambda z, g: z / torch.sqrt((z * z).mean(-1, keepdim=True) + QK_EPS) * g
    for i in range(cfg["num_layers"]):
        p = f"layers.{i}"
        h = plain_rmsnorm(x, w[f"{p}.n1.weight"], cfg["eps"])
        q = (h @ w[f"{p}.attn.q.weight"].T + w[f"{p}.attn.q.bias"]).view(t, hq, d)
        k = (h @ w[f"{p}.attn.k.weight"].T + w[f"{p}.attn.k.bias"]).view(t, hkv, d)
        v = (h @ w[f"{p}.attn.v.weight"].T + w[f"{p}.attn.v.bias"]).view(t, hkv, d)
        q = plain_rope(head_norm(q, w[f"{p}.attn.q_norm.weight"]), pos, inv_freq)
        k = plain_rope(head_norm(k, w[f"{p}.attn.k_norm.weight"]), pos, inv_freq)
        a = plain_attention(q, k, v, pos, pos).reshape(t, hq * d)
        x = x + a @ w[f"{p}.attn.o.weight"].T + w[f"{p}.attn.o.bias"]
        h = plain_rmsnorm(x, w[f"{p}.n2.weight"], cfg["eps"])
        x = x + plain_mlp(h, w, f"{p}.mlp")
    return plain_rmsnorm(x, w["norm.weight"], cfg["eps"]) @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(4, 2, 64), (3, 1, 48)])
def test_attention_with_biases_and_a_norm_of_every_head(dtype, heads, kv_heads, head_dim, tmp_path):
    from safetensors.torch import load_file

    from gllm_b200.config import ARCHITECTURES, load_config
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.weights import write_random_model

    register_biased()
    try:
        raw = dict(architectures=["ToyBiasedLM"], vocab_size=300, hidden_size=96, torch_dtype="bfloat16",
                   intermediate_size=128, num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, num_layers=2,
                   eps=1e-5)
        folder = write_random_model(str(tmp_path / "toy"), load_config(raw), seed=11, std=0.08, norm_jitter=0.3)
        weights = {k: v.float() for k, v in load_file(f"{folder}/model.safetensors").items()}
        assert float(weights["layers.0.attn.q.bias"].abs().min()) > 0.0
        _, runner = build_runner(folder, dtype, max_tokens=448, block_size=16)
        seqs = sequences(300, seed=4)
        plain = {k: plain_biased_forward(raw, weights, v) for k, v in seqs.items()}
        tol = (FP32_TOL, None) if dtype == "float32" else (BF16_TOL_MAX, BF16_TOL_MEAN)
        steps, index = single_request_steps(seqs)
        compare(run_steps(runner, steps), index, plain, *tol)
        steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
        compare(run_steps(runner, steps), index, plain, *tol)
        assert runner.graph_replays > 0
    finally:
        ARCHITECTURES.pop("ToyBiasedLM", None)
