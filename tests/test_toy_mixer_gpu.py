"""A toy mixer with a state of its own, defined here, is registered, built from a checkpoint and
stepped (portions, decoding, CUDA-graph decode steps, the engine's generate) without a change to the
package: the package only knows the Mixer interface and the state slots of the cache manager."""

import json
import os
from dataclasses import dataclass

import pytest
import torch

from plain_llama import plain_attention_layer, plain_inverse_frequencies, plain_mlp, plain_rmsnorm

pytestmark = pytest.mark.gpu

DECAY = 0.8


def register_toy():
    from gllm_b200 import ops
    from gllm_b200.config import register_architecture
    from gllm_b200.config.model_config import ModelConfig
    from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry
    from gllm_b200.parts import Mixer, StateRequirement, TensorExpectation, register_mixer

    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
        """y_t = W s_t with s_t = decay * s_{t-1} + x_t: one vector of state per request."""

        def __init__(self, names, hidden_size, decay):
            super().__init__(names)
            self.hidden_size, self.decay, self.w = hidden_size, decay, None

        def state_requirement(self):
            return StateRequirement((self.hidden_size,), torch.float32)

        def expected_tensors(self):
            return {self.names["w"]: TensorExpectation((self.hidden_size, self.hidden_size))}

        def load(self, get, dtype, device):
            self.w = get(self.names["w"], "matrix")

        def forward(self, x, ctx, cache):
            state, slots = cache.state, ctx.state_slots.long()
            if ctx.max_q_len == 1:                       # decoding (also inside a captured graph): no host loop
                s = state[slots] * self.decay + x.float()
                state[slots] = s
            else:
                rows = []
                off = 0
                for r, n in enumerate(ctx.q_lens_host):  # portions: a sequential scan per request
                    cur = state[slots[r]]
                    for t in range(n):
                        cur = cur * self.decay + x[off + t].float()
                        rows.append(cur)
                    state[slots[r]] = cur
                    off += n
                s = torch.stack(rows)
            return ops.linear(s.to(x.dtype), self.w)

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
        toy = PartSpec("toy_decay", dict(hidden_size=h, decay=DECAY), {"w": "layers.0.toy.weight"})
        attn = PartSpec("attention", dict(hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=cfg.num_heads,
                                          head_dim=cfg.head_dim,
                                          position=PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=10000.0))),
                        {n: f"layers.1.self_attn.{n}_proj.weight" for n in "qkvo"})
        layers = (
            LayerSpec("prenorm", dict(mixer=toy, feed_forward=ffn("layers.0"), mixer_norm=norm("layers.0.n1.weight"),
                                      feed_forward_norm=norm("layers.0.n2.weight"))),
            LayerSpec("prenorm", dict(mixer=attn, feed_forward=ffn("layers.1"), mixer_norm=norm("layers.1.n1.weight"),
                                      feed_forward_norm=norm("layers.1.n2.weight"))),
        )
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size, layers=layers,
                         plan=(PlanEntry(0), PlanEntry(1), PlanEntry(0)),      # the toy layer runs twice: two states
                         final_norm=norm("norm.weight"), embedding_name="embed.weight", head_name=None)

    register_architecture("ToyDecayLM", ToyConfig, build_spec)
    return ToyConfig


def plain_toy_forward(cfg, w, tokens):
    """Whole sequence, float64, no cache and no state slots."""
    w = {k: v.double() for k, v in w.items()}
    x = w["embed.weight"][torch.tensor(tokens)]
    t = x.shape[0]
    att_cfg = dict(num_attention_heads=cfg["num_heads"], num_key_value_heads=cfg["num_heads"], head_dim=cfg["head_dim"],
                   hidden_size=cfg["hidden_size"], rope_theta=10000.0)
    inv_freq = plain_inverse_frequencies(att_cfg)

    def toy(h):
        s = torch.zeros(cfg["hidden_size"], dtype=torch.float64)
        out = []
        for i in range(t):
            s = s * DECAY + h[i]
            out.append(s)
        return torch.stack(out) @ w["layers.0.toy.weight"].T

    for layer in (0, 1, 0):
        p = f"layers.{layer}"
        h = plain_rmsnorm(x, w[f"{p}.n1.weight"], cfg["eps"])
        if layer == 0:
            x = x + toy(h)
        else:
            x = x + plain_attention_layer(h, w, f"{p}.self_attn", att_cfg, torch.arange(t), inv_freq, None)[0]
        h = plain_rmsnorm(x, w[f"{p}.n2.weight"], cfg["eps"])
        x = x + plain_mlp(h, w, f"{p}.mlp")
    return plain_rmsnorm(x, w["norm.weight"], cfg["eps"]) @ w["embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state(dtype, tmp_path):
    from safetensors.torch import load_file

    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine
    from gllm_b200.cache import CacheManager
    from gllm_b200.config import ARCHITECTURES, load_config
    from gllm_b200.engine.step import StepEntry, StepRunner
    from gllm_b200.models.loading import load_model
    from gllm_b200.parts import MIXERS
    from gllm_b200.weights import write_random_model

    register_toy()
    try:
        raw = dict(architectures=["ToyDecayLM"], vocab_size=300, hidden_size=64, torch_dtype="bfloat16",
                   intermediate_size=96, num_heads=2, head_dim=32, eps=1e-5)
        folder = write_random_model(str(tmp_path / "toy"), load_config(raw), seed=21, std=0.06, norm_jitter=0.05)
        assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyDecayLM"]
        weights = load_file(os.path.join(folder, "model.safetensors"))
        assert "layers.0.toy.weight" in weights
        weights = {k: v.float() for k, v in weights.items()}
        config, model = load_model(folder, dtype, "cuda:0")
        reqs = model.cache_requirements()
        assert [(kv is not None, st is not None) for kv, st, _ in reqs] == [(False, True), (True, False), (False, True)]
        cache = CacheManager(reqs, 16, 32, 3, 512, model.dtype, "cuda:0")
        states = [c.state for c in cache.mixer_caches()]
        assert states[0] is not None and states[2] is not None and states[0].data_ptr() != states[2].data_ptr()
        runner = StepRunner(model, cache, 256)
        g = torch.Generator().manual_seed(4)
        seqs = {k: torch.randint(0, 300, (n,), generator=g).tolist() for k, n in (("a", 70), ("b", 41), ("c", 55))}
        want = {k: plain_toy_forward(raw, weights, v) for k, v in seqs.items()}
        scale = max(1.0, max(float(x.abs().max()) for x in want.values()))
        bound = 2e-4 * scale if dtype == "float32" else 5e-2 * scale
        # portions of a and b together, then token by token (graph steps), c joins late in a slot that was used
        cuts = {"a": [30, 2, 1, 1, 1, 1, 34], "b": [7, 30, 1, 1, 1, 1]}
        pos = {"a": 0, "b": 0}
        for step in range(7):
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
            if step == 5:
                runner.finish("b")
        got = runner.run([StepEntry("c", seqs["c"], list(range(55)))]).double().cpu()      # reuses b's slot: state starts at 0
        assert float((got - want["c"]).abs().max()) <= bound
        assert runner.graph_replays > 0
        # and through the engine
        engine = LLMEngine(folder, GeneratorParams(block_size=16, max_batch_size=2, max_seq_len=128, model_dtype=dtype),
                           device="cuda:0")
        out = engine.generate([GenerationRequest(prompt_token_ids=seqs["a"][:20], max_new_tokens=6, temperature=0.0)])[0]
        toks = seqs["a"][:20]
        for t in out.token_ids:
            logits = plain_toy_forward(raw, weights, toks)[-1]
            best = int(logits.argmax())
            assert t == best or float(logits[best] - logits[t]) < (1e-5 if dtype == "float32" else 0.05) * float(logits.abs().max())
            toks = toks + [t]
    finally:
        del ARCHITECTURES["ToyDecayLM"]
        del MIXERS["toy_decay"]
