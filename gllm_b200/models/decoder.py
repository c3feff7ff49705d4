"""The generic decoder: builds whatever a ModelSpec describes and runs it.

``forward`` is the model half of the step function: embedding lookup, the
layer plan, the final norm at the wanted rows only, and the output head in
fp32.  The reference computes logits at every position and slices afterwards
(gllm/llm/llm.py:335-340); here the final norm and the head see only the rows
whose logits were asked for.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.models.spec import ModelSpec
from gllm_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, build_part
from gllm_b200.parts.base import Block, MixerCache, Norm, StepContext, TensorExpectation


_TABLE_OF_KIND = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}


def _build_layer(layer_spec) -> Block:
    """The registered block of ``layer_spec.block`` with the parts it declares, each built from the
    spec of the same name."""
    try:
        block_cls = BLOCKS[layer_spec.block]
    except KeyError:
        raise KeyError(f"no block of kind {layer_spec.block!r} is registered; known: {sorted(BLOCKS)}") from None
    declared = block_cls.part_kinds
    missing = [n for n in declared if n not in layer_spec.parts]
    extra = [n for n in layer_spec.parts if n not in declared]
    if missing or extra:
        raise ValueError(f"block {layer_spec.block!r} declares parts {list(declared)}: the layer lacks {missing} "
                         f"and names {extra} beyond them")
    return block_cls(**{name: build_part(_TABLE_OF_KIND[kind], layer_spec.parts[name])
                        for name, kind in declared.items()})


def expected_tensors_of_spec(spec: ModelSpec) -> dict[str, TensorExpectation]:
    """Every checkpoint tensor the model will read, in declaration order."""
    spec.validate()
    exp: dict[str, TensorExpectation] = {
        spec.embedding_name: TensorExpectation((spec.vocab_size, spec.hidden_size), "matrix")
    }
    for layer_spec in spec.layers:
        for part in _build_layer(layer_spec).parts():
            exp.update(part.expected_tensors())
    exp.update(build_part(NORMS, spec.final_norm).expected_tensors())
    if spec.head_name is not None:
        exp[spec.head_name] = TensorExpectation((spec.vocab_size, spec.hidden_size), "matrix")
    return exp


class DecoderModel:
    """A stack of blocks between an embedding table and an output head."""

    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.layers: list[Block] = [_build_layer(s) for s in spec.layers]
        self.final_norm: Norm = build_part(NORMS, spec.final_norm)
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None

    @property
    def graph_safe_portions(self) -> bool:
        """True when every part (the mixers' position encodings included) may have its prompt portions
        captured in a CUDA graph (``Part.graph_safe_portions``)."""
        parts = [self.final_norm] + [p for block in self.layers for p in [block] + block.parts()]
        parts += [p.position for p in list(parts) if getattr(p, "position", None) is not None]
        return all(getattr(p, "graph_safe_portions", False) for p in parts)

    # ---------------------------------------------------------------- weights
    def expected_tensors(self) -> dict[str, TensorExpectation]:
        exp = {self.spec.embedding_name: TensorExpectation((self.spec.vocab_size, self.spec.hidden_size), "matrix")}
        for block in self.layers:
            for part in block.parts():
                exp.update(part.expected_tensors())
        exp.update(self.final_norm.expected_tensors())
        if self.spec.head_name is not None:
            exp[self.spec.head_name] = TensorExpectation((self.spec.vocab_size, self.spec.hidden_size), "matrix")
        return exp

    def load(self, checkpoint) -> None:
        checkpoint.validate(self.expected_tensors(), self.spec.ignorable_names)
        get = checkpoint.getter(self.dtype, self.device)
        self.embedding = get(self.spec.embedding_name, "matrix")
        for block in self.layers:
            for part in block.parts():
                part.load(get, self.dtype, self.device)
        self.final_norm.load(get, self.dtype, self.device)
        self.head = self.embedding if self.spec.head_name is None else get(self.spec.head_name, "matrix")

    # ------------------------------------------------------------------ cache
    def cache_requirements(self):
        """Per plan entry: (kv requirement | None, state requirement | None,
        reads_cache_of | None)."""
        out = []
        for entry in self.spec.plan:
            mixer = self.layers[entry.layer].cache_mixer()
            if mixer is None:
                out.append((None, None, entry.reads_cache_of))
            else:
                out.append((mixer.kv_requirement(), mixer.state_requirement(), entry.reads_cache_of))
        return out

    def kernel_needs(self) -> dict:
        """Union of what the parts will ask of the kernel modules (``Part.kernel_needs``)."""
        needs: dict = {}
        parts = [self.final_norm] + [p for block in self.layers for p in block.parts()]
        for part in parts:
            for key, values in part.kernel_needs().items():
                needs.setdefault(key, set()).update(values)
        return needs

    # ---------------------------------------------------------------- forward
    def forward(
        self,
        tokens: torch.Tensor,
        ctx: StepContext,
        caches: list[MixerCache],
        logit_rows: torch.Tensor,
        logits_out: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """Logits ``[len(logit_rows), vocab]`` fp32 of the flat batch ``tokens``."""
        resid = ops.embedding(tokens, self.embedding, sampled=ctx.sampled, token_row=ctx.token_row,
                              scale=1.0 if self.spec.embedding_scale is None else self.spec.embedding_scale)
        branch = None
        for entry_idx, entry in enumerate(self.spec.plan):
            branch, resid = self.layers[entry.layer].forward(branch, resid, ctx, caches[entry_idx])
        if logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        final = self.final_norm.forward(None if branch is ops.ADDED else branch, resid, self.dtype, rows=logit_rows)
        logits = ops.linear(final, self.head, out_dtype=torch.float32, out=logits_out)
        if self.spec.logit_scale is not None or self.spec.logit_softcap is not None:
            ops.scale_softcap(logits, 1.0 if self.spec.logit_scale is None else self.spec.logit_scale,
                              self.spec.logit_softcap)
        return logits
