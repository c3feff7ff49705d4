"""Architectures: each turns its typed configuration into a ModelSpec that the
generic decoder (gllm_b200.models.decoder) builds from registered parts."""

from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "PlanEntry"]
