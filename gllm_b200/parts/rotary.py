"""Rotary position encoding with optional llama3 frequency scaling.

Frequencies ``theta ** (-2m / rotary_dim)`` for m = 0 .. rotary_dim/2 - 1 as
gllm/model/model.py:119-123; each head's first ``rotary_dim`` dims are rotated
in pairs of its two halves (gllm/model/layers/attention.py:91-118) by
``position * frequency``.  The reference rounds a cos/sin table to the model
dtype (gllm/model/model.py:126-128) and ignores ``rope_scaling``; here the
frequencies are computed in float64 on the host, rounded once to fp32, and the
angle, sine and cosine are fp32 inside the kernel.
"""

from __future__ import annotations

import math

import torch

from gllm_b200.parts.base import PositionEncoding, register_position_encoding


def scaled_inverse_frequencies(
    rotary_dim: int,
    theta: float,
    scaling: dict | None = None,
) -> list[float]:
    """Float64 frequencies, llama3-scaled when ``scaling`` says so."""
    half = rotary_dim // 2
    freqs = [float(theta) ** (-2.0 * m / rotary_dim) for m in range(half)]
    if not scaling:
        return freqs
    kind = scaling.get("rope_type")
    if kind != "llama3":
        raise ValueError(f"rotary scaling {kind!r} is not supported")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            smooth = (original / wavelength - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe_portions = True

    def __init__(self, names=None, head_dim: int = 0, rotary_dim: int | None = None, theta: float = 10000.0,
                 scaling: dict | None = None, interleaved: bool = False):
        super().__init__(names)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.interleaved = bool(interleaved)
        self.inv_freq: torch.Tensor | None = None

    def load(self, get, dtype, device):
        freqs = scaled_inverse_frequencies(self.rotary_dim, self.theta, self.scaling)
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device)

    def rotary(self):
        return self.inv_freq, self.rotary_dim, self.interleaved


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    """Positions do not enter the mixer (keys and values are stored as they are)."""

    graph_safe_portions = True

    def __init__(self, names=None):
        super().__init__(names)
