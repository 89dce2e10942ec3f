"""Position encodings applied to queries and keys.

``rope_neox``: inv_freq[i] = 1 / theta^(2i/hd) for i < hd/2, angle[p, i] = p * inv_freq[i], all in
float32; cos and sin of the float32 angle; rotation of the pairs (i, i + hd/2)
(reference: src/layer/rotary_embedding.cpp:36-55, src/layer/rotary_embedding.cu:24-47).  The
tables stay float32 on the device (the reference rounds them to the model's type).

``rope_pairs``: rotation of adjacent pairs (2i, 2i + 1) on the first ``dims`` dimensions of a head, with
optional scaling of the frequencies by wavelength.

``none``: no encoding.
"""

from __future__ import annotations

import math

import torch

from ..config.errors import ConfigError
from ..config.spec import PositionSpec
from ..kernels import ops
from .base import PositionEncoding, register_position_encoding


def rope_tables(head_dim: int, max_positions: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, float32 [max_positions, head_dim/2], computed on the host in float32."""
    index = torch.arange(0, head_dim // 2, dtype=torch.float32)
    exponent = (2.0 * index) / torch.tensor(float(head_dim), dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angles = torch.arange(max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angles).contiguous(), torch.sin(angles).contiguous()


class RopeNeox(PositionEncoding):
    graph_safe = True

    kind = "rope_neox"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        if spec.head_dim <= 0 or spec.head_dim % 2 != 0:
            raise ConfigError("a rotary head size must be positive and even")
        theta = float(spec.params.get("theta", 10000.0))
        if not theta > 0.0 or theta == float("inf"):
            raise ConfigError("the rotary base must be finite and positive")
        self.head_dim = spec.head_dim
        self.max_positions = spec.max_positions
        cos, sin = rope_tables(spec.head_dim, spec.max_positions, theta)
        self.cos = cos.to(device)
        self.sin = sin.to(device)

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return ops.rope(x, heads, self.head_dim, self.cos, self.sin, positions, status)

    def as_rotation_tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


class NoPosition(PositionEncoding):
    graph_safe = True

    kind = "none"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        self.head_dim = spec.head_dim
        self.max_positions = spec.max_positions

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return x

    def as_rotation_tables(self) -> tuple[None, None]:
        return None, None


def scaled_frequencies(freqs: list[float], factor: float, low: float, high: float, original: float) -> list[float]:
    """Frequency scaling by wavelength (the scheme Llama 3.1 uses to stretch a context of ``original``
    positions): with wavelength l = 2 pi / f, a frequency is kept where l < original / high, divided by
    ``factor`` where l > original / low, and in between blended with s = (original / l - low) /
    (high - low) as (1 - s) f / factor + s f."""
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


class RopePairs(PositionEncoding):
    """Rotation of adjacent pairs: dimensions 2i and 2i + 1 of every head, for i < dims / 2, turn by the
    angle position * f_i with f_i = base^(-2i / dims); dimensions from ``dims`` on pass unchanged.
    (u, v) -> (u cos a - v sin a, v cos a + u sin a).  ``params``: base, dims (default: the head size),
    scaling (None, or factor / low / high / original as in ``scaled_frequencies``).  Frequencies are
    worked out in double precision on the host and kept as float32; angles are float32 products on the
    device.  The attention part hands the frequencies to the kernel that also norms and stores
    (``as_pair_frequencies``); ``apply`` is not offered apart from it."""

    graph_safe = True

    kind = "rope_pairs"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        dims = int(spec.params.get("dims", spec.head_dim))
        base = float(spec.params.get("base", 10000.0))
        if dims <= 0 or dims % 2 != 0 or dims > spec.head_dim:
            raise ConfigError("rotated dimensions must be even, positive and no more than the head size")
        if not base > 0.0 or base == float("inf"):
            raise ConfigError("the rotary base must be finite and positive")
        freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        scaling = spec.params.get("scaling")
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            if factor <= 0.0 or original <= 0.0 or high == low or low <= 0.0 or high <= 0.0:
                raise ConfigError("frequency scaling needs positive factor, low, high and original, and low != high")
            freqs = scaled_frequencies(freqs, factor, low, high, original)
        self.head_dim = spec.head_dim
        self.dims = dims
        self.max_positions = spec.max_positions
        self.freqs = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device)

    def as_pair_frequencies(self) -> tuple[torch.Tensor, int]:
        return self.freqs, self.dims

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        raise ConfigError("the rotation of adjacent pairs runs inside the attention's own kernel only")


register_position_encoding("rope_neox", RopeNeox)
register_position_encoding("rope_pairs", RopePairs)
register_position_encoding("none", NoPosition)
