"""Rotary position encoding with split-half pairing.

Parity: runtime/reference.py:9-15 and kernels/ops.cu:21-33: pair (i, i + D/2) turns
by pos * theta^(-2i/D); keys are cached already rotated.  The frequencies are taken
in float64 on the host and the angles in float64 on the device; the tables a step
uses are computed once per step and shared by all layers with the same constants.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .base import POSITIONS, PositionEncoding, Rotation, register


@register(POSITIONS, "rotary_half")
class RotaryHalf(PositionEncoding):
    """params: theta, dim (rotated width, at most the head size); scaling (optional, see `scaled_frequencies`)."""

    interleaved = False

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.theta = float(spec["theta"])
        self.dim = int(spec["dim"])
        if self.dim % 2:
            raise ValueError("rotary position encoding needs an even width")
        scaling = spec.get("scaling")
        self.scaling = dict(scaling) if scaling else None
        self.magnitude = 1.0
        self._inv_freq = None

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def inv_freq(self, device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != device:
            half = self.dim // 2
            host = self.theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / self.dim)
            if self.scaling:
                host, self.magnitude = scaled_frequencies(host, self.theta, self.dim, self.scaling)
            self._inv_freq = host.to(device)
        return self._inv_freq

    def rotation(self, ctx) -> Rotation:
        key = ("rotary", self.theta, self.dim, self.interleaved, tuple(sorted(self.scaling.items())) if self.scaling else None)
        cached = ctx.shared.get(key)
        if cached is None:
            half = self.dim // 2
            cos = torch.empty((ctx.n_tokens, half), dtype=torch.float32, device=ctx.device)
            sin = torch.empty_like(cos)
            inv_freq = self.inv_freq(ctx.device)          # also settles the magnitude
            kernels.rotary_tables(ctx.positions, inv_freq, cos, sin, self.magnitude)
            cached = Rotation(cos, sin, half, self.interleaved)
            ctx.shared[key] = cached
        return cached


def scaled_frequencies(freq: torch.Tensor, theta: float, dim: int, scaling) -> tuple:
    """Frequencies stretched for sequences longer than the `original` length, and the factor both tables are multiplied by.

    kind "yarn" (factor, original, fast, slow): pair i is the wave that makes `original * f_i / 2 pi` turns over the
    original length.  With pair(t) = dim * ln(original / (2 pi t)) / (2 ln theta) the pair that makes t turns,
    lo = max(floor(pair(fast)), 0) and hi = min(ceil(pair(slow)), dim - 1), pairs up to lo keep their frequency, pairs
    from hi on are slowed by `factor`, and those between are blended linearly:
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i' = f_i / factor * ramp_i + f_i * (1 - ramp_i).
    Both cos and sin are multiplied by 0.1 ln(factor) + 1."""
    import math

    kind = scaling.get("kind", "yarn")
    if kind == "wavelength":
        return frequencies_by_wavelength(freq, scaling), 1.0
    if kind != "yarn":
        raise ValueError(f"unknown rotary scaling {kind!r}")
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns: float) -> float:
        return dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dim - 1)
    index = torch.arange(freq.numel(), dtype=torch.float64)
    ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def frequencies_by_wavelength(freq: torch.Tensor, scaling) -> torch.Tensor:
    """kind "wavelength" (factor, low, high, original): a pair is judged by its wavelength l = 2 pi / f against the
    original length.  Waves shorter than original / high keep their frequency, waves longer than original / low are slowed
    by `factor`, and between the two the frequency is blended by s = (original / l - low) / (high - low):
    f' = (1 - s) f / factor + s f.  The tables' magnitude stays 1."""
    import math

    factor, low, high, original = (float(scaling[key]) for key in ("factor", "low", "high", "original"))
    wave = 2.0 * math.pi / freq
    blend = (original / wave - low) / (high - low)
    mixed = (1.0 - blend) * freq / factor + blend * freq
    return torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mixed))


@register(POSITIONS, "rotary_interleaved")
class RotaryInterleaved(RotaryHalf):
    """The same turn with neighbours paired: coordinates (2i, 2i + 1) turn by pos * theta^(-2i/dim).  params as above."""

    interleaved = True


@register(POSITIONS, "none")
class NoPosition(PositionEncoding):
    def rotation(self, ctx):
        return None
