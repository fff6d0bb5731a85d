"""Rotary position encoding as a (cos, sin) table, with either pairing of channels.

Pair i of a head's first ``rotary_dim`` channels turns by ``pos * theta^(-2i/rot)``
(native/include/flyweight_v2_native_kernels.hpp:993-1008 for the angle, :1034-1047
for the rotation; rot = min(rotary_dimension or hd, hd), native/src/v2_runtime.cpp:4232-4234).
LFM2 pairs channel i with channel i + rot/2 ("half-split", NEOX); the other common
convention pairs 2i with 2i+1 ("interleaved").  Which one is a parameter of the part and of
the kernel, not a property of the attention mixer.
flyweight evaluates powf/cosf/sinf in fp32 on a float position; here the angles are
computed once in float64 on the host and rounded to fp32, so that the rotation at
position 100 000 is as exact as at position 10 and every kernel reads the same values.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position


@register_position("rope")
class Rope(PositionEncoding):
    """params: theta, rotary_dim (even, <= head size), pairing ("half_split" | "interleaved"), and
    optionally ``scaling`` = {factor, low, high, original}: a frequency whose wavelength is shorter than
    original/high stays, one whose wavelength is longer than original/low is divided by ``factor``, and in
    between, with s = (original/wavelength - low) / (high - low), it becomes (1 - s) f/factor + s f.

    ``scaling`` = {factor, original, fast, slow} (no ``low``/``high``) is the other common rule, a ramp over
    the pair index: with c(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) the index of the pair that
    turns t times over ``original`` positions, lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)),
    rotary_dim - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i gets r_i f_i / factor +
    (1 - r_i) f_i, and every cos and sin of the table is multiplied by ``amplitude`` (0.1 ln(factor) + 1
    when the scaling does not name one)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(self.params["theta"])
        self.rotary_dim = int(self.params["rotary_dim"])
        self.pairing = str(self.params.get("pairing", self.pairing))
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        if self.pairing not in ("half_split", "interleaved"):
            raise ValueError(f"unknown rotary pairing {self.pairing!r}")
        self.scaling = dict(self.params["scaling"]) if self.params.get("scaling") else None
        self.ramp = self.scaling is not None and "fast" in self.scaling
        if self.ramp:
            missing = [key for key in ("factor", "original", "fast", "slow") if self.scaling.get(key) is None]
            if missing:
                raise ValueError("rotary frequency scaling is missing " + ", ".join(missing))
            if min(float(self.scaling[key]) for key in ("factor", "original", "fast", "slow")) <= 0 \
                    or self.theta <= 1.0:
                raise ValueError("rotary frequency scaling by a ramp needs positive factor, original, fast and "
                                 "slow, and theta > 1")
        elif self.scaling is not None:
            missing = [key for key in ("factor", "low", "high", "original") if self.scaling.get(key) is None]
            if missing:
                raise ValueError("rotary frequency scaling is missing " + ", ".join(missing))
            if float(self.scaling["high"]) == float(self.scaling["low"]) or float(self.scaling["factor"]) <= 0:
                raise ValueError("rotary frequency scaling needs high != low and a positive factor")

    def frequencies(self) -> torch.Tensor:
        """float64 [rotary_dim/2]: theta^(-2i/rotary_dim), scaled by wavelength when ``scaling`` is set."""
        half = self.rotary_dim // 2
        exponent = torch.arange(half, dtype=torch.float64) * (-2.0 / max(self.rotary_dim, 1))
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), exponent)
        if self.scaling is None:
            return freq
        if self.ramp:
            factor, original = float(self.scaling["factor"]), float(self.scaling["original"])

            def turn_index(turns: float) -> float:
                return self.rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turn_index(float(self.scaling["fast"]))), 0)
            hi = min(math.ceil(turn_index(float(self.scaling["slow"]))), self.rotary_dim - 1)
            ramp = torch.clamp((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            return freq / factor * ramp + freq * (1.0 - ramp)
        factor, low, high = (float(self.scaling[key]) for key in ("factor", "low", "high"))
        original = float(self.scaling["original"])
        wave = 2.0 * math.pi / freq
        blend = (original / wave - low) / (high - low)
        mixed = (1.0 - blend) * freq / factor + blend * freq
        return torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mixed))

    def amplitude(self) -> float:
        """What every cos and sin is multiplied by (1 unless the scaling is a ramp)."""
        if not self.ramp:
            return 1.0
        given = self.scaling.get("amplitude")
        return float(given) if given is not None else 0.1 * math.log(float(self.scaling["factor"])) + 1.0

    def table(self, n_positions: int, device):
        """[n_positions][rotary_dim/2][2] fp32: (cos, sin) of every angle, times ``amplitude()``."""
        inv_freq = self.frequencies()
        angle = torch.arange(n_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        table = (torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1) * self.amplitude()).to(torch.float32)
        return table.contiguous().to(device)


@register_position("rope_half_split")
class RopeHalfSplit(Rope):
    """params: theta, rotary_dim.  The pairing LFM2 uses."""
    pairing = "half_split"


@register_position("no_position")
class NoPosition(PositionEncoding):
    """Nothing turns: queries and keys go to the attention as the head norm left them."""
