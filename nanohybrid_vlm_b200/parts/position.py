"""Rotary position encoding: the fp32 cos/sin table of nanovllm/layers/rotary_embedding.py:83-89.

Parameters: ``theta`` (base), ``rotary_dim`` (how many leading elements of a head rotate;
the rest pass through), ``max_position``.  The angles are position * inv_freq in fp32, as
the reference computes them; mixers that rotate queries and keys read the table in their
fused kernel.
"""
from __future__ import annotations

import torch

from .base import POSITIONS, PositionEncoding


class RotaryTable(PositionEncoding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.max_position = int(spec["max_position"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        # Built once on the host in fp32 so that every device sees the same angles.
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
        t = torch.arange(self.max_position, dtype=torch.float32)
        freqs = t[:, None] * inv_freq[None, :]
        self.table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(env.device)

    def rotary(self):
        return self.table, self.rotary_dim


class BandedRotaryTable(PositionEncoding):
    """Rotary angles whose frequencies are rescaled by wavelength bands (the Llama 3.1 rule).  f_i = theta^(-2i/dims);
    with wavelength l = 2 pi / f: f stays where l < original / high, becomes f / factor where l > original / low,
    and in between (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  Parameters: ``theta``,
    ``rotary_dim``, and optionally ``factor``, ``low``, ``high``, ``original`` (all four or none).  The table covers
    the positions the engine can reach (``max_position`` of the build environment); frequencies, angles and their
    cosines are computed in float64 on the host and stored as the nearest float32."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        import math
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        band = [spec.get(k) for k in ("factor", "low", "high", "original")]
        if any(b is None for b in band) and not all(b is None for b in band):
            raise ValueError("frequency bands need factor, low, high and original together")
        half = self.rotary_dim // 2
        freqs = []
        for i in range(half):
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            if band[0] is not None:
                factor, low, high, original = (float(b) for b in band)
                wavelength = 2.0 * math.pi / f
                if wavelength > original / low:
                    f = f / factor
                elif wavelength >= original / high:
                    s = (original / wavelength - low) / (high - low)
                    f = (1.0 - s) * f / factor + s * f
            freqs.append(f)
        self.frequencies = torch.tensor(freqs, dtype=torch.float64)
        self.max_position = int(env.max_position)
        t = torch.arange(self.max_position, dtype=torch.float64)
        ang = t[:, None] * self.frequencies[None, :]
        self.table = torch.cat((ang.cos(), ang.sin()), dim=-1).to(torch.float32).contiguous().to(env.device)

    def rotary(self):
        return self.table, self.rotary_dim


class RampedRotaryTable(PositionEncoding):
    """Rotary angles whose frequencies are divided by ``factor`` along a linear ramp over the dimension index (the YaRN
    rule), with cosines and sines scaled.  f_i = theta^(-2i/dims).  The index at which a frequency makes t turns over
    ``original`` positions is dim(t) = dims ln(original / (2 pi t)) / (2 ln theta); lo = max(floor(dim(fast)), 0),
    hi = min(ceil(dim(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the frequency becomes
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by ``magnitude_slope`` ln(factor) + 1
    (the slope is 0.1 unless given).  Parameters: ``theta``, ``rotary_dim``, ``factor``, ``original``, ``fast``,
    ``slow``, ``magnitude_slope``.  Frequencies, angles and their cosines are computed in float64 on the host and stored
    as the nearest float32; the table covers the positions the engine can reach."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        import math
        self.rotary_dim = dims = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        if dims <= 0 or dims % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {dims}")
        factor, original = float(spec["factor"]), float(spec["original"])
        if factor <= 0 or original <= 0 or float(spec["fast"]) <= 0 or float(spec["slow"]) <= 0 or self.theta <= 1:
            raise ValueError("ramped rotary frequencies need positive factor, original, fast and slow, and theta > 1")

        def turn_dim(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(turn_dim(float(spec["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(spec["slow"]))), dims - 1)
        freqs = []
        for i in range(dims // 2):
            f = self.theta ** (-2.0 * i / dims)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freqs.append(f / factor * ramp + f * (1.0 - ramp))
        self.frequencies = torch.tensor(freqs, dtype=torch.float64)
        self.magnitude = float(spec.get("magnitude_slope", 0.1)) * math.log(factor) + 1.0
        self.max_position = int(env.max_position)
        t = torch.arange(self.max_position, dtype=torch.float64)
        ang = t[:, None] * self.frequencies[None, :]
        table = torch.cat((ang.cos(), ang.sin()), dim=-1) * self.magnitude
        self.table = table.to(torch.float32).contiguous().to(env.device)

    def rotary(self):
        return self.table, self.rotary_dim


class NoPosition(PositionEncoding):
    """No position signal at all (order then enters only through causality)."""


POSITIONS.register("rope", RotaryTable)
POSITIONS.register("rope_banded", BandedRotaryTable)
POSITIONS.register("rope_ramped", RampedRotaryTable)
POSITIONS.register("none", NoPosition)
