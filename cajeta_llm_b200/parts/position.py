"""Position encodings a mixer can be given.

A position part offers two things to the mixer that owns it: ``rotary_dim`` (how many
leading dims of each head are rotated; 0 = none) and ``inv_freq`` (float32,
``rotary_dim / 2`` entries).  The rotation itself happens in the mixer's kernel at each
row's absolute position, with the angle ``float32(p) * inv_freq[d]`` computed in
32-bit (model/Prim.cajeta:1917-1940).

``rope``: ``inv_freq[d] = theta^(-2d / rotary_dim)`` computed in float32 as the
reference does (model/Prim.cajeta:1866-1880; per-layer state, model/Attention.cajeta:72-99).
``scaling`` (optional, on ``rope``) stretches the slow frequencies (the YaRN form): with
``c(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(c(fast)), 0)``,
``hi = min(ceil(c(slow)), rotary_dim - 1)`` and ``ramp_d = clamp((d - lo) / max(hi - lo, 0.001), 0, 1)``
the frequency is ``f_d / factor * ramp_d + f_d (1 - ramp_d)``, and the part offers ``magnitude`` =
``0.1 ln(factor) + 1``, by which a mixer multiplies cos and sin (1 without scaling).  The table is worked
out in float64 and rounded once.
``scaling`` with ``"kind": "wavelength"`` (keys ``factor``, ``low``, ``high``, ``original``) is the other common form: with
the wavelength ``l = 2 pi / f``, a frequency stays where ``l < original / high``, becomes ``f / factor`` where
``l > original / low``, and in between ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``;
the magnitude stays 1.  Worked out in float64 and rounded once.
``none``: no rotation.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import Part, register_part


@register_part("position", "rope")
class RotaryEncoding(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.theta = float(spec["theta"])
        if self.rotary_dim % 2 != 0 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim must be even and within (0, head_dim={self.head_dim}], found {self.rotary_dim}")
        half = self.rotary_dim // 2
        d = np.arange(half, dtype=np.float32)
        exponent = (np.float32(0.0) - np.float32(2.0) * d) / np.float32(self.rotary_dim)
        inv = np.power(np.float32(self.theta), exponent).astype(np.float32)
        self.magnitude = 1.0
        scaling = spec.get("scaling")
        if scaling and scaling.get("kind") == "wavelength":
            factor, original = float(scaling["factor"]), float(scaling["original"])
            low, high = float(scaling["low"]), float(scaling["high"])
            if factor <= 0.0 or original <= 0.0 or not high > low >= 0.0:
                raise ValueError("rope scaling by wavelength needs a positive factor and original length and high > low >= 0")
            f = np.power(float(self.theta), -2.0 * np.arange(half, dtype=np.float64) / self.rotary_dim)
            wavelength = 2.0 * math.pi / f
            s = (original / wavelength - low) / (high - low)
            mid = (1.0 - s) * f / factor + s * f
            inv = np.where(wavelength < original / high, f, np.where(wavelength > (original / low if low > 0.0 else np.inf), f / factor, mid)).astype(np.float32)
        elif scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])
            if factor <= 0.0 or original <= 0.0 or self.theta <= 1.0:
                raise ValueError("rope scaling needs a positive factor and original length and theta > 1")

            def turns_dim(turns: float) -> float:
                return self.rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turns_dim(float(scaling["fast"]))), 0)
            hi = min(math.ceil(turns_dim(float(scaling["slow"]))), self.rotary_dim - 1)
            i = np.arange(half, dtype=np.float64)
            f = np.power(float(self.theta), -2.0 * i / self.rotary_dim)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv = (f / factor * ramp + f * (1.0 - ramp)).astype(np.float32)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.inv_freq = torch.from_numpy(inv).to(runtime.device)


@register_part("position", "none")
class NoPosition(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.rotary_dim = 0
        self.inv_freq = None
        self.magnitude = 1.0
