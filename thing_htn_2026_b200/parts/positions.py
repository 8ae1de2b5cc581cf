"""Rotary position encoding: the angle tables.  The rotation itself is fused into the
kernel that normalises q and k and writes the cache.

``inv_freq[i] = 1 / theta^(2i / rotary_dim)`` is computed once on the host in float32 with
the reference's expression (engine/engine.py:238-240); the device fills
``cos/sin[p, i]`` of ``p * inv_freq[i]`` in float32 (engine/engine.py:241-247).  The
tables cover the longest sequence of the cache and grow on demand (the reference grows
its tables the same way, engine/engine.py:232-251).

``layout`` says which entries of a head make a pair: "half" (entry i with entry
i + rotary_dim / 2, the default) or "interleaved" (entry 2i with entry 2i + 1).
``frequency_precision`` "float64" computes ``inv_freq`` in double precision before it is
rounded to float32 (one rounding instead of the float32 expression's several).
``angle_precision`` "float64": the angle ``p * inv_freq`` and its cosine and sine are computed in
double from the unrounded frequency and rounded once (the float32 product of a position in the
thousands carries an absolute error of 1e-4 of a turn's radian, which a score sums over a head).

``scaling`` (a mapping ``factor, original, fast, slow``) stretches the slow pairs for sequences
longer than ``original`` positions (YaRN).  With ``turn(t) = rotary_dim * ln(original / (2 pi t))
/ (2 ln theta)``, the pair index whose wavelength fits ``original`` positions t times,
``lo = max(floor(turn(fast)), 0)``, ``hi = min(ceil(turn(slow)), rotary_dim - 1)`` and
``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair i turns with
``inv_freq[i] / factor * ramp_i + inv_freq[i] * (1 - ramp_i)``, and cos and sin are both
multiplied by ``0.1 ln(factor) + 1`` (the tables carry that magnitude)."""

from __future__ import annotations

import math
from typing import List

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("position", "rope")
class Rope:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        return []

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        self.theta = float(spec.params["theta"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        self.layout = str(spec.params.get("layout", "half"))
        if self.layout not in ops.ROTARY_LAYOUTS:
            raise ValueError(f"rope: layout '{self.layout}' is not one of {sorted(ops.ROTARY_LAYOUTS)}")
        if spec.params.get("frequency_precision") == "float64":
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float64) / self.rotary_dim
            self.inv_freq = (self.theta ** -exponent).to(torch.float32).to(runtime.device)
        else:
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float32) / self.rotary_dim
            self.inv_freq = (1.0 / (self.theta ** exponent)).to(runtime.device)
        self.exact_angles = spec.params.get("angle_precision") == "float64"
        if self.exact_angles and spec.params.get("scaling"):
            raise ValueError("rope: angles in double are built without frequency scaling")
        self.inv_freq64 = (self.theta ** -(torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float64)
                                           / self.rotary_dim)).to(runtime.device)
        self.magnitude = 1.0
        scaling = spec.params.get("scaling")
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float64) / self.rotary_dim
            plain = self.theta ** -exponent

            def turn(t: float) -> float:
                return self.rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turn(float(scaling["fast"]))), 0)
            hi = min(math.ceil(turn(float(scaling["slow"]))), self.rotary_dim - 1)
            index = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            self.inv_freq = (plain / factor * ramp + plain * (1.0 - ramp)).to(torch.float32).to(runtime.device)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.device = runtime.device
        self._tables = None

    def ensure(self, n_positions: int) -> None:
        """Tables for positions ``[0, n_positions)``.  Call before a CUDA graph is captured."""
        have = 0 if self._tables is None else self._tables.cos.shape[0]
        if n_positions <= have:
            return
        size = max(64, 1 << (int(n_positions) - 1).bit_length())
        half = self.rotary_dim // 2
        cos = torch.empty((size, half), dtype=torch.float32, device=self.device)
        sin = torch.empty((size, half), dtype=torch.float32, device=self.device)
        if self.exact_angles:
            angle = torch.arange(size, dtype=torch.float64, device=self.device)[:, None] * self.inv_freq64[None, :]
            cos, sin = torch.cos(angle).to(torch.float32).contiguous(), torch.sin(angle).to(torch.float32).contiguous()
        else:
            ops.rope_table(cos, sin, self.inv_freq, 0, size)
        if self.magnitude != 1.0:
            cos.mul_(self.magnitude)
            sin.mul_(self.magnitude)
        self._tables = ops.RotaryTables(cos, sin, self.rotary_dim, self.layout)

    def tables(self) -> ops.RotaryTables:
        if self._tables is None:
            raise RuntimeError("rope: ensure(n_positions) has not been called")
        return self._tables
