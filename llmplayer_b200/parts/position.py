"""Position encodings of a mixer's queries and keys.

A position part owns the rule. It offers it in one of two forms: ``rotation()`` returns an
:class:`llmplayer_b200.kernels.ops.Rotation` when the rule is a rotation of feature pairs by
position x frequency, which the kernels that prepare queries and keys apply on the way; a part
whose rule is anything else returns None there and implements ``apply(ctx, qkv, num_heads=,
num_kv_heads=, head_dim=)``, which changes the query and key heads of the float32 projection
``qkv`` [T, (H + 2G) * hd] (or [T, H * hd] for a layer without keys of its own) in place, reading
the tokens' positions from ``ctx.positions``; the mixer then runs its kernels without rotation.

Rotary encoding: the per-pair frequencies the kernels rotate by.

Reference: inference/RoPE.java:80-105. f_i = 1 / theta^(2i / rotary_dim) is
computed in double and rounded to float32 (:83); a per-pair divisor may follow
(:85-87), which for "llama3" scaling is what the model file's converter derives
from the wavelength rule implemented here. The angle position * f_i is a
float32 product (:101), evaluated inside the kernel that rotates.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import ConfigError
from ..kernels import ops
from .base import POSITIONS, Part, Runtime
from .specs import Llama3Scaling, PositionSpec, YarnScaling


def inverse_frequencies(spec: PositionSpec) -> torch.Tensor:
    if spec.rotary_dim <= 0 or spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
        raise ConfigError(f"rotary width {spec.rotary_dim} does not fit a head of {spec.head_dim}")
    if not spec.theta > 0:
        raise ConfigError(f"rope theta must be positive, got {spec.theta}")
    freqs = []
    s = spec.scaling
    if s is not None and not isinstance(s, (Llama3Scaling, YarnScaling)):
        raise ConfigError(f"unknown scaling of rotary frequencies: {s!r}")
    lo = hi = 0
    if isinstance(s, YarnScaling):
        if not s.factor > 0 or s.original <= 0 or not s.fast > 0 or not s.slow > 0 or spec.theta == 1.0:
            raise ConfigError(f"rotary scaling needs positive factor, original, fast and slow and a base other than 1: {s!r}")
        # the pair that makes t turns over the original context, as a (fractional) pair index
        def turn(t: float) -> float:
            return spec.rotary_dim * math.log(s.original / (2.0 * math.pi * t)) / (2.0 * math.log(spec.theta))
        lo = max(math.floor(turn(s.fast)), 0)
        hi = min(math.ceil(turn(s.slow)), spec.rotary_dim - 1)
    for i in range(spec.rotary_dim // 2):
        f = 1.0 / math.pow(spec.theta, 2.0 * i / spec.rotary_dim)
        if isinstance(s, YarnScaling):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / s.factor * ramp + f * (1.0 - ramp)
        elif s is not None:
            wavelength = 2.0 * math.pi / f
            short = s.original_max_position / s.high_freq_factor
            long = s.original_max_position / s.low_freq_factor
            if wavelength > long:
                f = f / s.factor
            elif wavelength >= short:
                blend = (s.original_max_position / wavelength - s.low_freq_factor) / (
                    s.high_freq_factor - s.low_freq_factor)
                f = (1.0 - blend) * f / s.factor + blend * f
        freqs.append(f)
    return torch.tensor(freqs, dtype=torch.float64).to(torch.float32)


def rotation_magnitude(spec: PositionSpec) -> float:
    """The factor on both cosine and sine that a scaling rule brings along (one where it brings none)."""
    if isinstance(spec.scaling, YarnScaling):
        return 0.1 * math.log(spec.scaling.factor) + 1.0
    return 1.0


class Rotary(Part):
    """Rotation of query and key pairs by position x frequency: a rule the kernels apply themselves."""
    capture_safe = True

    def __init__(self, spec: PositionSpec):
        if spec.pairing not in ("split_half", "interleaved"):
            raise ConfigError(f"unknown rotary pairing {spec.pairing!r}")
        self.spec = spec
        self._rotation: Optional[ops.Rotation] = None

    def load(self, tensors, runtime: Runtime) -> None:
        super().load(tensors, runtime)
        # layers with equal specifications share one table of frequencies (and, per step, one table of angles)
        inv_freq = runtime.shared(("rotary", self.spec), lambda: inverse_frequencies(self.spec).to(runtime.device))
        self._rotation = ops.Rotation(inv_freq, self.spec.rotary_dim, self.spec.pairing == "interleaved",
                                      rotation_magnitude(self.spec))

    def rotation(self) -> Optional[ops.Rotation]:
        return self._rotation

    def apply(self, ctx, qkv, *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        raise ConfigError("a rotary encoding is applied by the kernels that take its rotation()")


class NoPosition(Part):
    """Queries and keys are used as projected."""
    capture_safe = True

    def __init__(self, spec: PositionSpec):
        self.spec = spec

    def rotation(self) -> Optional[ops.Rotation]:
        return ops.NO_ROTATION

    def apply(self, ctx, qkv, *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        pass


POSITIONS.register("rope", Rotary)
POSITIONS.register("none", NoPosition)
