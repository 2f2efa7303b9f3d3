"""Two mixers side by side: both read the same input, and the layer's result is
left_scale * left(x) + right_scale * right(x) with two constants.

Each member is any registered mixer and keeps what it keeps (pages of keys and values, a recurrent state, ...); the pair
asks the cache for both (a :class:`BundleRequest`) and hands each member its own view. A member stores its result in a
float32 buffer (or adds it into a zeroed one, if it can only add); one kernel then adds both, times their constants,
into the stream. A member that leaves its output map's additive vector to the caller (``bias_later``) has it added in
that kernel too.
"""
from __future__ import annotations

import inspect
from typing import Dict, Mapping

import torch

from ..cache.sequence_cache import BundleRequest
from ..kernels import ops
from .base import MIXERS, Part, PendingNorm, Runtime
from .specs import MixerPairSpec, TensorSpec


class MixerPair(Part):
    def __init__(self, spec: MixerPairSpec):
        self.spec = spec
        self.left = MIXERS.build(spec.left)
        self.right = MIXERS.build(spec.right)
        self._args = [inspect.signature(m.forward).parameters for m in (self.left, self.right)]

    def children(self):
        return (self.left, self.right)

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(m, "capture_safe", False)) for m in self.children())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for m in self.children():
            out.update(m.tensor_specs())
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        for m in self.children():
            m.load(tensors, runtime)

    def cache_request(self):
        return BundleRequest((self.left.cache_request(), self.right.cache_request()))

    def buffer_to_clear(self, ctx, tokens: int):
        ask = getattr(self.left, "buffer_to_clear", None)
        return ask(ctx, tokens) if ask is not None else None

    def _run(self, member, args, ctx, view, x, width: int, name: str, prefix: str):
        """Run a member into a float32 buffer of its own; returns (buffer, the vector it left to the caller or None)."""
        y = ctx.buffer(name, (x.shape[0], width), torch.float32)
        kwargs = {}
        if "overwrite" in args:
            kwargs["overwrite"] = True
        else:
            y.zero_()
        later = "bias_later" in args and "overwrite" in args and getattr(member, "output_bias", None) is not None
        if later:
            kwargs["bias_later"] = True
        with ops.section_prefix(prefix):
            member.forward(ctx, view, x, y, **kwargs)
        return y, (member.output_bias if later else None)

    def forward(self, ctx, cache, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the pair's result into ``residual`` (``overwrite``: the stream is set to zero first)."""
        if isinstance(x, PendingNorm):
            x = x.tensor()
        width = residual.shape[1]
        views = cache.members if cache is not None else (None, None)
        if overwrite:
            residual.zero_()
        a, a_vec = self._run(self.left, self._args[0], ctx, views[0], x, width, "pair_left", "left.")
        b, b_vec = self._run(self.right, self._args[1], ctx, views[1], x, width, "pair_right", "right.")
        with ops.section("mixer.sum"):
            ops.scaled_sum(residual, a, self.spec.left_scale, b, self.spec.right_scale, a_vector=a_vec, b_vector=b_vec)
        return False


MIXERS.register("mixer_pair", MixerPair)
