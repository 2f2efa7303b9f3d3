"""A selective state space per head behind a short causal convolution (the state-space-duality form of the Mamba family).

With inner = heads * head_dim, N the state size and G groups, one product of the layer's input gives
[z: inner | x: inner | B: G N | C: G N | dt: heads]. x, B and C pass a convolution over time per channel (a few taps,
the last one on the token itself, a bias) and silu. Per head h, which reads group h // (heads // G):

    dt_t = softplus(dt_t + dt_bias[h])                      a_t = exp(-exp(a_log[h]) * dt_t)
    S_t  = a_t S_(t-1) + dt_t B_t x_t^T                     (S: [N, head_dim], float32, zero at a sequence's start)
    y_t  = S_t^T C_t + skip[h] x_t

y, the heads side by side, is multiplied by silu(z), cut into equal parts that are each divided by their own root mean
square, multiplied by a gain and projected. The recurrence is the framework's linear-attention scan
(csrc/linear_attention.cu) with B as keys and C as queries shared by the heads of a group, one decay per head and dt as
the keys' gain, so long prompts run in chunks side by side like the other recurrences. What a sequence carries from
step to step is S and the convolution's last taps - 1 inputs. All kernels read the step from device tensors.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import BIAS, GAIN, MATRIX, StateSpaceSpec, TensorSpec


class StateSpace(Part):
    capture_safe = True

    def __init__(self, spec: StateSpaceSpec):
        s = spec
        if s.num_heads <= 0 or s.head_dim <= 0 or s.state_dim <= 0:
            raise ConfigError(f"a state space with {s.num_heads} heads of {s.head_dim} over states of {s.state_dim}")
        if s.groups <= 0 or s.num_heads % s.groups:
            raise ConfigError(f"{s.num_heads} heads cannot share {s.groups} groups")
        if not 1 <= s.conv_taps <= 8:
            raise ConfigError(f"a convolution of {s.conv_taps} taps (supported: 1 to 8)")
        if s.norm_groups <= 0 or (s.num_heads * s.head_dim) % s.norm_groups:
            raise ConfigError(f"{s.num_heads * s.head_dim} values cannot be normed in {s.norm_groups} equal parts")
        self.spec = spec
        self.inner = s.num_heads * s.head_dim
        self.conv_channels = self.inner + 2 * s.groups * s.state_dim
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        H = s.num_heads
        return {
            s.in_proj: TensorSpec((2 * self.inner + 2 * s.groups * s.state_dim + H, s.hidden_size), MATRIX),
            s.conv: TensorSpec((self.conv_channels, s.conv_taps), MATRIX),
            s.conv_bias: TensorSpec((self.conv_channels,), BIAS),
            s.dt_bias: TensorSpec((H,), BIAS),
            s.a_log: TensorSpec((H,), BIAS),
            s.skip: TensorSpec((H,), GAIN),
            s.out_norm: TensorSpec((self.inner,), GAIN),
            s.o: TensorSpec((s.hidden_size, self.inner), MATRIX),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        self.proj = Linear([tensors[s.in_proj]], runtime)
        self.taps = runtime.gain(tensors[s.conv])                # the taps take part in float32
        self.conv_bias = runtime.gain(tensors[s.conv_bias])
        self.dt_bias = runtime.gain(tensors[s.dt_bias])
        self.a_log = runtime.gain(tensors[s.a_log])
        self.skip = runtime.gain(tensors[s.skip])
        self.out_gain = runtime.gain(tensors[s.out_norm])
        self.out = Linear([tensors[s.o]], runtime)

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        s = self.spec
        # the state, stored [head, value column, state channel], and the convolution's last inputs
        return (StateRequest((s.num_heads, s.head_dim, s.state_dim), torch.float32),
                StateRequest((s.conv_taps - 1, self.conv_channels), torch.float32))

    # ------------------------------------------------------------------ step
    def buffer_to_clear(self, ctx, tokens: int):
        return self.proj.sums_into(ctx, tokens, "mixer_proj", ops.STORE)

    def forward(self, ctx, cache, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the mixer's output into ``residual`` (``overwrite``: stores it there instead)."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("a state space needs its per-sequence state")
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T = x.shape[0]
        H, P, N, G = s.num_heads, s.head_dim, s.state_dim, s.groups
        inner, C = self.inner, self.conv_channels
        proj = ctx.buffer("mixer_proj", (T, self.proj.out_features), torch.float32)
        with ops.section("recurrence.proj"):
            self.proj.store(x, proj, ctx)
        state, tail = cache.blocks
        mixed = ctx.buffer("conv_out", (T, C), torch.float32)            # [x | B | C] behind the convolution
        with ops.section("recurrence.conv"):
            ops.short_conv(proj[:, inner:inner + C], self.taps, self.conv_bias, tail, ctx.slots, ctx.q_start, mixed,
                           max_new=ctx.max_new)
        gates = ctx.buffer("decay_gates", (2, T, H), torch.float32)
        with ops.section("recurrence.gates"):
            ops.decay_gates(proj, inner + C, self.dt_bias, self.a_log, gates[0], dt=gates[1])
        raw = ctx.buffer("recurrence_raw", (T, inner), torch.float32)
        with ops.section("recurrence.scan"):
            ops.gla_scan(mixed, inner + G * N, inner, 0, gates[0], state, ctx.slots, ctx.q_start, raw, num_heads=H,
                         key_dim=N, value_dim=P, q_scale=1.0, max_new=ctx.max_new, scratch=ctx.buffer,
                         decay_per_head=True, key_gain=gates[1], qk_heads=G)
        o = ctx.buffer("attn_out", (T, inner), rt.act_dtype)
        with ops.section("recurrence.norm"):
            # an output product that sums partial results wants its target zero: this kernel clears it on the side
            clear = residual if overwrite and residual.dtype == torch.float32 and self.out.needs_zero(T) else None
            ops.gated_part_norm(raw, proj[:, :inner], self.out_gain, s.norm_eps, o, num_heads=H, head_dim=P,
                                parts=s.norm_groups, values=mixed[:, :inner], skip=self.skip, clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("recurrence.out"):
            if overwrite:
                self.out.store(o, residual, ctx)
            else:
                self.out.accumulate(o, residual, ctx)
        return False


MIXERS.register("state_space", StateSpace)
