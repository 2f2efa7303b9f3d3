"""A matrix state per head updated by the gated delta rule.

Queries and keys (``num_qk_heads`` heads of ``key_dim``) and values (``num_heads`` heads of ``value_dim``) each pass a
short causal convolution per channel and silu; queries and keys are then made unit vectors per head (queries also times
key_dim^-1/2). Per head h, which reads query / key head h // (num_heads // num_qk_heads):

    b_t = sigmoid(W_b x_t)                                  g_t = exp(-exp(a_log[h]) * softplus(W_a x_t + dt_bias[h]))
    S <- g_t S;   u = b_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          (S: [key_dim, value_dim])

so the read-out sees the token's own write. Each head's o_t is divided by its root mean square, multiplied by a gain
shared by the heads and by silu(W_g x_t), and projected. State, decays, strengths, unit norms and every sum are float32.
The recurrence is one more form of the framework's linear-attention scan (csrc/linear_attention.cu): a value column's
state entries live in the registers of a few threads, and the two read-outs S^T k and S^T q of a token are taken from
the state before it in one pass of shuffles; prompts of 256 tokens or more run in chunks of 128 side by side (a
chunk's effect on the state that enters it is S -> P S + L; the first pass forms P, a [key_dim, key_dim] matrix, beside
L, the chunks' start states follow in order, the second pass writes the outputs). What a sequence carries from step to step is S and the convolutions'
last taps - 1 inputs. All kernels read the step from device tensors.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import BIAS, GAIN, MATRIX, GatedDeltaRuleSpec, TensorSpec

UNIT_EPS = 1e-6         # inside the root of the heads' unit norm: the design fixes it


class GatedDeltaRule(Part):
    capture_safe = True

    def __init__(self, spec: GatedDeltaRuleSpec):
        s = spec
        if s.num_heads <= 0 or s.num_qk_heads <= 0 or s.num_heads % s.num_qk_heads:
            raise ConfigError(f"{s.num_heads} heads cannot share {s.num_qk_heads} query / key heads")
        if s.key_dim <= 0 or s.value_dim <= 0:
            raise ConfigError(f"a delta rule with heads of {s.key_dim} x {s.value_dim}")
        if not 1 <= s.conv_taps <= 8:
            raise ConfigError(f"a convolution of {s.conv_taps} taps (supported: 1 to 8)")
        self.spec = spec
        self.qk = s.num_qk_heads * s.key_dim
        self.values = s.num_heads * s.value_dim
        self.conv_channels = 2 * self.qk + self.values
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        d, H, K = s.hidden_size, s.num_heads, s.conv_taps
        return {
            s.q: TensorSpec((self.qk, d), MATRIX), s.q_conv: TensorSpec((self.qk, K), MATRIX),
            s.k: TensorSpec((self.qk, d), MATRIX), s.k_conv: TensorSpec((self.qk, K), MATRIX),
            s.v: TensorSpec((self.values, d), MATRIX), s.v_conv: TensorSpec((self.values, K), MATRIX),
            s.strength: TensorSpec((H, d), MATRIX),
            s.a_log: TensorSpec((H,), BIAS),
            s.out_norm: TensorSpec((s.value_dim,), GAIN),
            s.decay: TensorSpec((H, d), MATRIX),
            s.dt_bias: TensorSpec((H,), BIAS),
            s.gate: TensorSpec((self.values, d), MATRIX),
            s.o: TensorSpec((d, self.values), MATRIX),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        # one product of the normed input: queries, keys, values (the convolution's channels, in this order), then the
        # write strength's and the decay's pre-activations and the output gate
        self.proj = Linear([tensors[n] for n in (s.q, s.k, s.v, s.strength, s.decay, s.gate)], runtime)
        self.taps = runtime.gain(torch.cat([tensors[n].to(torch.float32) for n in (s.q_conv, s.k_conv, s.v_conv)], dim=0))
        self.a_log = runtime.gain(tensors[s.a_log])
        self.dt_bias = runtime.gain(tensors[s.dt_bias])
        self.out_gain = runtime.gain(tensors[s.out_norm])
        self.out = Linear([tensors[s.o]], runtime)

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        s = self.spec
        return (StateRequest((s.num_heads, s.value_dim, s.key_dim), torch.float32),      # [head, value column, key channel]
                StateRequest((s.conv_taps - 1, self.conv_channels), torch.float32))

    # ------------------------------------------------------------------ step
    def buffer_to_clear(self, ctx, tokens: int):
        return self.proj.sums_into(ctx, tokens, "mixer_proj", ops.STORE)

    def forward(self, ctx, cache, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the mixer's output into ``residual`` (``overwrite``: stores it there instead)."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("a delta rule needs its per-sequence state")
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T = x.shape[0]
        H, G, dk, dv = s.num_heads, s.num_qk_heads, s.key_dim, s.value_dim
        C = self.conv_channels
        b_off, a_off, g_off = C, C + H, C + 2 * H
        proj = ctx.buffer("mixer_proj", (T, self.proj.out_features), torch.float32)
        with ops.section("recurrence.proj"):
            self.proj.store(x, proj, ctx)
        state, tail = cache.blocks
        mixed = ctx.buffer("conv_out", (T, C), torch.float32)            # [q | k | v] behind the convolutions
        with ops.section("recurrence.conv"):
            ops.short_conv(proj[:, :C], self.taps, None, tail, ctx.slots, ctx.q_start, mixed, max_new=ctx.max_new)
            ops.head_unit_norm(mixed, 0, 2 * G, dk, UNIT_EPS, float(dk) ** -0.5, scaled_heads=G)
        gates = ctx.buffer("decay_gates", (2, T, H), torch.float32)
        with ops.section("recurrence.gates"):
            ops.decay_gates(proj, a_off, self.dt_bias, self.a_log, gates[0], strength=gates[1], b_off=b_off)
        raw = ctx.buffer("recurrence_raw", (T, self.values), torch.float32)
        with ops.section("recurrence.scan"):
            ops.gla_scan(mixed, 0, self.qk, 2 * self.qk, gates[0], state, ctx.slots, ctx.q_start, raw, num_heads=H,
                         key_dim=dk, value_dim=dv, q_scale=1.0, max_new=ctx.max_new, scratch=ctx.buffer, decay_per_head=True,
                         qk_heads=G, delta_strength=gates[1])
        o = ctx.buffer("attn_out", (T, self.values), rt.act_dtype)
        with ops.section("recurrence.norm"):
            clear = residual if overwrite and residual.dtype == torch.float32 and self.out.needs_zero(T) else None
            ops.gla_finish(raw, self.out_gain, s.norm_eps, proj[:, g_off:g_off + self.values], o, num_heads=H,
                           value_dim=dv, clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("recurrence.out"):
            if overwrite:
                self.out.store(o, residual, ctx)
            else:
                self.out.accumulate(o, residual, ctx)
        return False


MIXERS.register("gated_delta_rule", GatedDeltaRule)
