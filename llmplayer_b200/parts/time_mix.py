"""Time mixing with a matrix state per head and a token-dependent decay per key channel (the WKV recurrence of the
RWKV family, version 6).

With x' the previous token's input (zeros before a sequence's first token), each map reads its own blend

    b_s = x + (x' - x) * mu_s                                   s in r, k, v, g, w
    r, k, v = R b_r, K b_k, V b_v;   gate = silu(G b_g);   decay = exp(-exp(W2 tanh(W1 b_w) + w0))

and per head, with the bonus u for the current token,

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;    S_t = diag(decay_t) S_(t-1) + k_t v_t^T.

Each head's o_t is divided by its root mean square; the heads are multiplied by a gain over all heads' values and by
the gate, then projected. The state of a sequence is S (float32 [heads, value column, key channel]) and the last
token's input (float32 [hidden]); both start at zero. The blends are formed from the float32 stream, the decay, the
recurrence and the norm are float32.

The recurrence is the framework's gated-linear-attention scan (csrc/linear_attention.cu) with a bonus: the output of a
token is formed before the state takes the token in. All kernels read the step from device tensors (slots, offsets),
so one-token steps replay from captured graphs.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import ConfigError, WeightError
from ..kernels import ops
from .base import MIXERS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import ANY, BIAS, GAIN, MATRIX, TensorSpec, TimeMixSpec

BLENDS = ("r", "k", "v", "g", "w")


class TimeMix(Part):
    capture_safe = True
    reads_stream = True        # a block that lets its sublayers read the stream itself hands this part the float32 stream

    def __init__(self, spec: TimeMixSpec):
        s = spec
        if s.num_heads <= 0 or s.head_dim <= 0:
            raise ConfigError(f"time mixing with {s.num_heads} heads of {s.head_dim}")
        self.spec = spec
        self.maps: Dict[str, Linear] = {}
        self.out: Optional[Linear] = None
        self.decay_rank = 0

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        d, C = s.hidden_size, s.num_heads * s.head_dim
        specs = {s.mu + b: TensorSpec((d,), BIAS) for b in BLENDS}
        specs.update({
            s.r: TensorSpec((C, d), MATRIX), s.k: TensorSpec((C, d), MATRIX), s.v: TensorSpec((C, d), MATRIX),
            s.gate: TensorSpec((C, d), MATRIX), s.o: TensorSpec((d, C), MATRIX),
            s.decay_down: TensorSpec((ANY, d), MATRIX), s.decay_up: TensorSpec((C, ANY), MATRIX),
            s.decay_bias: TensorSpec((C,), BIAS), s.bonus: TensorSpec((s.num_heads, s.head_dim), BIAS),
            s.out_norm: TensorSpec((C,), GAIN),
        })
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        down, up = tensors[s.decay_down], tensors[s.decay_up]
        if down.shape[0] != up.shape[1]:
            raise WeightError(f"{s.decay_down} has {down.shape[0]} rows but {s.decay_up} has {up.shape[1]} columns")
        self.decay_rank = int(down.shape[0])
        self.mu = torch.stack([tensors[s.mu + b].to(torch.float32) for b in BLENDS]).to(runtime.device).contiguous()
        self.maps = {"r": Linear([tensors[s.r]], runtime), "k": Linear([tensors[s.k]], runtime),
                     "v": Linear([tensors[s.v]], runtime), "g": Linear([tensors[s.gate]], runtime),
                     "w": Linear([down], runtime)}
        self.decay_up = runtime.matrix(up)
        self.decay_bias = runtime.gain(tensors[s.decay_bias])
        self.bonus = runtime.gain(tensors[s.bonus])
        self.out_gain = runtime.gain(tensors[s.out_norm])
        self.out = Linear([tensors[s.o]], runtime)

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        s = self.spec
        # S stored [head, value column, key channel]; and the previous token's input
        return (StateRequest((s.num_heads, s.head_dim, s.head_dim), torch.float32),
                StateRequest((s.hidden_size,), torch.float32))

    # ------------------------------------------------------------------ step
    def forward(self, ctx, cache, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the mixer's output into ``residual`` (``overwrite``: stores it there instead). ``x``: the float32
        stream the layer reads (a block hands it over as it is: ``reads_stream``)."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("time mixing needs its per-sequence state")
        if isinstance(x, PendingNorm):
            x = x.tensor()
        if x.dtype != torch.float32:
            raise ConfigError("time mixing blends the float32 stream")
        T, d = x.shape
        H, n = s.num_heads, s.head_dim
        C = H * n
        state, last = cache.blocks
        blends = ctx.buffer("time_mix_blends", (len(BLENDS), T, d), rt.act_dtype)
        # the five maps write side by side into one float32 buffer: r | k | v | gate | decay factor (slices start
        # at multiples of 8 values). Maps that sum partial results want their slice zero: the blends' kernel clears
        # the whole buffer on the side
        width = -(-C // 8) * 8
        ld = 4 * width + -(-self.decay_rank // 8) * 8
        proj = ctx.buffer("mixer_proj", (T, ld), torch.float32)
        cleared = any(self.maps[b].needs_zero(T) for b in BLENDS)
        with ops.section("recurrence.shift"):
            ops.token_shift(x, last, self.mu, ctx.slots, ctx.q_start, ctx.seq_ids, blends, clear=proj if cleared else None)
        with ops.section("recurrence.proj"):
            for i, b in enumerate(BLENDS):
                m = self.maps[b]
                if cleared:
                    ctx.note_cleared()
                m.store(blends[i], proj[:, i * width:i * width + m.out_features], ctx)
            ctx.take_cleared()
        decay = ctx.buffer("gla_decay", (T, C), torch.float32)
        with ops.section("recurrence.decay"):
            ops.gla_decay(proj[:, 4 * width:4 * width + self.decay_rank], self.decay_up, self.decay_bias, decay,
                          double_exp=True)
        raw = ctx.buffer("gla_raw", (T, C), torch.float32)
        with ops.section("recurrence.scan"):
            ops.gla_scan(proj, 0, width, 2 * width, decay, state, ctx.slots, ctx.q_start, raw, num_heads=H, key_dim=n,
                         value_dim=n, q_scale=1.0, max_new=ctx.max_new, scratch=ctx.buffer, bonus=self.bonus)
        o = ctx.buffer("attn_out", (T, C), rt.act_dtype)
        with ops.section("recurrence.norm"):
            clear = residual if overwrite and residual.dtype == torch.float32 and self.out.needs_zero(T) else None
            ops.gla_finish(raw, self.out_gain, s.norm_eps, proj[:, 3 * width:3 * width + C], o, num_heads=H, value_dim=n,
                           gain_per_head=True, clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("recurrence.out"):
            if overwrite:
                self.out.store(o, residual, ctx)
            else:
                self.out.accumulate(o, residual, ctx)
        return False


MIXERS.register("time_mix", TimeMix)
