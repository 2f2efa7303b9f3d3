"""Dense gated feed-forward: residual += down(silu(gate x) * (up x)).

Gate and up are held as one stacked matrix so that one product yields both and
the activation is applied where the sums are formed.

Reference: inference/SwiGLUFFN.java:36-67, tensor/ScalarOps.java:69-73,
src/main/resources/kernels/cuda/silu_mul.cu:6-15.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..errors import ConfigError
from .base import FEED_FORWARDS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import BIAS, MATRIX, GatedDenseSpec, MixtureSpec, SquaredReLUSpec, SwiGLUSpec, TensorSpec, XIELUSpec


class SwiGLU(Part):
    capture_safe = True
    def __init__(self, spec: SwiGLUSpec):
        self.spec = spec
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        return {
            s.gate: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
            s.up: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
            s.down: TensorSpec((s.hidden_size, s.intermediate_size), MATRIX),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        self.gate_up = Linear([tensors[s.gate], tensors[s.up]], runtime, gated=True)
        self.down = Linear([tensors[s.down]], runtime)

    takes_pending_norm = True     # the gated product applies the norm of its input itself when a step is small

    def forward(self, ctx, x, residual: torch.Tensor, then_norm=None) -> bool:
        """Adds the feed-forward's output into ``residual``; returns whether ``then_norm`` was fused.
        ``x``: the normed stream, or a :class:`PendingNorm` of it."""
        from ..kernels import ops
        if isinstance(x, PendingNorm):
            T = residual.shape[0]
            if (self.runtime.fast and x.fusable and residual.dtype == torch.float32
                    and self.gate_up.can_few(T, ops.SWIGLU) and self.down.can_few(T, ops.ACCUMULATE)):
                h = ctx.buffer("ffn_hidden", (T, self.spec.intermediate_size), torch.bfloat16)
                with ops.section("ffn.gate_up"):
                    self.gate_up.few(x.source, h, ops.SWIGLU, norm=x.norm)
                with ops.section("ffn.down"):
                    self.down.few(h, residual, ops.ACCUMULATE)
                return False
            x = x.tensor()
        h = ctx.buffer("ffn_hidden", (x.shape[0], self.spec.intermediate_size), self.runtime.act_dtype)
        with ops.section("ffn.gate_up"):
            self.gate_up.swiglu(x, h, ctx)
        with ops.section("ffn.down"):
            return self.down.accumulate(h, residual, ctx, then_norm)


FEED_FORWARDS.register("swiglu", SwiGLU)


class GatedDense(Part):
    """down(act(gate x + b_g) * (up x + b_u)) + b_d with the tanh form of GELU (or silu) as the activation. Gate and up
    are one stacked product with float32 sums; the additive vectors and the activation are applied to those sums in
    float32 by one kernel. ``output_bias`` is what the down projection adds: a block that norms the result may add it
    in the kernel that reads the result (``bias_later``)."""
    capture_safe = True

    def __init__(self, spec: GatedDenseSpec):
        if spec.activation not in ("gelu_tanh", "silu"):
            raise ConfigError(f"unknown activation {spec.activation!r} of a gated feed-forward")
        if spec.intermediate_size <= 0:
            raise ConfigError(f"a feed-forward of {spec.intermediate_size} hidden values")
        self.spec = spec
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.bias: Optional[torch.Tensor] = None
        self.output_bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        out = {s.gate: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
               s.up: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
               s.down: TensorSpec((s.hidden_size, s.intermediate_size), MATRIX)}
        for name, size in ((s.gate_bias, s.intermediate_size), (s.up_bias, s.intermediate_size), (s.down_bias, s.hidden_size)):
            if name is not None:
                out[name] = TensorSpec((size,), BIAS)
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        self.gate_up = Linear([tensors[s.gate], tensors[s.up]], runtime)       # rows: gate, then up
        self.down = Linear([tensors[s.down]], runtime)
        if s.gate_bias is not None or s.up_bias is not None:
            self.bias = torch.cat([tensors[n].to(torch.float32) if n is not None else torch.zeros(s.intermediate_size)
                                   for n in (s.gate_bias, s.up_bias)]).to(runtime.device).contiguous()
        self.output_bias = runtime.gain(tensors[s.down_bias]) if s.down_bias is not None else None

    def buffer_to_clear(self, ctx, tokens: int):
        from ..kernels import ops
        return self.gate_up.sums_into(ctx, tokens, "ffn_up", ops.STORE)

    def forward(self, ctx, x, residual: torch.Tensor, overwrite: bool = False, bias_later: bool = False) -> bool:
        """Adds the feed-forward's output into ``residual`` (``overwrite``: stores it there instead; with
        ``bias_later`` the caller then adds ``output_bias`` itself)."""
        from ..kernels import ops
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T, F = x.shape[0], self.spec.intermediate_size
        z = ctx.buffer("ffn_up", (T, 2 * F), torch.float32)
        with ops.section("ffn.gate_up"):
            self.gate_up.store(x, z, ctx)
        h = ctx.buffer("ffn_hidden", (T, F), self.runtime.act_dtype)
        with ops.section("ffn.act"):
            clear = residual if overwrite and residual.dtype == torch.float32 and self.down.needs_zero(T) else None
            ops.gated_act(z, self.bias, h, self.spec.activation, clear=clear)
        with ops.section("ffn.down"):
            if clear is not None:
                ctx.note_cleared()
            if overwrite:
                self.down.store(h, residual, ctx)
            else:
                self.down.accumulate(h, residual, ctx)
            if self.output_bias is not None and not (overwrite and bias_later):
                ops.stream_add(residual, None, self.output_bias)
        return False


FEED_FORWARDS.register("gated_dense", GatedDense)


class XIELUFeedForward(Part):
    """down(act(up x)) with act(z) = softplus(p) z^2 + z / 2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
    otherwise; p and q are the layer's tensor ``act``. The activation is evaluated in float32 on the float32
    sums of the up projection.

    A block that projects its normed input for several consumers at once may take this part's ``up`` matrix
    into that product (:meth:`up_matrix`) and hand the sums to :meth:`forward_from_up`."""
    capture_safe = True

    def __init__(self, spec: XIELUSpec):
        self.spec = spec
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.numbers: Optional[torch.Tensor] = None
        self._up_host = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        return {
            s.up: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
            s.down: TensorSpec((s.hidden_size, s.intermediate_size), MATRIX),
            s.act: TensorSpec((2,), BIAS),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        self._up_host = tensors[s.up]
        self.down = Linear([tensors[s.down]], runtime)
        self.numbers = runtime.gain(tensors[s.act])

    def up_matrix(self):
        """The host tensor of the up projection, for a block that stacks it into a wider product."""
        return self._up_host

    def _own_up(self) -> Linear:
        if self.up is None:
            self.up = Linear([self._up_host], self.runtime)
        return self.up

    def forward_from_up(self, ctx, z: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``z``: the float32 sums up x [T, F] (may be a column slice); writes down(act(z)) to ``out`` float32 [T, d]."""
        from ..kernels import ops
        h = ctx.buffer("ffn_hidden", (z.shape[0], self.spec.intermediate_size), self.runtime.act_dtype)
        # a down product that sums partial results into `out` wants it zero: the activation clears it on the side
        clear = self.down.sums_into(ctx, z.shape[0], "ffn_out", ops.STORE)
        if clear is not None and clear.data_ptr() != out.data_ptr():
            clear = None
        with ops.section("ffn.act"):
            ops.xielu(z, self.numbers, h, clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("ffn.down"):
            self.down.store(h, out, ctx)
        return out

    def forward(self, ctx, x, residual: torch.Tensor) -> bool:
        from ..kernels import ops
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T = x.shape[0]
        z = ctx.buffer("ffn_up", (T, self.spec.intermediate_size), torch.float32)
        with ops.section("ffn.up"):
            self._own_up().store(x, z, ctx)
        out = ctx.buffer("ffn_out", tuple(residual.shape), torch.float32)
        self.forward_from_up(ctx, z, out)
        with ops.section("ffn.add"):
            ops.gated_sum(residual, out)
        return False


FEED_FORWARDS.register("xielu", XIELUFeedForward)


class SquaredReLU(Part):
    """down(relu(up x)^2); the activation is evaluated in float32 on the float32 sums of the up projection."""
    capture_safe = True

    def __init__(self, spec: SquaredReLUSpec):
        self.spec = spec
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        return {s.up: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
                s.down: TensorSpec((s.hidden_size, s.intermediate_size), MATRIX)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        self.up = Linear([tensors[self.spec.up]], runtime)
        self.down = Linear([tensors[self.spec.down]], runtime)

    def buffer_to_clear(self, ctx, tokens: int):
        from ..kernels import ops
        return self.up.sums_into(ctx, tokens, "ffn_up", ops.STORE)

    def forward(self, ctx, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the feed-forward's output into ``residual`` (``overwrite``: stores it there instead)."""
        from ..kernels import ops
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T, F = x.shape[0], self.spec.intermediate_size
        z = ctx.buffer("ffn_up", (T, F), torch.float32)
        with ops.section("ffn.up"):
            self.up.store(x, z, ctx)
        h = ctx.buffer("ffn_hidden", (T, F), self.runtime.act_dtype)
        with ops.section("ffn.act"):
            clear = residual if overwrite and residual.dtype == torch.float32 and self.down.needs_zero(T) else None
            ops.relu2(z, h, clear=clear)
        with ops.section("ffn.down"):
            if clear is not None:
                ctx.note_cleared()
            if overwrite:
                self.down.store(h, residual, ctx)
            else:
                self.down.accumulate(h, residual, ctx)
        return False


FEED_FORWARDS.register("squared_relu", SquaredReLU)


class Mixture(Part):
    """Mixture of gated experts. The router's logits are a product with float32 sums; the routing kernel turns them
    into one weight per token and expert (zero where the token did not choose the expert). The experts run as ONE
    stacked gated product over all of them (gate and up matrices of every expert, and of the shared expert, stacked
    by rows), whose hidden activations are multiplied by the token's weight for their expert, and ONE down product
    over the experts' down matrices stacked by columns, which sums the weighted outputs: every token passes through
    every expert, so the cost does not depend on the routing and the step has no host-side decisions (it replays
    from a captured graph); what a token did not choose is multiplied by zero."""
    capture_safe = True

    def __init__(self, spec: MixtureSpec):
        s, r = spec, spec.routing
        if r.scoring not in ("sigmoid_groups", "softmax_top", "softmax_groups"):
            raise ConfigError(f"unknown scoring {r.scoring!r} of a router")
        if r.scoring != "softmax_groups" and (r.correction is not None or r.identity_experts or r.weight_scale != 1.0):
            raise ConfigError("a correction of the choice, identity experts and a constant on the weights belong to "
                              "scoring 'softmax_groups'")
        if r.identity_experts < 0:
            raise ConfigError(f"{r.identity_experts} identity experts")
        if r.scoring == "softmax_groups" and (s.shared_size > 0 or s.activation != "silu"):
            raise ConfigError("scoring 'softmax_groups' comes with silu experts and without a shared expert")
        if s.activation not in ("silu", "clamped"):
            raise ConfigError(f"unknown activation {s.activation!r} of the experts")
        if s.activation == "clamped" and (not s.limit > 0 or (s.shared_size > 0 and not s.shared_limit > 0)):
            raise ConfigError(f"clamped experts need positive limits, got {s.limit} and {s.shared_limit}")
        if r.scoring == "softmax_top" and (r.groups != 1 or r.keep_groups != 1):
            raise ConfigError("a router that takes the largest logits has no groups")
        if r.router_bias is not None and r.scoring != "softmax_top":
            raise ConfigError("only a router that takes the largest logits adds a bias to them")
        if s.activation == "clamped" and s.shared_size > 0 and s.shared_gate is None:
            raise ConfigError("the shared expert of clamped experts comes with its gate")
        if s.shared_gate is not None and (s.shared_size <= 0 or r.scoring != "softmax_top" or s.activation != "clamped"):
            raise ConfigError("a gate of the shared expert belongs to clamped experts chosen by their largest logits")
        outputs = r.num_experts + r.identity_experts          # groups are formed over experts and identity experts together
        if r.num_experts <= 0 or r.groups <= 0 or outputs % r.groups:
            raise ConfigError(f"{outputs} experts cannot form {r.groups} equal groups")
        if not 0 < r.keep_groups <= r.groups:
            raise ConfigError(f"{r.keep_groups} of {r.groups} groups kept")
        if not 0 < r.top <= r.keep_groups * (outputs // r.groups):
            raise ConfigError(f"{r.top} experts cannot be chosen from {r.keep_groups} groups of {outputs // r.groups}")
        if s.expert_size <= 0 or s.shared_size < 0 or (s.shared_size > 0 and not s.shared_prefix):
            raise ConfigError(f"experts of {s.expert_size}, a shared expert of {s.shared_size}")
        self.spec = spec
        self.router: Optional[Linear] = None
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def _experts(self):
        s = self.spec
        names = [(f"{s.expert_prefix}e{e}.", s.expert_size) for e in range(s.routing.num_experts)]
        if s.shared_size > 0:
            names.append((s.shared_prefix, s.shared_size))
        return names

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        out: Dict[str, TensorSpec] = {}
        for prefix, size in self._experts():
            out[prefix + "gate"] = TensorSpec((size, s.hidden_size), MATRIX)
            out[prefix + "up"] = TensorSpec((size, s.hidden_size), MATRIX)
            out[prefix + "down"] = TensorSpec((s.hidden_size, size), MATRIX)
        out[s.routing.router] = TensorSpec((s.routing.num_experts + s.routing.identity_experts, s.hidden_size), MATRIX)
        if s.routing.correction is not None:
            out[s.routing.correction] = TensorSpec((s.routing.num_experts + s.routing.identity_experts,), BIAS)
        if s.routing.router_bias is not None:
            out[s.routing.router_bias] = TensorSpec((s.routing.num_experts,), BIAS)
        if s.shared_gate is not None:
            out[s.shared_gate] = TensorSpec((1, s.hidden_size), MATRIX)
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        experts = self._experts()
        gate = torch.cat([tensors[p + "gate"] for p, _ in experts], dim=0)
        up = torch.cat([tensors[p + "up"] for p, _ in experts], dim=0)
        down = torch.cat([tensors[p + "down"] for p, _ in experts], dim=1).contiguous()
        self.total = gate.shape[0]
        # the shared expert's gate is one more row of the router's product
        self.router = Linear([tensors[s.routing.router]] + ([tensors[s.shared_gate]] if s.shared_gate is not None else []),
                             runtime)
        self.router_bias = runtime.gain(tensors[s.routing.router_bias]) if s.routing.router_bias is not None else None
        self.correction = runtime.gain(tensors[s.routing.correction]) if s.routing.correction is not None else None
        # silu experts: the gated product applies the activation itself; clamped ones: float32 sums, then a kernel
        self.gate_up = Linear([gate, up], runtime, gated=s.activation == "silu")
        self.down = Linear([down], runtime)

    def buffer_to_clear(self, ctx, tokens: int):
        from ..kernels import ops
        return self.router.sums_into(ctx, tokens, "router_logits", ops.STORE)

    def forward(self, ctx, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the mixture's output into ``residual`` (``overwrite``: stores it there instead)."""
        from ..kernels import ops
        s, r = self.spec, self.spec.routing
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T = x.shape[0]
        columns = self.router.out_features              # the experts' logits (and the shared expert's gate)
        logits = ctx.buffer("router_logits", (T, columns), torch.float32)
        with ops.section("ffn.router"):
            self.router.store(x, logits, ctx)
            weights = ctx.buffer("router_weights", (T, columns), torch.float32)
            if r.scoring == "softmax_top":
                ops.route_top(logits, self.router_bias, weights, num_experts=r.num_experts, top=r.top)
            elif r.scoring == "softmax_groups":
                ops.route_softmax(logits, self.correction, weights, groups=r.groups, keep=r.keep_groups, top=r.top,
                                  scale=r.weight_scale)
            else:
                ops.route(logits, weights, groups=r.groups, keep=r.keep_groups, top=r.top)
        h = ctx.buffer("ffn_hidden", (T, self.total), self.runtime.act_dtype)
        clear = residual if overwrite and residual.dtype == torch.float32 and self.down.needs_zero(T) else None
        rides = False
        if s.activation == "clamped":
            z = ctx.buffer("ffn_up", (T, 2 * self.total), torch.float32)
            with ops.section("ffn.gate_up"):
                self.gate_up.store(x, z, ctx)
            with ops.section("ffn.weights"):
                ops.expert_act(z, weights, h, num_experts=r.num_experts, expert_size=s.expert_size, limit=s.limit,
                               limit_rest=s.shared_limit, clear=clear)
        else:
            with ops.section("ffn.gate_up"):
                self.gate_up.swiglu(x, h, ctx)
            # experts that are the identity (the feed-forward's input itself, times the token's weights for them) ride
            # along in the same launch when the experts' outputs are added to the stream afterwards
            rides = r.identity_experts > 0 and not overwrite and residual.dtype == torch.float32
            with ops.section("ffn.weights"):
                ops.expert_scale(h, weights, s.expert_size, clear=clear, num_experts=r.num_experts,
                                 identity=(residual, x, r.num_experts, r.identity_experts) if rides else None)
        with ops.section("ffn.down"):
            if clear is not None:
                ctx.note_cleared()
            if overwrite:
                self.down.store(h, residual, ctx)
            else:
                self.down.accumulate(h, residual, ctx)
        if r.identity_experts and not rides:
            # (a step that stores the experts' outputs adds the identities' share behind them)
            with ops.section("ffn.identity"):
                ops.identity_experts(residual, x, weights, r.num_experts, r.identity_experts)
        return False


FEED_FORWARDS.register("mixture", Mixture)
