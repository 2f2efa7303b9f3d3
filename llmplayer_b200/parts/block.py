"""One layer: the arrangement of its norms, its mixer and its feed-forward.

``parallel``: x += gate * mixer(norm(x)) + gate * feed_forward(norm(x)) from one norm, optionally followed by a
weighted sum over the results of all layers so far (:class:`ParallelBlock`).

``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream
x in float32 (inference/TransformerBlock.java:73-78, :109, :116-122, :149).
"""
from __future__ import annotations

import inspect
from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, FollowingNorm, Part, PendingNorm, Runtime
from ..errors import ConfigError
from .linear import Linear
from .specs import BIAS, GAIN, MATRIX, BlockSpec, ParallelBlockSpec, PostNormBlockSpec, SandwichBlockSpec, TensorSpec


class PreNormBlock(Part):
    def __init__(self, spec: BlockSpec):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        if (spec.ffn is None) != (spec.ffn_norm is None):
            raise ConfigError("a feed-forward comes with the norm in front of it, or not at all")
        self.ffn_norm = NORMS.build(spec.ffn_norm) if spec.ffn is not None else None
        self.ffn = FEED_FORWARDS.build(spec.ffn) if spec.ffn is not None else None
        # parts may offer to write the norm that follows them (a `then_norm` argument of forward)
        self._mixer_fuses = self.ffn is not None and "then_norm" in inspect.signature(self.mixer.forward).parameters
        self._ffn_fuses = self.ffn is not None and "then_norm" in inspect.signature(self.ffn.forward).parameters

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self.children())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.children():
            out.update(part.tensor_specs())
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        for part in self.children():
            part.load(tensors, runtime)

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, ctx, cache, residual: torch.Tensor, normed_ready: bool = False, next_block=None) -> bool:
        """Run the layer on the residual stream in place.

        ``normed_ready``: the previous block already left ``norm(residual)`` of this block's first
        norm in the shared "normed" buffer. ``next_block``: the block that runs next, so that this
        block's last product can write that block's first norm on the way. Returns whether it did.
        """
        act = self.runtime.act_dtype
        tokens = residual.shape[0]
        h = ctx.buffer("normed", tuple(residual.shape), act)

        def pending(norm, consumer):
            def run():
                self._norm(ctx, norm, consumer, residual, h)
                return h
            return PendingNorm(residual, norm, run)

        # a part that takes a pending norm gets (stream, norm) and may apply the norm in its first product
        mixer_pends = bool(getattr(self.mixer, "takes_pending_norm", False))
        ffn_pends = bool(getattr(self.ffn, "takes_pending_norm", False))
        if normed_ready:
            mixer_in = h
        elif mixer_pends:
            mixer_in = pending(self.mixer_norm, self.mixer)
        else:
            self._norm(ctx, self.mixer_norm, self.mixer, residual, h)
            mixer_in = h
        if self.ffn is None:                 # a layer without a feed-forward
            self.mixer.forward(ctx, cache, mixer_in, residual)
            return False
        fused = False
        if self._mixer_fuses and not ffn_pends:
            follow = FollowingNorm(self.ffn_norm, h, self._clear_for(ctx, self.ffn, tokens))
            fused = bool(self.mixer.forward(ctx, cache, mixer_in, residual, then_norm=follow))
            if fused and follow.clear is not None:
                ctx.note_cleared()
        else:
            self.mixer.forward(ctx, cache, mixer_in, residual)
        if fused:
            ffn_in = h
        elif ffn_pends:
            ffn_in = pending(self.ffn_norm, self.ffn)
        else:
            self._norm(ctx, self.ffn_norm, self.ffn, residual, h)
            ffn_in = h
        nxt = getattr(next_block, "mixer_norm", None)
        next_pends = bool(getattr(getattr(next_block, "mixer", None), "takes_pending_norm", False))
        if self._ffn_fuses and nxt is not None and getattr(next_block, "kind_prenorm", False) and not next_pends:
            follow = FollowingNorm(nxt, h, self._clear_for(ctx, next_block.mixer, tokens))
            done = bool(self.ffn.forward(ctx, ffn_in, residual, then_norm=follow))
            if done and follow.clear is not None:
                ctx.note_cleared()
            return done
        self.ffn.forward(ctx, ffn_in, residual)
        return False

    kind_prenorm = True

    @staticmethod
    def _clear_for(ctx, consumer, tokens):
        ask = getattr(consumer, "buffer_to_clear", None)
        return ask(ctx, tokens) if ask is not None else None

    @staticmethod
    def _norm(ctx, norm, consumer, residual, h) -> None:
        """Norm the residual stream for ``consumer``; if the consumer's first product wants a
        zeroed buffer (``buffer_to_clear(ctx, tokens)``), the norm clears it on the side."""
        clear = PreNormBlock._clear_for(ctx, consumer, residual.shape[0])
        with ops.section("norm"):
            if clear is not None:
                norm.apply(residual, h, clear=clear)
                ctx.note_cleared()
            else:
                norm.apply(residual, h)


class ParallelBlock(Part):
    """x <- x + gate_m * mixer(h) + gate_f * ffn(h) with h = norm(x): one norm, both sublayers read its output.
    Each gate (optional) is sigmoid(W h + b) per feature. With a depth mix, the layer's result X is kept and the
    stream that goes on is sum_j w[j] X_j over the embedding's output X_0 and every layer's result so far.

    Everything that multiplies h (the mixer's input projections if it offers them, the gates, the feed-forward's
    up projection) is stacked into one matrix, so a layer forms all of them in one product with float32 sums;
    gates, residual sum and depth mix are one kernel at the end. A mixer or feed-forward without those hooks
    is run through its ordinary ``forward`` into a zeroed buffer."""

    def __init__(self, spec: ParallelBlockSpec):
        self.spec = spec
        self.norm = NORMS.build(spec.norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.ffn = FEED_FORWARDS.build(spec.ffn) if spec.ffn is not None else None
        if spec.ffn_gate is not None and spec.ffn is None:
            raise ConfigError("a gate for a feed-forward that the layer does not have")
        if spec.depth_mix is not None and not 2 <= spec.depth_mix.count <= spec.depth_mix.total:
            raise ConfigError(f"a depth mix over {spec.depth_mix.count} of {spec.depth_mix.total} streams")
        self.proj: Optional[Linear] = None

    def children(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn) if p is not None)

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self.children())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        d = s.norm.size
        out: Dict[str, TensorSpec] = {}
        out.update(self.norm.tensor_specs())
        out.update(self.mixer.tensor_specs())
        if self.ffn is not None:
            out.update(self.ffn.tensor_specs())
        for gate in (s.mixer_gate, s.ffn_gate):
            if gate is not None:
                out[gate.weight] = TensorSpec((d, d), MATRIX)
                out[gate.bias] = TensorSpec((d,), BIAS)
        if s.depth_mix is not None:
            out[s.depth_mix.weights] = TensorSpec((s.depth_mix.count,), BIAS)
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        for part in self.children():
            part.load(tensors, runtime)
        stacked, at = [], 0
        self._mixer_at = self._mixer_gate_at = self._ffn_gate_at = self._up_at = None
        if hasattr(self.mixer, "input_projections"):
            self._mixer_at = at
            for m in self.mixer.input_projections():
                stacked.append(m)
                at += m.shape[0]
        self.mixer_gate_bias = self.ffn_gate_bias = None
        if s.mixer_gate is not None:
            self._mixer_gate_at, at = at, at + tensors[s.mixer_gate.weight].shape[0]
            stacked.append(tensors[s.mixer_gate.weight])
            self.mixer_gate_bias = runtime.gain(tensors[s.mixer_gate.bias])
        if s.ffn_gate is not None:
            self._ffn_gate_at, at = at, at + tensors[s.ffn_gate.weight].shape[0]
            stacked.append(tensors[s.ffn_gate.weight])
            self.ffn_gate_bias = runtime.gain(tensors[s.ffn_gate.bias])
        if self.ffn is not None and hasattr(self.ffn, "up_matrix"):
            self._up_at, at = at, at + self.ffn.up_matrix().shape[0]
            stacked.append(self.ffn.up_matrix())
        self.proj = Linear(stacked, runtime) if stacked else None
        self.depth_weights = runtime.gain(tensors[s.depth_mix.weights]) if s.depth_mix is not None else None

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, ctx, cache, residual: torch.Tensor) -> bool:
        s, act = self.spec, self.runtime.act_dtype
        T, d = residual.shape
        h = ctx.buffer("normed", (T, d), act)
        with ops.section("norm"):
            self.norm.apply(residual, h)
        proj = None
        if self.proj is not None:
            proj = ctx.buffer("layer_proj", (T, self.proj.out_features), torch.float32)
            with ops.section("layer.proj"):
                self.proj.store(h, proj, ctx)
        m = ctx.buffer("mixer_out", (T, d), torch.float32)
        if self._mixer_at is not None:
            self.mixer.forward_projected(ctx, cache, proj, self._mixer_at, m)
        else:
            m.zero_()
            self.mixer.forward(ctx, cache, h, m)
        f = None
        if self.ffn is not None:
            f = ctx.buffer("ffn_out", (T, d), torch.float32)
            if self._up_at is not None:
                width = self.ffn.up_matrix().shape[0]
                self.ffn.forward_from_up(ctx, proj[:, self._up_at:self._up_at + width], f)
            else:
                f.zero_()
                self.ffn.forward(ctx, h, f)
        m_gate = f_gate = None
        if self._mixer_gate_at is not None:
            m_gate = (proj[:, self._mixer_gate_at:self._mixer_gate_at + d], self.mixer_gate_bias)
        if self._ffn_gate_at is not None:
            f_gate = (proj[:, self._ffn_gate_at:self._ffn_gate_at + d], self.ffn_gate_bias)
        with ops.section("layer.sum"):
            if s.depth_mix is not None:
                streams = ctx.buffer("depth_streams", (s.depth_mix.total, T, d), torch.float32)
                ops.gated_sum(residual, m, m_gate, f, f_gate, streams=streams, mix=self.depth_weights,
                              count=s.depth_mix.count, keep_input=s.depth_mix.count == 2)
            else:
                ops.gated_sum(residual, m, m_gate, f, f_gate)
        return False


class SandwichBlock(Part):
    """x += post_norm(mixer(norm(x))); x += post_norm(ffn(norm(x))): a norm in front of and behind each sublayer.
    A sublayer stores its result in a float32 buffer (or adds it into the zeroed buffer, if it can only add); one kernel then norms that result, adds it into the
    stream and, when a further sublayer of this layer follows, writes that sublayer's input norm in the same pass.
    The norms are RMS norms (the kernel's rule); the feed-forward may be absent."""

    def __init__(self, spec: SandwichBlockSpec):
        self.spec = spec
        if (spec.ffn is None) != (spec.ffn_norm is None) or (spec.ffn is None) != (spec.post_ffn_norm is None):
            raise ConfigError("a feed-forward comes with the norms in front of and behind it, or not at all")
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.post_mixer_norm = NORMS.build(spec.post_mixer_norm)
        self.ffn_norm = NORMS.build(spec.ffn_norm) if spec.ffn is not None else None
        self.ffn = FEED_FORWARDS.build(spec.ffn) if spec.ffn is not None else None
        self.post_ffn_norm = NORMS.build(spec.post_ffn_norm) if spec.ffn is not None else None
        for norm in (self.mixer_norm, self.post_mixer_norm, self.ffn_norm, self.post_ffn_norm):
            if norm is not None and not getattr(norm, "fusable_rms", False):
                raise ConfigError("the norms of a sandwich block are RMS norms")
        # a part whose forward takes `overwrite` stores its result; any other adds it into a buffer zeroed first
        self._mixer_stores = "overwrite" in inspect.signature(self.mixer.forward).parameters
        self._ffn_stores = self.ffn is not None and "overwrite" in inspect.signature(self.ffn.forward).parameters

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.post_mixer_norm, self.ffn_norm, self.ffn,
                                 self.post_ffn_norm) if p is not None)

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self.children())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.children():
            out.update(part.tensor_specs())
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        for part in self.children():
            part.load(tensors, runtime)

    def cache_request(self):
        return self.mixer.cache_request()

    kind_sandwich = True

    def forward(self, ctx, cache, residual: torch.Tensor, normed_ready: bool = False, next_block=None) -> bool:
        """Run the layer on the residual stream in place. ``normed_ready``: the previous block already left this
        block's first norm of the stream in the shared "normed" buffer. ``next_block``: the block that runs next on
        the stream as this one leaves it; if it is of this kind, the kernel that adds this layer's last result also
        writes that block's first norm. Returns whether it did. A norm kernel also clears, on the side, the buffer
        that the product after it sums partial results into (``buffer_to_clear`` of the part that follows)."""
        act = self.runtime.act_dtype
        T = residual.shape[0]
        h = ctx.buffer("normed", tuple(residual.shape), act)
        y = ctx.buffer("sublayer_out", tuple(residual.shape), torch.float32)
        if not normed_ready:
            PreNormBlock._norm(ctx, self.mixer_norm, self.mixer, residual, h)
        if self._mixer_stores:
            self.mixer.forward(ctx, cache, h, y, overwrite=True)
        else:
            y.zero_()
            self.mixer.forward(ctx, cache, h, y)
        follower = next_block if getattr(next_block, "kind_sandwich", False) else None

        def add_normed(post, next_norm, consumer) -> bool:
            with ops.section("norm"):
                if next_norm is None:
                    ops.post_norm_add(y, post.weight, post.spec.eps, residual)
                    return False
                clear = PreNormBlock._clear_for(ctx, consumer, T)
                ops.post_norm_add(y, post.weight, post.spec.eps, residual, next_weight=next_norm.weight,
                                  next_eps=next_norm.spec.eps, next_out=h, clear=clear)
                if clear is not None:
                    ctx.note_cleared()
                return True

        if self.ffn is None:
            return add_normed(self.post_mixer_norm, follower.mixer_norm if follower else None, follower.mixer if follower else None)
        add_normed(self.post_mixer_norm, self.ffn_norm, self.ffn)
        if self._ffn_stores:
            self.ffn.forward(ctx, h, y, overwrite=True)
        else:
            y.zero_()
            self.ffn.forward(ctx, h, y)
        return add_normed(self.post_ffn_norm, follower.mixer_norm if follower else None, follower.mixer if follower else None)


class PostNormBlock(Part):
    """x += scale_m * norm_m(mixer(x)); x += scale_f * norm_f(ffn(x)): the sublayers read the stream itself, and each
    result is RMS-normed (and multiplied by a per-feature layer scale, if the layer has one) before it is added.

    A sublayer stores its result in a float32 buffer; ONE kernel then adds the additive vector of the sublayer's last
    map (if the sublayer left it to the block: ``bias_later``), norms, scales, adds into the stream and writes the new
    stream in the number format of the next sublayer's products (bfloat16 models; a float32 model's sublayers read the
    stream in place). A sublayer with ``reads_stream`` (one that blends neighbouring tokens in float32, say) is handed
    the float32 stream as it is. The feed-forward may be absent."""

    def __init__(self, spec: PostNormBlockSpec):
        self.spec = spec
        if (spec.ffn is None) != (spec.post_ffn_norm is None) or (spec.ffn is None and spec.ffn_scale is not None):
            raise ConfigError("a feed-forward comes with the norm behind it, or not at all")
        self.mixer = MIXERS.build(spec.mixer)
        self.post_mixer_norm = NORMS.build(spec.post_mixer_norm)
        self.ffn = FEED_FORWARDS.build(spec.ffn) if spec.ffn is not None else None
        self.post_ffn_norm = NORMS.build(spec.post_ffn_norm) if spec.ffn is not None else None
        for norm in (self.post_mixer_norm, self.post_ffn_norm):
            if norm is not None and not getattr(norm, "fusable_rms", False):
                raise ConfigError("the norms of a post-norm block are RMS norms")
        self.mixer_scale: Optional[torch.Tensor] = None
        self.ffn_scale: Optional[torch.Tensor] = None
        self._mixer_args = inspect.signature(self.mixer.forward).parameters
        self._ffn_args = inspect.signature(self.ffn.forward).parameters if self.ffn is not None else {}

    def children(self):
        return tuple(p for p in (self.mixer, self.post_mixer_norm, self.ffn, self.post_ffn_norm) if p is not None)

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self.children())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.children():
            out.update(part.tensor_specs())
        d = self.spec.post_mixer_norm.size
        for name in (self.spec.mixer_scale, self.spec.ffn_scale):
            if name is not None:
                out[name] = TensorSpec((d,), GAIN)
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        for part in self.children():
            part.load(tensors, runtime)
        s = self.spec
        self.mixer_scale = runtime.gain(tensors[s.mixer_scale]) if s.mixer_scale is not None else None
        self.ffn_scale = runtime.gain(tensors[s.ffn_scale]) if s.ffn_scale is not None else None

    def cache_request(self):
        return self.mixer.cache_request()

    kind_postnorm = True

    def wants_cast(self) -> bool:
        """Whether this block's first sublayer reads the stream in the products' number format (a copy that the
        kernel in front of it can write) rather than the float32 stream itself."""
        return self.runtime.act_dtype != torch.float32 and not getattr(self.mixer, "reads_stream", False)

    def _run(self, part, args, ctx, cache, source, y) -> Optional[torch.Tensor]:
        """Run a sublayer into ``y``; returns the additive vector it left to the block, if any."""
        kwargs = {}
        if "overwrite" in args:
            kwargs["overwrite"] = True
        else:
            y.zero_()
        later = "bias_later" in args and "overwrite" in args and getattr(part, "output_bias", None) is not None
        if later:
            kwargs["bias_later"] = True
        if cache is _NO_CACHE:
            part.forward(ctx, source, y, **kwargs)
        else:
            part.forward(ctx, cache, source, y, **kwargs)
        return part.output_bias if later else None

    def forward(self, ctx, cache, residual: torch.Tensor, normed_ready: bool = False, next_block=None) -> bool:
        """Run the layer on the residual stream in place. ``normed_ready``: the previous block already left the
        stream in the products' number format in the shared buffer. ``next_block``: the block that runs next; if it is
        of this kind and wants such a copy, the kernel that adds this layer's last result writes it. Returns whether
        it did."""
        act = self.runtime.act_dtype
        same = act == torch.float32                        # sublayers then read the stream in place
        h = residual if same else ctx.buffer("stream_copy", tuple(residual.shape), act)
        y = ctx.buffer("sublayer_out", tuple(residual.shape), torch.float32)
        if self.wants_cast() and not normed_ready:
            with ops.section("norm"):
                ops.stream_cast(residual, h)
        follower = next_block if getattr(next_block, "kind_postnorm", False) and not same else None
        to_follower = follower is not None and follower.wants_cast()

        def add_normed(post, scale, bias, copy: bool, consumer) -> bool:
            # the part that runs next may want the buffer of its first product zero: cleared here on the side
            clear = PreNormBlock._clear_for(ctx, consumer, residual.shape[0]) if consumer is not None else None
            with ops.section("norm"):
                ops.post_norm_add(y, post.weight, post.spec.eps, residual, next_out=h if copy else None, y_bias=bias,
                                  scale=scale, clear=clear)
            if clear is not None:
                ctx.note_cleared()
            return copy

        reads_stream = getattr(self.mixer, "reads_stream", False)
        bias = self._run(self.mixer, self._mixer_args, ctx, cache, residual if reads_stream else h, y)
        after = follower.mixer if follower is not None else None
        if self.ffn is None:
            return add_normed(self.post_mixer_norm, self.mixer_scale, bias, to_follower, after)
        ffn_reads_stream = getattr(self.ffn, "reads_stream", False)
        add_normed(self.post_mixer_norm, self.mixer_scale, bias, not same and not ffn_reads_stream, self.ffn)
        bias = self._run(self.ffn, self._ffn_args, ctx, _NO_CACHE, residual if ffn_reads_stream else h, y)
        return add_normed(self.post_ffn_norm, self.ffn_scale, bias, to_follower, after)


_NO_CACHE = object()


BLOCKS.register("postnorm", PostNormBlock)
BLOCKS.register("sandwich", SandwichBlock)
BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("parallel", ParallelBlock)
