"""Configuration of the ``Zasitar`` decoder: sliding-window attention layers (some of which attend over an earlier
layer's keys and values) and time-mixing (WKV) layers, in an order the configuration lists; dense or
mixture-of-experts feed-forwards.

``config.json`` holds ``architecture``, ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list of
``{"type", "mixer": {...}, "mlp": {...} or null}``; layer i's tensors start with ``l<i>.``, the mixer's with
``l<i>.mix.``, the feed-forward's with ``l<i>.mlp.``.

Every layer lets its sublayers read the stream itself and norms their results:
x += ls1 * rms_norm(mixer(x), norm1); x += ls2 * rms_norm(ffn(x), norm2), the layer scales ls being per-feature.

* type ``attention``: ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values), ``scale``,
  ``mask: {size}`` (a token sees itself and the size - 1 tokens before it), ``rot: {base, dims, scaling: {factor, low,
  high, original}}`` (pairs (i, i + dims/2) over the first ``dims`` features, frequencies stretched by wavelength).
  Projections with additive vectors; queries and keys RMS-normed per head with a gain shared by the heads, before the
  rotation; the softmax's denominator holds one more term of score zero. ``kv_from: j``: the layer has no key or
  value tensors and attends over layer j's keys and values.
* type ``wkv``: ``heads``, ``dim``: time mixing with a matrix state per head (see ``parts/time_mix.py``).
* mlp ``{"kind": "dense", "ff"}``: down(gelu_tanh(gate x + b) * (up x + b)) + b. mlp ``{"kind": "moe", "expert": {"ff",
  "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"}}``: clamped gated experts, the ``top`` largest router
  logits (with an additive vector) win and are weighted by the softmax over themselves; the shared expert runs for
  every token, times a sigmoid gate of its own.

The output is the model's norm ``final.norm`` and the matrix ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from ..parts.specs import (
    AttentionSpec, EmbeddingSpec, ExpertRoutingSpec, GatedDenseSpec, HeadSpec, Llama3Scaling, MixtureSpec, ModelLayout,
    NormSpec, PositionSpec, PostNormBlockSpec, ScheduleEntry, TimeMixSpec,
)
from .ramupel import _need
from .registry import ArchitectureConfig, register_architecture


@dataclass(frozen=True)
class RotationScaling:
    factor: float
    low: float
    high: float
    original: int


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]             # mask.size; None: every earlier token is seen
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotationScaling]
    kv_from: Optional[int] = None

    type = "attention"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "WindowAttentionConfig":
        rot = raw.get("rot")
        base, dims, scaling = 0.0, 0, None
        if rot is not None:
            rot = _need(raw, "rot", dict, where)
            dims = _need(rot, "dims", int, where + "rot.")
            base = _need(rot, "base", float, where + "rot.") if dims else 0.0
            if rot.get("scaling") is not None:
                sc = _need(rot, "scaling", dict, where + "rot.")
                w = where + "rot.scaling."
                scaling = RotationScaling(factor=_need(sc, "factor", float, w), low=_need(sc, "low", float, w),
                                          high=_need(sc, "high", float, w), original=_need(sc, "original", int, w))
        window = None
        if raw.get("mask") is not None:
            window = _need(_need(raw, "mask", dict, where), "size", int, where + "mask.")
        kv_from = raw.get("kv_from")
        if kv_from is not None:
            kv_from = _need(raw, "kv_from", int, where)
        return cls(heads=_need(raw, "heads", int, where), kv_heads=_need(raw, "kv_heads", int, where),
                   dim=_need(raw, "dim", int, where), vdim=_need(raw, "vdim", int, where),
                   scale=_need(raw, "scale", float, where), window=window, rot_base=base, rot_dims=dims,
                   rot_scaling=scaling, kv_from=kv_from)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            rot = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                sc = self.rot_scaling
                rot["scaling"] = {"factor": sc.factor, "low": sc.low, "high": sc.high, "original": sc.original}
            out["rot"] = rot
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out

    def validate(self, where: str) -> None:
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}heads {self.heads} is no multiple of kv_heads {self.kv_heads}")
        if self.window is not None and self.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive, got {self.window}")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ConfigError(f"{where}rot.dims {self.rot_dims} must be even and at most dim {self.dim}")
        if self.rot_dims and not self.rot_base > 0:
            raise ConfigError(f"{where}rot.base must be positive, got {self.rot_base}")
        sc = self.rot_scaling
        if sc is not None and (not sc.factor > 0 or sc.original <= 0 or not sc.low > 0 or not sc.high > sc.low):
            raise ConfigError(f"{where}rot.scaling needs factor > 0, original > 0 and 0 < low < high, got {sc}")


@dataclass(frozen=True)
class WKVConfig:
    heads: int
    dim: int

    type = "wkv"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "WKVConfig":
        return cls(heads=_need(raw, "heads", int, where), dim=_need(raw, "dim", int, where))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim}

    def validate(self, where: str) -> None:
        if self.heads <= 0 or self.dim <= 0:
            raise ConfigError(f"{where}heads {self.heads} and dim {self.dim} must be positive")


@dataclass(frozen=True)
class GeluMLPConfig:
    ff: int

    kind = "dense"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "GeluMLPConfig":
        return cls(ff=_need(raw, "ff", int, where))

    def to_dict(self) -> dict:
        return {"kind": self.kind, "ff": self.ff}

    def validate(self, where: str) -> None:
        if self.ff <= 0:
            raise ConfigError(f"{where}ff must be positive, got {self.ff}")


@dataclass(frozen=True)
class ClampedMoEConfig:
    expert_ff: int
    expert_limit: float
    experts: int
    top: int
    shared_ff: int            # 0: no shared expert
    shared_limit: float

    kind = "moe"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "ClampedMoEConfig":
        expert = _need(raw, "expert", dict, where)
        router = _need(raw, "router", dict, where)
        shared = raw.get("shared")
        if shared is not None and not isinstance(shared, dict):
            raise ConfigError(f"{where}shared must be an object or null")
        return cls(expert_ff=_need(expert, "ff", int, where + "expert."),
                   expert_limit=_need(expert, "limit", float, where + "expert."),
                   experts=_need(router, "experts", int, where + "router."), top=_need(router, "top", int, where + "router."),
                   shared_ff=_need(shared, "ff", int, where + "shared.") if shared is not None else 0,
                   shared_limit=_need(shared, "limit", float, where + "shared.") if shared is not None else 0.0)

    def to_dict(self) -> dict:
        out = {"kind": self.kind, "expert": {"ff": self.expert_ff, "limit": self.expert_limit},
               "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff > 0:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out

    def validate(self, where: str) -> None:
        for name in ("expert_ff", "experts", "top"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if self.top > self.experts:
            raise ConfigError(f"{where}{self.top} of {self.experts} experts cannot be chosen")
        if not self.expert_limit > 0:
            raise ConfigError(f"{where}expert.limit must be positive, got {self.expert_limit}")
        if self.shared_ff < 0 or (self.shared_ff > 0 and not self.shared_limit > 0):
            raise ConfigError(f"{where}shared needs a positive ff and limit, got {self.shared_ff} and {self.shared_limit}")


_MIXERS = {WindowAttentionConfig.type: WindowAttentionConfig, WKVConfig.type: WKVConfig}
_MLPS = {GeluMLPConfig.kind: GeluMLPConfig, ClampedMoEConfig.kind: ClampedMoEConfig}


@dataclass(frozen=True)
class ZasitarLayerConfig:
    mixer: object                      # WindowAttentionConfig or WKVConfig
    mlp: Optional[object]              # GeluMLPConfig, ClampedMoEConfig or None


@dataclass(frozen=True)
class ZasitarConfig(ArchitectureConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZasitarLayerConfig, ...]

    architecture = "Zasitar"
    # the design sets no limit on positions; this is the engine's default context when none is asked for
    DEFAULT_CONTEXT = 131072

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "ZasitarConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _need(entry, "type", str, where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}type {kind!r} is unknown; known: {', '.join(sorted(_MIXERS))}")
            mixer = _MIXERS[kind].from_dict(_need(entry, "mixer", dict, where), where + "mixer.")
            mlp_raw = entry.get("mlp")
            mlp = None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, dict):
                    raise ConfigError(f"{where}mlp must be an object or null")
                mlp_kind = _need(mlp_raw, "kind", str, where + "mlp.")
                if mlp_kind not in _MLPS:
                    raise ConfigError(f"{where}mlp.kind {mlp_kind!r} is unknown; known: {', '.join(sorted(_MLPS))}")
                mlp = _MLPS[mlp_kind].from_dict(mlp_raw, where + "mlp.")
            layers.append(ZasitarLayerConfig(mixer, mlp))
        cfg = cls(vocab=_need(raw, "vocab", int, ""), width=_need(raw, "width", int, ""),
                  norm_eps=_need(_need(raw, "norm", dict, ""), "eps", float, "norm."), layers=tuple(layers))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab {self.vocab} and width {self.width} must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}].mixer."
            layer.mixer.validate(where)
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp.")
            src = getattr(layer.mixer, "kv_from", None)
            if src is not None:
                if not 0 <= src < i:
                    raise ConfigError(f"{where}kv_from {src} must name an earlier layer")
                other = self.layers[src].mixer
                if not isinstance(other, WindowAttentionConfig) or other.kv_from is not None:
                    raise ConfigError(f"{where}kv_from {src} must name an attention layer with keys and values of its own")
                m = layer.mixer
                if (m.kv_heads, m.dim, m.vdim) != (other.kv_heads, other.dim, other.vdim):
                    raise ConfigError(f"{where}kv_from {src}: key/value heads and sizes of the two layers differ")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "layers": [{"type": layer.mixer.type, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    # ------------------------------------------------------------------ meaning
    def max_positions(self) -> int:
        return self.DEFAULT_CONTEXT

    def cache_window(self, index: int) -> Optional[int]:
        """How far back the cache of attention layer ``index`` must reach: the widest window among the layer itself
        and the layers that attend over its keys and values (None: everything)."""
        windows = [self.layers[index].mixer.window]
        windows += [l.mixer.window for l in self.layers if getattr(l.mixer, "kv_from", None) == index]
        return None if any(w is None for w in windows) else max(windows)

    def layout(self) -> ModelLayout:
        d, eps = self.width, self.norm_eps
        blocks, runs = [], []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer.mixer
            if isinstance(m, WindowAttentionConfig):
                scaling = None
                if m.rot_scaling is not None:
                    sc = m.rot_scaling
                    scaling = Llama3Scaling(factor=sc.factor, low_freq_factor=sc.low, high_freq_factor=sc.high,
                                            original_max_position=sc.original)
                position = (PositionSpec(kind="rope", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                         scaling=scaling, pairing="split_half")
                            if m.rot_dims > 0 else PositionSpec(kind="none", head_dim=m.dim))
                shares = m.kv_from is not None
                mixer = AttentionSpec(
                    hidden_size=d, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                    position=position, q=p + "mix.q", o=p + "mix.o", k=None if shares else p + "mix.k",
                    v=None if shares else p + "mix.v", window=m.window, shares_kv=shares, value_dim=m.vdim,
                    q_bias=p + "mix.q.b", k_bias=None if shares else p + "mix.k.b", v_bias=None if shares else p + "mix.v.b",
                    q_norm=p + "mix.q.norm", k_norm=None if shares else p + "mix.k.norm", qk_norm_eps=eps,
                    o_bias=p + "mix.o.b", sink_value=0.0, exact_weights=True,
                    cache_window="own" if shares else self.cache_window(i))
                runs.append(ScheduleEntry(i, reads_cache_of=m.kv_from))
            else:
                mixer = TimeMixSpec(
                    hidden_size=d, num_heads=m.heads, head_dim=m.dim, norm_eps=eps, mu=p + "mix.mu.", r=p + "mix.r",
                    k=p + "mix.k", v=p + "mix.v", gate=p + "mix.g", decay_down=p + "mix.w1", decay_up=p + "mix.w2",
                    decay_bias=p + "mix.w0", bonus=p + "mix.u", out_norm=p + "mix.norm", o=p + "mix.o")
                runs.append(ScheduleEntry(i))
            ffn = None
            if isinstance(layer.mlp, GeluMLPConfig):
                ffn = GatedDenseSpec(hidden_size=d, intermediate_size=layer.mlp.ff, gate=p + "mlp.gate", up=p + "mlp.up",
                                     down=p + "mlp.down", gate_bias=p + "mlp.gate.b", up_bias=p + "mlp.up.b",
                                     down_bias=p + "mlp.down.b", activation="gelu_tanh")
            elif isinstance(layer.mlp, ClampedMoEConfig):
                c = layer.mlp
                ffn = MixtureSpec(
                    hidden_size=d, expert_size=c.expert_ff,
                    routing=ExpertRoutingSpec(num_experts=c.experts, top=c.top, groups=1, keep_groups=1,
                                              router=p + "mlp.router", scoring="softmax_top",
                                              router_bias=p + "mlp.router.b"),
                    expert_prefix=p + "mlp.", shared_size=c.shared_ff,
                    shared_prefix=p + "mlp.shared." if c.shared_ff else None, activation="clamped",
                    limit=c.expert_limit, shared_limit=c.shared_limit,
                    shared_gate=p + "mlp.shared.sg" if c.shared_ff else None)
            blocks.append(PostNormBlockSpec(
                mixer=mixer, post_mixer_norm=NormSpec(d, eps, p + "norm1"), mixer_scale=p + "ls1", ffn=ffn,
                post_ffn_norm=NormSpec(d, eps, p + "norm2") if ffn is not None else None,
                ffn_scale=p + "ls2" if ffn is not None else None))
        return ModelLayout(
            embedding=EmbeddingSpec(self.vocab, d, "embed"), layers=tuple(blocks),
            head=HeadSpec(self.vocab, d, norm=NormSpec(d, eps, "final.norm"), weight="head"), schedule=tuple(runs))

    def ignorable_tensors(self) -> tuple:
        # a layer without a feed-forward has no use for the norm and the scale behind one, should a file carry them
        return tuple(f"l{i}.{n}" for i, layer in enumerate(self.layers) if layer.mlp is None for n in ("norm2", "ls2"))

    def describe(self) -> str:
        lines = [f"architecture: {self.architecture}", f"  vocab = {self.vocab}", f"  width = {self.width}",
                 f"  norm.eps = {self.norm_eps}"]
        for i, layer in enumerate(self.layers):
            sizes = ", ".join(f"{k}={v}" for k, v in layer.mixer.to_dict().items())
            lines.append(f"  layer {i}: {layer.mixer.type} ({sizes}), feed-forward {None if layer.mlp is None else layer.mlp.to_dict()}")
        return "\n".join(lines)


register_architecture(ZasitarConfig.architecture, ZasitarConfig)
