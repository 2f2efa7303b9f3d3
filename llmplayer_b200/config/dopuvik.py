"""Configuration of the ``Dopuvik`` decoder: state-space layers, latent-attention layers and layers whose mixer is a
softmax attention beside a gated delta rule, in an order the configuration lists; feed-forwards are mixtures of gated
experts, some of which are identities.

``config.json`` holds ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale`` and
``layers``, a list of ``{"type", "mixer": {...}, "mlp": {...} or null}``; layer i's tensors start with ``l<i>.``, the
mixer's with ``l<i>.mix.``, the feed-forward's with ``l<i>.mlp.``. Every layer is pre-norm with layer norms (a gain,
no bias): x += mixer(ln(x, norm1)); x += ffn(ln(x, norm2)).

* type ``mamba2``: ``heads``, ``vdim`` (values per head), ``state``, ``groups``, ``conv`` (taps), ``norm_groups``:
  a selective state space per head (see ``parts/state_space.py``).
* type ``latent_attention``: ``heads``, ``dim`` (unrotated) and ``rot_dim`` (rotated) query / key sizes per head,
  ``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``mask: {size}`` (a token sees itself and the size - 1 tokens before it),
  ``rot: {base, dims, scaling: {factor, original, fast, slow}}``: neighbouring pairs (2i, 2i + 1) rotate, frequencies
  stretched by the number of turns over the original context, cosine and sine times 0.1 ln(factor) + 1. Queries go
  through an RMS-normed latent of their own; keys and values come from one cached RMS-normed latent plus one rotated key
  part shared by the heads.
* type ``parallel``: ``left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask: {size, keep_first}``,
  ``rot: {base, dims}`` with pairs (i, i + dims/2); projections with additive vectors; the window also keeps a sequence's
  first ``keep_first`` tokens) and ``right`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``: a gated delta rule, see
  ``parts/delta_rule.py``), summed as ``left_scale`` * left + ``right_scale`` * right.
* mlp ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity", "scale", "groups": {"count",
  "keep"}}}``: scores are the softmax over all router outputs (``experts`` + ``identity``); the choice adds a correction
  vector and is limited to the best groups; the weights are the chosen scores times ``scale``.

The output is the model's layer norm ``final.norm``, the matrix ``head`` and the constant ``logit_scale``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from ..parts.specs import (
    AttentionSpec, BlockSpec, EmbeddingSpec, ExpertRoutingSpec, GatedDeltaRuleSpec, HeadSpec, LatentAttentionSpec,
    MixerPairSpec, MixtureSpec, ModelLayout, NormSpec, PositionSpec, ScheduleEntry, StateSpaceSpec, YarnScaling,
)
from .ramupel import _need
from .registry import ArchitectureConfig, register_architecture


def _optional(raw: dict, key: str, kind, where: str, default):
    return default if raw.get(key) is None else _need(raw, key, kind, where)


def _positive(where: str, **values) -> None:
    for name, value in values.items():
        if value <= 0:
            raise ConfigError(f"{where}{name} must be positive, got {value}")


@dataclass(frozen=True)
class YarnConfig:
    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class RotationConfig:
    """``dims`` == 0: no rotation."""
    base: float
    dims: int
    scaling: Optional[YarnConfig] = None

    @classmethod
    def from_dict(cls, raw: Optional[dict], where: str) -> "RotationConfig":
        if raw is None:
            return cls(0.0, 0)
        if not isinstance(raw, dict):
            raise ConfigError(f"{where[:-1]} must be an object or null")
        dims = _need(raw, "dims", int, where)
        base = _need(raw, "base", float, where) if dims else 0.0
        scaling = None
        if raw.get("scaling") is not None:
            sc, w = _need(raw, "scaling", dict, where), where + "scaling."
            scaling = YarnConfig(factor=_need(sc, "factor", float, w), original=_need(sc, "original", int, w),
                                 fast=_need(sc, "fast", float, w), slow=_need(sc, "slow", float, w))
        return cls(base, dims, scaling)

    def to_dict(self) -> Optional[dict]:
        if not self.dims:
            return None
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            sc = self.scaling
            out["scaling"] = {"factor": sc.factor, "original": sc.original, "fast": sc.fast, "slow": sc.slow}
        return out

    def validate(self, where: str, most: int) -> None:
        if self.dims < 0 or self.dims % 2 or self.dims > most:
            raise ConfigError(f"{where}dims {self.dims} must be even and at most {most}")
        if self.dims and (not self.base > 0 or self.base == 1.0):
            raise ConfigError(f"{where}base must be positive and not 1, got {self.base}")
        sc = self.scaling
        if sc is not None and (not sc.factor > 0 or sc.original <= 0 or not sc.fast > 0 or not sc.slow > 0):
            raise ConfigError(f"{where}scaling needs positive factor, original, fast and slow, got {sc}")

    def position(self, head_dim: int, pairing: str) -> PositionSpec:
        if not self.dims:
            return PositionSpec(kind="none", head_dim=head_dim)
        sc = self.scaling
        scaling = None if sc is None else YarnScaling(factor=sc.factor, original=sc.original, fast=sc.fast, slow=sc.slow)
        return PositionSpec(kind="rope", head_dim=head_dim, rotary_dim=self.dims, theta=self.base, scaling=scaling,
                            pairing=pairing)


def _mask(raw: dict, where: str):
    """(size or None, keep_first) of a layer's ``mask``."""
    mask = raw.get("mask")
    if mask is None:
        return None, 0
    mask = _need(raw, "mask", dict, where)
    size = _optional(mask, "size", int, where + "mask.", None)
    return size, _optional(mask, "keep_first", int, where + "mask.", 0)


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    type = "mamba2"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "StateSpaceConfig":
        return cls(heads=_need(raw, "heads", int, where), vdim=_need(raw, "vdim", int, where),
                   state=_need(raw, "state", int, where), groups=_need(raw, "groups", int, where),
                   conv=_need(raw, "conv", int, where), norm_groups=_need(raw, "norm_groups", int, where))

    def to_dict(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}

    def validate(self, where: str) -> None:
        _positive(where, heads=self.heads, vdim=self.vdim, state=self.state, groups=self.groups, conv=self.conv,
                  norm_groups=self.norm_groups)
        if self.heads % self.groups:
            raise ConfigError(f"{where}heads {self.heads} is no multiple of groups {self.groups}")
        if (self.heads * self.vdim) % self.norm_groups:
            raise ConfigError(f"{where}norm_groups {self.norm_groups} does not divide heads * vdim = {self.heads * self.vdim}")
        if self.conv > 8:
            raise ConfigError(f"{where}conv {self.conv}: at most 8 taps are supported")

    def spec(self, p: str, width: int, eps: float):
        return StateSpaceSpec(
            hidden_size=width, num_heads=self.heads, head_dim=self.vdim, state_dim=self.state, groups=self.groups,
            conv_taps=self.conv, norm_groups=self.norm_groups, norm_eps=eps, in_proj=p + "in", conv=p + "conv",
            conv_bias=p + "conv.b", dt_bias=p + "dt_bias", a_log=p + "A_log", skip=p + "D", out_norm=p + "norm", o=p + "o")


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: Optional[int]
    rot: RotationConfig

    type = "latent_attention"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "LatentConfig":
        window, _ = _mask(raw, where)
        return cls(heads=_need(raw, "heads", int, where), dim=_need(raw, "dim", int, where),
                   rot_dim=_need(raw, "rot_dim", int, where), vdim=_need(raw, "vdim", int, where),
                   kv_rank=_need(raw, "kv_rank", int, where), q_rank=_need(raw, "q_rank", int, where),
                   scale=_need(raw, "scale", float, where), window=window,
                   rot=RotationConfig.from_dict(raw.get("rot"), where + "rot."))

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
               "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot.dims:
            out["rot"] = self.rot.to_dict()
        return out

    def validate(self, where: str) -> None:
        _positive(where, heads=self.heads, vdim=self.vdim, kv_rank=self.kv_rank, q_rank=self.q_rank)
        if self.dim < 0 or self.rot_dim < 0 or self.dim + self.rot_dim <= 0:
            raise ConfigError(f"{where}dim {self.dim} and rot_dim {self.rot_dim}: a head needs some of either")
        if self.window is not None and self.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive, got {self.window}")
        self.rot.validate(where + "rot.", self.rot_dim)

    def spec(self, p: str, width: int, eps: float):
        return LatentAttentionSpec(
            hidden_size=width, num_heads=self.heads, nope_dim=self.dim, rope_dim=self.rot_dim, value_dim=self.vdim,
            kv_rank=self.kv_rank, scale=self.scale, norm_eps=eps, position=self.rot.position(self.rot_dim, "interleaved"),
            q=p + "uq", kv_down=p + "dkv", latent_norm=p + "dkv.norm", k_up=p + "uk", v_up=p + "uv", o=p + "o",
            q_down=p + "dq", q_norm=p + "dq.norm", q_rank=self.q_rank, window=self.window, exact_weights=True)


@dataclass(frozen=True)
class KeptWindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    keep_first: int
    rot: RotationConfig

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "KeptWindowAttentionConfig":
        window, keep = _mask(raw, where)
        return cls(heads=_need(raw, "heads", int, where), kv_heads=_need(raw, "kv_heads", int, where),
                   dim=_need(raw, "dim", int, where), vdim=_need(raw, "vdim", int, where),
                   scale=_need(raw, "scale", float, where), window=window, keep_first=keep,
                   rot=RotationConfig.from_dict(raw.get("rot"), where + "rot."))

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.rot.dims:
            out["rot"] = self.rot.to_dict()
        return out

    def validate(self, where: str) -> None:
        _positive(where, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}heads {self.heads} is no multiple of kv_heads {self.kv_heads}")
        if self.window is not None and self.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive, got {self.window}")
        if self.keep_first < 0 or (self.keep_first > 0 and self.window is None):
            raise ConfigError(f"{where}mask.keep_first {self.keep_first} needs a mask.size and must not be negative")
        if self.rot.scaling is not None:
            raise ConfigError(f"{where}rot.scaling: this attention's rotation is not stretched")
        self.rot.validate(where + "rot.", self.dim)

    def spec(self, p: str, width: int):
        return AttentionSpec(
            hidden_size=width, num_heads=self.heads, num_kv_heads=self.kv_heads, head_dim=self.dim, scale=self.scale,
            position=self.rot.position(self.dim, "split_half"), q=p + "q", o=p + "o", k=p + "k", v=p + "v",
            window=self.window, value_dim=self.vdim, q_bias=p + "q.b", k_bias=p + "k.b", v_bias=p + "v.b",
            o_bias=p + "o.b", exact_weights=True, keep_first=self.keep_first or None)


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "DeltaRuleConfig":
        return cls(heads=_need(raw, "heads", int, where), kv_heads=_need(raw, "kv_heads", int, where),
                   dim=_need(raw, "dim", int, where), vdim=_need(raw, "vdim", int, where),
                   conv=_need(raw, "conv", int, where))

    def to_dict(self) -> dict:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}

    def validate(self, where: str) -> None:
        _positive(where, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, conv=self.conv)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}heads {self.heads} is no multiple of kv_heads {self.kv_heads}")
        if self.conv > 8:
            raise ConfigError(f"{where}conv {self.conv}: at most 8 taps are supported")
        if self.dim > 512:
            raise ConfigError(f"{where}dim {self.dim}: at most 512 key channels per head are supported")

    def spec(self, p: str, width: int, eps: float):
        return GatedDeltaRuleSpec(
            hidden_size=width, num_heads=self.heads, num_qk_heads=self.kv_heads, key_dim=self.dim, value_dim=self.vdim,
            conv_taps=self.conv, norm_eps=eps, q=p + "q", k=p + "k", v=p + "v", q_conv=p + "q.conv", k_conv=p + "k.conv",
            v_conv=p + "v.conv", strength=p + "b", decay=p + "a", a_log=p + "A_log", dt_bias=p + "dt_bias", gate=p + "g",
            out_norm=p + "norm", o=p + "o")


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: KeptWindowAttentionConfig
    right: DeltaRuleConfig
    left_scale: float
    right_scale: float

    type = "parallel"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "ParallelMixerConfig":
        return cls(left=KeptWindowAttentionConfig.from_dict(_need(raw, "left", dict, where), where + "left."),
                   right=DeltaRuleConfig.from_dict(_need(raw, "right", dict, where), where + "right."),
                   left_scale=_need(raw, "left_scale", float, where), right_scale=_need(raw, "right_scale", float, where))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}

    def validate(self, where: str) -> None:
        self.left.validate(where + "left.")
        self.right.validate(where + "right.")

    def spec(self, p: str, width: int, eps: float):
        return MixerPairSpec(left=self.left.spec(p + "left.", width), right=self.right.spec(p + "right.", width, eps),
                             left_scale=self.left_scale, right_scale=self.right_scale)


@dataclass(frozen=True)
class IdentityMoEConfig:
    expert_ff: int
    experts: int
    top: int
    identity: int
    scale: float
    group_count: int
    group_keep: int

    kind = "moe"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "IdentityMoEConfig":
        expert = _need(raw, "expert", dict, where)
        router = _need(raw, "router", dict, where)
        count = keep = 1
        if router.get("groups") is not None:
            groups = _need(router, "groups", dict, where + "router.")
            count = _need(groups, "count", int, where + "router.groups.")
            keep = _need(groups, "keep", int, where + "router.groups.")
        return cls(expert_ff=_need(expert, "ff", int, where + "expert."),
                   experts=_need(router, "experts", int, where + "router."), top=_need(router, "top", int, where + "router."),
                   identity=_optional(router, "identity", int, where + "router.", 0),
                   scale=_optional(router, "scale", float, where + "router.", 1.0), group_count=count, group_keep=keep)

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.expert_ff}, "kind": self.kind,
                "router": {"experts": self.experts, "groups": {"count": self.group_count, "keep": self.group_keep},
                           "identity": self.identity, "scale": self.scale, "top": self.top}}

    def validate(self, where: str) -> None:
        _positive(where, expert_ff=self.expert_ff, experts=self.experts, top=self.top, group_count=self.group_count,
                  group_keep=self.group_keep)
        if self.identity < 0:
            raise ConfigError(f"{where}router.identity must not be negative, got {self.identity}")
        outputs = self.experts + self.identity
        if outputs % self.group_count:
            raise ConfigError(f"{where}router.groups.count {self.group_count} does not divide the {outputs} router outputs")
        if self.group_keep > self.group_count:
            raise ConfigError(f"{where}router.groups.keep {self.group_keep} of {self.group_count} groups")
        if self.top > self.group_keep * (outputs // self.group_count):
            raise ConfigError(f"{where}router.top {self.top} cannot be chosen from {self.group_keep} groups of "
                              f"{outputs // self.group_count}")

    def spec(self, p: str, width: int):
        return MixtureSpec(
            hidden_size=width, expert_size=self.expert_ff,
            routing=ExpertRoutingSpec(num_experts=self.experts, top=self.top, groups=self.group_count,
                                      keep_groups=self.group_keep, router=p + "router", scoring="softmax_groups",
                                      correction=p + "correction", weight_scale=self.scale, identity_experts=self.identity),
            expert_prefix=p)


_MIXERS = {c.type: c for c in (StateSpaceConfig, LatentConfig, ParallelMixerConfig)}
_MLPS = {IdentityMoEConfig.kind: IdentityMoEConfig}


@dataclass(frozen=True)
class DopuvikLayerConfig:
    mixer: object                      # StateSpaceConfig, LatentConfig or ParallelMixerConfig
    mlp: Optional[object]              # IdentityMoEConfig or None


@dataclass(frozen=True)
class DopuvikConfig(ArchitectureConfig):
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[DopuvikLayerConfig, ...]

    architecture = "Dopuvik"
    # the design sets no limit on positions; this is the engine's default context when none is asked for
    DEFAULT_CONTEXT = 131072

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "DopuvikConfig":
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
            mlp_raw, mlp = entry.get("mlp"), None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, dict):
                    raise ConfigError(f"{where}mlp must be an object or null")
                mlp_kind = _need(mlp_raw, "kind", str, where + "mlp.")
                if mlp_kind not in _MLPS:
                    raise ConfigError(f"{where}mlp.kind {mlp_kind!r} is unknown; known: {', '.join(sorted(_MLPS))}")
                mlp = _MLPS[mlp_kind].from_dict(mlp_raw, where + "mlp.")
            layers.append(DopuvikLayerConfig(mixer, mlp))
        embedding = raw.get("embedding")
        cfg = cls(vocab=_need(raw, "vocab", int, ""), width=_need(raw, "width", int, ""),
                  norm_eps=_need(_need(raw, "norm", dict, ""), "eps", float, "norm."),
                  embedding_scale=_optional(embedding, "scale", float, "embedding.", 1.0) if isinstance(embedding, dict) else 1.0,
                  logit_scale=_optional(raw, "logit_scale", float, "", 1.0), layers=tuple(layers))
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
            layer.mixer.validate(f"layers[{i}].mixer.")
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp.")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict(),
                        "type": layer.mixer.type} for layer in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    # ------------------------------------------------------------------ meaning
    def max_positions(self) -> int:
        return self.DEFAULT_CONTEXT

    def layout(self) -> ModelLayout:
        d, eps = self.width, self.norm_eps
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            has_ffn = layer.mlp is not None
            blocks.append(BlockSpec(
                mixer_norm=NormSpec(d, eps, p + "norm1", kind="layernorm"), mixer=layer.mixer.spec(p + "mix.", d, eps),
                ffn_norm=NormSpec(d, eps, p + "norm2", kind="layernorm") if has_ffn else None,
                ffn=layer.mlp.spec(p + "mlp.", d) if has_ffn else None))
        return ModelLayout(
            embedding=EmbeddingSpec(self.vocab, d, "embed", scale=self.embedding_scale), layers=tuple(blocks),
            head=HeadSpec(self.vocab, d, norm=NormSpec(d, eps, "final.norm", kind="layernorm"), weight="head",
                          logit_scale=self.logit_scale),
            schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))))

    def ignorable_tensors(self) -> tuple:
        # a layer without a feed-forward has no use for the norm in front of one, should a file carry it
        return tuple(f"l{i}.norm2" for i, layer in enumerate(self.layers) if layer.mlp is None)

    def describe(self) -> str:
        lines = [f"architecture: {self.architecture}", f"  vocab = {self.vocab}", f"  width = {self.width}",
                 f"  norm.eps = {self.norm_eps}", f"  embedding.scale = {self.embedding_scale}",
                 f"  logit_scale = {self.logit_scale}"]
        for i, layer in enumerate(self.layers):
            lines.append(f"  layer {i}: {layer.mixer.type} {layer.mixer.to_dict()}, feed-forward "
                         f"{None if layer.mlp is None else layer.mlp.to_dict()}")
        return "\n".join(lines)


register_architecture(DopuvikConfig.architecture, DopuvikConfig)
