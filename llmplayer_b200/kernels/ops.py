"""The operations of a step, as calls into the compiled CUDA libraries.

Each function checks the tensors it is given (device, dtype, shape, layout),
then launches on torch's current stream. There is no other implementation
behind them: without a GPU and the compiled library they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..errors import ExtensionMissing, KernelError
from . import build

F32, BF16 = 0, 1
STORE, ACCUMULATE, SWIGLU = 0, 1, 2
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_P, _I, _F = c_void_p, c_int, c_float
_SIGNATURES = {
    "elementwise": {
        "lp_embed": [_P, _I, _P, _P, _I, _I, _F, _P],
        "lp_layernorm": [_P, _P, _P, _P, _I, _I, _I, _F, _P, ctypes.c_longlong, _P],
        "lp_scaled_sum": [_P, _P, _P, _F, _P, _P, _F, _I, _I, _P],
        "lp_xielu": [_P, _I, _P, _P, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "lp_gated_sum": [_P, _P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
        "lp_rmsnorm": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _F, _P, ctypes.c_longlong, _P],
        "lp_rope_cache_write": [_P, _I, _P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
        "lp_advance": [_P, _P, _P, _P, _I, _P],
        "lp_rope_angles": [_P, _P, _P, _I, _I, _P],
        "lp_qkv_prepare": [_P, _I, _P, _P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P,
                           ctypes.c_longlong, _P, _P, _F, _P],
        "lp_post_norm_add": [_P, _P, _F, _P, _P, _F, _P, _I, _I, _I, _P, ctypes.c_longlong, _P, _P, _P],
        "lp_gated_act": [_P, _I, _P, _P, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "lp_stream_cast": [_P, _P, _I, ctypes.c_longlong, _P, ctypes.c_longlong, _P],
        "lp_stream_add": [_P, _P, _P, _I, _I, _P],
        "lp_relu2": [_P, _I, _P, _I, _I, _I, _P, ctypes.c_longlong, _P],
    },
    "routing": {
        "lp_route": [_P, _I, _P, _I, _I, _I, _I, _I, _I, _P],
        "lp_expert_scale": [_P, _I, _I, _P, _I, _I, _I, _I, _P, ctypes.c_longlong, _P, _P, _I, _I, _I, _I, _P],
        "lp_route_top": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
        "lp_expert_act": [_P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _F, _F, _P, ctypes.c_longlong, _P],
        "lp_route_softmax": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P],
        "lp_identity_experts": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _P],
    },
    "gemm_plain": {
        "lp_gemm_plain": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    },
    "attention_plain": {
        "lp_attention_plain": [_P, _P, _I, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _F, _P, _I, _P],
    },
    "gemm_tcgen05": {
        "lp_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P,
                            ctypes.c_longlong, _P, _P],
        "lp_gemm_persistent": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "lp_gemm_fewtok": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P, _I, _P],
        "lp_gemm_configure": [_I, _I, _I, _I, _I],
        "lp_gemm_qkv_rope": [_P, _P, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    },
    "attention_mma": {
        "lp_attention_prefill": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _F, _P, _I, _I, _P],
        "lp_attention_decode": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _F, _P, _I, _P],
        "lp_attention_decode_fitted": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _F, _P, _I, _I, _P],
        "lp_attention_decode_fused": [_P, _I, _P, _I, _I, _P, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I,
                                      _I, _I, _I, _P, _F, _I, ctypes.c_longlong, _P, _P],
    },
    "attention_tcgen05": {
        "lp_attention_prefill_tc": [_P, _P, _P, ctypes.c_longlong, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I,
                                    _P, _P],
    },
    "latent_attention": {
        "lp_latent_prepare": [_P, _I, _I, _I, _P, _F, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P,
                              _I, _P, _I, _I, _F, _P],
        "lp_latent_heads_to_pages": [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
        "lp_latent_gate_heads": [_P, _P, _I, _P, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "lp_latent_absorb": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _P],
        "lp_latent_attend_rows": [],
        "lp_latent_attend": [_P, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P],
        "lp_latent_merge": [_P, _I, _P, _I, _I, _P],
        "lp_latent_query_norm": [_P, _I, _I, _I, _P, _F, _P, _I, _I, _P],
        "lp_latent_expand": [_P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
    },
    "linear_attention": {
        "lp_gla_decay": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _F, _I, _P],
        "lp_gla_scan": [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, _I, _P, _I, _P, _I, _P, _P],
        "lp_short_conv": [_P, _I, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "lp_decay_gates": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _P],
        "lp_head_unit_norm": [_P, _I, _I, _I, _I, _F, _F, _I, _I, _P],
        "lp_gated_part_norm": [_P, _P, _I, _P, _P, _I, _P, _F, _P, _I, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "lp_token_shift": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "lp_gla_finish": [_P, _P, _F, _P, _I, _P, _I, _I, _I, _I, _P, ctypes.c_longlong, _I, _I, _I, _P, _P],
        "lp_exp_gates": [_P, _I, _I, _I, _P, _P, _F, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    },
    "host_loop": {
        "lp_decode_loop": [_P, _P, _P, _I, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P],
        "lp_decode_loop_sampled": [_P, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P,
                                   _P, _P, _P, _P, _P, _P],
    },
    "sampling": {
        "lp_sample": [_P, ctypes.c_longlong, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P],
        "lp_sample_params_size": [],
        "lp_sample_select_words": [],
        "lp_sample_slice_capacity": [_I],
        "lp_argmax": [_P, ctypes.c_longlong, _I, _I, _P, _P, _P],
        "lp_sample_fetch": [_P, _P, _I, _I, _I, _I, _P],
    },
}

_libs: Dict[str, ctypes.CDLL] = {}


def _env_int(name: str, default: int) -> int:
    import os
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


@dataclass
class KernelSettings:
    """Switches of the kernels, one set per process (the compiled libraries are shared by every engine of the
    process). The defaults are what was measured best; the environment variables of the same meaning
    (``LLMPLAYER_B200_PDL``, ``_FEW_TOKENS``, ``_FEWTOK``, ``_RING_SHARED``, ``_RING_ALONE``) set the initial
    values, :func:`configure` (which the engine's options call) changes them.

    ``pdl``: programmatic dependent launch between the kernels of a step. ``few_tokens``: up to how many tokens
    the parts put the RMS norm inside the consuming product and use the few-token kernel. ``fewtok_kernel``:
    whether 16-token tiles of the general product go to the mma.sync few-token kernel. ``ring_shared`` /
    ``ring_alone``: stages of that kernel's ring when two CTAs share an SM / when a CTA has one to itself.
    ``ring_alone_tile``: the most stages the one-tile tcgen05 product takes when its grid has no more CTAs than SMs
    (0, the default: never more than what lets two CTAs share an SM; a deeper ring measured slower).
    ``ring_normed``: the same for the tcgen05 product with the norm on the way in (9 to 64 tokens), whose stages
    also hold a float32 tile of x; there the deeper ring measured faster."""
    pdl: bool = True
    few_tokens: int = 32
    fewtok_kernel: bool = True
    ring_shared: int = 6
    ring_alone: int = 10
    ring_alone_tile: int = 0
    ring_normed: int = 6

    @classmethod
    def from_env(cls) -> "KernelSettings":
        return cls(pdl=_env_int("LLMPLAYER_B200_PDL", 1) != 0, few_tokens=_env_int("LLMPLAYER_B200_FEW_TOKENS", 32),
                   fewtok_kernel=_env_int("LLMPLAYER_B200_FEWTOK", 1) != 0,
                   ring_shared=_env_int("LLMPLAYER_B200_RING_SHARED", 6),
                   ring_alone=_env_int("LLMPLAYER_B200_RING_ALONE", 10),
                   ring_alone_tile=_env_int("LLMPLAYER_B200_RING_ALONE_TILE", 0),
                   ring_normed=_env_int("LLMPLAYER_B200_RING_NORMED", 6))


settings = KernelSettings.from_env()


def _apply_settings(name: str, lib: ctypes.CDLL) -> None:
    lib.lp_set_pdl.argtypes = [c_int]
    lib.lp_set_pdl.restype = None
    lib.lp_set_pdl(1 if settings.pdl else 0)
    if name == "gemm_tcgen05":
        lib.lp_gemm_configure(1 if settings.fewtok_kernel else 0, int(settings.ring_shared), int(settings.ring_alone),
                              int(settings.ring_alone_tile), int(settings.ring_normed))


def configure(**changes) -> KernelSettings:
    """Change kernel settings (fields of :class:`KernelSettings`) for this process, now and for libraries
    loaded later. Graphs captured before the change keep what they were captured with."""
    global FEW_TOKENS
    for key, value in changes.items():
        if value is None:
            continue
        if not hasattr(settings, key):
            raise KernelError(f"unknown kernel setting {key!r}")
        setattr(settings, key, type(getattr(settings, key))(value))
    FEW_TOKENS = max(0, min(int(settings.few_tokens), FEW_TOKENS_MAX))
    for name, lib in _libs.items():
        _apply_settings(name, lib)
    return settings


def library(name: str) -> ctypes.CDLL:
    """The loaded library ``name``; compiled first if it is missing or stale."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    path = build.ensure_built(name)
    try:
        lib = ctypes.CDLL(path)
    except OSError as exc:
        raise ExtensionMissing(f"cannot load {path}: {exc}") from None
    for fn, args in _SIGNATURES.get(name, {}).items():
        f = getattr(lib, fn)
        f.argtypes = args
        f.restype = c_int
    lib.lp_last_error.restype = ctypes.c_char_p
    _apply_settings(name, lib)
    _libs[name] = lib
    return lib


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise ExtensionMissing("no CUDA device: this library runs on the GPU only and has no CPU path")


# --------------------------------------------------------------------------- profile mode
class _NoSection:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SECTION = _NoSection()


class StepProfiler:
    """Device time per section of the model walk, from CUDA-event pairs around each section.

    The reference's ``-Dcuda.profile=true`` puts stream barriers between the sections of a token's forward
    pass and prints milliseconds per section (java21 inference/CudaForwardPass.java:1431-1456, :1646-1737);
    graph replay is off meanwhile (:1761). Here a section is a ``with ops.section(name):`` block in a part;
    the events between sections also keep neighbouring kernels from overlapping, so the times add up to
    the step's, and steps run directly instead of from captured graphs."""

    def __init__(self):
        self._pairs = []            # (name, start event, end event), resolved when a report is asked for
        self._totals: Dict[str, list] = {}
        self.steps = 0

    class _Section:
        def __init__(self, owner, name):
            self.owner, self.name = owner, name

        def __enter__(self):
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
            return self

        def __exit__(self, *exc):
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.owner._pairs.append((self.name, self.start, end))
            return False

    def section(self, name: str):
        return StepProfiler._Section(self, name)

    def _resolve(self) -> None:
        if self._pairs:
            torch.cuda.synchronize()
            for name, start, end in self._pairs:
                entry = self._totals.setdefault(name, [0.0, 0])
                entry[0] += start.elapsed_time(end)
                entry[1] += 1
            self._pairs = []

    def report(self) -> dict:
        """{"steps": n, "total_ms": t, "sections": {name: {"ms": total, "calls": c, "ms_per_step": m}}}"""
        self._resolve()
        steps = max(1, self.steps)
        sections = {name: {"ms": ms, "calls": calls, "ms_per_step": ms / steps}
                    for name, (ms, calls) in sorted(self._totals.items(), key=lambda kv: -kv[1][0])}
        return {"steps": self.steps, "total_ms": sum(v["ms"] for v in sections.values()), "sections": sections}

    def reset(self) -> None:
        self._resolve()
        self._totals = {}
        self.steps = 0


_profiler: Optional[StepProfiler] = None


def set_profiler(profiler: Optional[StepProfiler]) -> None:
    global _profiler
    _profiler = profiler


_section_prefix = ""


class section_prefix:
    """``with ops.section_prefix("left."):`` around a part that runs inside another: the sections it opens are
    reported under that prefix, so that two members of the same kind keep their times apart."""

    def __init__(self, prefix: str):
        self.prefix = prefix

    def __enter__(self):
        global _section_prefix
        self.before = _section_prefix
        _section_prefix = self.before + self.prefix
        return self

    def __exit__(self, *exc):
        global _section_prefix
        _section_prefix = self.before
        return False


def section(name: str):
    """``with ops.section("attention.qkv"):`` around the launches of one section of the model walk; costs
    nothing unless a profiler is set."""
    return _NO_SECTION if _profiler is None else _profiler.section(_section_prefix + name)


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched by this process."""
    return _launches


def count_launches(n: int) -> None:
    """Kernels launched by replaying captured graphs from native code (the host loop) are counted here."""
    global _launches
    _launches += int(n)


def _check(lib: ctypes.CDLL, code: int) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(lib.lp_last_error().decode("utf-8", "replace") or f"kernel call failed with code {code}")


_device_index = None


def current_stream() -> int:
    return _stream()


def _stream() -> int:
    """The raw handle of torch's current stream (asked of torch's C layer directly: this is on the path of
    every launch)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    try:
        return torch._C._cuda_getCurrentRawStream(_device_index)
    except AttributeError:                        # a torch without that entry
        return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _want(t: torch.Tensor, what: str, dtype=None, ndim: Optional[int] = None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: expected a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected dtype {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what}: expected {ndim} dimensions, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous tensor, got strides {t.stride()}")
    return t


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------- embedding
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = float32(table[tokens[t], :]) * scale."""
    _want(table, "embed table", ndim=2)
    _want(tokens, "embed tokens", torch.int32, 1)
    _want(out, "embed out", torch.float32, 2)
    T, d = out.shape
    if tokens.numel() != T or table.shape[1] != d:
        raise KernelError(f"embed: {tokens.numel()} tokens, table {tuple(table.shape)}, out {tuple(out.shape)}")
    lib = library("elementwise")
    _check(lib, lib.lp_embed(table.data_ptr(), _code(table, "embed table"), tokens.data_ptr(), out.data_ptr(),
                             T, d, float(scale), _stream()))
    return out


# --------------------------------------------------------------------------- norm
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None,
            clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = x[rows[r]] / sqrt(mean(x^2) + eps) * weight, float32 inside.

    ``add`` (same shape as x) is first added into x in place: the residual sum
    fused with the norm that follows it. ``clear``: a float32 buffer that is set to
    zero on the side (for a product after the norm that sums partial results into it).
    """
    _want(x, "rmsnorm x", torch.float32, 2)
    _want(weight, "rmsnorm weight", torch.float32, 1)
    _want(out, "rmsnorm out", ndim=2)
    d = x.shape[1]
    R = out.shape[0]
    if weight.numel() != d or out.shape[1] != d:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _want(rows, "rmsnorm rows", torch.int32, 1)
        if rows.numel() != R:
            raise KernelError(f"rmsnorm: {rows.numel()} row indices for {R} output rows")
    elif x.shape[0] != R:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)} and out {tuple(out.shape)} differ in rows")
    add_code = F32
    if add is not None:
        _want(add, "rmsnorm add", ndim=2)
        if add.shape != x.shape:
            raise KernelError(f"rmsnorm: add {tuple(add.shape)} does not match x {tuple(x.shape)}")
        add_code = _code(add, "rmsnorm add")
    if clear is not None:
        _want(clear, "rmsnorm clear", torch.float32)
    lib = library("elementwise")
    _check(lib, lib.lp_rmsnorm(x.data_ptr(), _ptr(add), add_code, _ptr(rows), weight.data_ptr(), out.data_ptr(),
                               _code(out, "rmsnorm out"), R, d, float(eps), _ptr(clear),
                               clear.numel() if clear is not None else 0, _stream()))
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
              rows: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = (x[rows[r]] - mean) / sqrt(variance + eps) * weight, float32 inside; the variance is the mean
    of the squared deviations from the mean. ``clear``: a float32 buffer zeroed on the side."""
    _want(x, "layernorm x", torch.float32, 2)
    _want(weight, "layernorm weight", torch.float32, 1)
    _want(out, "layernorm out", ndim=2)
    d, R = x.shape[1], out.shape[0]
    if weight.numel() != d or out.shape[1] != d:
        raise KernelError(f"layernorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _want(rows, "layernorm rows", torch.int32, 1)
        if rows.numel() != R:
            raise KernelError(f"layernorm: {rows.numel()} row indices for {R} output rows")
    elif x.shape[0] != R:
        raise KernelError(f"layernorm: x {tuple(x.shape)} and out {tuple(out.shape)} differ in rows")
    lib = library("elementwise")
    _check(lib, lib.lp_layernorm(x.data_ptr(), _ptr(rows), weight.data_ptr(), out.data_ptr(), _code(out, "layernorm out"),
                                 R, d, float(eps), *_clear_args(clear, "layernorm"), _stream()))
    return out


def _slice(t: torch.Tensor, what: str):
    """(pointer, row stride) of a float32 matrix that may be a column slice of a wider one."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2:
        raise KernelError(f"{what}: expected a float32 CUDA matrix")
    if t.stride(1) != 1 and t.shape[1] > 1:
        raise KernelError(f"{what}: columns must lie together, got strides {t.stride()}")
    return t.data_ptr(), int(t.stride(0))


def _out_matrix(t: torch.Tensor, what: str):
    """(pointer, row stride) of a product's output: a matrix whose columns lie together; it may be a column slice of a
    wider one, so that several products write side by side into one buffer."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dim() != 2:
        raise KernelError(f"{what}: expected a CUDA matrix")
    if t.shape[1] > 1 and t.stride(1) != 1:
        raise KernelError(f"{what}: columns must lie together, got strides {t.stride()}")
    return t.data_ptr(), int(t.stride(0)) if t.shape[0] > 1 or t.stride(0) >= t.shape[1] else int(t.shape[1])


def _clear_args(clear: Optional[torch.Tensor], what: str):
    """(pointer, count) of a float32 buffer that a kernel zeroes on the side, or (None, 0)."""
    if clear is None:
        return None, 0
    _want(clear, f"{what} clear", torch.float32)
    return clear.data_ptr(), clear.numel()


def xielu(z: torch.Tensor, pq: torch.Tensor, out: torch.Tensor, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = softplus(p) z^2 + z / 2 where z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 elsewhere;
    ``z``: float32 [T, F] (may be a column slice), ``pq``: float32 [2] on the device. ``clear``: a float32 buffer zeroed
    on the side (for the product after it, when that sums partial results into its output)."""
    zp, ldz = _slice(z, "xielu z")
    _want(pq, "xielu numbers", torch.float32, 1)
    _want(out, "xielu out", ndim=2)
    if out.shape != z.shape or pq.numel() != 2:
        raise KernelError(f"xielu: z {tuple(z.shape)}, out {tuple(out.shape)}, {pq.numel()} numbers")
    lib = library("elementwise")
    _check(lib, lib.lp_xielu(zp, ldz, pq.data_ptr(), out.data_ptr(), _code(out, "xielu out"), z.shape[0], z.shape[1],
                             *_clear_args(clear, "xielu"), _stream()))
    return out


def gated_sum(x: torch.Tensor, a: Optional[torch.Tensor], a_gate=None, b: Optional[torch.Tensor] = None, b_gate=None, *,
              streams: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None, count: int = 0,
              keep_input: bool = False) -> torch.Tensor:
    """x <- x + a * sigmoid(ga + ba) + b * sigmoid(gb + bb), float32, in place. ``a_gate`` / ``b_gate``:
    ``(logits [T, d], may be a column slice; bias [d] or None)`` or None for an ungated branch; ``b`` may be None.
    ``streams`` [>= count, T, d] with ``mix`` [count]: the sum is kept as stream ``count - 1`` and x becomes
    sum_j mix[j] * streams[j]; ``keep_input`` first stores the incoming x as stream ``count - 2``."""
    _want(x, "gated_sum x", torch.float32, 2)
    T, d = x.shape

    def branch(t, gate, what):
        if t is None:
            return None, None, 0, None
        _want(t, f"gated_sum {what}", torch.float32, 2)
        if t.shape != x.shape:
            raise KernelError(f"gated_sum: {what} {tuple(t.shape)} does not match x {tuple(x.shape)}")
        if gate is None:
            return t.data_ptr(), None, 0, None
        logits, bias = gate
        gp, ldg = _slice(logits, f"gated_sum {what} gate")
        if logits.shape != x.shape:
            raise KernelError(f"gated_sum: {what} gate {tuple(logits.shape)} does not match x {tuple(x.shape)}")
        if bias is not None:
            _want(bias, f"gated_sum {what} gate bias", torch.float32, 1)
            if bias.numel() != d:
                raise KernelError(f"gated_sum: a gate bias of {bias.numel()} values for rows of {d}")
        return t.data_ptr(), gp, ldg, _ptr(bias)

    ap, agp, ald, abp = branch(a, a_gate, "a")
    bp, bgp, bld, bbp = branch(b, b_gate, "b")
    if streams is not None:
        _want(streams, "gated_sum streams", torch.float32, 3)
        _want(mix, "gated_sum mix", torch.float32, 1)
        if streams.shape[1:] != x.shape or streams.shape[0] < count or mix.numel() != count or count < 1:
            raise KernelError(f"gated_sum: streams {tuple(streams.shape)}, {mix.numel()} weights, count {count}")
    lib = library("elementwise")
    _check(lib, lib.lp_gated_sum(x.data_ptr(), ap, agp, ald, abp, bp, bgp, bld, bbp, _ptr(streams), _ptr(mix), int(count),
                                 1 if keep_input else 0, T, d, _stream()))
    return x


# --------------------------------------------------------------------------- rotation + cache write
@dataclass(frozen=True)
class Rotation:
    """What the kernels that prepare queries and keys can do to them on the way: rotate the first
    ``rotary_dim`` features of every head by ``position * inv_freq[pair]``, the pairs being
    (i, i + rotary_dim / 2) or, ``interleaved``, (2i, 2i + 1). ``rotary_dim == 0``: nothing.
    A position encoding that is such a rotation hands this to the kernels; any other rule is
    applied by its own part before they run."""
    inv_freq: Optional[torch.Tensor] = None      # float32 [rotary_dim / 2] on the device
    rotary_dim: int = 0
    interleaved: bool = False
    magnitude: float = 1.0                       # a factor on both cosine and sine (wavelength-stretched encodings)

    def checked(self, what: str, takes_magnitude: bool = False):
        """(pointer or None, rotary_dim, interleaved as int) after checking the frequencies."""
        if self.magnitude != 1.0 and not takes_magnitude:
            raise KernelError(f"{what}: a rotation with a factor of {self.magnitude} on cosine and sine is not supported here")
        if self.rotary_dim <= 0:
            return None, 0, 0
        _want(self.inv_freq, f"{what} inv_freq", torch.float32, 1)
        if self.inv_freq.numel() != self.rotary_dim // 2:
            raise KernelError(f"{what}: {self.inv_freq.numel()} frequencies for a rotary width of {self.rotary_dim}")
        return self.inv_freq.data_ptr(), int(self.rotary_dim), 1 if self.interleaved else 0


NO_ROTATION = Rotation()


def rope_cache_write(qkv: torch.Tensor, rotation: Rotation, positions: torch.Tensor,
                     seq_ids: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor,
                     pages: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate queries (and keys), write queries to ``q_out`` [T, H*hd] and keys and
    values into ``pages`` [num_pages, 2, G, page_size, hd]. ``pages=None``: queries only."""
    _want(qkv, "rope qkv", torch.float32, 2)
    _want(positions, "rope positions", torch.int32, 1)
    _want(seq_ids, "rope seq_ids", torch.int32, 1)
    _want(page_table, "rope page_table", torch.int32, 2)
    _want(q_out, "rope q_out", ndim=2)
    T = qkv.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if positions.numel() != T or seq_ids.numel() != T or q_out.shape != (T, H * hd):
        raise KernelError(f"rope: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}, {positions.numel()} positions")
    page_size, kv_code = 0, F32
    if pages is not None:
        _want(pages, "rope pages", ndim=5)
        if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
            raise KernelError(f"rope: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
        page_size, kv_code = pages.shape[3], _code(pages, "rope pages")
    freq_ptr, rotary_dim, interleaved = rotation.checked("rope")
    lib = library("elementwise")
    _check(lib, lib.lp_rope_cache_write(
        qkv.data_ptr(), qkv.shape[1], freq_ptr, positions.data_ptr(),
        seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], q_out.data_ptr(), _code(q_out, "rope q_out"),
        _ptr(pages), kv_code, T, H, G, hd, rotary_dim, interleaved, page_size, _stream()))


def rope_angles(positions: torch.Tensor, rotation: Rotation, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = (cos, sin) of float(positions[t]) * inv_freq[i], float32 [T, rotary_dim / 2, 2]: the angles of a
    step's tokens, formed once for a product whose epilogue rotates (:func:`gemm_qkv_rope`)."""
    _want(positions, "rope_angles positions", torch.int32, 1)
    _want(out, "rope_angles out", torch.float32, 3)
    freq_ptr, rotary_dim, _ = rotation.checked("rope_angles")
    T, half = positions.numel(), rotary_dim // 2
    if out.shape != (T, half, 2) or half == 0:
        raise KernelError(f"rope_angles: out {tuple(out.shape)} for {T} tokens and a rotary width of {rotary_dim}")
    lib = library("elementwise")
    _check(lib, lib.lp_rope_angles(positions.data_ptr(), freq_ptr, out.data_ptr(), T, half, _stream()))
    return out


QKV_ROPE_HEAD_SIZES = (32, 64, 128, 256)


def qkv_rope_serves(rotation: Rotation, head_dim: int) -> bool:
    """Whether :func:`gemm_qkv_rope` can apply this rotation to heads of this size in its epilogue."""
    if head_dim not in QKV_ROPE_HEAD_SIZES or rotation.rotary_dim not in (0, head_dim) or rotation.magnitude != 1.0:
        return False
    return rotation.rotary_dim == 0 or rotation.interleaved or head_dim >= 64


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, angles: Optional[torch.Tensor], interleaved: bool,
                  positions: torch.Tensor, seq_ids: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor,
                  pages: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """The fused projection of a step with many tokens on the tensor cores, with what follows it in its epilogue:
    ``x`` [T, K] x ``w`` [(H + 2G) * hd, K]^T (rows of queries, keys, values; ``[H * hd, K]`` and ``pages=None``
    for a layer without keys of its own), queries and keys rotated by ``angles`` (from :func:`rope_angles`;
    None: no rotation), queries written to ``q_out`` [T, H * hd], keys and values into ``pages`` at the tokens'
    positions. All bfloat16."""
    _want(x, "gemm_qkv_rope x", torch.bfloat16, 2)
    _want(w, "gemm_qkv_rope w", torch.bfloat16, 2)
    _want(q_out, "gemm_qkv_rope q_out", torch.bfloat16, 2)
    _want(positions, "gemm_qkv_rope positions", torch.int32, 1)
    _want(seq_ids, "gemm_qkv_rope seq_ids", torch.int32, 1)
    _want(page_table, "gemm_qkv_rope page_table", torch.int32, 2)
    T, K = x.shape
    H, G, hd = num_heads, num_kv_heads, head_dim
    heads = H + 2 * G if pages is not None else H
    if w.shape != (heads * hd, K) or q_out.shape != (T, H * hd) or positions.numel() != T or seq_ids.numel() != T:
        raise KernelError(f"gemm_qkv_rope: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}")
    page_size = 0
    if pages is not None:
        _want(pages, "gemm_qkv_rope pages", torch.bfloat16, 5)
        if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
            raise KernelError(f"gemm_qkv_rope: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
        page_size = pages.shape[3]
    half = 0
    if angles is not None:
        _want(angles, "gemm_qkv_rope angles", torch.float32, 3)
        half = angles.shape[1]
        if angles.shape != (T, half, 2):
            raise KernelError(f"gemm_qkv_rope: angles {tuple(angles.shape)} for {T} tokens")
    lib = library("gemm_tcgen05")
    _check(lib, lib.lp_gemm_qkv_rope(
        x.data_ptr(), w.data_ptr(), T, K, K, K, _ptr(angles), half, 1 if interleaved else 0, positions.data_ptr(),
        seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], q_out.data_ptr(), _ptr(pages), H, G, hd,
        page_size, kernel_status().data_ptr(), _stream()))


# --------------------------------------------------------------------------- matrix products
def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STORE) -> torch.Tensor:
    """out (=|+=) a @ w.T with float32 multiply-adds in increasing k.

    ``SWIGLU``: ``w`` is [2N, K], gate rows then up rows; out = silu(a gate^T) * (a up^T).
    """
    _want(a, "gemm a", ndim=2)
    _want(w, "gemm w", ndim=2)
    out_ptr, ldc = _out_matrix(out, "gemm out")
    M, K = a.shape
    N = out.shape[1]
    rows = 2 * N if mode == SWIGLU else N
    if w.shape != (rows, K) or out.shape[0] != M:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, mode {mode}")
    lib = library("gemm_plain")
    _check(lib, lib.lp_gemm_plain(a.data_ptr(), _code(a, "gemm a"), w.data_ptr(), _code(w, "gemm w"), out_ptr,
                                  _code(out, "gemm out"), M, N, K, K, K, ldc, mode, _stream()))
    return out


_num_sms = None


def num_sms() -> int:
    """Streaming multiprocessors of the current device (asked once)."""
    global _num_sms
    if _num_sms is None:
        require_gpu()
        _num_sms = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return _num_sms


_status = None


def kernel_status() -> torch.Tensor:
    """One int32 in device memory that kernels with bounded waits set when a wait runs out."""
    global _status
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status


def check_kernel_status() -> None:
    """Raise if a kernel reported a wait that ran out. Reads the word back, which synchronises."""
    if _status is not None and int(_status.item()) != 0:
        code = int(_status.item())
        _status.zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting on a barrier (code {code}: "
                          "1 = loader, 2 = MMA issuer, 3 = epilogue, 4-5 = operand maker; 2x the same in the "
                          "persistent product; 6 = a page of the decode attention)")


def _token_tile(tokens: int, gated: bool) -> int:
    # up to 64 tokens: the smallest tile that holds them; beyond: 128, of which two CTAs share an SM
    # (so one's epilogue runs under the other's MMAs); 256 remains available to callers
    for tile in (16, 32, 64):
        if tokens <= tile:
            return tile
    return 128


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The weight layout of the tensor-core gated product: for every 64 output features, their 64
    gate rows followed by their 64 up rows (features padded with zero rows to a multiple of 64)."""
    F, K = gate.shape
    if up.shape != gate.shape:
        raise KernelError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} differ")
    pad = -F % 64
    if pad:
        zeros = torch.zeros((pad, K), dtype=gate.dtype, device=gate.device)
        gate, up = torch.cat([gate, zeros]), torch.cat([up, zeros])
    blocks = (F + pad) // 64
    return torch.stack([gate.view(blocks, 64, K), up.view(blocks, 64, K)], dim=1).reshape(2 * (F + pad), K).contiguous()


def gemm_plan(tokens: int, features: int, k: int, mode: int):
    """(token tile, splits) that :func:`gemm` uses for these sizes."""
    k_blocks = -(-k // 64)
    tile = _token_tile(tokens, mode == SWIGLU)
    if mode == SWIGLU:
        return tile, 1
    ctas = -(-features // 128) * -(-tokens // tile)
    sms = num_sms()
    if ctas >= sms // 2 or k_blocks < 8:
        return tile, 1
    return tile, max(1, min(sms // ctas, k_blocks // 4))


FUSED_NORM_MAX_TOKENS = 4
PERSISTENT_MIN_TOKENS = 512


def _persistent_pays(tokens: int, features: int, k: int, mode: int) -> bool:
    """Whether the persistent form (one CTA per SM walking 128 x 256 tiles, 128 x 128 x 2 when gated)
    fills the SMs at least as well as separate CTAs of 128 x 128 tiles, two to an SM."""
    feat_tiles = -(-features // 128)
    persistent_tiles = feat_tiles * -(-tokens // (128 if mode == SWIGLU else 256))
    separate_ctas = feat_tiles * -(-tokens // 128)
    sms = num_sms()
    fill_p = persistent_tiles / (-(-persistent_tiles // sms) * sms)
    fill_s = separate_ctas / (-(-separate_ctas // (2 * sms)) * 2 * sms)
    # at equal fill the persistent form wins when the SMs are well filled (its tiles are twice as large and one
    # tile's epilogue hides under the next one's MMAs) or the K loop is long
    return fill_p > fill_s + 0.02 or (fill_p >= fill_s and (fill_p >= 0.8 or k >= 4096))


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STORE, *, block_tok: int = 0,
         splits: int = 0, cleared: bool = False, norm_after=None) -> torch.Tensor:
    """out (=|+=) a @ w.T on the tensor cores (bfloat16 in, float32 accumulation).

    ``a`` [tokens, K] and ``w`` [features, K] are bfloat16; for ``SWIGLU``, ``w`` is the
    interleaved gate/up matrix of :func:`interleave_gate_up` and ``out`` [tokens, features] gets
    silu(gate) * up. When few CTAs would cover the output, the K range is split over more of
    them and the partial sums meet in float32 atomics; ``cleared`` says that ``out`` is already
    zero for that. ``block_tok`` / ``splits`` override the plan (tests).

    ``norm_after = (gain, eps, normed_out, clear, counter)`` (``ACCUMULATE`` only, at most
    ``FUSED_NORM_MAX_TOKENS`` rows): once all CTAs have added their parts, the last one writes
    the RMS norm of every row of ``out`` to ``normed_out`` (bfloat16) and zeroes ``clear``
    (a float32 tensor or None). ``counter``: one int32 on the device that is zero between uses
    (the CTAs count themselves there; the last one sets it back).
    """
    _want(a, "gemm a", torch.bfloat16, 2)
    _want(w, "gemm w", torch.bfloat16, 2)
    out_ptr, ldc = _out_matrix(out, "gemm out")          # may be a column slice of a wider buffer
    M, K = a.shape
    N = out.shape[1]
    rows = 128 * (-(-N // 64)) if mode == SWIGLU else N
    if w.shape != (rows, K) or out.shape[0] != M:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, mode {mode}")
    if M == 0:
        return out
    if ldc != N and norm_after is not None:
        raise KernelError("gemm: a following norm needs an output of whole rows")
    lib = library("gemm_tcgen05")
    status = kernel_status()
    if (M >= PERSISTENT_MIN_TOKENS and not block_tok and not splits and norm_after is None
            and _persistent_pays(M, N, K, mode)):
        # many tokens: one CTA per SM walks over the tiles, epilogue and MMAs of neighbouring tiles overlap
        if mode == ACCUMULATE and out.dtype != torch.float32:
            raise KernelError("gemm: accumulation needs a float32 output")
        _check(lib, lib.lp_gemm_persistent(a.data_ptr(), w.data_ptr(), out_ptr, _code(out, "gemm out"), M, N, K,
                                           K, K, ldc, mode, status.data_ptr(), _stream()))
        return out
    tile, n_splits = gemm_plan(M, N, K, mode)
    tile = block_tok or tile
    n_splits = 1 if mode == SWIGLU else (splits or n_splits)
    if mode == ACCUMULATE:
        if out.dtype != torch.float32:
            raise KernelError("gemm: accumulation needs a float32 output")
    elif mode == STORE and n_splits > 1:
        if out.dtype != torch.float32:
            n_splits = 1
        elif not cleared:
            out.zero_()
    norm_args = (None, 0.0, None, None, 0, None)
    if norm_after is not None:
        gain, eps, normed, clear, counter = norm_after
        if mode != ACCUMULATE or M > FUSED_NORM_MAX_TOKENS:
            raise KernelError("gemm: a following norm needs an accumulating product of few rows")
        _want(gain, "gemm norm gain", torch.float32, 1)
        _want(normed, "gemm normed out", torch.bfloat16, 2)
        if gain.numel() != N or normed.shape != (M, N):
            raise KernelError(f"gemm: norm gain {tuple(gain.shape)}, normed out {tuple(normed.shape)} for [{M}, {N}]")
        if clear is not None:
            _want(clear, "gemm norm clear", torch.float32)
        _want(counter, "gemm norm counter", torch.int32, 1)
        norm_args = (gain.data_ptr(), float(eps), normed.data_ptr(), _ptr(clear),
                     clear.numel() if clear is not None else 0, counter.data_ptr())
    _check(lib, lib.lp_gemm_tcgen05(a.data_ptr(), w.data_ptr(), out_ptr, _code(out, "gemm out"), M, N, K,
                                    K, K, ldc, mode, tile, n_splits, status.data_ptr(), *norm_args, _stream()))
    return out


FEW_TOKENS_MAX = 64                  # what the few-token entry takes
# Up to where the parts choose it with the norm inside (``settings.few_tokens``). Measured at the 1B shape (ms per
# step, norm inside against separate norm kernels): 8 tokens 0.68 / 0.76 (the mma.sync kernel); 12 tokens
# 0.79 / 0.87, 16 tokens 0.80 / 0.88, 20 tokens 0.84 / 0.89, 32 tokens 0.86 / 0.94 (the tcgen05 kernel with operand
# makers); 48 tokens 1.07 / 0.99 and 64 tokens 1.14 / 1.06: beyond 32 tokens the norm kernels stay.
FEW_TOKENS = max(0, min(int(settings.few_tokens), FEW_TOKENS_MAX))


def gemm_few(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STORE, *, norm=None,
             sumsq: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None) -> bool:
    """out (=|+=) f(x) @ w.T for at most ``FEW_TOKENS_MAX`` rows, with what a decode step fuses around it
    (up to 16 rows, 8 with a norm, the mma.sync kernel; beyond that the one-tile tcgen05 kernels).

    ``norm = (gain, eps)``: ``x`` is the float32 residual stream and the product applies the RMS norm on
    the way in. If the K range is then shared out over CTAs (few output features), ``out`` still lacks each
    row's factor: ``sumsq`` [rows] (zero beforehand) receives the rows' sums of squares, the reader applies
    ``1 / sqrt(sumsq / K + eps)``, and the function returns True. ``out`` must be zero beforehand in that
    case, as for any ``STORE`` whose partial sums meet in atomics. ``zero``: a float32 buffer cleared on the
    side. Without ``norm``, ``x`` is bfloat16."""
    _want(w, "gemm_few w", torch.bfloat16, 2)
    _want(out, "gemm_few out", ndim=2)
    _want(x, "gemm_few x", torch.float32 if norm is not None else torch.bfloat16, 2)
    M, K = x.shape
    N = out.shape[1]
    rows = 128 * (-(-N // 64)) if mode == SWIGLU else N
    if w.shape != (rows, K) or out.shape[0] != M or M > FEW_TOKENS_MAX:
        raise KernelError(f"gemm_few: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, mode {mode}")
    _, splits = gemm_plan(M, N, K, mode)
    if mode == STORE and splits > 1 and out.dtype != torch.float32:
        splits = 1
    gain = eps = None
    if norm is not None:
        gain, eps = norm
        _want(gain, "gemm_few gain", torch.float32, 1)
        if gain.numel() != K:
            raise KernelError(f"gemm_few: a gain of {gain.numel()} values for rows of {K}")
        if splits > 1 and sumsq is None:
            splits = 1
    deferred = norm is not None and splits > 1
    if deferred:
        _want(sumsq, "gemm_few sumsq", torch.float32, 1)
        if sumsq.numel() < M:
            raise KernelError(f"gemm_few: {sumsq.numel()} sums of squares for {M} rows")
    if zero is not None:
        _want(zero, "gemm_few zero", torch.float32)
    lib = library("gemm_tcgen05")
    _check(lib, lib.lp_gemm_fewtok(
        x.data_ptr(), _code(x, "gemm_few x"), w.data_ptr(), out.data_ptr(), _code(out, "gemm_few out"), M, N, K, K, K, N,
        mode, splits, kernel_status().data_ptr(), _ptr(gain), float(eps) if eps is not None else 0.0,
        sumsq.data_ptr() if deferred else None, _ptr(zero), zero.numel() if zero is not None else 0, _stream()))
    return deferred


# --------------------------------------------------------------------------- attention
def attention_plain(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor,
                    seq_ids: torch.Tensor, positions: torch.Tensor, *, num_heads: int, num_kv_heads: int,
                    head_dim: int, scale: float, window: Optional[int], softcap: Optional[float] = None,
                    sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """Each query token attends over the cached keys of its sequence up to its own
    position (and within ``window``, if given). ``softcap``: scores become softcap * tanh(score / softcap) after the
    scale; ``sinks``: float32 [H], a logit per head that enters the softmax's denominator once. ``keep_first`` (with a
    window): the sequence's first ``keep_first`` tokens stay visible to every later query."""
    _check_sinks(sinks, num_heads, "attention")
    _want(q, "attention q", ndim=2)
    _want(out, "attention out", q.dtype, 2)
    _want(pages, "attention pages", ndim=5)
    _want(page_table, "attention page_table", torch.int32, 2)
    _want(seq_ids, "attention seq_ids", torch.int32, 1)
    _want(positions, "attention positions", torch.int32, 1)
    T = q.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if q.shape != (T, H * hd) or out.shape != q.shape or seq_ids.numel() != T or positions.numel() != T:
        raise KernelError(f"attention: q {tuple(q.shape)}, out {tuple(out.shape)} for {H} heads of {hd}")
    if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
        raise KernelError(f"attention: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
    lib = library("attention_plain")
    _check(lib, lib.lp_attention_plain(
        q.data_ptr(), out.data_ptr(), _code(q, "attention q"), pages.data_ptr(), _code(pages, "attention pages"),
        page_table.data_ptr(), page_table.shape[1], seq_ids.data_ptr(), positions.data_ptr(), T, H, G, hd,
        pages.shape[3], float(scale), int(window) if window else 0, float(softcap or 0.0), _ptr(sinks),
        int(keep_first) if window else 0, _stream()))
    return out


def _check_sinks(sinks: Optional[torch.Tensor], num_heads: int, what: str) -> None:
    if sinks is not None:
        _want(sinks, f"{what} sinks", torch.float32, 1)
        if sinks.numel() != num_heads:
            raise KernelError(f"{what}: {sinks.numel()} sinks for {num_heads} heads")


def _check_attention(q, out, pages, page_table, H, G, hd, what):
    _want(q, f"{what} q", torch.bfloat16, 2)
    _want(out, f"{what} out", torch.bfloat16, 2)
    _want(pages, f"{what} pages", torch.bfloat16, 5)
    _want(page_table, f"{what} page_table", torch.int32, 2)
    if q.shape[1] != H * hd or out.shape != q.shape:
        raise KernelError(f"{what}: q {tuple(q.shape)}, out {tuple(out.shape)} for {H} heads of {hd}")
    if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
        raise KernelError(f"{what}: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")


tcgen05_attention = True      # tests switch it off to reach the mma.sync kernel at every size


def attention_prefill(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, max_new: int, *, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                      softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None,
                      exact_weights: bool = False, keep_first: int = 0) -> torch.Tensor:
    """Tensor-core attention for a step that brings several tokens per sequence. ``keep_first`` (with a window): the
    sequence's first ``keep_first`` tokens stay visible to every later query.
    ``q_start`` [B+1]: offsets of each sequence's new tokens; ``kv_len`` [B]: lengths after the step.
    ``exact_weights``: the softmax weights enter the product with the values at float32 precision (as a bfloat16
    value plus a bfloat16 rest, two products) instead of rounded to bfloat16."""
    _check_attention(q, out, pages, page_table, num_heads, num_kv_heads, head_dim, "attention_prefill")
    _want(q_start, "attention_prefill q_start", torch.int32, 1)
    _want(kv_len, "attention_prefill kv_len", torch.int32, 1)
    B = kv_len.numel()
    if q_start.numel() != B + 1 or page_table.shape[0] != B:
        raise KernelError(f"attention_prefill: {B} sequences, {q_start.numel()} offsets, table {tuple(page_table.shape)}")
    _check_sinks(sinks, num_heads, "attention_prefill")
    keep_first = int(keep_first) if window else 0
    if (head_dim in (64, 128) and max_new > 64 and tcgen05_attention and not softcap and sinks is None and not exact_weights
            and not keep_first):
        # long runs of new tokens with heads of 64 or 128: scores and P V on the tcgen05 tensor cores
        lib = library("attention_tcgen05")
        _check(lib, lib.lp_attention_prefill_tc(
            q.data_ptr(), out.data_ptr(), pages.data_ptr(), pages.shape[0], page_table.data_ptr(),
            page_table.shape[1], q_start.data_ptr(), kv_len.data_ptr(), B, q.shape[0], int(max_new), num_heads,
            num_kv_heads, head_dim, pages.shape[3], float(scale), int(window) if window else 0,
            kernel_status().data_ptr(), _stream()))
        return out
    lib = library("attention_mma")
    _check(lib, lib.lp_attention_prefill(
        q.data_ptr(), out.data_ptr(), pages.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        q_start.data_ptr(), kv_len.data_ptr(), B, int(max_new), num_heads, num_kv_heads, head_dim, pages.shape[3],
        float(scale), int(window) if window else 0, float(softcap or 0.0), _ptr(sinks), 1 if exact_weights else 0,
        keep_first, _stream()))
    return out


MIN_SHARE_PAGES = 8
LONG_SHARE_PAGES = 14


def decode_split(batch: int, num_kv_heads: int, num_heads: int, table_width: int):
    """How a decode step's pages are shared out over CTAs: (pages per share, shares) for page tables of
    ``table_width`` entries. A share and the merge of shares cost several dependent round trips to memory, so a
    sequence is cut only into shares of at least ``MIN_SHARE_PAGES`` pages, and into no more CTAs than there are SMs
    (the kernel then gives each CTA 16 warps), or twice that for shares of twice the pages. This is the most shares
    a sequence can get; the kernels fit the
    number to each sequence's own length (at batch 8 and a context of 600 in a table of 16 pages: one share,
    0.69 ms per step, against 0.75 with two shares of 8 pages)."""
    groups = decode_groups(batch, num_heads, num_kv_heads)
    shares = max(1, min(table_width // MIN_SHARE_PAGES, num_sms() // groups))
    # long sequences: up to two CTAs per SM (8 warps each) if every share still has LONG_SHARE_PAGES pages. Measured with the pages
    # brought by TMA, ms per step at contexts of 3.5 k / 1 k: batch 4: 0.771 -> 0.756 / 0.716 -> 0.711, batch 8:
    # 0.837 -> 0.818 / unchanged, batch 16: 1.080 -> 1.048 / 0.828 (0.856 with shares of 8 pages there)
    shares = max(shares, min(table_width // LONG_SHARE_PAGES, 2 * num_sms() // groups))
    per = -(-table_width // shares)
    return per, -(-table_width // per)


def attention_decode(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor,
                     kv_len: torch.Tensor, scratch, *, num_heads: int, num_kv_heads: int, head_dim: int,
                     scale: float, window: Optional[int], pages_per_split: int = 0, num_splits: int = 0,
                     softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None,
                     exact_weights: bool = False, keep_first: int = 0) -> torch.Tensor:
    """Tensor-core attention for a step of one token per sequence. ``scratch(name, shape, dtype)``
    supplies the float32 buffer for the partial results of the shares. ``keep_first`` (with a window, shares fitted to
    the sequences): the sequence's first ``keep_first`` tokens stay visible; their pages are visited first."""
    _check_attention(q, out, pages, page_table, num_heads, num_kv_heads, head_dim, "attention_decode")
    _want(kv_len, "attention_decode kv_len", torch.int32, 1)
    _check_sinks(sinks, num_heads, "attention_decode")
    B = kv_len.numel()
    if q.shape[0] != B or page_table.shape[0] != B:
        raise KernelError(f"attention_decode: {B} sequences, q {tuple(q.shape)}, table {tuple(page_table.shape)}")
    fitted = not pages_per_split or not num_splits
    keep_first = int(keep_first) if window else 0
    if keep_first and not fitted:
        raise KernelError("attention_decode: kept first tokens need shares fitted to the sequences")
    if fitted:
        pages_per_split, num_splits = decode_split(B, num_kv_heads, num_heads, page_table.shape[1])
    buf = scratch("attention_partials", (B * num_heads * num_splits * (head_dim + 2),), torch.float32)
    lib = library("attention_mma")
    if fitted:
        _check(lib, lib.lp_attention_decode_fitted(
            q.data_ptr(), out.data_ptr(), pages.data_ptr(), page_table.data_ptr(), page_table.shape[1],
            kv_len.data_ptr(), buf.data_ptr(), B, num_heads, num_kv_heads, head_dim, pages.shape[3], float(scale),
            int(window) if window else 0, num_splits, MIN_SHARE_PAGES, float(softcap or 0.0), _ptr(sinks),
            1 if exact_weights else 0, keep_first, _stream()))
        return out
    _check(lib, lib.lp_attention_decode(
        q.data_ptr(), out.data_ptr(), pages.data_ptr(), page_table.data_ptr(), page_table.shape[1], kv_len.data_ptr(),
        buf.data_ptr(), B, num_heads, num_kv_heads, head_dim, pages.shape[3], float(scale),
        int(window) if window else 0, pages_per_split, num_splits, float(softcap or 0.0), _ptr(sinks),
        1 if exact_weights else 0, _stream()))
    return out


DECODE_HEAD_ROWS = 8          # query heads that one CTA of a decode step serves (HEAD_ROWS of the kernels)


def decode_groups(batch: int, num_heads: int, num_kv_heads: int) -> int:
    """How many groups of CTAs a fused decode step has (each merges its own shares and counts them in a
    counter of its own)."""
    return batch * num_kv_heads * (-(-(num_heads // num_kv_heads) // DECODE_HEAD_ROWS))


def attention_decode_fused(qkv: torch.Tensor, rotation: Rotation, out: torch.Tensor,
                           pages: torch.Tensor, page_table: torch.Tensor, kv_len: torch.Tensor, scratch,
                           counters: torch.Tensor, *,
                           num_heads: int, num_kv_heads: int, head_dim: int,
                           write_kv: bool, scale: float, window: Optional[int], pages_per_split: int = 0,
                           num_splits: int = 0, row_sumsq: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                           norm_width: int = 0) -> torch.Tensor:
    """A decode step's attention from the float32 fused projection ``qkv`` [B, (H + 2G) * hd]
    (``[B, H * hd]`` when ``write_kv`` is false): rotates the queries, rotates and stores the new
    key, stores the new value, attends over the pages and merges the shares, in one kernel.
    ``counters``: int32, at least ``decode_groups(B, H, G)`` entries, zero between uses (the shares of a
    group count themselves there and the last one sets the counter back).
    Without ``pages_per_split`` / ``num_splits`` the shares are fitted to each sequence's own length.
    ``row_sumsq`` [B]: ``qkv`` still lacks the factor of the RMS norm of its input; row b is scaled by
    ``1 / sqrt(row_sumsq[b] / norm_width + norm_eps)`` as it is read."""
    _want(qkv, "attention_decode_fused qkv", torch.float32, 2)
    _want(out, "attention_decode_fused out", torch.bfloat16, 2)
    _want(pages, "attention_decode_fused pages", torch.bfloat16, 5)
    _want(page_table, "attention_decode_fused page_table", torch.int32, 2)
    _want(kv_len, "attention_decode_fused kv_len", torch.int32, 1)
    _want(counters, "attention_decode_fused counters", torch.int32, 1)
    H, G, hd = num_heads, num_kv_heads, head_dim
    B = kv_len.numel()
    heads = H + 2 * G if write_kv else H
    if qkv.shape != (B, heads * hd) or out.shape != (B, H * hd) or page_table.shape[0] != B:
        raise KernelError(f"attention_decode_fused: qkv {tuple(qkv.shape)}, out {tuple(out.shape)}, {B} sequences")
    if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
        raise KernelError(f"attention_decode_fused: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
    freq_ptr, rotary_dim, interleaved = rotation.checked("attention_decode_fused")
    fitted = not pages_per_split or not num_splits
    if fitted:                       # as many shares as the tables allow; the kernel fits them to each sequence
        _, num_splits = decode_split(B, G, H, page_table.shape[1])
        pages_per_split = page_table.shape[1]
    if counters.numel() < decode_groups(B, H, G):
        raise KernelError(f"attention_decode_fused: {counters.numel()} counters for {decode_groups(B, H, G)} groups")
    buf = scratch("attention_partials", (B * H * num_splits * (hd + 2),), torch.float32)
    lib = library("attention_mma")
    _check(lib, lib.lp_attention_decode_fused(
        qkv.data_ptr(), qkv.shape[1], freq_ptr, rotary_dim, interleaved,
        out.data_ptr(), pages.data_ptr(), 1 if write_kv else 0, page_table.data_ptr(), page_table.shape[1],
        kv_len.data_ptr(), buf.data_ptr(), counters.data_ptr(), B, H, G, hd, pages.shape[3], float(scale),
        int(window) if window else 0, pages_per_split, num_splits, MIN_SHARE_PAGES if fitted else 0, _ptr(row_sumsq),
        float(norm_eps), int(norm_width), pages.shape[0], kernel_status().data_ptr(), _stream()))
    return out


def attention(ctx, q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor, *,
              num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
              fast: bool, softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None,
              exact_weights: bool = False, keep_first: int = 0) -> torch.Tensor:
    """Attention of the step's tokens over the cache; picks the kernel for the step's shape. ``keep_first`` (with a
    window): the first tokens of a sequence that stay visible beyond the window."""
    tensor_cores = (fast and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16
                    and head_dim % 16 == 0 and head_dim <= 256)
    keep_first = int(keep_first) if window else 0
    if tensor_cores and ctx.all_single:
        return attention_decode(q, out, pages, page_table, ctx.kv_len, ctx.buffer, num_heads=num_heads,
                                num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window,
                                softcap=softcap, sinks=sinks, exact_weights=exact_weights, keep_first=keep_first)
    if tensor_cores and not ctx.all_single:
        return attention_prefill(q, out, pages, page_table, ctx.q_start, ctx.kv_len, ctx.max_new,
                                 num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale,
                                 window=window, softcap=softcap, sinks=sinks, exact_weights=exact_weights,
                                 keep_first=keep_first)
    return attention_plain(q, out, pages, page_table, ctx.seq_ids, ctx.positions, num_heads=num_heads,
                           num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window, softcap=softcap,
                           sinks=sinks, keep_first=keep_first)


# --------------------------------------------------------------------------- latent attention
def latent_prepare(proj: torch.Tensor, q_off: int, kv_off: int, gain: torch.Tensor, eps: float, rotation: Rotation,
                   positions: torch.Tensor, seq_ids: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor,
                   pages: torch.Tensor, *, num_heads: int, nope_dim: int, rope_dim: int, kv_rank: int,
                   latent_out: Optional[torch.Tensor] = None, shared_out: Optional[torch.Tensor] = None,
                   q_half: Optional[torch.Tensor] = None, q_from: Optional[torch.Tensor] = None) -> None:
    """From the float32 projection ``proj`` [T, F] (queries at column ``q_off``, [H, nope + rope]; latent and
    shared key part at ``kv_off``, [rank + rope]): RMS-norm the latent with ``gain``, rotate the shared key
    part and write both into ``pages`` [num_pages, page_size, rank + rope] at the tokens' positions; rotate the
    queries' rope parts and write the queries to ``q_out`` float32 [T, H, nope + rope]. Optional bfloat16 copies
    that lie together, for a step that forms every head's keys and values outright: ``latent_out`` [T, rank],
    ``shared_out`` [T, rope], ``q_half`` [T, H * hd] with hd >= nope + rope (heads padded with zeros).
    ``q_from``: float32 [T, H * (nope + rope)] (may be a column slice): the queries, when they come from a product
    of their own (queries formed through a latent) instead of from ``proj``."""
    _want(proj, "latent_prepare proj", torch.float32, 2)
    _want(gain, "latent_prepare gain", torch.float32, 1)
    _want(positions, "latent_prepare positions", torch.int32, 1)
    _want(seq_ids, "latent_prepare seq_ids", torch.int32, 1)
    _want(page_table, "latent_prepare page_table", torch.int32, 2)
    _want(q_out, "latent_prepare q_out", torch.float32, 3)
    _want(pages, "latent_prepare pages", ndim=3)
    T = proj.shape[0]
    H, dn, dr, rank = num_heads, nope_dim, rope_dim, kv_rank
    if (q_out.shape != (T, H, dn + dr) or pages.shape[2] != rank + dr or gain.numel() != rank
            or positions.numel() != T or seq_ids.numel() != T):
        raise KernelError(f"latent_prepare: proj {tuple(proj.shape)}, q_out {tuple(q_out.shape)}, pages "
                          f"{tuple(pages.shape)} for {H} heads of {dn} + {dr} over rank {rank}")
    for extra, shape, what in ((latent_out, (T, rank), "latent_out"), (shared_out, (T, dr), "shared_out")):
        if extra is not None:
            _want(extra, f"latent_prepare {what}", torch.bfloat16, 2)
            if extra.shape != shape:
                raise KernelError(f"latent_prepare: {what} {tuple(extra.shape)}, expected {shape}")
    q_half_hd = 0
    if q_half is not None:
        _want(q_half, "latent_prepare q_half", torch.bfloat16, 2)
        q_half_hd = q_half.shape[1] // H
        if q_half.shape[0] != T or q_half.shape[1] != H * q_half_hd or q_half_hd < dn + dr:
            raise KernelError(f"latent_prepare: q_half {tuple(q_half.shape)} for {H} heads of {dn + dr}")
    freq_ptr, rot, interleaved = rotation.checked("latent_prepare", takes_magnitude=True)
    q_ptr, ldq = None, 0
    if q_from is not None:
        q_ptr, ldq = _slice(q_from, "latent_prepare q_from")
        if q_from.shape != (T, H * (dn + dr)):
            raise KernelError(f"latent_prepare: queries {tuple(q_from.shape)} for {H} heads of {dn + dr}")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_prepare(
        proj.data_ptr(), proj.shape[1], int(q_off), int(kv_off), gain.data_ptr(), float(eps), freq_ptr, rot,
        positions.data_ptr(), seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], q_out.data_ptr(),
        pages.data_ptr(), _code(pages, "latent_prepare pages"), T, H, dn, dr, rank, pages.shape[1], _ptr(latent_out),
        _ptr(shared_out), _ptr(q_half), q_half_hd, q_ptr, ldq, interleaved, float(rotation.magnitude), _stream()))


def latent_query_norm(proj: torch.Tensor, offset: int, gain: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[t] = rms_norm(proj[t, offset:offset + rank]) * gain for the float32 projection ``proj`` [T, F]: the norm of
    the latent that queries go through. ``out``: [T, rank], float32 or bfloat16."""
    _want(proj, "latent_query_norm proj", torch.float32, 2)
    _want(gain, "latent_query_norm gain", torch.float32, 1)
    _want(out, "latent_query_norm out", ndim=2)
    rank = gain.numel()
    if out.shape != (proj.shape[0], rank):
        raise KernelError(f"latent_query_norm: out {tuple(out.shape)} for {proj.shape[0]} tokens and rank {rank}")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_query_norm(proj.data_ptr(), proj.shape[1], int(offset), rank, gain.data_ptr(), float(eps),
                                         out.data_ptr(), _code(out, "latent_query_norm out"), proj.shape[0], _stream()))
    return out


def latent_heads_to_pages(kv: torch.Tensor, shared_part: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                          table: torch.Tensor, kv_len: torch.Tensor, pages: torch.Tensor, *, num_heads: int, nope_dim: int,
                          rope_dim: int, value_dim: int) -> None:
    """Lay the heads' keys and values of a step's tokens out as pages of ordinary keys and values
    [num_pages, 2, H, page_size, hd] with hd >= nope + rope: key of head h = [kv[t, h * nope + :] | shared_part[t]],
    value of head h = kv[t, H * nope + h * dv + :], both padded with zeros. All bfloat16; ``table`` [B, W] names the pages. The step
    holds every position of its sequences (``kv_len`` [B]); the rest of each sequence's last page is cleared."""
    H, dn, dr, dv = num_heads, nope_dim, rope_dim, value_dim
    _want(kv, "latent_heads_to_pages kv", torch.bfloat16, 2)
    _want(shared_part, "latent_heads_to_pages shared part", torch.bfloat16, 2)
    _want(pages, "latent_heads_to_pages pages", torch.bfloat16, 5)
    _want(table, "latent_heads_to_pages table", torch.int32, 2)
    _want(kv_len, "latent_heads_to_pages kv_len", torch.int32, 1)
    T = kv.shape[0]
    if (kv.shape[1] != H * (dn + dv) or shared_part.shape != (T, dr) or pages.shape[1] != 2 or pages.shape[2] != H
            or pages.shape[4] < dn + dr or positions.numel() != T or seq_ids.numel() != T):
        raise KernelError(f"latent_heads_to_pages: kv {tuple(kv.shape)}, shared part {tuple(shared_part.shape)}, pages "
                          f"{tuple(pages.shape)}")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_heads_to_pages(kv.data_ptr(), shared_part.data_ptr(), positions.data_ptr(), seq_ids.data_ptr(),
                                             table.data_ptr(), table.shape[1], kv_len.data_ptr(), pages.data_ptr(), T, H, dn, dr, dv,
                                             pages.shape[3], pages.shape[4], _stream()))


def latent_gate_heads(heads: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, *, num_heads: int,
                      head_dim: int, value_dim: int, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h * dv + v] = heads[t, h * hd + v] * sigmoid(gate[t, h]) (bfloat16; ``gate`` float32 [T, H], may be a
    column slice, or None)."""
    _want(heads, "latent_gate_heads heads", torch.bfloat16, 2)
    _want(out, "latent_gate_heads out", torch.bfloat16, 2)
    T = heads.shape[0]
    if heads.shape[1] != num_heads * head_dim or out.shape != (T, num_heads * value_dim):
        raise KernelError(f"latent_gate_heads: heads {tuple(heads.shape)}, out {tuple(out.shape)}")
    gp, ldg = (None, 0)
    if gate is not None:
        gp, ldg = _slice(gate, "latent_gate_heads gate")
        if gate.shape != (T, num_heads):
            raise KernelError(f"latent_gate_heads: gate {tuple(gate.shape)} for {T} tokens and {num_heads} heads")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_gate_heads(heads.data_ptr(), gp, ldg, out.data_ptr(), T, num_heads, head_dim, value_dim,
                                         *_clear_args(clear, "latent_gate_heads"), _stream()))
    return out


def latent_absorb(q: torch.Tensor, k_up: torch.Tensor, out: torch.Tensor, *, nope_dim: int, rope_dim: int) -> torch.Tensor:
    """out[t, h] = [k_up[h]^T q[t, h, :nope] | q[t, h, nope:]]: float32 [T, H, rank + rope] from ``q`` float32
    [T, H, nope + rope] and ``k_up`` [H * nope, rank]."""
    _want(q, "latent_absorb q", torch.float32, 3)
    _want(k_up, "latent_absorb k_up", ndim=2)
    _want(out, "latent_absorb out", torch.float32, 3)
    T, H, hd = q.shape
    rank = k_up.shape[1]
    if hd != nope_dim + rope_dim or k_up.shape[0] != H * nope_dim or out.shape != (T, H, rank + rope_dim):
        raise KernelError(f"latent_absorb: q {tuple(q.shape)}, k_up {tuple(k_up.shape)}, out {tuple(out.shape)}")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_absorb(q.data_ptr(), k_up.data_ptr(), _code(k_up, "latent_absorb k_up"), out.data_ptr(),
                                     T, H, nope_dim, rope_dim, rank, _stream()))
    return out


def latent_shares(batch: int, max_new: int, num_heads: int, table_width: int, page_size: int) -> int:
    """Into how many shares :func:`latent_attend` cuts a sequence's keys: one while the (token, head) rows
    alone fill the SMs, else as many as the SMs have room for, down to shares of one block of 32 keys."""
    rows = library("latent_attention").lp_latent_attend_rows()
    ctas = batch * -(-max_new * num_heads // rows)
    return max(1, min(num_sms() // max(ctas, 1), table_width * (page_size // 32)))


def latent_attend(q_abs: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor, q_start: torch.Tensor,
                  kv_len: torch.Tensor, partials: torch.Tensor, *, max_new: int, kv_rank: int, scale: float,
                  window: Optional[int] = None) -> torch.Tensor:
    """Causal softmax attention of the absorbed queries ``q_abs`` float32 [T, H, rank + rope] over the rows of
    ``pages`` [num_pages, page_size, rank + rope]; ``partials`` float32 [T, H, shares, rank + 2] receives each
    share's unnormalised latent sum, maximum and sum of weights. ``window``: a query at position p sees the keys at
    positions p - window + 1 .. p only."""
    _want(q_abs, "latent_attend q", torch.float32, 3)
    _want(pages, "latent_attend pages", ndim=3)
    _want(page_table, "latent_attend page_table", torch.int32, 2)
    _want(q_start, "latent_attend q_start", torch.int32, 1)
    _want(kv_len, "latent_attend kv_len", torch.int32, 1)
    _want(partials, "latent_attend partials", torch.float32, 4)
    T, H, Dk = q_abs.shape
    B = kv_len.numel()
    shares = partials.shape[2]
    if (pages.shape[2] != Dk or kv_rank > Dk or partials.shape != (T, H, shares, kv_rank + 2)
            or q_start.numel() != B + 1 or page_table.shape[0] != B):
        raise KernelError(f"latent_attend: q {tuple(q_abs.shape)}, pages {tuple(pages.shape)}, partials "
                          f"{tuple(partials.shape)}, {B} sequences")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_attend(q_abs.data_ptr(), pages.data_ptr(), _code(pages, "latent_attend pages"),
                                     page_table.data_ptr(), page_table.shape[1], q_start.data_ptr(), kv_len.data_ptr(),
                                     partials.data_ptr(), B, int(max_new), H, kv_rank, Dk - kv_rank, pages.shape[1],
                                     float(scale), shares, int(window) if window else 0, _stream()))
    return partials


LATENT_ROWS_FORM_TOKENS = 64      # up to here latent_expand runs one CTA per (token, head) row and merges the shares itself


def latent_merge(partials: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The shares of every (token, head) row of ``partials`` [T, H, shares, rank + 2] merged into one share
    ``out`` [T, H, 1, rank + 2] whose sum of weights is one."""
    _want(partials, "latent_merge partials", torch.float32, 4)
    _want(out, "latent_merge out", torch.float32, 4)
    T, H, shares, width = partials.shape
    if out.shape != (T, H, 1, width):
        raise KernelError(f"latent_merge: partials {tuple(partials.shape)}, out {tuple(out.shape)}")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_merge(partials.data_ptr(), shares, out.data_ptr(), T * H, width - 2, _stream()))
    return out


def latent_expand(partials: torch.Tensor, v_up: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, *,
                  value_dim: int, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h * dv + v] = sigmoid(gate[t, h]) * (v_up[h] latent[t, h])[v], the latent being the merge of the
    shares in ``partials``; ``gate``: float32 [T, H] (may be a column slice) or None."""
    _want(partials, "latent_expand partials", torch.float32, 4)
    _want(v_up, "latent_expand v_up", ndim=2)
    _want(out, "latent_expand out", ndim=2)
    T, H, shares, width = partials.shape
    rank = width - 2
    if v_up.shape != (H * value_dim, rank) or out.shape != (T, H * value_dim):
        raise KernelError(f"latent_expand: partials {tuple(partials.shape)}, v_up {tuple(v_up.shape)}, out {tuple(out.shape)}")
    gp, ldg = (None, 0)
    if gate is not None:
        gp, ldg = _slice(gate, "latent_expand gate")
        if gate.shape != (T, H):
            raise KernelError(f"latent_expand: gate {tuple(gate.shape)} for {T} tokens and {H} heads")
    lib = library("latent_attention")
    _check(lib, lib.lp_latent_expand(partials.data_ptr(), shares, v_up.data_ptr(), _code(v_up, "latent_expand v_up"), gp, ldg,
                                     out.data_ptr(), _code(out, "latent_expand out"), T, H, rank, value_dim,
                                     *_clear_args(clear, "latent_expand"), _stream()))
    return out


# --------------------------------------------------------------------------- gated linear attention
def gla_decay(low: torch.Tensor, up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, tau: float = 1.0,
              double_exp: bool = False) -> torch.Tensor:
    """out[t, c] = sigmoid(up[c] . low[t] + bias[c]) ** (1 / tau), float32; ``low``: float32 [T, R] (may be a column
    slice), ``up``: [C, R]. ``double_exp``: out[t, c] = exp(-exp(up[c] . tanh(low[t]) + bias[c])) instead (the decay of
    the time-mixing family)."""
    lp, ldl = _slice(low, "gla_decay low")
    _want(up, "gla_decay up", ndim=2)
    _want(out, "gla_decay out", torch.float32, 2)
    T, R = low.shape
    C = up.shape[0]
    if up.shape[1] != R or out.shape != (T, C):
        raise KernelError(f"gla_decay: low {tuple(low.shape)}, up {tuple(up.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _want(bias, "gla_decay bias", torch.float32, 1)
        if bias.numel() != C:
            raise KernelError(f"gla_decay: a bias of {bias.numel()} values for {C} channels")
    lib = library("linear_attention")
    _check(lib, lib.lp_gla_decay(lp, ldl, up.data_ptr(), _code(up, "gla_decay up"), _ptr(bias), out.data_ptr(), T, C, R,
                                 float(tau), 1 if double_exp else 0, _stream()))
    return out


GLA_CHUNK = 128               # tokens per chunk of a long prompt's recurrence
GLA_CHUNKED_FROM = 256        # from how many new tokens of a sequence on the chunks run side by side


def gla_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor, state: torch.Tensor,
             slots: torch.Tensor, q_start: torch.Tensor, out: torch.Tensor, *, num_heads: int, key_dim: int,
             value_dim: int, q_scale: float, max_new: int = 0, scratch=None, decay_per_head: bool = False,
             key_gain: Optional[torch.Tensor] = None, ones_column: bool = False,
             bonus: Optional[torch.Tensor] = None, qk_heads: Optional[int] = None,
             delta_strength: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The recurrence S <- diag(decay_t) S + k_t v_t^T, out_t = S^T (q_t * q_scale) over the step's tokens of every
    sequence, from and into ``state`` float32 [slots, H, dv, dk] (row ``slots[b]`` for sequence b; a value column's
    key channels lie together). ``proj``: float32
    [T, F] with queries, keys and values at the given columns; ``decay``: float32 [T, H * dk]; ``out``: float32 [T, H * dv].
    With ``max_new`` (the most new tokens of a sequence) of ``GLA_CHUNKED_FROM`` or more and ``scratch(name, shape,
    dtype)`` for buffers, the sequences are cut into chunks of ``GLA_CHUNK`` tokens that run side by side: each
    chunk's own contribution from a zero state, then the chunks' start states in order, then the outputs.

    ``decay_per_head``: ``decay`` is float32 [T, H], one decay per token and head for all its key channels.
    ``key_gain``: float32 [T, H], multiplied into the token's keys (an input gate). ``ones_column``: the last of the
    ``value_dim`` columns of state and output is fed the constant 1 instead of a value (the projection then holds
    ``value_dim - 1`` values per head): its output is q . (decayed sum of the gated keys), a normaliser.
    ``bonus``: float32 [H, dk]; a token's output then comes from the state BEFORE the token plus bonus_c k_c v_j for the
    token itself, out_t = (S + diag(bonus) k_t v_t^T)^T q_t, and the state is updated afterwards.
    ``qk_heads``: the projection holds that many query / key heads (a divisor of ``num_heads``); head h reads query / key
    head h // (num_heads // qk_heads). ``delta_strength``: float32 [T, H]; the recurrence is then the gated delta rule
    (one decay a per head): S <- a S; u = strength * (v - S^T k); S <- S + k u^T; out = S^T q; long prompts run in
    chunks side by side here too (a chunk's effect on the state that enters it is S -> P S + L with a [dk, dk] matrix P,
    which the first pass forms beside L)."""
    _want(proj, "gla_scan proj", torch.float32, 2)
    _want(decay, "gla_scan decay", torch.float32, 2)
    _want(state, "gla_scan state", torch.float32, 4)
    _want(slots, "gla_scan slots", torch.int32, 1)
    _want(q_start, "gla_scan q_start", torch.int32, 1)
    _want(out, "gla_scan out", torch.float32, 2)
    T = proj.shape[0]
    H, dk, dv = num_heads, key_dim, value_dim
    B = slots.numel()
    if bonus is not None:
        _want(bonus, "gla_scan bonus", torch.float32, 2)
        if bonus.shape != (H, dk):
            raise KernelError(f"gla_scan: a bonus of {tuple(bonus.shape)} for {H} heads of {dk} channels")
    if key_gain is not None:
        _want(key_gain, "gla_scan key_gain", torch.float32, 2)
        if key_gain.shape != (T, H):
            raise KernelError(f"gla_scan: key gains {tuple(key_gain.shape)} for {T} tokens and {H} heads")
    if (decay.shape != (T, H if decay_per_head else H * dk) or state.shape[1:] != (H, dv, dk) or out.shape != (T, H * dv)
            or q_start.numel() != B + 1):
        raise KernelError(f"gla_scan: proj {tuple(proj.shape)}, decay {tuple(decay.shape)}, state {tuple(state.shape)}, "
                          f"out {tuple(out.shape)}, {B} sequences")
    if delta_strength is not None:
        _want(delta_strength, "gla_scan delta_strength", torch.float32, 2)
        if delta_strength.shape != (T, H) or not decay_per_head:
            raise KernelError(f"gla_scan: write strengths {tuple(delta_strength.shape)} for {T} tokens and {H} heads "
                              f"(the delta rule takes one decay per head)")
    if qk_heads is not None and (qk_heads <= 0 or H % qk_heads):
        raise KernelError(f"gla_scan: {H} heads over {qk_heads} query / key heads")
    chunks, chunk_state, chunk_decay = 1, None, None
    # the delta rule's passes are bound by their chain of tokens, not by arithmetic: shorter chunks, more of them
    # (measured at 4 heads of 64 x 64 over 2,048 tokens: chunks of 128 / 64 / 32: 0.28 / 0.22 / 0.34 ms; the chunks'
    # combination, a chain over the chunks, costs about 5 us per chunk)
    chunk = GLA_CHUNK // 2 if delta_strength is not None else GLA_CHUNK
    if scratch is not None and max_new >= GLA_CHUNKED_FROM and B * -(-max_new // chunk) <= 65535:
        chunks = -(-max_new // chunk)
        # the delta rule's chunks also carry their [dk, dk] transition, as dk more columns per head
        chunk_state = scratch("gla_chunk_states", (B, chunks, H, dv + (dk if delta_strength is not None else 0), dk), torch.float32)
        chunk_decay = scratch("gla_chunk_decays", (B, chunks, H, dk), torch.float32) if delta_strength is None else None
    lib = library("linear_attention")
    _check(lib, lib.lp_gla_scan(proj.data_ptr(), proj.shape[1], int(q_off), int(k_off), int(v_off), decay.data_ptr(),
                                state.data_ptr(), slots.data_ptr(), q_start.data_ptr(), out.data_ptr(), B, H, dk, dv,
                                float(q_scale), chunks, chunk, _ptr(chunk_state), _ptr(chunk_decay),
                                1 if decay_per_head else 0, _ptr(key_gain), 1 if ones_column else 0, _ptr(bonus),
                                int(qk_heads or H), _ptr(delta_strength), _stream()))
    if chunks > 1:
        count_launches(2)
    return out


def gla_finish(o: torch.Tensor, gain: torch.Tensor, eps: float, gate: Optional[torch.Tensor], out: torch.Tensor, *,
               num_heads: int, value_dim: int, clear: Optional[torch.Tensor] = None, gain_per_head: bool = False,
               gate_sigmoid: bool = False, max_row: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h] = rmsnorm(o[t, h]) * gain * silu(gate[t, h]) per head of ``value_dim`` values; ``gate``: float32
    [T, H * dv] (may be a column slice) or None. ``gain_per_head``: ``gain`` is [H * dv]. ``gate_sigmoid``: the gate's
    sigmoid instead of its silu. ``max_row`` (float32 [T, H]): ``o`` is [T, H * (dv + 1)], a head's last column being
    its normaliser n; o[t, h] is first divided by max(|n|, exp(-max_row[t, h])) + 1e-6."""
    _want(o, "gla_finish o", torch.float32, 2)
    _want(gain, "gla_finish gain", torch.float32, 1)
    _want(out, "gla_finish out", ndim=2)
    T = o.shape[0]
    xs = value_dim + (1 if max_row is not None else 0)
    if max_row is not None:
        _want(max_row, "gla_finish max_row", torch.float32, 2)
        if max_row.shape != (T, num_heads):
            raise KernelError(f"gla_finish: maxima {tuple(max_row.shape)} for {T} tokens and {num_heads} heads")
    if (o.shape != (T, num_heads * xs) or out.shape != (T, num_heads * value_dim)
            or gain.numel() != (num_heads * value_dim if gain_per_head else value_dim)):
        raise KernelError(f"gla_finish: o {tuple(o.shape)}, out {tuple(out.shape)}, gain {tuple(gain.shape)}")
    gp, ldg = (None, 0)
    if gate is not None:
        gp, ldg = _slice(gate, "gla_finish gate")
        if gate.shape != out.shape:
            raise KernelError(f"gla_finish: gate {tuple(gate.shape)} does not match out {tuple(out.shape)}")
    lib = library("linear_attention")
    _check(lib, lib.lp_gla_finish(o.data_ptr(), gain.data_ptr(), float(eps), gp, ldg, out.data_ptr(),
                                  _code(out, "gla_finish out"), T, num_heads, value_dim, *_clear_args(clear, "gla_finish"),
                                  xs, 1 if gain_per_head else 0, 1 if gate_sigmoid else 0, _ptr(max_row), _stream()))
    return out


def short_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], tail: torch.Tensor, slots: torch.Tensor,
               q_start: torch.Tensor, out: torch.Tensor, *, max_new: int, silu: bool = True) -> torch.Tensor:
    """A short causal convolution over time, per channel, continued from step to step: out[t, c] = act(bias[c] +
    sum_j taps[c, j] * x[t - (K - 1) + j, c]), the last tap on the token itself, zeros before a sequence's start.
    ``x``: float32 [T, C] (may be a column slice); ``taps``: [C, K]; ``tail``: float32 [slots, K - 1, C], the last
    K - 1 inputs of every sequence (zero at its start), read and renewed here; ``out``: float32 [T, C] (may be a slice)."""
    xp, ldx = _slice(x, "short_conv x")
    op, ldo = _slice(out, "short_conv out")
    _want(taps, "short_conv taps", ndim=2)
    _want(tail, "short_conv tail", torch.float32, 3)
    _want(slots, "short_conv slots", torch.int32, 1)
    _want(q_start, "short_conv q_start", torch.int32, 1)
    T, C = x.shape
    K = taps.shape[1]
    B = slots.numel()
    if taps.shape[0] != C or out.shape != x.shape or tail.shape[1:] != (K - 1, C) or q_start.numel() != B + 1:
        raise KernelError(f"short_conv: x {tuple(x.shape)}, taps {tuple(taps.shape)}, tail {tuple(tail.shape)}, out "
                          f"{tuple(out.shape)}, {B} sequences")
    if bias is not None:
        _want(bias, "short_conv bias", torch.float32, 1)
        if bias.numel() != C:
            raise KernelError(f"short_conv: a bias of {bias.numel()} values for {C} channels")
    lib = library("linear_attention")
    _check(lib, lib.lp_short_conv(xp, ldx, taps.data_ptr(), _code(taps, "short_conv taps"), _ptr(bias), tail.data_ptr(),
                                  slots.data_ptr(), q_start.data_ptr(), op, ldo, B, int(max_new), C, K, 1 if silu else 0,
                                  _stream()))
    return out


def decay_gates(proj: torch.Tensor, z_off: int, dt_bias: Optional[torch.Tensor], a_log: torch.Tensor, decay: torch.Tensor,
                dt: Optional[torch.Tensor] = None, strength: Optional[torch.Tensor] = None, b_off: int = 0) -> None:
    """Per token and head, from float32 columns of ``proj``: step = softplus(proj[:, z_off + h] + dt_bias[h]) (no
    clamp), decay = exp(-exp(a_log[h]) * step); optionally strength = sigmoid(proj[:, b_off + h]). ``decay``, ``dt``,
    ``strength``: float32 [T, H]."""
    _want(proj, "decay_gates proj", torch.float32, 2)
    _want(a_log, "decay_gates a_log", torch.float32, 1)
    _want(decay, "decay_gates decay", torch.float32, 2)
    T, H = decay.shape
    if proj.shape[0] != T or a_log.numel() != H:
        raise KernelError(f"decay_gates: proj {tuple(proj.shape)}, decay {tuple(decay.shape)}, {a_log.numel()} heads")
    for name, t in (("dt", dt), ("strength", strength)):
        if t is not None:
            _want(t, f"decay_gates {name}", torch.float32, 2)
            if t.shape != decay.shape:
                raise KernelError(f"decay_gates: {name} {tuple(t.shape)} for {tuple(decay.shape)}")
    if dt_bias is not None:
        _want(dt_bias, "decay_gates dt_bias", torch.float32, 1)
        if dt_bias.numel() != H:
            raise KernelError(f"decay_gates: {dt_bias.numel()} biases for {H} heads")
    lib = library("linear_attention")
    _check(lib, lib.lp_decay_gates(proj.data_ptr(), proj.shape[1], int(z_off), int(b_off), _ptr(dt_bias), a_log.data_ptr(),
                                   decay.data_ptr(), _ptr(dt), _ptr(strength), T, H, _stream()))


def head_unit_norm(x: torch.Tensor, offset: int, heads: int, dim: int, eps: float, scale: float = 1.0,
                   scaled_heads: Optional[int] = None) -> torch.Tensor:
    """In place, for ``heads`` heads of ``dim`` values from column ``offset`` of the float32 matrix ``x``: every head
    becomes x / sqrt(sum(x^2) + eps); the first ``scaled_heads`` of them (all, if None) are also multiplied by ``scale``."""
    _want(x, "head_unit_norm x", torch.float32, 2)
    lib = library("linear_attention")
    _check(lib, lib.lp_head_unit_norm(x.data_ptr(), x.shape[1], int(offset), int(heads), int(dim), float(eps), float(scale),
                                      int(heads if scaled_heads is None else scaled_heads), x.shape[0], _stream()))
    return x


def gated_part_norm(raw: torch.Tensor, gate: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor, *,
                    num_heads: int, head_dim: int, parts: int, values: Optional[torch.Tensor] = None,
                    skip: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = (raw + skip[h] * values) * silu(gate), then each of ``parts`` equal parts of a row is divided by its own root
    mean square (``eps`` inside the root) and multiplied by ``gain``. ``raw``: float32 [T, H * P]; ``gate`` and ``values``:
    float32 [T, H * P] (may be column slices); ``skip``: float32 [H]; ``gain``: float32 [H * P]. The gate comes before the
    norm. ``clear``: a float32 buffer zeroed on the side."""
    _want(raw, "gated_part_norm raw", torch.float32, 2)
    _want(gain, "gated_part_norm gain", torch.float32, 1)
    _want(out, "gated_part_norm out", ndim=2)
    T, W = raw.shape
    gp, ldg = _slice(gate, "gated_part_norm gate")
    if W != num_heads * head_dim or gate.shape != raw.shape or out.shape != raw.shape or gain.numel() != W or parts <= 0 or W % parts:
        raise KernelError(f"gated_part_norm: raw {tuple(raw.shape)}, gate {tuple(gate.shape)}, out {tuple(out.shape)}, "
                          f"{num_heads} heads of {head_dim} in {parts} parts")
    vp, ldv = None, 0
    if (values is None) != (skip is None):
        raise KernelError("gated_part_norm: a skip comes with the values it multiplies")
    if values is not None:
        vp, ldv = _slice(values, "gated_part_norm values")
        _want(skip, "gated_part_norm skip", torch.float32, 1)
        if values.shape != raw.shape or skip.numel() != num_heads:
            raise KernelError(f"gated_part_norm: values {tuple(values.shape)}, {skip.numel()} skips for {num_heads} heads")
    lib = library("linear_attention")
    _check(lib, lib.lp_gated_part_norm(raw.data_ptr(), vp, ldv, _ptr(skip), gp, ldg, gain.data_ptr(), float(eps), out.data_ptr(),
                                       _code(out, "gated_part_norm out"), T, num_heads, head_dim, int(parts),
                                       *_clear_args(clear, "gated_part_norm"), _stream()))
    return out


def exp_gates(proj: torch.Tensor, i_off: int, f_off: int, bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor],
              cap: Optional[float], mstate: torch.Tensor, slots: torch.Tensor, q_start: torch.Tensor,
              decay: torch.Tensor, gain: torch.Tensor, max_row: torch.Tensor) -> None:
    """Exponential gates with a running maximum, per token and head, in token order for every sequence of the step:
    i = cap * tanh((zi + bias_i) / cap), f = logsigmoid(cap * tanh((zf + bias_f) / cap)) from the float32 columns
    ``i_off`` / ``f_off`` of ``proj`` (H each), m_t = max(f + m_(t-1), i) from and into ``mstate`` float32 [slots, H];
    writes decay = exp(f + m_(t-1) - m_t), gain = exp(i - m_t) and max_row = m_t, each float32 [T, H]."""
    _want(proj, "exp_gates proj", torch.float32, 2)
    _want(mstate, "exp_gates mstate", torch.float32, 2)
    _want(slots, "exp_gates slots", torch.int32, 1)
    _want(q_start, "exp_gates q_start", torch.int32, 1)
    T, H, B = proj.shape[0], mstate.shape[1], slots.numel()
    for name, t in (("decay", decay), ("gain", gain), ("max_row", max_row)):
        _want(t, f"exp_gates {name}", torch.float32, 2)
        if t.shape != (T, H):
            raise KernelError(f"exp_gates: {name} {tuple(t.shape)} for {T} tokens and {H} heads")
    for name, t in (("bias_i", bias_i), ("bias_f", bias_f)):
        if t is not None:
            _want(t, f"exp_gates {name}", torch.float32, 1)
            if t.numel() != H:
                raise KernelError(f"exp_gates: {name} of {t.numel()} values for {H} heads")
    if q_start.numel() != B + 1:
        raise KernelError(f"exp_gates: {q_start.numel()} offsets for {B} sequences")
    lib = library("linear_attention")
    _check(lib, lib.lp_exp_gates(proj.data_ptr(), proj.shape[1], int(i_off), int(f_off), _ptr(bias_i), _ptr(bias_f),
                                 float(cap or 0.0), mstate.data_ptr(), slots.data_ptr(), q_start.data_ptr(),
                                 decay.data_ptr(), gain.data_ptr(), max_row.data_ptr(), B, H, _stream()))


def token_shift(x: torch.Tensor, last: torch.Tensor, mu: torch.Tensor, slots: torch.Tensor, q_start: torch.Tensor,
                seq_ids: torch.Tensor, out: torch.Tensor, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s] for the S rows of ``mu`` (float32 [S, d]); the token before a
    sequence's first new token is the row of its slot in ``last`` (float32 [slots, d]), which then receives the
    sequence's last new token. ``x``: float32 [T, d]; ``out``: [S, T, d]. ``clear``: a float32 buffer zeroed on the side."""
    _want(x, "token_shift x", torch.float32, 2)
    _want(last, "token_shift last", torch.float32, 2)
    _want(mu, "token_shift mu", torch.float32, 2)
    _want(slots, "token_shift slots", torch.int32, 1)
    _want(q_start, "token_shift q_start", torch.int32, 1)
    _want(seq_ids, "token_shift seq_ids", torch.int32, 1)
    _want(out, "token_shift out", ndim=3)
    T, d = x.shape
    S = mu.shape[0]
    if last.shape[1] != d or mu.shape[1] != d or out.shape != (S, T, d) or seq_ids.numel() != T or q_start.numel() != slots.numel() + 1:
        raise KernelError(f"token_shift: x {tuple(x.shape)}, last {tuple(last.shape)}, mu {tuple(mu.shape)}, out {tuple(out.shape)}")
    lib = library("linear_attention")
    _check(lib, lib.lp_token_shift(x.data_ptr(), last.data_ptr(), mu.data_ptr(), slots.data_ptr(), q_start.data_ptr(),
                                   seq_ids.data_ptr(), out.data_ptr(), _code(out, "token_shift out"), T, d, S,
                                   *_clear_args(clear, "token_shift"), _stream()))
    return out


# --------------------------------------------------------------------------- general attention heads, sublayer norms
def qkv_prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], rotation: Rotation, positions: torch.Tensor,
                seq_ids: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor, pages: torch.Tensor, *,
                num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, unit_norm_eps: Optional[float],
                clear: Optional[torch.Tensor] = None, q_gain: Optional[torch.Tensor] = None,
                k_gain: Optional[torch.Tensor] = None, gain_eps: float = 0.0, write_kv: bool = True) -> None:
    """From the float32 projection ``qkv`` [T, H * dk + G * dk + G * dv]: add ``bias`` (float32, same width, or None),
    rotate queries and keys, divide each query and key head by its root mean square (``unit_norm_eps`` not None), and
    store queries to ``q_out`` [T, H * hdp] and keys and values into ``pages`` [num_pages, 2, G, page_size, hdp], every
    head padded with zeros to the pages' head size hdp. ``q_gain`` / ``k_gain`` (float32 [dk], shared by the heads):
    before the rotation, query / key heads are RMS-normed over dk with that gain and ``gain_eps``. ``write_kv=False``:
    ``qkv`` [T, H * dk] holds queries only (a layer that attends over another layer's keys and values); ``pages`` only
    says how queries are stored."""
    _want(qkv, "qkv_prepare qkv", torch.float32, 2)
    _want(positions, "qkv_prepare positions", torch.int32, 1)
    _want(seq_ids, "qkv_prepare seq_ids", torch.int32, 1)
    _want(page_table, "qkv_prepare page_table", torch.int32, 2)
    _want(q_out, "qkv_prepare q_out", ndim=2)
    _want(pages, "qkv_prepare pages", q_out.dtype, 5)
    T = qkv.shape[0]
    H, G, dk, dv = num_heads, num_kv_heads, key_dim, value_dim
    hdp = pages.shape[4]
    if pages.shape[1] != 2 or pages.shape[2] != G:
        raise KernelError(f"qkv_prepare: pages {tuple(pages.shape)} for {G} key heads")
    if not write_kv:
        G = 0
    F = (H + G) * dk + G * dv
    for name, gain in (("q_gain", q_gain), ("k_gain", k_gain)):
        if gain is not None:
            _want(gain, f"qkv_prepare {name}", torch.float32, 1)
            if gain.numel() != dk:
                raise KernelError(f"qkv_prepare: {name} of {gain.numel()} values for heads of {dk}")
    if qkv.shape[1] != F or q_out.shape != (T, H * hdp):
        raise KernelError(f"qkv_prepare: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}, pages {tuple(pages.shape)}")
    if bias is not None:
        _want(bias, "qkv_prepare bias", torch.float32, 1)
        if bias.numel() != F:
            raise KernelError(f"qkv_prepare: a bias of {bias.numel()} values for {F} features")
    freq_ptr, rotary_dim, interleaved = rotation.checked("qkv_prepare")
    lib = library("elementwise")
    _check(lib, lib.lp_qkv_prepare(
        qkv.data_ptr(), qkv.shape[1], _ptr(bias), freq_ptr, positions.data_ptr(), seq_ids.data_ptr(),
        page_table.data_ptr(), page_table.shape[1], q_out.data_ptr(), _code(q_out, "qkv_prepare q_out"),
        pages.data_ptr() if write_kv else None, _code(pages, "qkv_prepare pages"), T, H, G, dk, dv, hdp, rotary_dim, interleaved,
        0 if unit_norm_eps is None else 1, float(unit_norm_eps or 0.0), pages.shape[3], *_clear_args(clear, "qkv_prepare"),
        _ptr(q_gain), _ptr(k_gain) if write_kv else None, float(gain_eps), _stream()))


def post_norm_add(y: torch.Tensor, weight: torch.Tensor, eps: float, x: torch.Tensor, *, next_weight: Optional[torch.Tensor] = None,
                  next_eps: float = 0.0, next_out: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None,
                  y_bias: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += y / sqrt(mean(y^2) + eps) * weight, float32 in place; with ``next_weight``, also
    next_out = x / sqrt(mean(x^2) + next_eps) * next_weight of the new x (the norm in front of the next sublayer).
    ``y_bias`` (float32 [d]) is added to y first; ``scale`` (float32 [d]) multiplies the normed y once more (a layer
    scale); ``next_out`` without ``next_weight`` receives the new x as it is, in ``next_out``'s number format."""
    _want(y, "post_norm_add y", torch.float32, 2)
    _want(x, "post_norm_add x", torch.float32, 2)
    _want(weight, "post_norm_add weight", torch.float32, 1)
    T, d = x.shape
    if y.shape != x.shape or weight.numel() != d:
        raise KernelError(f"post_norm_add: y {tuple(y.shape)}, x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    code = F32
    if next_weight is not None:
        _want(next_weight, "post_norm_add next_weight", torch.float32, 1)
        if next_weight.numel() != d or next_out is None:
            raise KernelError("post_norm_add: a next norm needs its gain over whole rows and its output")
    if next_out is not None:
        _want(next_out, "post_norm_add next_out", ndim=2)
        if next_out.shape != x.shape:
            raise KernelError(f"post_norm_add: next output {tuple(next_out.shape)} for x {tuple(x.shape)}")
        code = _code(next_out, "post_norm_add next_out")
    for name, vec in (("y_bias", y_bias), ("scale", scale)):
        if vec is not None:
            _want(vec, f"post_norm_add {name}", torch.float32, 1)
            if vec.numel() != d:
                raise KernelError(f"post_norm_add: {name} of {vec.numel()} values for rows of {d}")
    lib = library("elementwise")
    _check(lib, lib.lp_post_norm_add(y.data_ptr(), weight.data_ptr(), float(eps), x.data_ptr(), _ptr(next_weight),
                                     float(next_eps), _ptr(next_out), code, T, d,
                                     *_clear_args(clear, "post_norm_add"), _ptr(y_bias), _ptr(scale), _stream()))
    return x


def gated_act(z: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, form: str = "gelu_tanh",
              clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, f] = act(z[t, f] + bias[f]) * (z[t, F + f] + bias[F + f]) from the float32 sums ``z`` [T, 2 F] of a stacked
    gate | up product (may be a column slice); ``bias``: float32 [2 F] or None. ``form``: ``"gelu_tanh"``
    (0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))) or ``"silu"``. Everything in float32 until ``out`` is stored."""
    zp, ldz = _slice(z, "gated_act z")
    _want(out, "gated_act out", ndim=2)
    T, F = out.shape
    if z.shape != (T, 2 * F):
        raise KernelError(f"gated_act: z {tuple(z.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _want(bias, "gated_act bias", torch.float32, 1)
        if bias.numel() != 2 * F:
            raise KernelError(f"gated_act: a bias of {bias.numel()} values for 2 x {F} sums")
    forms = {"gelu_tanh": 0, "silu": 1}
    if form not in forms:
        raise KernelError(f"gated_act: unknown form {form!r}")
    lib = library("elementwise")
    _check(lib, lib.lp_gated_act(zp, ldz, _ptr(bias), out.data_ptr(), _code(out, "gated_act out"), T, F, forms[form],
                                 *_clear_args(clear, "gated_act"), _stream()))
    return out


def stream_cast(x: torch.Tensor, out: torch.Tensor, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x in ``out``'s number format; ``x``: float32, same shape."""
    _want(x, "stream_cast x", torch.float32)
    _want(out, "stream_cast out")
    if out.shape != x.shape:
        raise KernelError(f"stream_cast: x {tuple(x.shape)}, out {tuple(out.shape)}")
    lib = library("elementwise")
    _check(lib, lib.lp_stream_cast(x.data_ptr(), out.data_ptr(), _code(out, "stream_cast out"), x.numel(),
                                   *_clear_args(clear, "stream_cast"), _stream()))
    return out


def stream_add(x: torch.Tensor, other: Optional[torch.Tensor] = None, vector: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[t] += other[t] + vector, float32 in place; either may be None."""
    _want(x, "stream_add x", torch.float32, 2)
    T, d = x.shape
    if other is not None:
        _want(other, "stream_add other", torch.float32, 2)
        if other.shape != x.shape:
            raise KernelError(f"stream_add: other {tuple(other.shape)} does not match x {tuple(x.shape)}")
    if vector is not None:
        _want(vector, "stream_add vector", torch.float32, 1)
        if vector.numel() != d:
            raise KernelError(f"stream_add: a vector of {vector.numel()} values for rows of {d}")
    lib = library("elementwise")
    _check(lib, lib.lp_stream_add(x.data_ptr(), _ptr(other), _ptr(vector), T, d, _stream()))
    return x


def scaled_sum(x: torch.Tensor, a: torch.Tensor, a_scale: float, b: Optional[torch.Tensor] = None, b_scale: float = 0.0, *,
               a_vector: Optional[torch.Tensor] = None, b_vector: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x <- x + a_scale * (a + a_vector) + b_scale * (b + b_vector), float32 [T, d] in place; the vectors [d] and ``b``
    are optional."""
    _want(x, "scaled_sum x", torch.float32, 2)
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _want(t, f"scaled_sum {name}", torch.float32, 2)
            if t.shape != x.shape:
                raise KernelError(f"scaled_sum: {name} {tuple(t.shape)} does not match x {tuple(x.shape)}")
    for name, t in (("a_vector", a_vector), ("b_vector", b_vector)):
        if t is not None:
            _want(t, f"scaled_sum {name}", torch.float32, 1)
            if t.numel() != x.shape[1]:
                raise KernelError(f"scaled_sum: {name} of {t.numel()} values for rows of {x.shape[1]}")
    lib = library("elementwise")
    _check(lib, lib.lp_scaled_sum(x.data_ptr(), a.data_ptr(), _ptr(a_vector), float(a_scale), _ptr(b), _ptr(b_vector),
                                  float(b_scale), x.shape[0], x.shape[1], _stream()))
    return x


def relu2(z: torch.Tensor, out: torch.Tensor, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = max(z, 0)^2; ``z``: float32 [T, F] (may be a column slice)."""
    zp, ldz = _slice(z, "relu2 z")
    _want(out, "relu2 out", ndim=2)
    if out.shape != z.shape:
        raise KernelError(f"relu2: z {tuple(z.shape)}, out {tuple(out.shape)}")
    lib = library("elementwise")
    _check(lib, lib.lp_relu2(zp, ldz, out.data_ptr(), _code(out, "relu2 out"), z.shape[0], z.shape[1],
                             *_clear_args(clear, "relu2"), _stream()))
    return out


# --------------------------------------------------------------------------- routing of a mixture of experts
def route(logits: torch.Tensor, weights: torch.Tensor, *, groups: int, keep: int, top: int) -> torch.Tensor:
    """weights[t, e] = the weight of expert e for token t (zero if it was not chosen) from the router's float32
    ``logits`` [T, E] (may be a column slice): scores sigmoid(logit); a group of E / groups neighbours scores the sum
    of its two largest; the ``top`` largest scores within the ``keep`` best groups win; weights are the winners'
    scores divided by their sum."""
    zp, ldz = _slice(logits, "route logits")
    _want(weights, "route weights", torch.float32, 2)
    if weights.shape != logits.shape:
        raise KernelError(f"route: logits {tuple(logits.shape)}, weights {tuple(weights.shape)}")
    lib = library("routing")
    _check(lib, lib.lp_route(zp, ldz, weights.data_ptr(), weights.shape[1], logits.shape[0], logits.shape[1], int(groups),
                             int(keep), int(top), _stream()))
    return weights


def route_softmax(logits: torch.Tensor, correction: Optional[torch.Tensor], weights: torch.Tensor, *, groups: int, keep: int,
                  top: int, scale: float) -> torch.Tensor:
    """Scores softmax(logits) over all E router outputs; the choice is made on score + correction inside the best
    ``keep`` of ``groups`` groups of neighbours (a group's score is its largest choice score), the ``top`` largest win;
    weights[t, e] = score * ``scale`` for the chosen, zero otherwise (not renormalised). ``logits``: float32 [T, E] (may
    be a column slice); ``correction``: float32 [E] or None; ``weights``: float32 [T, E]."""
    zp, ldz = _slice(logits, "route_softmax logits")
    _want(weights, "route_softmax weights", torch.float32, 2)
    T, E = logits.shape
    if weights.shape != (T, E):
        raise KernelError(f"route_softmax: logits {tuple(logits.shape)}, weights {tuple(weights.shape)}")
    if correction is not None:
        _want(correction, "route_softmax correction", torch.float32, 1)
        if correction.numel() != E:
            raise KernelError(f"route_softmax: a correction of {correction.numel()} values for {E} experts")
    lib = library("routing")
    _check(lib, lib.lp_route_softmax(zp, ldz, _ptr(correction), weights.data_ptr(), weights.shape[1], T, E, int(groups),
                                     int(keep), int(top), float(scale), _stream()))
    return weights


def identity_experts(x: torch.Tensor, h: torch.Tensor, weights: torch.Tensor, first: int, count: int) -> torch.Tensor:
    """x[t] += h[t] * sum(weights[t, first:first + count]): experts that pass their input on. ``x``: float32 [T, d];
    ``h``: [T, d]; ``weights``: float32 [T, E]."""
    _want(x, "identity_experts x", torch.float32, 2)
    _want(h, "identity_experts h", ndim=2)
    _want(weights, "identity_experts weights", torch.float32, 2)
    if h.shape != x.shape or weights.shape[0] != x.shape[0] or first < 0 or first + count > weights.shape[1]:
        raise KernelError(f"identity_experts: x {tuple(x.shape)}, h {tuple(h.shape)}, weights {tuple(weights.shape)}, "
                          f"columns {first}..{first + count - 1}")
    lib = library("routing")
    _check(lib, lib.lp_identity_experts(x.data_ptr(), h.data_ptr(), _code(h, "identity_experts h"), weights.data_ptr(),
                                        weights.shape[1], int(first), int(count), x.shape[0], x.shape[1], _stream()))
    return x


def expert_scale(hidden: torch.Tensor, weights: torch.Tensor, expert_size: int, clear: Optional[torch.Tensor] = None,
                 num_experts: Optional[int] = None, identity=None) -> torch.Tensor:
    """hidden[t, e * expert_size + j] *= weights[t, e] in place for the E experts of ``weights`` [T, E] (``num_experts``:
    for its first so many columns only); columns of ``hidden`` beyond E * expert_size are left as they are.
    ``identity`` = (x, h, first, count): in the same launch x[t] += h[t] * sum(weights[t, first:first + count]), as
    :func:`identity_experts` does (x float32 [T, d], h [T, d])."""
    _want(hidden, "expert_scale hidden", ndim=2)
    _want(weights, "expert_scale weights", torch.float32, 2)
    T, ldw = weights.shape
    E = ldw if num_experts is None else int(num_experts)
    if hidden.shape[0] != T or hidden.shape[1] < E * expert_size or not 0 < E <= ldw:
        raise KernelError(f"expert_scale: hidden {tuple(hidden.shape)} for {E} experts of {expert_size}")
    id_args = (None, None, 0, 0, 0, 0)
    if identity is not None:
        x, h, first, count = identity
        _want(x, "expert_scale identity x", torch.float32, 2)
        _want(h, "expert_scale identity h", ndim=2)
        if h.shape != x.shape or x.shape[0] != T or first < 0 or first + count > ldw:
            raise KernelError(f"expert_scale: identity x {tuple(x.shape)}, h {tuple(h.shape)}, columns {first}..{first + count - 1} of {ldw}")
        id_args = (x.data_ptr(), h.data_ptr(), _code(h, "expert_scale identity h"), int(first), int(count), x.shape[1])
    lib = library("routing")
    _check(lib, lib.lp_expert_scale(hidden.data_ptr(), _code(hidden, "expert_scale hidden"), hidden.shape[1],
                                    weights.data_ptr(), ldw, T, E, int(expert_size), *_clear_args(clear, "expert_scale"),
                                    *id_args, _stream()))
    return hidden


def route_top(logits: torch.Tensor, bias: Optional[torch.Tensor], weights: torch.Tensor, *, num_experts: int, top: int) -> torch.Tensor:
    """weights[t, e] for the E = ``num_experts`` experts: the ``top`` largest of logits[t, e] + bias[e] are chosen and
    weighted by the softmax over the chosen logits alone (zero elsewhere). Columns of ``logits`` beyond E are gates of
    experts that every token uses: weights[t, E + i] = sigmoid(logits[t, E + i]). ``logits``: float32 [T, E + extra]
    (may be a column slice); ``weights``: float32, same shape."""
    zp, ldz = _slice(logits, "route_top logits")
    _want(weights, "route_top weights", torch.float32, 2)
    E = int(num_experts)
    if weights.shape != logits.shape or logits.shape[1] < E:
        raise KernelError(f"route_top: logits {tuple(logits.shape)}, weights {tuple(weights.shape)}, {E} experts")
    if bias is not None:
        _want(bias, "route_top bias", torch.float32, 1)
        if bias.numel() != E:
            raise KernelError(f"route_top: a bias of {bias.numel()} values for {E} experts")
    lib = library("routing")
    _check(lib, lib.lp_route_top(zp, ldz, _ptr(bias), weights.data_ptr(), weights.shape[1], logits.shape[0], E, int(top),
                                 logits.shape[1] - E, _stream()))
    return weights


def expert_act(z: torch.Tensor, weights: Optional[torch.Tensor], hidden: torch.Tensor, *, num_experts: int, expert_size: int,
               limit: float, limit_rest: float = 0.0, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Hidden activations of clamped gated experts from the float32 sums ``z`` [T, 2 * total] of one stacked product
    (all gate sums, then all up sums): with g = min(gate, limit), u = clamp(up, -limit, limit),
    hidden[t, c] = g * sigmoid(1.702 g) * (u + 1) * weights[t, expert of c]. The first ``num_experts * expert_size``
    columns belong to the routed experts; the rest to one more expert (weights[:, num_experts], ``limit_rest``)."""
    zp, ldz = _slice(z, "expert_act z")
    _want(hidden, "expert_act hidden", ndim=2)
    T, total = hidden.shape
    if z.shape != (T, 2 * total):
        raise KernelError(f"expert_act: z {tuple(z.shape)}, hidden {tuple(hidden.shape)}")
    ldw = 0
    if weights is not None:
        _want(weights, "expert_act weights", torch.float32, 2)
        ldw = weights.shape[1]
        if weights.shape[0] != T:
            raise KernelError(f"expert_act: weights {tuple(weights.shape)} for {T} tokens")
    lib = library("routing")
    _check(lib, lib.lp_expert_act(zp, ldz, total, hidden.data_ptr(), _code(hidden, "expert_act hidden"), _ptr(weights), ldw,
                                  T, int(num_experts), int(expert_size), float(limit), float(limit_rest),
                                  *_clear_args(clear, "expert_act"), _stream()))
    return hidden


# --------------------------------------------------------------------------- sampling
def sample_select_words() -> int:
    """4-byte words of scratch per row that ``sample`` wants for finding top-k candidates with several blocks."""
    return library("sampling").lp_sample_select_words()


def sample_slice_capacity(vocab: int) -> int:
    """The largest top-k whose candidates several blocks per row find together (0: none at this vocabulary)."""
    return library("sampling").lp_sample_slice_capacity(int(vocab))


def sample(logits: torch.Tensor, work: torch.Tensor, params: torch.Tensor, edit_token: torch.Tensor,
           edit_subtract: torch.Tensor, edit_factor: torch.Tensor, out_token: torch.Tensor,
           out_prob: torch.Tensor, select: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``params`` (packed LpSampleParams records) from the float32 ``logits``.
    ``select``: int32 scratch of ``sample_select_words()`` per row; with it, rows whose top-k is at most
    ``sample_slice_capacity(vocab)`` have their candidates found by several blocks each."""
    _want(logits, "sample logits", torch.float32, 2)
    _want(work, "sample work", torch.float32, 2)
    _want(params, "sample params", torch.uint8, 1)
    _want(edit_token, "sample edit tokens", torch.int32, 1)
    _want(edit_subtract, "sample edit amounts", torch.float32, 1)
    _want(edit_factor, "sample edit factors", torch.float32, 1)
    _want(out_token, "sample out tokens", torch.int32, 1)
    _want(out_prob, "sample out probabilities", torch.float32, 1)
    lib = library("sampling")
    record = lib.lp_sample_params_size()
    B = out_token.numel()
    V = logits.shape[1]
    if params.numel() != B * record or work.shape != (B, V) or out_prob.numel() != B:
        raise KernelError(f"sample: {params.numel()} parameter bytes, work {tuple(work.shape)} for {B} rows of {V}")
    select_ptr = 0
    if select is not None:
        _want(select, "sample select scratch", torch.int32, 1)
        if select.numel() < B * lib.lp_sample_select_words():
            raise KernelError(f"sample: select scratch of {select.numel()} words for {B} rows")
        select_ptr = select.data_ptr()
    _check(lib, lib.lp_sample(logits.data_ptr(), V, work.data_ptr(), V, params.data_ptr(), B, edit_token.data_ptr(),
                              edit_subtract.data_ptr(), edit_factor.data_ptr(), select_ptr, out_token.data_ptr(),
                              out_prob.data_ptr(), _stream()))


def sample_fetch(host_block: torch.Tensor, dev_block: torch.Tensor, batch: int, cap: int, record_words: int,
                 field_count: int) -> None:
    """Bring a step's sampler block (records, then ``cap`` edit tokens, amounts and factors per sequence) from
    page-locked host memory: each record and as many edits as it names."""
    _want(dev_block, "sample_fetch device block", torch.int32, 1)
    if host_block.dtype != torch.int32 or not host_block.is_pinned() or host_block.numel() != dev_block.numel():
        raise KernelError("sample_fetch: the host block must be page-locked int32 of the device block's size")
    if dev_block.numel() != batch * (record_words + 3 * cap):
        raise KernelError(f"sample_fetch: a block of {dev_block.numel()} words for {batch} records of {record_words} "
                          f"words and {cap} edits each")
    lib = library("sampling")
    _check(lib, lib.lp_sample_fetch(host_block.data_ptr(), dev_block.data_ptr(), batch, cap, record_words, field_count,
                                    _stream()))


def advance(tokens: torch.Tensor, positions: torch.Tensor, kv_len: torch.Tensor, sampled: torch.Tensor) -> None:
    """tokens <- sampled; positions += 1; kv_len += 1 (a decoding batch moves on by one token)."""
    B = tokens.numel()
    for t, what in ((tokens, "tokens"), (positions, "positions"), (kv_len, "kv_len"), (sampled, "sampled")):
        _want(t, f"advance {what}", torch.int32, 1)
        if t.numel() != B:
            raise KernelError(f"advance: {what} has {t.numel()} entries, tokens {B}")
    lib = library("elementwise")
    _check(lib, lib.lp_advance(tokens.data_ptr(), positions.data_ptr(), kv_len.data_ptr(), sampled.data_ptr(), B,
                               _stream()))


def argmax(logits: torch.Tensor, scratch: torch.Tensor, out_token: torch.Tensor) -> None:
    """out_token[b] = index of the first maximum of row b of the float32 ``logits``.
    ``scratch``: at least 64 float32 per row."""
    _want(logits, "argmax logits", torch.float32, 2)
    _want(scratch, "argmax scratch", torch.float32, 1)
    _want(out_token, "argmax out", torch.int32, 1)
    B, V = logits.shape
    if out_token.numel() != B or scratch.numel() < 64 * B:
        raise KernelError(f"argmax: {B} rows, {out_token.numel()} outputs, scratch of {scratch.numel()}")
    lib = library("sampling")
    _check(lib, lib.lp_argmax(logits.data_ptr(), V, V, B, scratch.data_ptr(), out_token.data_ptr(), _stream()))
