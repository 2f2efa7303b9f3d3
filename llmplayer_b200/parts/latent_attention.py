"""Softmax attention over a cache of low-rank latents.

Each position keeps one row: the RMS-normed latent c (``kv_rank`` values) and one rotated key part
(``rope_dim`` values) shared by all heads. Head h's key is [k_up[h] c | shared rotated part], its value
v_up[h] c; its query is [nope_dim unrotated | rope_dim rotated]. The kernels apply k_up to the query
instead of to every cached latent, attend over the cached rows with all heads at once, and apply v_up to
the weighted sum of latents (csrc/latent_attention.cu). An optional output gate scales head h's output by
sigmoid(out_gate[h] . x). A step of prompts that start at their first token, in bfloat16, instead forms every
head's keys and values from the latents in one product and runs the tensor-core attention of ordinary heads
over them; the cache is written the same either way.

The part offers its input projections to the block (``input_projections``), so that a block whose
sublayers all read one normed input can form them in one product, and takes the product's float32 sums
back (``forward_projected``); used alone (``forward``) it forms them itself.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache.sequence_cache import RowsRequest
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, POSITIONS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import GAIN, MATRIX, LatentAttentionSpec, TensorSpec


class LatentAttention(Part):
    def __init__(self, spec: LatentAttentionSpec):
        s = spec
        if s.num_heads <= 0 or s.kv_rank <= 0 or s.value_dim <= 0:
            raise ConfigError(f"latent attention with {s.num_heads} heads, rank {s.kv_rank}, values of {s.value_dim}")
        if s.nope_dim < 0 or s.rope_dim < 0 or s.nope_dim + s.rope_dim <= 0:
            raise ConfigError(f"latent attention: query heads of {s.nope_dim} + {s.rope_dim}")
        if (s.q_down is None) != (s.q_norm is None) or (s.q_down is not None and s.q_rank <= 0):
            raise ConfigError("queries through a latent need its map, its norm's gain and its rank together")
        if s.window is not None and s.window <= 0:
            raise ConfigError(f"attention window must be positive or absent, got {s.window}")
        self.spec = spec
        self.position = POSITIONS.build(s.position)
        self._inputs: List[torch.Tensor] = []
        self._own: Optional[Linear] = None
        self.out: Optional[Linear] = None

    @property
    def capture_safe(self) -> bool:
        return bool(getattr(self.position, "capture_safe", False))

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        specs = {
            s.q: TensorSpec((s.num_heads * (s.nope_dim + s.rope_dim), s.q_rank if s.q_down is not None else s.hidden_size), MATRIX),
            s.kv_down: TensorSpec((s.kv_rank + s.rope_dim, s.hidden_size), MATRIX),
            s.latent_norm: TensorSpec((s.kv_rank,), GAIN),
            s.k_up: TensorSpec((s.num_heads * s.nope_dim, s.kv_rank), MATRIX),
            s.v_up: TensorSpec((s.num_heads * s.value_dim, s.kv_rank), MATRIX),
        }
        if s.out_gate is not None:
            specs[s.out_gate] = TensorSpec((s.num_heads, s.hidden_size), MATRIX)
        if s.q_down is not None:
            specs[s.q_down] = TensorSpec((s.q_rank, s.hidden_size), MATRIX)
            specs[s.q_norm] = TensorSpec((s.q_rank,), GAIN)
        specs[s.o] = TensorSpec((s.hidden_size, s.num_heads * s.value_dim), MATRIX)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        # what multiplies the mixer's input: the queries' map (or, where queries go through a latent, that latent's
        # map, in the same place), the latent's map, the output gate
        self._inputs = ([tensors[s.q_down] if s.q_down is not None else tensors[s.q], tensors[s.kv_down]]
                        + ([tensors[s.out_gate]] if s.out_gate is not None else []))
        self.q_up = Linear([tensors[s.q]], runtime) if s.q_down is not None else None
        self.q_gain = runtime.gain(tensors[s.q_norm]) if s.q_down is not None else None
        self.k_up = runtime.matrix(tensors[s.k_up])
        self.v_up = runtime.matrix(tensors[s.v_up])
        self._k_up_host, self._v_up_host = tensors[s.k_up], tensors[s.v_up]
        self._up = None                     # both maps stacked, for steps that form every head's keys and values
        self.latent_gain = runtime.gain(tensors[s.latent_norm])
        self.out = Linear([tensors[s.o]], runtime)
        self.position.load(tensors, runtime)
        self._own = None

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        return RowsRequest(self.spec.kv_rank + self.spec.rope_dim, self.spec.window)

    # ------------------------------------------------------------------ step
    def input_projections(self) -> List[torch.Tensor]:
        """The matrices that multiply the mixer's input, in the order ``forward_projected`` expects their sums."""
        return list(self._inputs)

    def forward_projected(self, ctx, cache, proj: torch.Tensor, offset: int, out: torch.Tensor, add: bool = False) -> torch.Tensor:
        """``proj``: float32 [T, F] holding, from column ``offset``, the sums of :meth:`input_projections`;
        writes the mixer's result (before any residual gate) to ``out`` float32 [T, hidden] (``add``: adds it there)."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("latent attention needs its cache of latent rows")
        T = proj.shape[0]
        H, dn, dr, dv, rank = s.num_heads, s.nope_dim, s.rope_dim, s.value_dim, s.kv_rank
        q_off = offset
        kv_off = q_off + (s.q_rank if s.q_down is not None else H * (dn + dr))
        gate_off = kv_off + rank + dr
        rotation = self.position.rotation()
        if rotation is None:
            raise ConfigError("latent attention takes position encodings that are rotations")
        table = ctx.page_tables[cache.group_index]
        q_from = None
        if s.q_down is not None:
            # queries through their own latent: its RMS norm (float32), then the queries' map
            with ops.section("attention.qkv"):
                q_latent = ctx.buffer("latent_q_latent", (T, s.q_rank), rt.act_dtype)
                ops.latent_query_norm(proj, q_off, self.q_gain, s.norm_eps, q_latent)
                q_from = ctx.buffer("latent_q_proj", (T, H * (dn + dr)), torch.float32)
                self.q_up.store(q_latent, q_from, ctx)
        q = ctx.buffer("latent_q", (T, H, dn + dr), torch.float32)
        if self._forms_heads(ctx, cache):
            return self._forward_heads(ctx, cache, proj, q_off, kv_off, gate_off, rotation, table, q, out, q_from, add)
        with ops.section("attention.position"):
            ops.latent_prepare(proj, q_off, kv_off, self.latent_gain, s.norm_eps, rotation, ctx.positions, ctx.seq_ids,
                               table, q, cache.pages, num_heads=H, nope_dim=dn, rope_dim=dr, kv_rank=rank, q_from=q_from)
        q_abs = ctx.buffer("latent_q_absorbed", (T, H, rank + dr), torch.float32)
        with ops.section("attention.absorb"):
            ops.latent_absorb(q, self.k_up, q_abs, nope_dim=dn, rope_dim=dr)
        shares = ops.latent_shares(ctx.num_sequences, ctx.max_new, H, table.shape[1], cache.pages.shape[1])
        if s.window is not None:
            shares = min(shares, -(-s.window // 32) + 1)        # a row sees that many blocks of 32 keys at most
        partials = ctx.buffer("latent_partials", (T, H, shares, rank + 2), torch.float32)
        with ops.section("attention.scores"):
            ops.latent_attend(q_abs, cache.pages, table, ctx.q_start, ctx.kv_len, partials, max_new=ctx.max_new,
                              kv_rank=rank, scale=s.scale, window=s.window)
        o = ctx.buffer("attn_out", (T, H * dv), rt.act_dtype)
        gate = proj[:, gate_off:gate_off + H] if s.out_gate is not None else None
        clear = None if add else self._out_to_clear(ctx, T, out)
        with ops.section("attention.values"):
            if shares > 2 and T > ops.LATENT_ROWS_FORM_TOKENS:
                # many shares in a long step: one CTA per row merges them, so that the value map's CTAs (a tile of
                # tokens each) need not each do it; a short step merges inside the value map's kernel, a CTA per row
                merged = ctx.buffer("latent_merged", (T, H, 1, rank + 2), torch.float32)
                partials = ops.latent_merge(partials, merged)
            ops.latent_expand(partials, self.v_up, gate, o, value_dim=dv, clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("attention.out"):
            if add:
                self.out.accumulate(o, out, ctx)
            else:
                self.out.store(o, out, ctx)
        return out

    def _out_to_clear(self, ctx, tokens: int, out: torch.Tensor):
        """``out`` if the output product will sum partial results into it (the kernel before it then clears it on the
        side), else None."""
        clear = self.out.sums_into(ctx, tokens, "mixer_out", ops.STORE)
        return clear if clear is not None and clear.data_ptr() == out.data_ptr() else None

    # ------------------------------------------------------------------ prompts: every head's keys and values outright
    HEADS_MIN_TOKENS = 48

    def _forms_heads(self, ctx, cache) -> bool:
        """Whether this step forms every head's keys and values and runs the tensor-core attention of ordinary
        heads over them: the bfloat16 path, every sequence at its first token (nothing cached to attend over),
        enough tokens for it to pay, and head sizes that kernel takes."""
        s, rt = self.spec, self.runtime
        hd = self._padded_head()
        return (rt.fast and cache.pages.dtype == torch.bfloat16 and ctx.max_new >= self.HEADS_MIN_TOKENS
                and all(p == 0 for p in ctx.first_positions) and hd is not None and s.value_dim <= hd
                and s.kv_rank % 8 == 0)

    def _padded_head(self):
        """The head size the prompt attention runs at: the next of 64, 128, 192, 256 (the sizes its kernels know at
        compile time), queries, keys and values padded with zeros."""
        need = self.spec.nope_dim + self.spec.rope_dim
        return next((size for size in (64, 128, 192, 256) if need <= size), None)

    def _forward_heads(self, ctx, cache, proj, q_off, kv_off, gate_off, rotation, table, q, out, q_from=None, add=False):
        s = self.spec
        T = proj.shape[0]
        H, dn, dr, dv, rank = s.num_heads, s.nope_dim, s.rope_dim, s.value_dim, s.kv_rank
        hd = self._padded_head()
        page = cache.pages.shape[1]
        latent = ctx.buffer("latent_rows", (T, rank), torch.bfloat16)
        shared = ctx.buffer("latent_shared_key", (T, dr), torch.bfloat16)
        q_half = ctx.buffer("q", (T, H * hd), torch.bfloat16)
        with ops.section("attention.position"):
            ops.latent_prepare(proj, q_off, kv_off, self.latent_gain, s.norm_eps, rotation, ctx.positions, ctx.seq_ids,
                               table, q, cache.pages, num_heads=H, nope_dim=dn, rope_dim=dr, kv_rank=rank,
                               latent_out=latent, shared_out=shared, q_half=q_half, q_from=q_from)
        if self._up is None:
            self._up = Linear([self._k_up_host, self._v_up_host], self.runtime)
        kv = ctx.buffer("latent_heads", (T, H * (dn + dv)), torch.bfloat16)
        with ops.section("attention.heads"):
            self._up.store(latent, kv, ctx)
        # pages of this step only: sequence after sequence, each from a page of its own
        counts = [-(-n // page) for n in ctx.new_counts]
        width = max(counts)
        rows, base = [], 0
        for c in counts:
            rows.append([base + i for i in range(c)] + [0] * (width - c))
            base += c
        step_table = torch.tensor(rows, dtype=torch.int32).to(proj.device, non_blocking=True)
        step_pages = ctx.buffer("latent_head_pages", (base, 2, H, page, hd), torch.bfloat16)
        with ops.section("attention.heads"):
            ops.latent_heads_to_pages(kv, shared, ctx.positions, ctx.seq_ids, step_table, ctx.kv_len, step_pages, num_heads=H,
                                      nope_dim=dn, rope_dim=dr, value_dim=dv)
        heads = ctx.buffer("latent_head_out", (T, H * hd), torch.bfloat16)
        with ops.section("attention.scores"):
            ops.attention_prefill(q_half, heads, step_pages, step_table, ctx.q_start, ctx.kv_len, ctx.max_new, num_heads=H,
                                  num_kv_heads=H, head_dim=hd, scale=s.scale, window=s.window,
                                  exact_weights=s.exact_weights)
        o = ctx.buffer("attn_out", (T, H * dv), torch.bfloat16)
        gate = proj[:, gate_off:gate_off + H] if s.out_gate is not None else None
        clear = None if add else self._out_to_clear(ctx, T, out)
        with ops.section("attention.values"):
            ops.latent_gate_heads(heads, gate, o, num_heads=H, head_dim=hd, value_dim=dv, clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("attention.out"):
            if add:
                self.out.accumulate(o, out, ctx)
            else:
                self.out.store(o, out, ctx)
        return out

    def buffer_to_clear(self, ctx, tokens: int):
        if self._own is None:
            self._own = Linear(self._inputs, self.runtime)
        return self._own.sums_into(ctx, tokens, "mixer_proj", ops.STORE)

    def forward(self, ctx, cache, x, residual: torch.Tensor) -> bool:
        """Adds the mixer's output into ``residual`` (for blocks that hand over a normed input only)."""
        if isinstance(x, PendingNorm):
            x = x.tensor()
        if self._own is None:
            self._own = Linear(self._inputs, self.runtime)
        proj = ctx.buffer("mixer_proj", (x.shape[0], self._own.out_features), torch.float32)
        with ops.section("attention.qkv"):
            self._own.store(x, proj, ctx)
        self.forward_projected(ctx, cache, proj, 0, residual, add=True)      # the output product adds into the stream itself
        return False


MIXERS.register("latent_attention", LatentAttention)
