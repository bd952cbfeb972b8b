"""Softmax attention over a cache of low-rank latents.

Each position keeps one row: the RMS-normed latent c (``kv_rank`` values) and one rotated key part
(``rope_dim`` values) shared by all heads. Head h's key is [k_up[h] c | shared rotated part], its value
v_up[h] c; its query is [nope_dim unrotated | rope_dim rotated]. The kernels apply k_up to the query
instead of to every cached latent, attend over the cached rows with all heads at once, and apply v_up to
the weighted sum of latents (csrc/latent_attention.cu). An optional output gate scales head h's output by
sigmoid(out_gate[h] . x).

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
            s.q: TensorSpec((s.num_heads * (s.nope_dim + s.rope_dim), s.hidden_size), MATRIX),
            s.kv_down: TensorSpec((s.kv_rank + s.rope_dim, s.hidden_size), MATRIX),
            s.latent_norm: TensorSpec((s.kv_rank,), GAIN),
            s.k_up: TensorSpec((s.num_heads * s.nope_dim, s.kv_rank), MATRIX),
            s.v_up: TensorSpec((s.num_heads * s.value_dim, s.kv_rank), MATRIX),
        }
        if s.out_gate is not None:
            specs[s.out_gate] = TensorSpec((s.num_heads, s.hidden_size), MATRIX)
        specs[s.o] = TensorSpec((s.hidden_size, s.num_heads * s.value_dim), MATRIX)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        self._inputs = [tensors[s.q], tensors[s.kv_down]] + ([tensors[s.out_gate]] if s.out_gate is not None else [])
        self.k_up = runtime.matrix(tensors[s.k_up])
        self.v_up = runtime.matrix(tensors[s.v_up])
        self.latent_gain = runtime.gain(tensors[s.latent_norm])
        self.out = Linear([tensors[s.o]], runtime)
        self.position.load(tensors, runtime)
        self._own = None

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        return RowsRequest(self.spec.kv_rank + self.spec.rope_dim)

    # ------------------------------------------------------------------ step
    def input_projections(self) -> List[torch.Tensor]:
        """The matrices that multiply the mixer's input, in the order ``forward_projected`` expects their sums."""
        return list(self._inputs)

    def forward_projected(self, ctx, cache, proj: torch.Tensor, offset: int, out: torch.Tensor) -> torch.Tensor:
        """``proj``: float32 [T, F] holding, from column ``offset``, the sums of :meth:`input_projections`;
        writes the mixer's result (before any residual gate) to ``out`` float32 [T, hidden]."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("latent attention needs its cache of latent rows")
        T = proj.shape[0]
        H, dn, dr, dv, rank = s.num_heads, s.nope_dim, s.rope_dim, s.value_dim, s.kv_rank
        q_off = offset
        kv_off = q_off + H * (dn + dr)
        gate_off = kv_off + rank + dr
        rotation = self.position.rotation()
        if rotation is None:
            raise ConfigError("latent attention takes position encodings that are rotations")
        table = ctx.page_tables[cache.group_index]
        q = ctx.buffer("latent_q", (T, H, dn + dr), torch.float32)
        with ops.section("attention.position"):
            ops.latent_prepare(proj, q_off, kv_off, self.latent_gain, s.norm_eps, rotation, ctx.positions, ctx.seq_ids,
                               table, q, cache.pages, num_heads=H, nope_dim=dn, rope_dim=dr, kv_rank=rank)
        q_abs = ctx.buffer("latent_q_absorbed", (T, H, rank + dr), torch.float32)
        with ops.section("attention.absorb"):
            ops.latent_absorb(q, self.k_up, q_abs, nope_dim=dn, rope_dim=dr)
        shares = ops.latent_shares(ctx.num_sequences, ctx.max_new, H, table.shape[1], cache.pages.shape[1])
        partials = ctx.buffer("latent_partials", (T, H, shares, rank + 2), torch.float32)
        with ops.section("attention.scores"):
            ops.latent_attend(q_abs, cache.pages, table, ctx.q_start, ctx.kv_len, partials, max_new=ctx.max_new,
                              kv_rank=rank, scale=s.scale)
        o = ctx.buffer("attn_out", (T, H * dv), rt.act_dtype)
        gate = proj[:, gate_off:gate_off + H] if s.out_gate is not None else None
        with ops.section("attention.values"):
            ops.latent_expand(partials, self.v_up, gate, o, value_dim=dv)
        with ops.section("attention.out"):
            self.out.store(o, out, ctx)
        return out

    def forward(self, ctx, cache, x, residual: torch.Tensor) -> bool:
        """Adds the mixer's output into ``residual`` (for blocks that hand over a normed input only)."""
        if isinstance(x, PendingNorm):
            x = x.tensor()
        if self._own is None:
            self._own = Linear(self._inputs, self.runtime)
        proj = ctx.buffer("mixer_proj", (x.shape[0], self._own.out_features), torch.float32)
        with ops.section("attention.qkv"):
            self._own.store(x, proj, ctx)
        out = ctx.buffer("mixer_out", tuple(residual.shape), torch.float32)
        self.forward_projected(ctx, cache, proj, 0, out)
        ops.gated_sum(residual, out)
        return False


MIXERS.register("latent_attention", LatentAttention)
