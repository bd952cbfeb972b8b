"""Gated linear attention: a float32 matrix state per head and sequence, decayed per key channel.

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T (q_t * key_dim^-1/2)
    a_t = sigmoid(up(down(x_t)) + bias)^(1 / temperature)

Each head's o_t is RMS-normed over its values with one gain shared by the heads, multiplied by
silu(gate x_t), and the heads are projected by ``o``. The state (kept as [heads, value_dim, key_dim]) starts at zero
(the cache zeroes a slot's row when it is taken) and is carried from step to step; the kernels read the
row of each sequence's slot from the device, so one-token steps replay from captured graphs
(csrc/linear_attention.cu).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import ConfigError, WeightError
from ..kernels import ops
from .base import MIXERS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import ANY, BIAS, GAIN, MATRIX, GatedLinearAttentionSpec, TensorSpec


class GatedLinearAttention(Part):
    capture_safe = True

    def __init__(self, spec: GatedLinearAttentionSpec):
        s = spec
        if s.num_heads <= 0 or s.key_dim <= 0 or s.value_dim <= 0:
            raise ConfigError(f"gated linear attention with {s.num_heads} heads of {s.key_dim} x {s.value_dim}")
        if not s.decay.temperature > 0:
            raise ConfigError(f"decay temperature must be positive, got {s.decay.temperature}")
        self.spec = spec
        self._inputs: List[torch.Tensor] = []
        self._own: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.decay_rank = 0

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        return {
            s.q: TensorSpec((s.num_heads * s.key_dim, s.hidden_size), MATRIX),
            s.k: TensorSpec((s.num_heads * s.key_dim, s.hidden_size), MATRIX),
            s.v: TensorSpec((s.num_heads * s.value_dim, s.hidden_size), MATRIX),
            s.gate: TensorSpec((s.num_heads * s.value_dim, s.hidden_size), MATRIX),
            s.o: TensorSpec((s.hidden_size, s.num_heads * s.value_dim), MATRIX),
            s.out_norm: TensorSpec((s.value_dim,), GAIN),
            s.decay.down: TensorSpec((ANY, s.hidden_size), MATRIX),
            s.decay.up: TensorSpec((s.num_heads * s.key_dim, ANY), MATRIX),
            s.decay.bias: TensorSpec((s.num_heads * s.key_dim,), BIAS),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        down, up = tensors[s.decay.down], tensors[s.decay.up]
        if down.shape[0] != up.shape[1]:
            raise WeightError(f"{s.decay.down} has {down.shape[0]} rows but {s.decay.up} has {up.shape[1]} columns")
        self.decay_rank = int(down.shape[0])
        self._inputs = [tensors[s.q], tensors[s.k], tensors[s.v], tensors[s.gate], down]
        self.decay_up = runtime.matrix(up)
        self.decay_bias = runtime.gain(tensors[s.decay.bias])
        self.out_gain = runtime.gain(tensors[s.out_norm])
        self.out = Linear([tensors[s.o]], runtime)
        self._own = None

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        s = self.spec
        return StateRequest((s.num_heads, s.value_dim, s.key_dim), torch.float32)     # stored [head, value column, key channel]

    # ------------------------------------------------------------------ step
    def input_projections(self) -> List[torch.Tensor]:
        """The matrices that multiply the mixer's input, in the order ``forward_projected`` expects their sums."""
        return list(self._inputs)

    def forward_projected(self, ctx, cache, proj: torch.Tensor, offset: int, out: torch.Tensor) -> torch.Tensor:
        """``proj``: float32 [T, F] holding, from column ``offset``, the sums of :meth:`input_projections`;
        writes the mixer's result (before any residual gate) to ``out`` float32 [T, hidden]."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("gated linear attention needs its per-sequence state")
        T = proj.shape[0]
        H, dk, dv = s.num_heads, s.key_dim, s.value_dim
        q_off = offset
        k_off = q_off + H * dk
        v_off = k_off + H * dk
        g_off = v_off + H * dv
        a_off = g_off + H * dv
        decay = ctx.buffer("gla_decay", (T, H * dk), torch.float32)
        with ops.section("recurrence.decay"):
            ops.gla_decay(proj[:, a_off:a_off + self.decay_rank], self.decay_up, self.decay_bias, decay, s.decay.temperature)
        raw = ctx.buffer("gla_raw", (T, H * dv), torch.float32)
        with ops.section("recurrence.scan"):
            ops.gla_scan(proj, q_off, k_off, v_off, decay, cache.rows, ctx.slots, ctx.q_start, raw, num_heads=H,
                         key_dim=dk, value_dim=dv, q_scale=float(dk) ** -0.5, max_new=ctx.max_new, scratch=ctx.buffer)
        o = ctx.buffer("attn_out", (T, H * dv), rt.act_dtype)
        # an output product that sums partial results into `out` wants it zero: the kernel before it clears it
        clear = self.out.sums_into(ctx, T, "mixer_out", ops.STORE)
        if clear is not None and clear.data_ptr() != out.data_ptr():
            clear = None
        with ops.section("recurrence.norm"):
            ops.gla_finish(raw, self.out_gain, s.norm_eps, proj[:, g_off:g_off + H * dv], o, num_heads=H, value_dim=dv,
                           clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("recurrence.out"):
            self.out.store(o, out, ctx)
        return out

    def forward(self, ctx, cache, x, residual: torch.Tensor) -> bool:
        """Adds the mixer's output into ``residual`` (for blocks that hand over a normed input only)."""
        if isinstance(x, PendingNorm):
            x = x.tensor()
        if self._own is None:
            self._own = Linear(self._inputs, self.runtime)
        proj = ctx.buffer("mixer_proj", (x.shape[0], self._own.out_features), torch.float32)
        with ops.section("recurrence.proj"):
            self._own.store(x, proj, ctx)
        out = ctx.buffer("mixer_out", tuple(residual.shape), torch.float32)
        self.forward_projected(ctx, cache, proj, 0, out)
        ops.gated_sum(residual, out)
        return False


MIXERS.register("gated_linear_attention", GatedLinearAttention)
