"""Matrix memory with exponential gates (the mLSTM of the xLSTM family): per head a float32 state S [dk, dv], a
normaliser n [dk] and a running maximum m of the gates' logarithms.

    i_t = cap * tanh((W_i x_t + b_i) / cap)                     log input gate, per head
    f_t = logsigmoid(cap * tanh((W_f x_t + b_f) / cap))         log forget gate, per head
    m_t = max(f_t + m_(t-1), i_t)                               m starts at 0
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),     q_t scaled by dk^-1/2

Each head's o_t is divided by its root mean square; the heads are multiplied by a gain over all heads' values
and by sigmoid(W_g x_t), then projected. State, gates, decays and every sum are float32.

The recurrence is the framework's gated-linear-attention scan (csrc/linear_attention.cu) with one decay per head,
the input gate as a gain of the keys, and n as one more value column that is fed the constant 1; the gates and
the maximum come from a kernel of their own that walks a sequence's tokens in order. All kernels read the step
from device tensors (slots, offsets), so one-token steps replay from captured graphs.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import BIAS, GAIN, MATRIX, MatrixMemorySpec, TensorSpec


class MatrixMemory(Part):
    capture_safe = True

    def __init__(self, spec: MatrixMemorySpec):
        s = spec
        if s.num_heads <= 0 or s.key_dim <= 0 or s.value_dim <= 0:
            raise ConfigError(f"matrix memory with {s.num_heads} heads of {s.key_dim} x {s.value_dim}")
        if s.gate_cap is not None and not s.gate_cap > 0:
            raise ConfigError(f"gate cap must be positive or absent, got {s.gate_cap}")
        self.spec = spec
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        H, d = s.num_heads, s.hidden_size
        return {
            s.q: TensorSpec((H * s.key_dim, d), MATRIX),
            s.k: TensorSpec((H * s.key_dim, d), MATRIX),
            s.v: TensorSpec((H * s.value_dim, d), MATRIX),
            s.gate: TensorSpec((H * s.value_dim, d), MATRIX),
            s.o: TensorSpec((d, H * s.value_dim), MATRIX),
            s.out_norm: TensorSpec((H * s.value_dim,), GAIN),
            s.input_gate: TensorSpec((H, d), MATRIX),
            s.input_gate_bias: TensorSpec((H,), BIAS),
            s.forget_gate: TensorSpec((H, d), MATRIX),
            s.forget_gate_bias: TensorSpec((H,), BIAS),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        # one product of the normed input: queries, keys, values, output gate, and the two gates' pre-activations
        self.proj = Linear([tensors[n] for n in (s.q, s.k, s.v, s.gate, s.input_gate, s.forget_gate)], runtime)
        self.bias_i = runtime.gain(tensors[s.input_gate_bias])
        self.bias_f = runtime.gain(tensors[s.forget_gate_bias])
        self.out_gain = runtime.gain(tensors[s.out_norm])
        self.out = Linear([tensors[s.o]], runtime)

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        s = self.spec
        # S and n together, stored [head, value column (the last one is n), key channel]; and m per head
        return (StateRequest((s.num_heads, s.value_dim + 1, s.key_dim), torch.float32),
                StateRequest((s.num_heads,), torch.float32))

    # ------------------------------------------------------------------ step
    def buffer_to_clear(self, ctx, tokens: int):
        return self.proj.sums_into(ctx, tokens, "mixer_proj", ops.STORE)

    def forward(self, ctx, cache, x, residual: torch.Tensor, overwrite: bool = False) -> bool:
        """Adds the mixer's output into ``residual`` (``overwrite``: stores it there instead)."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("a matrix memory needs its per-sequence state")
        if isinstance(x, PendingNorm):
            x = x.tensor()
        T = x.shape[0]
        H, dk, dv = s.num_heads, s.key_dim, s.value_dim
        proj = ctx.buffer("mixer_proj", (T, self.proj.out_features), torch.float32)
        with ops.section("recurrence.proj"):
            self.proj.store(x, proj, ctx)
        q_off, k_off, v_off = 0, H * dk, 2 * H * dk
        g_off = v_off + H * dv
        i_off = g_off + H * dv
        f_off = i_off + H
        state, maxima = cache.blocks
        gates = ctx.buffer("exp_gates", (3, T, H), torch.float32)
        with ops.section("recurrence.gates"):
            ops.exp_gates(proj, i_off, f_off, self.bias_i, self.bias_f, s.gate_cap, maxima, ctx.slots, ctx.q_start,
                          gates[0], gates[1], gates[2])
        raw = ctx.buffer("memory_raw", (T, H * (dv + 1)), torch.float32)
        with ops.section("recurrence.scan"):
            ops.gla_scan(proj, q_off, k_off, v_off, gates[0], state, ctx.slots, ctx.q_start, raw, num_heads=H,
                         key_dim=dk, value_dim=dv + 1, q_scale=float(dk) ** -0.5, max_new=ctx.max_new, scratch=ctx.buffer,
                         decay_per_head=True, key_gain=gates[1], ones_column=True)
        o = ctx.buffer("attn_out", (T, H * dv), rt.act_dtype)
        with ops.section("recurrence.norm"):
            # an output product that sums partial results wants its target zero: this kernel clears it on the side
            clear = residual if overwrite and residual.dtype == torch.float32 and self.out.needs_zero(T) else None
            ops.gla_finish(raw, self.out_gain, s.norm_eps, proj[:, g_off:g_off + H * dv], o, num_heads=H, value_dim=dv,
                           gain_per_head=True, gate_sigmoid=True, max_row=gates[2], clear=clear)
        if clear is not None:
            ctx.note_cleared()
        with ops.section("recurrence.out"):
            if overwrite:
                self.out.store(o, residual, ctx)
            else:
                self.out.accumulate(o, residual, ctx)
        return False


MIXERS.register("matrix_memory", MatrixMemory)
