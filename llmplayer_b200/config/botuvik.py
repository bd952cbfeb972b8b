"""Configuration of the ``Botuvik`` decoder: attention layers with a score cap and a sink, and matrix-memory
(mLSTM) layers, in an order the configuration lists; dense or mixture-of-experts feed-forwards; a span of layers
that may run several times with the same weights.

``config.json`` holds ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``layers`` and optionally ``loop``.
``layers[i]`` = ``{"type", "mixer": {...}, "mlp": {...} or null}``; layer i's tensors start with ``l<i>.``, the
mixer's with ``l<i>.mix.``, the feed-forward's with ``l<i>.mlp.``.

Every layer has an RMS norm in front of and behind each sublayer (``norm1``, ``norm1b``, ``norm2``, ``norm2b``).

* type ``attention``: ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values), ``scale``, ``softcap``,
  ``rot: {base, dims}`` (interleaved pairs over the first ``dims`` features). Projections with biases; queries and
  keys divided by their root mean square per head after the rotation; a learned sink per head.
* type ``mlstm``: ``heads``, ``dim``, ``vdim``, ``gate_cap``.
* mlp ``{"kind": "dense", "ff"}``: down(relu(up x)^2). mlp ``{"kind": "moe", "expert": {"ff"}, "router":
  {"experts", "top", "groups": {"count", "keep"}}, "shared": {"ff"}}``: gated experts chosen by sigmoid scores within
  the best groups, plus a shared expert.
* ``loop: {start, stop, times}``: layers start .. stop-1 run ``times`` times in a row, each pass with a cache of its
  own; before each pass but the first the embedding's output is added to the stream, and before every pass row
  ``pass`` of the tensor ``loop.step`` [times, width].

The output is the model's norm ``final.norm`` and the matrix ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from ..parts.specs import (
    AttentionSpec, EmbeddingSpec, ExpertRoutingSpec, HeadSpec, MatrixMemorySpec, MixtureSpec, ModelLayout, NormSpec,
    PositionSpec, SandwichBlockSpec, ScheduleEntry, SquaredReLUSpec,
)
from .ramupel import _need
from .registry import ArchitectureConfig, register_architecture


@dataclass(frozen=True)
class CappedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    rot_base: float
    rot_dims: int

    type = "attention"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "CappedAttentionConfig":
        rot = _need(raw, "rot", dict, where)
        return cls(heads=_need(raw, "heads", int, where), kv_heads=_need(raw, "kv_heads", int, where),
                   dim=_need(raw, "dim", int, where), vdim=_need(raw, "vdim", int, where),
                   scale=_need(raw, "scale", float, where), softcap=_need(raw, "softcap", float, where),
                   rot_base=_need(rot, "base", float, where + "rot."), rot_dims=_need(rot, "dims", int, where + "rot."))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "softcap": self.softcap, "rot": {"base": self.rot_base, "dims": self.rot_dims}}

    def validate(self, where: str) -> None:
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}heads {self.heads} is no multiple of kv_heads {self.kv_heads}")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ConfigError(f"{where}rot.dims {self.rot_dims} must be even and at most dim {self.dim}")
        if self.rot_dims and not self.rot_base > 0:
            raise ConfigError(f"{where}rot.base must be positive, got {self.rot_base}")
        if not self.softcap > 0:
            raise ConfigError(f"{where}softcap must be positive, got {self.softcap}")


@dataclass(frozen=True)
class MLSTMConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    type = "mlstm"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "MLSTMConfig":
        return cls(heads=_need(raw, "heads", int, where), dim=_need(raw, "dim", int, where),
                   vdim=_need(raw, "vdim", int, where), gate_cap=_need(raw, "gate_cap", float, where))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}

    def validate(self, where: str) -> None:
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if not self.gate_cap > 0:
            raise ConfigError(f"{where}gate_cap must be positive, got {self.gate_cap}")


@dataclass(frozen=True)
class DenseMLPConfig:
    ff: int

    kind = "dense"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "DenseMLPConfig":
        return cls(ff=_need(raw, "ff", int, where))

    def to_dict(self) -> dict:
        return {"kind": self.kind, "ff": self.ff}

    def validate(self, where: str) -> None:
        if self.ff <= 0:
            raise ConfigError(f"{where}ff must be positive, got {self.ff}")


@dataclass(frozen=True)
class MoEMLPConfig:
    expert_ff: int
    experts: int
    top: int
    groups: int
    keep: int
    shared_ff: int            # 0: no shared expert

    kind = "moe"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "MoEMLPConfig":
        router = _need(raw, "router", dict, where)
        groups = _need(router, "groups", dict, where + "router.")
        shared = raw.get("shared")
        if shared is not None and not isinstance(shared, dict):
            raise ConfigError(f"{where}shared must be an object or null")
        return cls(expert_ff=_need(_need(raw, "expert", dict, where), "ff", int, where + "expert."),
                   experts=_need(router, "experts", int, where + "router."), top=_need(router, "top", int, where + "router."),
                   groups=_need(groups, "count", int, where + "router.groups."),
                   keep=_need(groups, "keep", int, where + "router.groups."),
                   shared_ff=_need(shared, "ff", int, where + "shared.") if shared is not None else 0)

    def to_dict(self) -> dict:
        return {"kind": self.kind, "expert": {"ff": self.expert_ff},
                "router": {"experts": self.experts, "top": self.top, "groups": {"count": self.groups, "keep": self.keep}},
                "shared": {"ff": self.shared_ff} if self.shared_ff > 0 else None}

    def validate(self, where: str) -> None:
        for name in ("expert_ff", "experts", "top", "groups", "keep"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if self.shared_ff < 0:
            raise ConfigError(f"{where}shared.ff must not be negative, got {self.shared_ff}")
        if self.experts % self.groups:
            raise ConfigError(f"{where}{self.experts} experts cannot form {self.groups} equal groups")
        if self.keep > self.groups:
            raise ConfigError(f"{where}{self.keep} of {self.groups} groups kept")
        if self.top > self.keep * (self.experts // self.groups):
            raise ConfigError(f"{where}{self.top} experts cannot be chosen from {self.keep} groups of {self.experts // self.groups}")


_MIXERS = {CappedAttentionConfig.type: CappedAttentionConfig, MLSTMConfig.type: MLSTMConfig}
_MLPS = {DenseMLPConfig.kind: DenseMLPConfig, MoEMLPConfig.kind: MoEMLPConfig}


@dataclass(frozen=True)
class BotuvikLayerConfig:
    mixer: object                      # CappedAttentionConfig or MLSTMConfig
    mlp: Optional[object]              # DenseMLPConfig, MoEMLPConfig or None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BotuvikConfig(ArchitectureConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BotuvikLayerConfig, ...]
    loop: Optional[LoopConfig] = None

    architecture = "Botuvik"
    # the design sets no limit on positions; this is the engine's default context when none is asked for
    DEFAULT_CONTEXT = 131072

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "BotuvikConfig":
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
            layers.append(BotuvikLayerConfig(mixer, mlp))
        loop = None
        loop_raw = raw.get("loop")
        if loop_raw is not None:
            if not isinstance(loop_raw, dict):
                raise ConfigError("loop must be an object or null")
            loop = LoopConfig(start=_need(loop_raw, "start", int, "loop."), stop=_need(loop_raw, "stop", int, "loop."),
                              times=_need(loop_raw, "times", int, "loop."))
        cfg = cls(vocab=_need(raw, "vocab", int, ""), width=_need(raw, "width", int, ""),
                  norm_eps=_need(_need(raw, "norm", dict, ""), "eps", float, "norm."), layers=tuple(layers), loop=loop)
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
        if self.loop is not None:
            lp = self.loop
            if not 0 <= lp.start < lp.stop <= len(self.layers):
                raise ConfigError(f"loop over layers {lp.start} .. {lp.stop - 1} of {len(self.layers)}")
            if lp.times <= 0:
                raise ConfigError(f"loop.times must be positive, got {lp.times}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        out = {
            "architecture": self.architecture,
            "layers": [{"type": layer.mixer.type, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    # ------------------------------------------------------------------ meaning
    def max_positions(self) -> int:
        return self.DEFAULT_CONTEXT

    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """The runs of the layers: the looped span ``times`` times in a row (every pass is a run of its own, so it has
        a cache and state of its own), the embedding's output added before every pass but the first, and the pass's
        row of ``loop.step`` before every pass."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(ScheduleEntry(i) for i in range(n))
        lp = self.loop
        runs = [ScheduleEntry(i) for i in range(lp.start)]
        for t in range(lp.times):
            for i in range(lp.start, lp.stop):
                if i == lp.start:
                    runs.append(ScheduleEntry(i, add_embedding=t > 0, add_vector="loop.step", add_row=t))
                else:
                    runs.append(ScheduleEntry(i))
        runs.extend(ScheduleEntry(i) for i in range(lp.stop, n))
        return tuple(runs)

    def layout(self) -> ModelLayout:
        d, eps = self.width, self.norm_eps
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer.mixer
            if isinstance(m, CappedAttentionConfig):
                position = (PositionSpec(kind="rope", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                         pairing="interleaved")
                            if m.rot_dims > 0 else PositionSpec(kind="none", head_dim=m.dim))
                mixer = AttentionSpec(
                    hidden_size=d, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                    position=position, q=p + "mix.q", k=p + "mix.k", v=p + "mix.v", o=p + "mix.o", value_dim=m.vdim,
                    q_bias=p + "mix.q.b", k_bias=p + "mix.k.b", v_bias=p + "mix.v.b", unit_norm_eps=eps,
                    softcap=m.softcap, sink=p + "mix.sink", exact_weights=True)
            else:
                mixer = MatrixMemorySpec(
                    hidden_size=d, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, norm_eps=eps, gate_cap=m.gate_cap,
                    q=p + "mix.q", k=p + "mix.k", v=p + "mix.v", gate=p + "mix.g", input_gate=p + "mix.i",
                    input_gate_bias=p + "mix.i.b", forget_gate=p + "mix.f", forget_gate_bias=p + "mix.f.b",
                    out_norm=p + "mix.norm", o=p + "mix.o")
            ffn = None
            if isinstance(layer.mlp, DenseMLPConfig):
                ffn = SquaredReLUSpec(hidden_size=d, intermediate_size=layer.mlp.ff, up=p + "mlp.up", down=p + "mlp.down")
            elif isinstance(layer.mlp, MoEMLPConfig):
                c = layer.mlp
                ffn = MixtureSpec(
                    hidden_size=d, expert_size=c.expert_ff,
                    routing=ExpertRoutingSpec(num_experts=c.experts, top=c.top, groups=c.groups, keep_groups=c.keep,
                                              router=p + "mlp.router"),
                    expert_prefix=p + "mlp.", shared_size=c.shared_ff, shared_prefix=p + "mlp.shared." if c.shared_ff else None)
            blocks.append(SandwichBlockSpec(
                mixer_norm=NormSpec(d, eps, p + "norm1"), mixer=mixer, post_mixer_norm=NormSpec(d, eps, p + "norm1b"),
                ffn_norm=NormSpec(d, eps, p + "norm2") if ffn is not None else None, ffn=ffn,
                post_ffn_norm=NormSpec(d, eps, p + "norm2b") if ffn is not None else None))
        return ModelLayout(
            embedding=EmbeddingSpec(self.vocab, d, "embed"), layers=tuple(blocks),
            head=HeadSpec(self.vocab, d, norm=NormSpec(d, eps, "final.norm"), weight="head"), schedule=self.schedule())

    def ignorable_tensors(self) -> tuple:
        # a layer without a feed-forward has no use for the norms around one, nor a model without a loop for the
        # passes' vectors, should a file carry them
        spare = [f"l{i}.{n}" for i, layer in enumerate(self.layers) if layer.mlp is None for n in ("norm2", "norm2b")]
        if self.loop is None:
            spare.append("loop.step")
        return tuple(spare)

    def describe(self) -> str:
        lines = [f"architecture: {self.architecture}", f"  vocab = {self.vocab}", f"  width = {self.width}",
                 f"  norm.eps = {self.norm_eps}"]
        for i, layer in enumerate(self.layers):
            sizes = ", ".join(f"{k}={v}" for k, v in layer.mixer.to_dict().items())
            lines.append(f"  layer {i}: {layer.mixer.type} ({sizes}), feed-forward {None if layer.mlp is None else layer.mlp.to_dict()}")
        if self.loop is not None:
            lines.append(f"  layers {self.loop.start} .. {self.loop.stop - 1} run {self.loop.times} times")
        return "\n".join(lines)


register_architecture(BotuvikConfig.architecture, BotuvikConfig)
