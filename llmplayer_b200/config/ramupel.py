"""Configuration of the ``Ramupel`` decoder: a hybrid of latent-attention layers and gated-linear-attention
layers in an order the configuration lists.

``config.json`` holds ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and ``layers``, a list
of ``{"type", "mixer": {...sizes and constants of the mixer...}, "mlp": {"kind": "dense", "ff": n} or null}``.
Tensors of layer i start with ``l<i>.``; the mixer's with ``l<i>.mix.``, the feed-forward's with ``l<i>.mlp.``.

Every layer is a parallel block: one layer norm (gain, no bias) whose output the mixer and the feed-forward
both read, each result multiplied by a sigmoid gate computed from the same normed input, and after the
residual sum a learned weighted sum over the embedding's output and all layers' results so far. The token
embedding is multiplied by a constant; the output is the model's norm followed by the embedding table as the
head (without that constant).

Mixer ``latent_attention``: ``heads``, ``dim`` unrotated and ``rot_dim`` rotated query/key sizes, ``vdim``,
``kv_rank``, ``scale``, ``rot: {base, dims}`` (split-half pairs over the first ``dims`` of the rotated part), a
sigmoid gate per head on the output. Mixer ``gla``: ``heads``, ``dim``, ``vdim``, decay temperature ``tau``; the
width of the decay's low-rank factor is read off the tensors. Feed-forward: dense, xIELU activation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from ..parts.specs import (
    DepthMixSpec, EmbeddingSpec, GatedLinearAttentionSpec, HeadSpec, LatentAttentionSpec, LowRankDecaySpec,
    ModelLayout, NormSpec, ParallelBlockSpec, PositionSpec, ResidualGateSpec, XIELUSpec,
)
from .registry import ArchitectureConfig, register_architecture


def _need(raw: dict, key: str, kind, where: str):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks {where}{key!r}")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"{where}{key} must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{where}{key} must be a number, got {value!r}")
        return float(value)
    if kind is dict:
        if not isinstance(value, dict):
            raise ConfigError(f"{where}{key} must be an object, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"{where}{key} must be a string, got {value!r}")
        return value
    raise AssertionError(kind)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int

    type = "latent_attention"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "LatentMixerConfig":
        rot = _need(raw, "rot", dict, where)
        return cls(heads=_need(raw, "heads", int, where), dim=_need(raw, "dim", int, where),
                   rot_dim=_need(raw, "rot_dim", int, where), vdim=_need(raw, "vdim", int, where),
                   kv_rank=_need(raw, "kv_rank", int, where), scale=_need(raw, "scale", float, where),
                   rot_base=_need(rot, "base", float, where + "rot."), rot_dims=_need(rot, "dims", int, where + "rot."))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}

    def validate(self, where: str) -> None:
        for name in ("heads", "vdim", "kv_rank"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if self.dim < 0 or self.rot_dim < 0 or self.dim + self.rot_dim <= 0:
            raise ConfigError(f"{where}dim {self.dim} and rot_dim {self.rot_dim} leave no query")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ConfigError(f"{where}rot.dims {self.rot_dims} must be even and at most rot_dim {self.rot_dim}")
        if self.rot_dims and not self.rot_base > 0:
            raise ConfigError(f"{where}rot.base must be positive, got {self.rot_base}")


@dataclass(frozen=True)
class GLAMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float

    type = "gla"

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "GLAMixerConfig":
        return cls(heads=_need(raw, "heads", int, where), dim=_need(raw, "dim", int, where),
                   vdim=_need(raw, "vdim", int, where), tau=_need(raw, "tau", float, where))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}

    def validate(self, where: str) -> None:
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}{name} must be positive, got {getattr(self, name)}")
        if not self.tau > 0:
            raise ConfigError(f"{where}tau must be positive, got {self.tau}")


_MIXERS = {LatentMixerConfig.type: LatentMixerConfig, GLAMixerConfig.type: GLAMixerConfig}


@dataclass(frozen=True)
class RamupelLayerConfig:
    mixer: object                      # LatentMixerConfig or GLAMixerConfig
    ff: Optional[int]                  # width of the dense feed-forward, None for a layer without one


@dataclass(frozen=True)
class RamupelConfig(ArchitectureConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[RamupelLayerConfig, ...]

    architecture = "Ramupel"
    # the design sets no limit on positions; this is the engine's default context when none is asked for
    DEFAULT_CONTEXT = 131072

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "RamupelConfig":
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
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{where}mlp must be an object or null")
                mlp_kind = _need(mlp, "kind", str, where + "mlp.")
                if mlp_kind != "dense":
                    raise ConfigError(f"{where}mlp.kind {mlp_kind!r} is unknown; known: dense")
                ff = _need(mlp, "ff", int, where + "mlp.")
            layers.append(RamupelLayerConfig(mixer, ff))
        cfg = cls(vocab=_need(raw, "vocab", int, ""), width=_need(raw, "width", int, ""),
                  embedding_scale=_need(_need(raw, "embedding", dict, ""), "scale", float, "embedding."),
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
            layer.mixer.validate(f"layers[{i}].mixer.")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive, got {layer.ff}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": layer.mixer.type, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}}
                       for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    # ------------------------------------------------------------------ meaning
    def max_positions(self) -> int:
        return self.DEFAULT_CONTEXT

    def ignorable_tensors(self) -> tuple:
        # a layer without a feed-forward has no use for the feed-forward's gate, should a file carry one
        return tuple(f"l{i}.rg2{suffix}" for i, layer in enumerate(self.layers) if layer.ff is None for suffix in ("", ".b"))

    def layout(self) -> ModelLayout:
        d = self.width
        total = len(self.layers) + 1
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer.mixer
            if isinstance(m, LatentMixerConfig):
                position = (PositionSpec(kind="rope", head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                         pairing="split_half")
                            if m.rot_dims > 0 else PositionSpec(kind="none", head_dim=m.rot_dim))
                mixer = LatentAttentionSpec(
                    hidden_size=d, num_heads=m.heads, nope_dim=m.dim, rope_dim=m.rot_dim, value_dim=m.vdim,
                    kv_rank=m.kv_rank, scale=m.scale, norm_eps=self.norm_eps, position=position,
                    q=p + "mix.q", kv_down=p + "mix.dkv", latent_norm=p + "mix.dkv.norm", k_up=p + "mix.uk",
                    v_up=p + "mix.uv", o=p + "mix.o", out_gate=p + "mix.g")
            else:
                mixer = GatedLinearAttentionSpec(
                    hidden_size=d, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, norm_eps=self.norm_eps,
                    decay=LowRankDecaySpec(temperature=m.tau, down=p + "mix.a1", up=p + "mix.a2", bias=p + "mix.a2.b"),
                    q=p + "mix.q", k=p + "mix.k", v=p + "mix.v", gate=p + "mix.g", out_norm=p + "mix.norm", o=p + "mix.o")
            ffn = None
            if layer.ff is not None:
                ffn = XIELUSpec(hidden_size=d, intermediate_size=layer.ff, up=p + "mlp.up", down=p + "mlp.down",
                                act=p + "mlp.act")
            blocks.append(ParallelBlockSpec(
                norm=NormSpec(d, self.norm_eps, p + "norm1", kind="layernorm"), mixer=mixer, ffn=ffn,
                mixer_gate=ResidualGateSpec(p + "rg1", p + "rg1.b"),
                ffn_gate=ResidualGateSpec(p + "rg2", p + "rg2.b") if ffn is not None else None,
                depth_mix=DepthMixSpec(p + "dwa", i + 2, total)))
        return ModelLayout(
            embedding=EmbeddingSpec(self.vocab, d, "embed", scale=self.embedding_scale),
            layers=tuple(blocks),
            head=HeadSpec(self.vocab, d, norm=NormSpec(d, self.norm_eps, "final.norm", kind="layernorm"), weight="embed"))

    def describe(self) -> str:
        lines = [f"architecture: {self.architecture}", f"  vocab = {self.vocab}", f"  width = {self.width}",
                 f"  embedding.scale = {self.embedding_scale}", f"  norm.eps = {self.norm_eps}"]
        for i, layer in enumerate(self.layers):
            sizes = ", ".join(f"{k}={v}" for k, v in layer.mixer.to_dict().items())
            lines.append(f"  layer {i}: {layer.mixer.type} ({sizes}), feed-forward {layer.ff}")
        return "\n".join(lines)


register_architecture(RamupelConfig.architecture, RamupelConfig)
