"""Typed configuration of the Pitolix decoder, read from config.json.

A Pitolix model is a list of layers whose two sublayers run side by side, each behind a norm of its own:
x += mixer(norm1 x) + ff(norm2 x).  Two mixers, both grouped-query softmax attention over every earlier position:
"attention" (no rotation; unit-RMS queries and keys; a query factor that grows by steps with the position; a learned sink in
the softmax's denominator; a gate per element of the heads' outputs) and "attention_2" (biased projections; a rotation over
the leading part of each head, element i paired with i + dims/2; plain softmax; a gate per head).  The feed-forward is gated
with SiLU, or absent.  A span of layers may run several times with the same weights: from the second pass on the embedding's
output joins the stream again, and every pass adds a vector of its own.  Every size and every constant that can differ
between models is a field here; the parts and kernels carry none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError
from .turudra import LoopConfig, _get

NAME = "Pitolix"


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int              # positions per step of the factor 1 + coef ln(floor((p + 1) / every) + 1)

    @classmethod
    def from_dict(cls, d, where):
        c = cls(coef=_get(d, "coef", float, where), every=_get(d, "every", int, where))
        if c.every < 1:
            raise ConfigError(f"config.json: {where}.every must be positive")
        return c


def _sizes(d, where):
    heads = _get(d, "heads", int, where)
    kv_heads = _get(d, "kv_heads", int, where, heads)
    dim = _get(d, "dim", int, where)
    vdim = _get(d, "vdim", int, where, dim)
    if min(heads, kv_heads, dim, vdim) < 1 or heads % kv_heads:
        raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
    return heads, kv_heads, dim, vdim


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                # query/key elements per head
    vdim: int               # value elements per head
    scale: float
    q_temp: Optional[QueryTemperature]
    kind: str = "attention"

    @classmethod
    def from_dict(cls, d, where):
        heads, kv_heads, dim, vdim = _sizes(d, where)
        qt = d.get("q_temp")
        return cls(heads, kv_heads, dim, vdim, scale=_get(d, "scale", float, where),
                   q_temp=QueryTemperature.from_dict(qt, where + ".q_temp") if qt else None)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.q_temp is not None:
            d["q_temp"] = {"coef": self.q_temp.coef, "every": self.q_temp.every}
        return d


@dataclass(frozen=True)
class RotaryAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int           # leading elements of a head that are rotated, i paired with i + rot_dims / 2 (0: none)
    kind: str = "attention_2"

    @classmethod
    def from_dict(cls, d, where):
        heads, kv_heads, dim, vdim = _sizes(d, where)
        rot = d.get("rot")
        base, dims = 10000.0, 0
        if rot:
            base, dims = _get(rot, "base", float, where + ".rot"), _get(rot, "dims", int, where + ".rot")
        if dims % 2 or dims > dim or not base > 0:
            raise ConfigError(f"config.json: {where}.rot: dims must be even and at most dim, base positive")
        return cls(heads, kv_heads, dim, vdim, scale=_get(d, "scale", float, where), rot_base=base, rot_dims=dims)

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where, "dense")
        if kind != "dense":
            raise ConfigError(f"config.json: {where}.kind '{kind}' is not supported (known: dense)")
        c = cls(ff=_get(d, "ff", int, where))
        if c.ff < 1:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return c


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                       # SinkAttentionConfig | RotaryAttentionConfig
    mlp: Optional[DenseConfig]


@dataclass(frozen=True)
class PitolixConfig:
    architecture: str
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    loop: Optional[LoopConfig]
    embedding_scale: float
    norm_eps: float
    torch_dtype: str = "bfloat16"

    MIXERS = {"attention": SinkAttentionConfig, "attention_2": RotaryAttentionConfig}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "PitolixConfig":
        top = "top level"
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(raw):
            where = f"layers[{i}]"
            kind = _get(lr, "type", str, where)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not supported (known: {', '.join(sorted(cls.MIXERS))})")
            if not isinstance(lr.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} lacks 'mixer'")
            mixer = cls.MIXERS[kind].from_dict(lr["mixer"], where + ".mixer")
            mlp = DenseConfig.from_dict(lr["mlp"], where + ".mlp") if lr.get("mlp") else None
            layers.append(LayerConfig(mixer, mlp))
        loop = None
        if d.get("loop"):
            lp = d["loop"]
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"), _get(lp, "times", int, "loop"))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError("config.json: loop needs 0 <= start < stop <= number of layers and times >= 1")
        emb = d.get("embedding") or {}
        norm = d.get("norm") or {}
        cfg = cls(architecture=NAME, vocab=_get(d, "vocab", int, top), width=_get(d, "width", int, top), layers=tuple(layers),
                  loop=loop, embedding_scale=_get(emb, "scale", float, "embedding", 1.0), norm_eps=_get(norm, "eps", float, "norm"),
                  torch_dtype=_get(d, "torch_dtype", str, top, "bfloat16"))
        if cfg.vocab < 1 or cfg.width < 1:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    def layer_runs(self):
        """[(layer index, number of the pass it opens or None)] in the order the layers run."""
        L = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(L)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        runs = [(i, None) for i in range(a)]
        for t in range(times):
            runs += [(i, t if i == a else None) for i in range(a, b)]
        return runs + [(i, None) for i in range(b, L)]

    def to_dict(self) -> dict:
        """The config.json of this configuration."""
        return {"architecture": NAME, "vocab": self.vocab, "width": self.width, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(),
                            "mlp": None if l.mlp is None else {"kind": "dense", "ff": l.mlp.ff}} for l in self.layers],
                "loop": None if self.loop is None else {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times},
                "torch_dtype": self.torch_dtype}
