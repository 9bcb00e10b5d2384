"""Typed configuration of the Buzarax decoder, read from config.json.

A Buzarax model is a list of layers whose norms act on the sublayers' outputs: x += norm1(mixer(x)), x += norm2(ff(x)), each
norm an RMS norm with ONE gain; behind every layer the stream becomes a learned mixture of the embedding's output and of what
every layer so far has left.  The embedding adds a row of a second table chosen by a hash of the previous and the current
token.  Two mixers: "rglru" (a gated branch beside a short convolution and a real-gated linear recurrence per channel, its gates
block-diagonal) and "parallel" (softmax attention and linear attention with a per-head decay side by side, each with a scale).
The attention rotates part of every query and key head with wavelength-interpolated frequencies, divides the rotated heads by
their root mean square, rotates its values over their whole length and turns the sums back, caps its scores and has a sink of
score zero.  The feed-forward is dense (a clamped gated activation) or a mixture of experts chosen by sigmoid scores plus a
correction, weighted by the scores as they are; or absent.  The logits are capped.  Every size and every constant that can
differ between models is a field here; the parts and kernels carry none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError
from .turudra import _get

NAME = "Buzarax"


@dataclass(frozen=True)
class YarnConfig:
    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, d, where):
        c = cls(factor=_get(d, "factor", float, where), original=_get(d, "original", float, where),
                fast=_get(d, "fast", float, where), slow=_get(d, "slow", float, where))
        if not (c.factor > 0 and c.original > 0 and c.fast > 0 and c.slow > 0):
            raise ConfigError(f"config.json: {where}: factor, original, fast and slow must be positive")
        return c

    def to_dict(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int                          # leading elements of a query/key head that are rotated, element i with i + dims/2
    scaling: Optional[YarnConfig]

    @classmethod
    def from_dict(cls, d, where):
        if d is None:
            return cls(10000.0, 0, None)
        sc = d.get("scaling") if isinstance(d, Mapping) else None
        c = cls(base=_get(d, "base", float, where), dims=_get(d, "dims", int, where),
                scaling=YarnConfig.from_dict(sc, where + ".scaling") if sc else None)
        if c.dims % 2 or not c.base > 1:
            raise ConfigError(f"config.json: {where}: dims must be even and base above one")
        return c

    def to_dict(self):
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = self.scaling.to_dict()
        return d


@dataclass(frozen=True)
class SoftmaxSideConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    rot: RotationConfig

    @classmethod
    def from_dict(cls, d, where):
        heads = _get(d, "heads", int, where)
        c = cls(heads=heads, kv_heads=_get(d, "kv_heads", int, where, heads), dim=_get(d, "dim", int, where),
                vdim=_get(d, "vdim", int, where), scale=_get(d, "scale", float, where),
                softcap=_get(d, "softcap", float, where, None), rot=RotationConfig.from_dict(d.get("rot"), where + ".rot"))
        if min(c.heads, c.kv_heads, c.dim, c.vdim) < 1 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        if c.rot.dims > c.dim:
            raise ConfigError(f"config.json: {where}.rot.dims exceeds dim")
        if c.vdim % 2:
            raise ConfigError(f"config.json: {where}.vdim must be even (the values are rotated in pairs)")
        if c.softcap is not None and not c.softcap > 0:
            raise ConfigError(f"config.json: {where}.softcap must be positive")
        return c

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": self.rot.to_dict()}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class DecaySideConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, d, where):
        raw = d.get("decay") if isinstance(d, Mapping) else None
        if not isinstance(raw, list) or not all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in raw):
            raise ConfigError(f"config.json: {where}.decay must be a list of numbers, one per head")
        c = cls(heads=_get(d, "heads", int, where), dim=_get(d, "dim", int, where), vdim=_get(d, "vdim", int, where),
                decay=tuple(float(v) for v in raw))
        if min(c.heads, c.dim, c.vdim) < 1 or len(c.decay) != c.heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and decay hold one number per head")
        return c

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class ParallelConfig:
    left: SoftmaxSideConfig
    right: DecaySideConfig
    left_scale: float
    right_scale: float
    kind: str = "parallel"

    @classmethod
    def from_dict(cls, d, where):
        return cls(left=SoftmaxSideConfig.from_dict(_get(d, "left", dict, where), where + ".left"),
                   right=DecaySideConfig.from_dict(_get(d, "right", dict, where), where + ".right"),
                   left_scale=_get(d, "left_scale", float, where, 1.0), right_scale=_get(d, "right_scale", float, where, 1.0))

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale, "right_scale": self.right_scale}


@dataclass(frozen=True)
class RecurrentConfig:
    width: int                 # channels of the recurrence
    blocks: int                # diagonal blocks of the gates' matrices
    conv: int                  # taps of the convolution
    kind: str = "rglru"

    @classmethod
    def from_dict(cls, d, where):
        c = cls(width=_get(d, "width", int, where), blocks=_get(d, "blocks", int, where), conv=_get(d, "conv", int, where))
        if min(c.width, c.blocks, c.conv) < 1 or c.width % c.blocks:
            raise ConfigError(f"config.json: {where}: sizes must be positive and width a multiple of blocks")
        return c

    def to_dict(self):
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float
    kind: str = "dense"

    @classmethod
    def from_dict(cls, d, where):
        c = cls(ff=_get(d, "ff", int, where), limit=_get(d, "limit", float, where))
        if c.ff < 1 or not c.limit > 0:
            raise ConfigError(f"config.json: {where}: ff and limit must be positive")
        return c

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    kind: str = "moe"

    @classmethod
    def from_dict(cls, d, where):
        r = _get(d, "router", dict, where)
        c = cls(experts=_get(r, "experts", int, where + ".router"), top=_get(r, "top", int, where + ".router"),
                ff=_get(_get(d, "expert", dict, where), "ff", int, where + ".expert"))
        if c.ff < 1 or not (1 <= c.top <= c.experts):
            raise ConfigError(f"config.json: {where}: expert.ff must be positive and 1 <= router.top <= router.experts")
        return c

    def to_dict(self):
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                       # ParallelConfig | RecurrentConfig
    mlp: Any                         # DenseConfig | ExpertsConfig | None


@dataclass(frozen=True)
class BuzaraxConfig:
    architecture: str
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    logit_softcap: Optional[float]
    torch_dtype: str = "bfloat16"

    MIXERS = {"parallel": ParallelConfig, "rglru": RecurrentConfig}
    MLPS = {"dense": DenseConfig, "moe": ExpertsConfig}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BuzaraxConfig":
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
            mixer = cls.MIXERS[kind].from_dict(_get(lr, "mixer", dict, where), where + ".mixer")
            mlp = None
            if lr.get("mlp"):
                mk = _get(lr["mlp"], "kind", str, where + ".mlp", "dense")
                if mk not in cls.MLPS:
                    raise ConfigError(f"config.json: {where}.mlp.kind '{mk}' is not supported (known: {', '.join(sorted(cls.MLPS))})")
                mlp = cls.MLPS[mk].from_dict(lr["mlp"], where + ".mlp")
            layers.append(LayerConfig(mixer, mlp))
        norm = d.get("norm") or {}
        big = _get(_get(d, "embedding", dict, top), "bigram", dict, "embedding")
        cfg = cls(architecture=NAME, vocab=_get(d, "vocab", int, top), width=_get(d, "width", int, top), layers=tuple(layers),
                  norm_eps=_get(norm, "eps", float, "norm"), buckets=_get(big, "buckets", int, "embedding.bigram"),
                  mul_prev=_get(big, "mul_prev", int, "embedding.bigram"), mul_cur=_get(big, "mul_cur", int, "embedding.bigram"),
                  logit_softcap=_get(d, "logit_softcap", float, top, None), torch_dtype=_get(d, "torch_dtype", str, top, "bfloat16"))
        if cfg.vocab < 1 or cfg.width < 1 or cfg.buckets < 1:
            raise ConfigError("config.json: vocab, width and embedding.bigram.buckets must be positive")
        if cfg.logit_softcap is not None and not cfg.logit_softcap > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        return cfg

    def to_dict(self) -> dict:
        """The config.json of this configuration."""
        d = {"architecture": NAME, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
             "layers": [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                        for l in self.layers],
             "torch_dtype": self.torch_dtype}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
