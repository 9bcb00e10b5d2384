"""The Buzarax decoder as a list of parts chosen from its configuration.

Fixed by the design: norms on the sublayers' outputs with one gain each; the depth average behind every layer; rotations pair
element i with i + dims/2; the rotated queries and keys are divided by their root mean square; the values are rotated over their
whole length with the keys' base and no scaling; the attention's sink has score zero; the recurrence's rate constant 8 and its
tanh-GELU gate; the dense feed-forward's activation g sigmoid(1.702 g) (u + 1) on clamped g and u; experts gated with SiLU,
chosen by sigmoid score plus correction and weighted by the score.  Everything else -- sizes, the order and kinds of the layers,
bases, scaling, caps, decays, scales, the hash's multipliers -- comes from the configuration.
Tensor names: embed, bigram, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.dwa, final.norm, head.
"""
from __future__ import annotations

from ..config.buzarax import NAME, BuzaraxConfig, DenseConfig, ExpertsConfig, ParallelConfig, RecurrentConfig
from ..config.registry import register_architecture
from ..engine.model import ModelPlan, ScheduleEntry
from ..parts import (DecayLinearAttention, DepthAverage, GatedFeedForward, GatedLinearRecurrence, GQAAttention, Head, OutputNormBlock,
                     PairEmbedding, RoutedExperts, ScalarRMSNorm, SideBySide, YarnRope)
from ..weights.loader import TensorSpec

# no position table limits a request's length: the rotations take any position and the recurrences have none
MAX_POSITIONS = 1 << 30
RECURRENCE_RATE = 8.0


class _Block(OutputNormBlock):
    """A layer without a feed-forward lets a checkpoint carry a second gain that nothing reads."""

    def __init__(self, *parts, spare: str = None):
        super().__init__(*parts)
        self.spare = spare

    def tensors(self):
        out = super().tensors()
        if self.spare is not None:
            out[self.spare] = TensorSpec((), kind="vector", init="ones", optional=True)
        return out


def _softmax_side(W, m, eps, prefix, out_scale):
    sc = m.rot.scaling
    position = YarnRope(m.dim, m.rot.base, m.rot.dims, factor=None if sc is None else sc.factor,
                        original=0.0 if sc is None else sc.original, fast=32.0 if sc is None else sc.fast,
                        slow=1.0 if sc is None else sc.slow, pairing="half")
    return GQAAttention(W, m.heads, m.kv_heads, m.dim, position=position, prefix=prefix, scale=m.scale, q="q", k="k", v="v", o="o",
                        weight_suffix="", value_dim=m.vdim, qk_norm="unit", norm_eps=eps, norm_after_rotation=True,
                        value_rotation=(m.rot.base, "half"), softcap=m.softcap, sink=0.0, out_scale=out_scale)


def build_buzarax(cfg: BuzaraxConfig) -> ModelPlan:
    W, eps, depth = cfg.width, cfg.norm_eps, len(cfg.layers)
    blocks, schedule, averages = [], [], []
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = lay.mixer
        if isinstance(m, ParallelConfig):
            mixer = SideBySide(_softmax_side(W, m.left, eps, p + "mix.left.", m.left_scale),
                               DecayLinearAttention(W, m.right.heads, m.right.dim, m.right.vdim, m.right.decay, eps,
                                                    prefix=p + "mix.right.", out_scale=m.right_scale))
        elif isinstance(m, RecurrentConfig):
            mixer = GatedLinearRecurrence(W, m.width, m.blocks, m.conv, prefix=p + "mix.", rate=RECURRENCE_RATE)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {type(m).__name__}")
        norm1 = ScalarRMSNorm(W, eps, p + "norm1")
        if lay.mlp is None:
            blocks.append(_Block(norm1, mixer, spare=p + "norm2"))
        else:
            if isinstance(lay.mlp, DenseConfig):
                ff = GatedFeedForward(W, lay.mlp.ff, p + "mlp.", "swish_clamp", gate="gate", up="up", down="down", limit=lay.mlp.limit)
            elif isinstance(lay.mlp, ExpertsConfig):
                ff = RoutedExperts(W, lay.mlp.experts, lay.mlp.top, lay.mlp.ff, p + "mlp.", activation="silu", scoring="sigmoid",
                                   correction="correction")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward configuration {type(lay.mlp).__name__}")
            blocks.append(_Block(norm1, mixer, ScalarRMSNorm(W, eps, p + "norm2"), ff))
        # the stream behind the last layer goes to the final norm, which reads float32: no rounded copy of it
        averages.append(DepthAverage(W, p + "dwa", i + 1, depth, cast=i + 1 < depth))
        schedule.append(ScheduleEntry(layer=i, after=i))
    return ModelPlan(embedding=PairEmbedding(cfg.vocab, W, "embed", "bigram", cfg.buckets, cfg.mul_prev, cfg.mul_cur), blocks=blocks,
                     schedule=schedule, final_norm=ScalarRMSNorm(W, eps, "final.norm"),
                     head=Head(cfg.vocab, W, name="head", softcap=cfg.logit_softcap), width=W, vocab_size=cfg.vocab,
                     max_positions=MAX_POSITIONS, stream_parts=averages)


register_architecture(NAME, BuzaraxConfig.from_dict, build_buzarax, replace=True)
