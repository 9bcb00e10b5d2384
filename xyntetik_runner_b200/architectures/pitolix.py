"""The Pitolix decoder as a list of parts chosen from its configuration.

Fixed by the design: every layer runs its mixer and its feed-forward side by side, each behind an RMSNorm of its own whose
stored weight is an offset from one (factor 1 + w), and adds both to the stream; the feed-forward is gated with SiLU; the
rotation pairs element i with i + dims/2; the sink counts once in a softmax's denominator; a looped span's passes add the
embedding's output (from the second pass on) and row t of a table to the stream before their first layer.  Everything else
-- sizes, the order and kinds of the layers, the loop, scales, the rotation's base and extent, the query factor's constants
-- comes from the configuration.
Tensor names: embed, loop.step, l<i>.norm1, l<i>.norm2, l<i>.mix.{q,k,v,g,o} (+ .b on q, k, v; sink), l<i>.mlp.{gate,up,down},
final.norm, head.
"""
from __future__ import annotations

from ..config.pitolix import NAME, PitolixConfig, RotaryAttentionConfig, SinkAttentionConfig
from ..config.registry import register_architecture
from ..engine.model import ModelPlan, ScheduleEntry
from ..parts import (Embedding, GatedFeedForward, GQAAttention, Head, NoPosition, ParallelBlock, RMSNorm, Rope, StreamStep)
from ..weights.loader import TensorSpec

# no position table limits a request's length: the rotation and the query factor take any position
MAX_POSITIONS = 1 << 30


class _Block(ParallelBlock):
    """A layer without a feed-forward lets a checkpoint carry a second norm weight that nothing reads."""

    def __init__(self, *parts, spare: str = None, **options):
        super().__init__(*parts, **options)
        self.spare = spare

    def tensors(self):
        out = super().tensors()
        if self.spare is not None:
            out[self.spare] = TensorSpec((self.norm.width,), kind="vector", init="zeros", optional=True)
        return out


def build_pitolix(cfg: PitolixConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    blocks = []
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = lay.mixer
        names = dict(prefix=p + "mix.", q="q", k="k", v="v", o="o", g="g", weight_suffix="", value_dim=m.vdim, scale=m.scale)
        if isinstance(m, SinkAttentionConfig):
            mixer = GQAAttention(W, m.heads, m.kv_heads, m.dim, position=NoPosition(), qk_norm="unit", norm_eps=eps,
                                 q_temp=None if m.q_temp is None else (m.q_temp.coef, m.q_temp.every), sink="sink", gate="each",
                                 **names)
        elif isinstance(m, RotaryAttentionConfig):
            position = Rope(m.dim, m.rot_base, rotary_dim=m.rot_dims, pairing="half") if m.rot_dims else NoPosition()
            mixer = GQAAttention(W, m.heads, m.kv_heads, m.dim, position=position, bias=True, bias_suffix=".b", out_bias=False,
                                 gate="head", **names)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {type(m).__name__}")
        ff = ff_norm = None
        if lay.mlp is not None:
            ff = GatedFeedForward(W, lay.mlp.ff, p + "mlp.", "silu", gate="gate", up="up", down="down")
            ff_norm = RMSNorm(W, eps, p + "norm2", one_plus=True)
        blocks.append(_Block(RMSNorm(W, eps, p + "norm1", one_plus=True), mixer, ff, ff_norm=ff_norm, direct=True,
                             spare=None if ff is not None else p + "norm2"))
    # one stream part per pass of the loop: the embedding's output from the second pass on, and the pass's vector
    stream_parts = []
    if cfg.loop is not None:
        stream_parts = [StreamStep(W, "loop.step", cfg.loop.times, t, add_embedding=t > 0) for t in range(cfg.loop.times)]
    schedule = [ScheduleEntry(layer=i, before=t) for i, t in cfg.layer_runs()]
    return ModelPlan(embedding=Embedding(cfg.vocab, W, "embed", scale=cfg.embedding_scale), blocks=blocks, schedule=schedule,
                     final_norm=RMSNorm(W, eps, "final.norm", one_plus=True), head=Head(cfg.vocab, W, name="head"), width=W,
                     vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, stream_parts=stream_parts)


register_architecture(NAME, PitolixConfig.from_dict, build_pitolix, replace=True)
