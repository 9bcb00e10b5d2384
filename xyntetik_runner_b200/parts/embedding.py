"""Token embedding and the output head.

Embedding: x[t] = E[id_t], ids outside the table read row 0, no scale (src/model.c:6148-6162).
Head: logits = W_out . norm(x) at the wanted rows; when the model ties its head to the embedding
the same tensor serves both (src/model.c:2353-2354).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, StateNeed
from .linear import Linear


class Embedding(Part):
    graph_safe = True
    def __init__(self, vocab: int, width: int, name: str, scale: float = 1.0):
        """`scale` multiplies every embedded row (1: none)."""
        self.vocab, self.width, self.name, self.scale = vocab, width, name, float(scale)
        self.table = None

    def tensors(self):
        return {self.name: TensorSpec((self.vocab, self.width), kind="matrix")}

    def bind(self, tensors, rt):
        self.table = tensors[self.name]

    def forward(self, ctx, ids: torch.Tensor, x: torch.Tensor) -> None:
        # ids below zero stand for tokens an earlier step left on the device (the step context's `token_feed`)
        kernels.embed(self.table, ids, x, getattr(ctx, "token_feed", None), self.scale)


class PairEmbedding(Embedding):
    """x[t] = E[id_t] + P[row_t]: a second table read by a hash of (previous token, token),
    row_t = (prev_t * mul_prev + id_t * mul_cur) mod buckets; the first token of a request reads row `buckets`, the table's last.
    The token before a portion's first is part of the request's state: one int32 per request slot, which the engine keeps
    (``state_need``) and hands over as ``ctx.embedding_state``; it is set behind every step."""

    def __init__(self, vocab: int, width: int, name: str, pairs_name: str, buckets: int, mul_prev: int, mul_cur: int):
        super().__init__(vocab, width, name)
        if buckets < 1:
            raise ValueError("the pair table needs at least one bucket")
        self.pairs_name, self.buckets, self.mul_prev, self.mul_cur = pairs_name, int(buckets), int(mul_prev), int(mul_cur)
        self.pairs = None

    def state_need(self):
        return StateNeed((1,), torch.int32)

    def tensors(self):
        t = super().tensors()
        t[self.pairs_name] = TensorSpec((self.buckets + 1, self.width), kind="matrix")
        return t

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.pairs = tensors[self.pairs_name]
        if self.pairs.dtype != self.table.dtype:
            self.table, self.pairs = self.table.to(torch.float32), self.pairs.to(torch.float32)

    def forward(self, ctx, ids: torch.Tensor, x: torch.Tensor) -> None:
        feed = getattr(ctx, "token_feed", None)
        last = ctx.embedding_state
        kernels.embed_pair(self.table, self.pairs, ids, ctx.positions, ctx.tok_seg, ctx.seg_start, ctx.seg_slot, last, x,
                           self.mul_prev, self.mul_cur, feed)
        kernels.last_token(ids, ctx.seg_start, ctx.seg_len, ctx.seg_slot, last, ctx.n_seg, self.vocab, feed)


class Head(Part):
    graph_safe = True
    """`tied_to` set: no tensor of its own, multiplies by the embedding table."""

    def __init__(self, vocab: int, width: int, name: str = None, tied_to: Embedding = None, softcap: float = None):
        """`softcap` c: the logits become c tanh(logits / c) (None or 0: as they are)."""
        assert (name is None) != (tied_to is None)
        self.vocab, self.width, self.name, self.tied_to = vocab, width, name, tied_to
        self.softcap = float(softcap) if softcap else None
        self.linear = None

    def tensors(self):
        return {} if self.tied_to is not None else {self.name: TensorSpec((self.vocab, self.width), kind="matrix")}

    def bind(self, tensors, rt):
        # a tied head multiplies by the embedding table; the gather keeps reading the table as stored
        self.linear = Linear(self.tied_to.table if self.tied_to is not None else tensors[self.name]).prepare(
            rt, keep_plain=self.tied_to is not None)

    def weight_bytes(self):
        return self.linear.nbytes()

    def forward(self, ctx, h: torch.Tensor, logits: torch.Tensor) -> None:
        self.linear.forward(h, logits)
        if self.softcap is not None:
            kernels.softcap(logits, self.softcap)
