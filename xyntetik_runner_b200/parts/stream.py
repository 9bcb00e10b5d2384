"""Parts that act on the residual stream between layers.

``StreamJoin``: x <- W [x; x0], one product over the stream and the embedding's output side by side (W is
[width, 2 width], the stream's columns first).  A model that runs a span of layers several times with the same
weights feeds the embedding back in this way at the start of every pass.

``StreamStep``: x <- x (+ x0) + v, v one row of a table [passes, width]: such a model may instead add the embedding's
output (from the second pass on) and a vector of the pass, in float32.

``DepthAverage``: x <- sum_(j=0..k) w[j] X_j behind layer k - 1, where X_0 is the embedding's output and X_j what layer j - 1 left
BEFORE its own average: every layer reads a learned mixture of all the streams so far.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part
from .linear import Linear


class StreamJoin(Part):
    graph_safe = True

    def __init__(self, width: int, name: str):
        self.width, self.name = width, name
        self.linear = None

    def tensors(self):
        return {self.name: TensorSpec((self.width, 2 * self.width))}

    def bind(self, tensors, rt):
        self.linear = Linear(tensors[self.name]).prepare(rt)

    def weight_bytes(self):
        return self.linear.nbytes()

    def forward(self, ctx, x: torch.Tensor, x0: torch.Tensor) -> None:
        ctx.materialize(x)
        both = ctx.buf("stream_join", (x.shape[0], 2 * self.width), ctx.act_dtype)
        kernels.concat_cast(x, x0, both)
        self.linear.forward(both, x)


class StreamStep(Part):
    """x += x0 + table[row] (`add_embedding`), or x += table[row] alone; `name` None: no table, the embedding alone."""
    graph_safe = True

    def __init__(self, width: int, name: str, rows: int, row: int, add_embedding: bool):
        if name is None and not add_embedding:
            raise ValueError("a stream step adds the embedding's output, a row of a table, or both")
        if name is not None and not (0 <= row < rows):
            raise ValueError(f"row {row} of a table of {rows}")
        self.width, self.name, self.rows, self.row, self.add_embedding = width, name, rows, row, bool(add_embedding)
        self.vector = None

    def tensors(self):
        return {} if self.name is None else {self.name: TensorSpec((self.rows, self.width), kind="vector", init="zeros_jitter")}

    def bind(self, tensors, rt):
        if self.name is not None:
            self.vector = tensors[self.name][self.row].to(torch.float32).contiguous()

    def weight_bytes(self):
        return 0 if self.name is None else self.width * 4

    def forward(self, ctx, x: torch.Tensor, x0: torch.Tensor) -> None:
        ctx.materialize(x)
        kernels.stream_step(x, x0 if self.add_embedding else None, self.vector)


class DepthAverage(Part):
    """Behind the k-th layer run (k from 1): keep x as X_k and set x <- w[0] X_0 + ... + w[k] X_k, in float32.  The streams X_1 ..
    X_(depth) of a step live in one buffer of the step; X_0 is the embedding's output, which the engine keeps.  In the serving
    precision the new x is also left in the activation dtype for the layer that follows (``ctx.stream_cast``)."""
    graph_safe = True

    def __init__(self, width: int, name: str, k: int, depth: int, cast: bool = True):
        if not (1 <= k <= depth):
            raise ValueError(f"{name}: layer run {k} of {depth}")
        self.width, self.name, self.k, self.depth, self.cast = width, name, k, depth, bool(cast)
        self.weights = None

    def tensors(self):
        return {self.name: TensorSpec((self.k + 1,), kind="vector", init="ones_jitter")}

    def bind(self, tensors, rt):
        self.weights = tensors[self.name].to(torch.float32).contiguous()

    def weight_bytes(self):
        return (self.k + 1) * 4

    def forward(self, ctx, x: torch.Tensor, x0: torch.Tensor) -> None:
        ctx.materialize(x)
        n = x.shape[0]
        hist = ctx.buf("depth_streams", (self.depth, n, self.width), torch.float32)
        h = None
        if self.cast and ctx.act_dtype != torch.float32:
            h = ctx.buf("block_normed", (n, self.width), ctx.act_dtype)
        kernels.depth_average(x, x0, hist, self.weights, self.k, cast=h)
        ctx.stream_cast = x.data_ptr() if h is not None else None
