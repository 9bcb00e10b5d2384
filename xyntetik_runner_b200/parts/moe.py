"""Routed experts with an optional shared expert.

    z = W_router h (float32);  the `top` experts with the largest z;  weights = softmax over the chosen z alone
    out = sum_j weight_j * expert_{e_j}(h)  (+ shared(h))
    expert(h) = W_down gate_act(W_gate h, W_up h), no biases
With ``scoring="sigmoid"`` the scores are s = sigmoid(z); the `top` largest s + correction are chosen (`correction`: a tensor of
one number per expert, or None) and the weights are the chosen experts' s, not renormalised.
The activation is one of ``kernels.ACTIVATIONS`` (with its `limit` where it has one).  Experts' matrices are kept as
[experts, rows, columns] arrays; the (token, choice) pairs are put in the order of their experts on the device and every
expert multiplies the rows that chose it (csrc/moe.cu), so no step waits for the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_feed_forward
from .feed_forward import GatedFeedForward, _act_id
from . import linear_tc
from .linear import Linear


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, width: int, experts: int, top: int, inner: int, prefix: str, activation: str = "silu",
                 limit: float = 0.0, shared: Optional[GatedFeedForward] = None, router: str = "router",
                 expert: str = "e{}.", gate: str = "gate", up: str = "up", down: str = "down", scoring: str = "softmax",
                 correction: Optional[str] = None):
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"{prefix}: scoring is 'softmax' (over the chosen logits) or 'sigmoid'")
        if correction is not None and scoring != "sigmoid":
            raise ValueError(f"{prefix}: a correction of the choice goes with sigmoid scores")
        if not (1 <= top <= experts):
            raise ValueError(f"{prefix}: top {top} of {experts} experts")
        self.width, self.E, self.top, self.inner, self.prefix = width, experts, top, inner, prefix
        self.act, self.limit, self.shared = _act_id(activation), float(limit), shared
        self.router_name = prefix + router
        self.sigmoid, self.correction_name, self.correction = scoring == "sigmoid", None if correction is None else prefix + correction, None
        self.expert_names = [tuple(prefix + expert.format(e) + s for s in (gate, up, down)) for e in range(experts)]
        self.router = self.w_gate_up = self.w_down = None
        self.tensor_cores, self._nbytes = False, 0

    def tensors(self):
        t = {self.router_name: TensorSpec((self.E, self.width))}
        if self.correction_name is not None:
            t[self.correction_name] = TensorSpec((self.E,), "vector", "zeros")
        for g, u, d in self.expert_names:
            t[g] = TensorSpec((self.inner, self.width))
            t[u] = TensorSpec((self.inner, self.width))
            t[d] = TensorSpec((self.width, self.inner))
        if self.shared is not None:
            t.update(self.shared.tensors())
        return t

    def bind(self, tensors, rt):
        self.router = Linear(tensors[self.router_name]).prepare(rt)
        if self.correction_name is not None:
            self.correction = tensors[self.correction_name].to(torch.float32).contiguous()
        ws = [tensors.pop(n) for names in self.expert_names for n in names]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        # [E][2F][width]: an expert's gate rows, then its up rows; [E][width][F]
        gate_up = torch.stack([torch.cat([ws[3 * e], ws[3 * e + 1]], dim=0) for e in range(self.E)]).contiguous()
        down = torch.stack([ws[3 * e + 2] for e in range(self.E)]).contiguous()
        del ws
        self._nbytes = (gate_up.numel() + down.numel()) * down.element_size()
        # bfloat16 serving: the tensor-core product over rows sorted by expert, on matrices re-laid tile by tile
        self.tensor_cores = (linear_tc.ENABLED and rt.act_dtype == torch.bfloat16 and down.dtype == torch.bfloat16 and down.is_cuda
                             and self.width % 8 == 0 and self.inner % 8 == 0)
        if self.tensor_cores:
            self.w_gate_up = kernels.pack_weight_groups(gate_up, halves=2)
            self.w_down = kernels.pack_weight_groups(down)
        else:
            self.w_gate_up, self.w_down = gate_up, down
        if self.shared is not None:
            self.shared.bind(tensors, rt)

    def weight_bytes(self):
        # a step reads the router, the shared expert, and at most all experts
        return self.router.nbytes() + self._nbytes + (self.shared.weight_bytes() if self.shared is not None else 0)

    @staticmethod
    def _row_tile(pairs: int, experts: int) -> int:
        """Rows per tile of the tensor-core product: about what an expert gets when the choices spread evenly."""
        avg = pairs / experts
        return 16 if avg <= 16 else (32 if avg <= 32 else (64 if avg <= 64 else 128))

    def forward(self, ctx, h, x):
        n, top, E = h.shape[0], self.top, self.E
        pairs = n * top
        z = ctx.buf("moe_logits", (n, E), torch.float32)
        self.router.forward(h, z)
        ids = ctx.buf("moe_ids", (n, top), torch.int32)
        wts = ctx.buf("moe_weights", (n, top), torch.float32)
        if self.sigmoid:
            kernels.route_topk(z, ids, wts, top, sigmoid_scores=True, correction=self.correction)
        else:
            kernels.route_topk(z, ids, wts, top)
        align = self._row_tile(pairs, E) if self.tensor_cores else kernels.moe_tile_rows()
        max_tiles = kernels.moe_max_tiles(pairs, E, align)
        rows = max_tiles * align
        row_src = ctx.buf("moe_row_src", (rows,), torch.int32)
        pair_row = ctx.buf("moe_pair_row", (pairs,), torch.int32)
        tile_group = ctx.buf("moe_tile_group", (max_tiles,), torch.int32)
        kernels.moe_plan(ids, row_src, pair_row, tile_group, E, align)
        y = ctx.buf("moe_act", (rows, self.inner), ctx.act_dtype)
        zz = ctx.buf("moe_out", (rows, self.width), torch.float32)
        if self.tensor_cores:
            xs = ctx.buf("moe_rows", (rows, self.width), ctx.act_dtype)
            kernels.moe_gather(h, xs, row_src, tile_group, top, align)
            kernels.gemm_tc_grouped(xs, self.w_gate_up, y, tile_group, align, self.inner, kernels.EPI_GATED, self.act, self.limit)
            kernels.gemm_tc_grouped(y, self.w_down, zz, tile_group, align, self.width)
        else:
            kernels.moe_gemm(h, self.w_gate_up, y, row_src, tile_group, top, True, self.act, self.limit)
            kernels.moe_gemm(y, self.w_down, zz, row_src, tile_group, top, False)
        ctx.materialize(x)
        kernels.moe_combine(x, zz, wts, pair_row, top)
        if self.shared is not None:
            self.shared.forward(ctx, h, x)


register_feed_forward("routed_experts", RoutedExperts)
