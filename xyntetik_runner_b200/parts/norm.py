"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, computed in float32 (src/model.c:3386-3392).  With `one_plus` the
stored weight is an offset from one: the factor is 1 + w."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True
    def __init__(self, width: int, eps: float, name: str, one_plus: bool = False):
        self.width, self.eps, self.name, self.one_plus = width, float(eps), name, bool(one_plus)
        self.weight = None

    def tensors(self):
        return {self.name: TensorSpec((self.width,), kind="vector", init="zeros_jitter" if self.one_plus else "ones_jitter")}

    def bind(self, tensors, rt):
        # norm weights are used in float32 whatever they were stored in (src/model.c:2830-2831)
        self.weight = tensors[self.name].to(torch.float32).contiguous()
        if self.one_plus:
            self.weight = (1.0 + self.weight).contiguous()      # the factor itself, made once in float32

    def weight_bytes(self):
        return self.width * 4

    def forward(self, ctx, x, out, rows=None, second=None, out2=None):
        """`second` (another RMSNorm of the same width and eps) with `out2`: both norms of the same rows in one kernel."""
        w2 = None
        if second is not None:
            if second.eps != self.eps or second.width != self.width:
                raise ValueError(f"{self.name} and {second.name}: two norms share a pass only with the same width and eps")
            w2 = second.weight
        pend = ctx.take_pending(x)
        if pend is not None and rows is None:
            # the product before this norm left partial sums: sum, add into x and normalise in one pass
            kernels.finish_add_rmsnorm(pend.partial, pend.splits, pend.bias, x, self.weight, out, self.eps, w2, out2)
            pend.release()
            return
        if pend is not None:
            pend.finish()
        kernels.rmsnorm(x, self.weight, out, self.eps, rows, w2, out2)


class ScalarRMSNorm(RMSNorm):
    """RMSNorm whose weight is ONE number for all coordinates: y = x * rsqrt(mean(x^2) + eps) * g.  The number is spread over the
    width when the part binds, and the kernels are the RMSNorm's."""

    def tensors(self):
        return {self.name: TensorSpec((), kind="vector", init="ones_jitter")}

    def bind(self, tensors, rt):
        g = tensors[self.name].to(torch.float32).reshape(1)
        self.gain = g.contiguous()
        self.weight = g.expand(self.width).contiguous()


register_norm("rmsnorm", RMSNorm)
register_norm("scalar_rmsnorm", ScalarRMSNorm)
