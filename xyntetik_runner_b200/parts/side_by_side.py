"""Two mixers side by side: both read the same input and add into the same stream.  Each applies its own output scale (a
constructor argument of the mixers that have one), so the result is scale_a a(h) + scale_b b(h).  At most one of the two keeps
keys and values in pages and at most one keeps a state per request: a layer has one cache entry and one state array."""
from __future__ import annotations

from .base import Mixer, register_mixer


class SideBySide(Mixer):
    def __init__(self, first: Mixer, second: Mixer):
        if first.kv_need() is not None and second.kv_need() is not None:
            raise ValueError("two mixers side by side: only one may keep keys and values")
        if first.state_need() is not None and second.state_need() is not None:
            raise ValueError("two mixers side by side: only one may keep a state per request")
        self.first, self.second = first, second

    @property
    def graph_safe(self):
        return self.first.graph_safe and self.second.graph_safe

    def kv_need(self):
        return self.first.kv_need() or self.second.kv_need()

    def state_need(self):
        return self.first.state_need() or self.second.state_need()

    def tensors(self):
        return {**self.first.tensors(), **self.second.tensors()}

    def bind(self, tensors, rt):
        self.first.bind(tensors, rt)
        self.second.bind(tensors, rt)

    def weight_bytes(self):
        return self.first.weight_bytes() + self.second.weight_bytes()

    def forward(self, ctx, h, x, lay):
        self.first.forward(ctx, h, x, lay)
        self.second.forward(ctx, h, x, lay)


register_mixer("side_by_side", SideBySide)
