"""Pre-norm block: x -> norm -> mixer -> +x -> norm -> feed-forward -> +x
(src/model.c:6206-6208, 6350-6352, 6366-6368, 6421-6423).  The two additions happen in float32
inside the last product of the mixer and of the feed-forward."""
from __future__ import annotations

import torch

from .base import Block, FeedForward, Mixer, Norm, register_block
from .norm import RMSNorm, ScalarRMSNorm


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm = None, feed_forward: FeedForward = None):
        """`feed_forward` None: a layer of the mixer alone (no second norm either)."""
        if (ff_norm is None) != (feed_forward is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = mixer_norm, mixer, ff_norm, feed_forward

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def tensors(self):
        out = {}
        for p in self.parts():
            out.update(p.tensors())
        return out

    def bind(self, tensors, rt):
        for p in self.parts():
            p.bind(tensors, rt)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts())

    def forward(self, ctx, x, lay):
        # A norm finishes whatever sum the part before it left pending on x (see StepContext.set_pending),
        # so x is complete whenever a mixer or a feed-forward runs.
        h = ctx.buf("block_normed", (x.shape[0], x.shape[1]), ctx.act_dtype)
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, lay)
        if self.feed_forward is not None:
            self.ff_norm.forward(ctx, x, h)
            self.feed_forward.forward(ctx, h, x)


register_block("prenorm", PreNormBlock)


class ParallelBlock(Block):
    """Mixer and feed-forward side by side, both reading the same x:  x += m (mixer(norm(x)) + ff(norm'(x))), norm' the
    same norm, or with `ff_norm` a second one with a weight of its own.  With a multiplier m other than one the sublayers
    add into a float32 stream of their own, which is added to x once, times m.  `direct` (m = 1 only): the norms are taken
    first and the sublayers' last products add into x themselves, one after the other, with no stream in between."""

    def __init__(self, norm: Norm, mixer: Mixer, feed_forward, residual_mult: float = 1.0, ff_norm: Norm = None,
                 direct: bool = False):
        if ff_norm is not None and feed_forward is None:
            raise ValueError("a second norm comes with a feed-forward")
        if direct and float(residual_mult) != 1.0:
            raise ValueError("sublayers add into x directly only with a residual multiplier of one")
        self.norm, self.mixer, self.feed_forward, self.mult, self.ff_norm = norm, mixer, feed_forward, float(residual_mult), ff_norm
        self.direct = bool(direct)

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def tensors(self):
        out = {}
        for p in self.parts():
            out.update(p.tensors())
        return out

    def bind(self, tensors, rt):
        for p in self.parts():
            p.bind(tensors, rt)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts())

    def forward(self, ctx, x, lay):
        from .. import kernels
        n, width = x.shape
        h = ctx.buf("block_normed", (n, width), ctx.act_dtype)
        h2 = h
        if self.ff_norm is None:
            self.norm.forward(ctx, x, h)
        else:
            # the second norm reads the x the first one reads, before any sublayer adds to it: one kernel takes the row's root
            # mean square once and writes both
            h2 = ctx.buf("block_normed_ff", (n, width), ctx.act_dtype)
            if isinstance(self.norm, RMSNorm) and isinstance(self.ff_norm, RMSNorm) and self.norm.eps == self.ff_norm.eps:
                self.norm.forward(ctx, x, h, second=self.ff_norm, out2=h2)
            else:
                self.norm.forward(ctx, x, h)
                self.ff_norm.forward(ctx, x, h2)
        if self.direct:
            self.mixer.forward(ctx, h, x, lay)
            if self.feed_forward is not None:
                self.feed_forward.forward(ctx, h2, x)
            return
        d = ctx.buf("block_sum", (n, width), torch.float32)
        d.zero_()
        self.mixer.forward(ctx, h, d, lay)
        if self.feed_forward is not None:
            self.feed_forward.forward(ctx, h2, d)
        ctx.materialize(d)
        kernels.scaled_add(x, d, self.mult)


register_block("parallel", ParallelBlock)


class OutputNormBlock(Block):
    """Norms on the sublayers' OUTPUTS: x += norm1(mixer(x)), then x += norm2(ff(x)).  The sublayers read the stream itself (in the
    activation dtype); each adds into a float32 sum of its own, whose norm (a ``ScalarRMSNorm``: one gain for all coordinates) is
    added into x in one pass, in float32.  The same pass writes the new x in the activation dtype for the sublayer that follows;
    a layer reads its input from ``ctx.stream_cast`` where the part ahead of it left one (see ``parts.stream.DepthAverage``)."""

    def __init__(self, mixer_norm: ScalarRMSNorm, mixer: Mixer, ff_norm: ScalarRMSNorm = None, feed_forward: FeedForward = None):
        if (ff_norm is None) != (feed_forward is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = mixer_norm, mixer, ff_norm, feed_forward

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def tensors(self):
        out = {}
        for p in self.parts():
            out.update(p.tensors())
        return out

    def bind(self, tensors, rt):
        for p in self.parts():
            p.bind(tensors, rt)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts())

    def forward(self, ctx, x, lay):
        from .. import kernels
        n, width = x.shape
        ctx.materialize(x)
        narrow = ctx.act_dtype != torch.float32
        # what the sublayers read: the stream itself in the true 32-bit path, its rounding otherwise
        h = x
        if narrow:
            h = ctx.buf("block_normed", (n, width), ctx.act_dtype)
            if getattr(ctx, "stream_cast", None) != x.data_ptr():
                kernels.cast_rows(x, h)
        ctx.stream_cast = None
        d = ctx.buf("block_sum", (n, width), torch.float32)
        # the sum starts at zero once a step; every norm clears it behind its read
        ctx.once(("output_norm_sum", d.data_ptr()), lambda: (d.zero_(), True)[1])
        self.mixer.forward(ctx, h, d, lay)
        last = self.feed_forward is None
        self._norm_add(ctx, d, x, self.mixer_norm, cast=h if narrow and not last else None)
        if not last:
            self.feed_forward.forward(ctx, h, d)
            self._norm_add(ctx, d, x, self.ff_norm, cast=None)

    @staticmethod
    def _norm_add(ctx, d, x, norm, cast):
        """x += norm(d); partial sums that the sublayer's last products left on d are taken in the same pass."""
        from .. import kernels
        pend = ctx.take_pending(d)
        if pend is None:
            kernels.norm_add(d, x, norm.gain, norm.eps, cast=cast, clear=True)
            return
        kernels.norm_add(d, x, norm.gain, norm.eps, cast=cast, clear=True, partial=pend.partial, splits=pend.splits, bias=pend.bias)
        pend.release()


register_block("output_norm", OutputNormBlock)
