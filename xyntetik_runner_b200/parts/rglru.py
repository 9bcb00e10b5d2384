"""Griffin's recurrent block: a gated branch beside a short convolution and a real-gated linear recurrent unit.

With h the mixer's input, R channels in B blocks of R / B, a causal convolution of `taps` taps per channel (the last column of
its weight is the current token's, zeros before a request's first token) and a constant c:
    y = gelu_tanh(W_y h + b_y),   u = conv(W_x h + b_x) + conv bias                      (no activation behind the convolution)
    r = sigmoid(Wa[b] u_b + ba[b]),   i = sigmoid(Wi[b] u_b + bi[b])                     per block b; Wa[b], Wi[b] square, [out, in]
    a = exp(-c r softplus(lam)),   S <- a S + sqrt(1 - a^2) (i u),   out = W_o (S * y)
S starts at zero (the first token takes no other path) and lives in float32 in the request's state slot together with the last
taps - 1 rows that entered the convolution.  The projections leave their product in float32, and everything behind them is
float32 in both precisions (csrc/recurrent.cu).  The state after a token does not depend on how tokens were cut into steps.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear


class GatedLinearRecurrence(Mixer):
    graph_safe = True

    def __init__(self, width: int, channels: int, blocks: int, taps: int, prefix: str, rate: float = 8.0,
                 y: str = "y", x: str = "x", conv: str = "conv", ra: str = "ra", ri: str = "ri", lam: str = "lam", o: str = "o",
                 bias_suffix: str = ".b"):
        if channels % blocks:
            raise ValueError(f"{prefix}: {channels} channels do not divide into {blocks} blocks")
        if not (1 <= taps <= 16):
            raise ValueError(f"{prefix}: the convolution takes 1 to 16 taps")
        self.width, self.R, self.B, self.taps, self.prefix = width, channels, blocks, taps, prefix
        self.rate = float(rate)
        self.names = {k: prefix + v for k, v in dict(y=y, x=x, conv=conv, ra=ra, ri=ri, lam=lam, o=o).items()}
        self.b = bias_suffix
        self.proj = self.out = None

    def state_need(self):
        return StateNeed((kernels.rglru_state_floats(self.R, self.taps),), torch.float32)

    def tensors(self):
        n, R, B, W, b = self.names, self.R, self.B, self.width, self.b
        Bs = R // B
        return {n["y"]: TensorSpec((R, W)), n["y"] + b: TensorSpec((R,), "vector", "zeros"),
                n["x"]: TensorSpec((R, W)), n["x"] + b: TensorSpec((R,), "vector", "zeros"),
                n["conv"]: TensorSpec((R, self.taps), "vector", "normal"), n["conv"] + b: TensorSpec((R,), "vector", "zeros"),
                n["ra"]: TensorSpec((B, Bs, Bs), "vector", "normal"), n["ra"] + b: TensorSpec((B, Bs), "vector", "zeros"),
                n["ri"]: TensorSpec((B, Bs, Bs), "vector", "normal"), n["ri"] + b: TensorSpec((B, Bs), "vector", "zeros"),
                n["lam"]: TensorSpec((R,), "vector", "normal"), n["o"]: TensorSpec((W, R))}

    def bind(self, tensors, rt):
        n, b = self.names, self.b
        ws = [tensors.pop(n["y"]), tensors.pop(n["x"])]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        f32 = lambda name: tensors[name].to(torch.float32).contiguous()
        # one product for both branches (the gated branch's rows first); its sums stay float32
        self.proj = Linear(torch.cat(ws, dim=0), torch.cat([f32(n["y"] + b), f32(n["x"] + b)])).prepare(rt)
        del ws
        self.out = Linear(tensors[n["o"]]).prepare(rt)
        self.conv_w, self.conv_b = f32(n["conv"]), f32(n["conv"] + b)
        # the gates' matrices transposed, [block][in][out]: a warp then reads consecutive outputs of one input
        self.wa, self.wi = f32(n["ra"]), f32(n["ri"])
        self.wa_t = self.wa.transpose(1, 2).contiguous()
        self.wi_t = self.wi.transpose(1, 2).contiguous()
        self.ba, self.bi, self.lam = f32(n["ra"] + b).reshape(-1), f32(n["ri"] + b).reshape(-1), f32(n["lam"])
        self._small = (self.wa_t.numel() + self.wi_t.numel() + self.conv_w.numel() + 4 * self.R) * 4

    def weight_bytes(self):
        return self.proj.nbytes() + self.out.nbytes() + self._small

    def forward(self, ctx, h, x, lay):
        n, R = h.shape[0], self.R
        ld = -(-2 * R // 8) * 8
        proj = ctx.buf("rglru_proj", (n, ld), torch.float32)[:, :2 * R]
        self.proj.forward(h, proj)
        a_s = ctx.buf("rglru_a", (n, R), torch.float32)
        b_s = ctx.buf("rglru_b", (n, R), torch.float32)
        u_s = ctx.buf("rglru_u", (n, R), torch.float32)
        y = ctx.buf("rglru_out", (n, R), ctx.act_dtype)
        kernels.rglru(proj, self.conv_w, self.conv_b, self.wa_t, self.wi_t, self.wa, self.wi, self.ba, self.bi, self.lam, lay.state, ctx.tok_seg,
                      ctx.seg_start, ctx.seg_len, ctx.seg_slot, a_s, b_s, u_s, y, ctx.n_seg, R, self.B, self.taps, self.rate)
        ctx.set_pending(x, self.out.forward(y, x, accumulate=True, defer=True))


register_mixer("gated_linear_recurrence", GatedLinearRecurrence)
