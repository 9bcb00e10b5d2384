"""Linear attention with a constant decay per head ("lightning attention") as a mixer with a fixed-size state per request.

With h the mixer's input, H heads, key size D and value size V:
    q = silu(W_q h),  k = silu(W_k h),  v = silu(W_v h)                       laid out head by head
    S <- decay_h S + k v^T,   o = S^T q                                       S [D, V] per head, no other scale
    y = W_o (rms_norm(concat_h o_h) * w * sigmoid(W_g h)) * out_scale         one norm over all heads together, w of H V values
S starts at zero and lives in float32 in the request's state slot.  The projections leave their product in float32; the
activations, the recurrence, the norm and the gate are float32 in both precisions (csrc/recurrent.cu).  The state after a token
does not depend on how tokens were cut into steps.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear


class DecayLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float, prefix: str,
                 out_scale: float = 1.0, q: str = "q", k: str = "k", v: str = "v", g: str = "g", o: str = "o", norm: str = "norm"):
        if len(decay) != heads:
            raise ValueError(f"{prefix}: {len(decay)} decays for {heads} heads")
        if dim > 256:
            raise ValueError(f"{prefix}: key size {dim}: the recurrence kernel takes up to 256")
        self.width, self.H, self.D, self.V = width, heads, dim, vdim
        self.decay_values, self.eps, self.prefix, self.out_scale = [float(d) for d in decay], float(eps), prefix, float(out_scale)
        self.names = {a: prefix + b for a, b in dict(q=q, k=k, v=v, g=g, o=o, norm=norm).items()}
        self.proj = self.out = self.norm_w = self.decay = None

    def state_need(self):
        return StateNeed((self.H * self.D * self.V,), torch.float32)

    def tensors(self):
        n, H, D, V, W = self.names, self.H, self.D, self.V, self.width
        return {n["q"]: TensorSpec((H * D, W)), n["k"]: TensorSpec((H * D, W)), n["v"]: TensorSpec((H * V, W)),
                n["g"]: TensorSpec((H * V, W)), n["o"]: TensorSpec((W, H * V)), n["norm"]: TensorSpec((H * V,), "vector", "ones_jitter")}

    def bind(self, tensors, rt):
        n = self.names
        ws = [tensors.pop(n[a]) for a in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0)).prepare(rt)
        del ws
        self.out = Linear(tensors[n["o"]]).prepare(rt)
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)

    def weight_bytes(self):
        return self.proj.nbytes() + self.out.nbytes()

    def forward(self, ctx, h, x, lay):
        n, H, D, V = h.shape[0], self.H, self.D, self.V
        total = 2 * H * D + 2 * H * V
        proj = ctx.buf("decay_proj", (n, -(-total // 8) * 8), torch.float32)[:, :total]
        self.proj.forward(h, proj)
        o = ctx.buf("decay_o", (n, H * V), torch.float32)
        kernels.decay_attention(proj, (0, H * D, 2 * H * D), self.decay, lay.state, ctx.seg_start, ctx.seg_len, ctx.seg_slot, o,
                                ctx.n_seg, H, D, V)
        y = ctx.buf("decay_out", (n, H * V), ctx.act_dtype)
        kernels.row_norm_gate(o, proj, 2 * H * D + H * V, self.norm_w, y, self.eps, scale=self.out_scale)
        ctx.set_pending(x, self.out.forward(y, x, accumulate=True, defer=True))


register_mixer("decay_linear_attention", DecayLinearAttention)
