"""Grouped-query causal attention over the paged cache.

q = Wq h (+bq), k = Wk h (+bk), v = Wv h (+bv) as one fused product; Q and K are
rotated by the position encoding after the projection and before the cache
write, V is stored as it is (src/model.c:6243-6310).  Query head h reads kv
head h / (H/K); scores are (q . k) * scale over the keys t0..p, softmax in
float32, weighted sum of V (src/model.c:3548-3589); then x += Wo o (+bo)
(src/model.c:6338, 6350-6352).  Heads, kv heads, head size, scale, window and
position encoding are all arguments.

Options: `qk_norm` puts an RMSNorm over every query and key head (one weight of head_dim values for all query heads,
one for all key heads, eps `norm_eps`) between the projection and the rotation; `value_dim` gives the value heads
another size than the query/key heads.  With either, the projection's rows go through one kernel that norms, rotates
(angles from float64 products) and stores; keys and values are then cached with one head size, the larger of the two
rounded up to a multiple of 16 and filled with zeros, which changes no score and no sum, and the output product's
matrix gets zero columns to match.

Further options, all on that general path.  `qk_norm="unit"`: every query and key head is divided by its root mean square,
without a weight.  `q_temp=(c, n)`: the queries at position p are multiplied by 1 + c ln(floor((p + 1) / n) + 1), a factor
that grows by steps with the position.  `sink`: a learned logit per query head that joins the softmax's denominator once
and has no key and no value (every attention kernel adds exp(sink - m) to a row's sum when the row is complete).  `gate`:
the heads' outputs are multiplied by sigmoid(W_g h) before the output product, "each" element by its own gate (W_g of
H x Vd rows) or "head" by head (W_g of H rows); W_g's rows ride in the fused projection.  Biases (`bias`, with
`bias_suffix`; `out_bias` for the output product's) combine with all of these.

`norm_after_rotation` (with `qk_norm="unit"`): the heads are rotated first and divided by their root mean square afterwards, which
differs from the other order when the position encoding scales its cosines and sines.  `value_rotation=(base, pairing)`: the
value of position j is turned by j over all its Vd elements (pair m by j base^(-2m/Vd)) before it is cached, and every head's sum
at position i is turned back by -i, so that what a query reads of a value depends on their distance.  `softcap` c: every scaled
score s becomes c tanh(s / c).  `sink=0.0` (a number instead of a tensor's name): a sink of that logit for every head, which adds
exp(sink) to every softmax's denominator.  `out_scale` multiplies the heads' outputs before the output product.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import numpy as np
import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, PositionEncoding, register_mixer
from .linear import Linear

# Which attention kernels the mixer may use (module attributes, so that a test can compare paths): the mma.sync kernels
# for bfloat16 (else the float32-arithmetic kernel), the tcgen05 kernel for prompt portions, bulk copies in the decode
# kernel.  XRB200_NO_TMA_ATTENTION=1 (read once) keeps the decode kernel on per-thread cp.async gathers: a test runs
# generation both ways in child processes and compares the tokens.
USE_MMA = True
USE_TC = True
USE_TMA = os.environ.get("XRB200_NO_TMA_ATTENTION", "0") in ("", "0")
counters = {"mma": 0, "simt": 0, "tcgen05": 0}


class GQAAttention(Mixer):
    graph_safe = True
    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int, position: PositionEncoding,
                 prefix: str, bias: bool = False, window: Optional[int] = None, scale: Optional[float] = None,
                 q: str = "q_proj", k: str = "k_proj", v: str = "v_proj", o: str = "o_proj", weight_suffix: str = ".weight",
                 value_dim: Optional[int] = None, qk_norm=False, norm_eps: float = 1e-6,
                 q_norm: str = "q.norm", k_norm: str = "k.norm", bias_suffix: str = ".bias", out_bias: Optional[bool] = None,
                 q_temp: Optional[tuple] = None, sink=None, gate: Optional[str] = None, g: str = "g",
                 norm_after_rotation: bool = False, value_rotation: Optional[tuple] = None, softcap: Optional[float] = None,
                 out_scale: float = 1.0):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if qk_norm not in (False, True, "unit"):
            raise ValueError(f"{prefix}: qk_norm is False, True (a weight per element) or 'unit' (no weight)")
        if gate not in (None, "head", "each"):
            raise ValueError(f"{prefix}: gate is None, 'head' or 'each'")
        if q_temp is not None and (len(q_temp) != 2 or int(q_temp[1]) < 1):
            raise ValueError(f"{prefix}: q_temp is (coefficient, positions per step >= 1)")
        if norm_after_rotation and qk_norm != "unit":
            raise ValueError(f"{prefix}: norm_after_rotation goes with qk_norm='unit'")
        if value_rotation is not None and (len(value_rotation) != 2 or value_rotation[1] not in ("half", "adjacent")):
            raise ValueError(f"{prefix}: value_rotation is (base, 'half' or 'adjacent')")
        self.D = head_dim                                      # query/key elements per head
        self.Vd = head_dim if value_dim is None else value_dim  # value elements per head
        # the general path: a norm per head, or values of another size than keys
        self.general = bool(qk_norm) or self.Vd != self.D or q_temp is not None or gate is not None or value_rotation is not None
        # head size of the cache and of the attention kernels
        hd = -(-max(self.D, self.Vd) // 16) * 16 if self.general else head_dim
        if not (1 <= hd <= 256):
            raise ValueError(f"head_dim {hd}: the attention kernels take head sizes up to 256")
        self.width, self.H, self.K, self.hd = width, heads, kv_heads, hd
        self.position, self.prefix, self.bias, self.window = position, prefix, bias, window
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)   # src/model.h:464-467
        self.proj = (q, k, v, o)
        self.suffix = weight_suffix
        self.qk_norm, self.unit_norm, self.norm_eps = qk_norm is True, qk_norm == "unit", float(norm_eps)
        self.norm_names = (prefix + q_norm, prefix + k_norm)
        self.bias_suffix, self.out_bias = bias_suffix, bool(bias) if out_bias is None else bool(out_bias)
        self.q_temp = None if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        self.sink_name = prefix + sink if isinstance(sink, str) else None
        self.sink_value = float(sink) if sink is not None and not isinstance(sink, str) else None
        self.norm_after, self.value_rotation = bool(norm_after_rotation), value_rotation
        self.softcap = float(softcap) if softcap else 0.0
        self.out_scale = float(out_scale)
        if value_rotation is not None and self.Vd % 2:
            raise ValueError(f"{prefix}: rotated values need an even value size")
        self.vfreq64 = None
        self.gate, self.gate_name = gate, prefix + g
        self.gate_cols = 0 if gate is None else (heads * self.Vd if gate == "each" else heads)
        self.sink = None
        self.qkv = self.out = None
        self.rot = None
        self.q_norm_w = self.k_norm_w = self.freq64 = None

    def kv_need(self):
        return KVNeed(self.K, self.hd, self.window)

    def tensors(self):
        q, k, v, o = (self.prefix + n for n in self.proj)
        sfx = self.suffix
        qd, kd, vd = self.H * self.D, self.K * self.D, self.K * self.Vd
        t = {q + sfx: TensorSpec((qd, self.width)), k + sfx: TensorSpec((kd, self.width)),
             v + sfx: TensorSpec((vd, self.width)), o + sfx: TensorSpec((self.width, self.H * self.Vd))}
        b = self.bias_suffix
        if self.bias:
            t.update({q + b: TensorSpec((qd,), "vector", "zeros"), k + b: TensorSpec((kd,), "vector", "zeros"),
                      v + b: TensorSpec((vd,), "vector", "zeros")})
        if self.out_bias:
            t[o + b] = TensorSpec((self.width,), "vector", "zeros")
        if self.qk_norm:
            t.update({n: TensorSpec((self.D,), "vector", "ones_jitter") for n in self.norm_names})
        if self.gate is not None:
            t[self.gate_name + sfx] = TensorSpec((self.gate_cols, self.width))
        if self.sink_name is not None:
            t[self.sink_name] = TensorSpec((self.H,), "vector")
        return t

    def bind(self, tensors, rt):
        q, k, v, o = (self.prefix + n for n in self.proj)
        sfx = self.suffix
        # the gate's rows ride in the same product, behind Q, K and V
        fused = (q, k, v) + ((self.gate_name,) if self.gate is not None else ())
        ws = [tensors.pop(n + sfx) for n in fused]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        bias = obias = None
        if self.bias:
            bias = torch.cat([tensors[n + self.bias_suffix].to(torch.float32) for n in (q, k, v)])
            if self.gate is not None:
                bias = torch.cat([bias, torch.zeros(self.gate_cols, dtype=torch.float32, device=bias.device)])
        if self.out_bias:
            obias = tensors[o + self.bias_suffix]
        if self.sink_name is not None:
            self.sink = tensors[self.sink_name].to(torch.float32).contiguous()
        elif self.sink_value is not None:
            self.sink = torch.full((self.H,), self.sink_value, dtype=torch.float32, device=rt.device)
        if self.value_rotation is not None:
            vf = np.power(float(self.value_rotation[0]), -2.0 * np.arange(self.Vd // 2, dtype=np.float64) / float(self.Vd))
            self.vfreq64 = torch.from_numpy(vf).to(rt.device)
        self.qkv = Linear(torch.cat(ws, dim=0), bias).prepare(rt)
        del ws
        wo = tensors[o + sfx]
        if self.hd != self.Vd:
            # the attention's output rows hold hd values a head, of which the first Vd are the head's: zero columns for the rest
            wide = torch.zeros((self.width, self.H, self.hd), dtype=wo.dtype, device=wo.device)
            wide[:, :, :self.Vd] = wo.view(self.width, self.H, self.Vd)
            wo = wide.view(self.width, self.H * self.hd)
        self.out = Linear(wo, obias).prepare(rt)
        self._out_bytes = self.width * self.H * self.Vd * wo.element_size()
        if self.qk_norm:
            self.q_norm_w, self.k_norm_w = (tensors[n].to(torch.float32).contiguous() for n in self.norm_names)
        self.position.prepare(rt)
        try:
            rot = self.position.rotary()
        except NotImplementedError as e:
            raise ValueError(f"{self.prefix}: this mixer takes position encodings that rotate query and key pairs, or "
                             f"none ({e}); another kind needs a mixer of its own") from None
        if rot is not None and rot.rotary_dim > self.D:
            raise ValueError(f"{self.prefix}: rotary_dim {rot.rotary_dim} exceeds head_dim {self.D}")
        # (rotary_dim, inv_freq, adjacent pairs, mscale) as the rotation kernels take them
        self.rot = (0, None, False, 1.0) if rot is None or rot.rotary_dim == 0 else \
            (rot.rotary_dim, rot.inv_freq, rot.pairing == "adjacent", rot.mscale)
        if self.general and self.rot[0]:
            f64 = getattr(self.position, "inv_freq64_host", None)
            f64 = rot.inv_freq.double().cpu().numpy() if f64 is None else f64
            self.freq64 = torch.from_numpy(np.ascontiguousarray(f64, dtype=np.float64)).to(rt.device)

    def weight_bytes(self):
        return self.qkv.nbytes() + self._out_bytes

    @staticmethod
    def _portions(ctx, G):
        """(some portion has at most 16 packed rows, some has more, the longest portion, the row tiles of the longer
        ones in tiles of 128 and of 64 rows)"""
        seg_len = ctx.host["seg_len"]
        rows = seg_len * G
        return (bool((rows <= 16).any()), bool((rows > 16).any()), int(seg_len.max()),
                kernels.long_row_tiles(seg_len, G, 128), kernels.long_row_tiles(seg_len, G, 64))

    def forward(self, ctx, h, x, lay):
        n = h.shape[0]
        qkv_dim = (self.H + 2 * self.K) * self.hd
        qkv = ctx.buf("attn_qkv", (n, qkv_dim), ctx.act_dtype)
        k_ptr, page_stride, v_offset = ctx.cache_layer(lay)
        bt = ctx.block_tables[lay.group]
        store_ptr = k_ptr if lay.writes_cache else None
        rot_dim, rot_freq, adjacent, mscale = self.rot
        if self.general:
            # the projection's rows [Q | K | V] in their own sizes; norm, rotation and store in one kernel, Q into `qkv`
            # (and the gate's columns behind them, which the gate kernel reads after the attention)
            gate_at = (self.H + self.K) * self.D + self.K * self.Vd
            cols = gate_at + self.gate_cols
            proj = ctx.buf("attn_proj", (n, -(-cols // 8) * 8), ctx.act_dtype)[:, :cols]
            # (a product that was cut along K leaves its partial sums to the same kernel; not where the values are turned first)
            pend = self.qkv.forward(h, proj, defer=self.value_rotation is None)
            if self.value_rotation is not None:
                kernels.rotate_heads(proj, (self.H + self.K) * self.D, self.K, self.Vd, self.Vd, self.Vd, self.value_rotation[1] == "adjacent",
                                     self.vfreq64, ctx.positions)
            coef, every = self.q_temp if self.q_temp is not None else (0.0, 0)
            kernels.qk_norm_rope_store(proj, qkv, ctx.positions, ctx.tok_seg, bt, self.freq64, self.q_norm_w, self.k_norm_w, store_ptr,
                                       page_stride, v_offset, self.H, self.K, self.D, self.Vd, self.hd, rot_dim, ctx.max_pages,
                                       ctx.page_size, adjacent, self.norm_eps, self.unit_norm, coef, every,
                                       partial=None if pend is None else pend.partial, splits=0 if pend is None else pend.splits,
                                       bias=None if pend is None else pend.bias, mscale=mscale, norm_after=self.norm_after)
            if pend is not None:
                pend.release()
        else:
            pend = self.qkv.forward(h, qkv, defer=True)
            if pend is not None and lay.writes_cache:
                # the product was split along K: its finish, the rotation and the page store are one kernel
                kernels.finish_rope_store(pend.partial, pend.splits, pend.bias, qkv, ctx.positions, ctx.tok_seg, bt,
                                          rot_freq, store_ptr, page_stride, v_offset, self.H, self.K, self.hd,
                                          rot_dim, ctx.max_pages, ctx.page_size, adjacent, mscale)
                pend.release()
            else:
                if pend is not None:
                    pend.finish()
                kernels.rope_store(qkv, ctx.positions, ctx.tok_seg, bt, rot_freq, store_ptr, page_stride,
                                   v_offset, self.H, self.K, self.hd, rot_dim, ctx.max_pages, ctx.page_size, adjacent, mscale)
        o = ctx.buf("attn_out", (n, self.H * self.hd), ctx.act_dtype)
        # Q is read in place from the fused rows (row stride = qkv_dim)
        G = self.H // self.K
        if USE_MMA and kernels.attention_mma_supported(ctx.act_dtype, self.H, self.K, self.hd):
            # (what the portions' lengths say is the same for every layer of the step)
            any_short, any_long, longest, tiles_tc, tiles_rows = ctx.once(("gqa_portions", G), lambda: self._portions(ctx, G))
            splits = ctx.once(("gqa_splits", self.window or 0, self.K),
                              lambda: kernels.attention_mma_splits(ctx.max_kv_len, self.window or 0, ctx.n_seg * self.K))
            pa = pm = None
            if any_short:
                pa = ctx.buf("attn_part_acc", (ctx.n_seg * self.K * splits * 16 * self.hd,), torch.float32)
                pm = ctx.buf("attn_part_ml", (ctx.n_seg * self.K * splits * 32,), torch.float32)
            if any_long and USE_TC and kernels.attention_tc_supported(ctx.act_dtype, self.H, self.K, self.hd, ctx.page_size):
                # prompt portions: S = Q K^T and O += P V on tcgen05
                kernels.attention_tc(qkv, o, ctx.seg_start, ctx.seg_len, ctx.seg_pos0, bt, ctx.cache_group(lay), self.H,
                                     self.K, self.hd, ctx.max_pages, ctx.page_size, self.window or 0, self.scale, ctx.n_seg,
                                     longest, row_tiles=tiles_tc, sink=self.sink, softcap=self.softcap)
                counters["tcgen05"] += 1
                any_long = False
            if any_short or any_long:
                kernels.attention_mma(qkv, qkv_dim, o, k_ptr, ctx.seg_start, ctx.seg_len, ctx.seg_pos0, bt, pa, pm,
                                      page_stride, v_offset, self.H, self.K, self.hd, ctx.max_pages, ctx.page_size,
                                      self.window or 0, self.scale, ctx.n_seg, longest, ctx.max_kv_len, splits,
                                      any_short, any_long, group=ctx.cache_group(lay) if USE_TMA else None, uneven=ctx.uneven,
                                      row_tiles=tiles_rows, sink=self.sink, softcap=self.softcap)
                counters["mma"] += 1
        else:
            kernels.attention_simt(qkv, qkv_dim, o, k_ptr, ctx.positions, ctx.tok_seg, bt, page_stride, v_offset,
                                   self.H, self.K, self.hd, ctx.max_pages, ctx.page_size, self.window or 0, self.scale, sink=self.sink, softcap=self.softcap)
            counters["simt"] += 1
        if self.gate is not None:
            kernels.sigmoid_gate(o, proj[:, gate_at:gate_at + self.gate_cols], self.H, self.hd, self.Vd, self.gate == "each")
        if self.value_rotation is not None:
            # the sums are turned back by their own position (and scaled in the same pass)
            kernels.rotate_heads(o, 0, self.H, self.hd, self.Vd, self.Vd, self.value_rotation[1] == "adjacent", self.vfreq64, ctx.positions,
                                 sign=-1.0, scale=self.out_scale)
        elif self.out_scale != 1.0:
            kernels.rotate_heads(o, 0, self.H, self.hd, 0, self.hd, False, self.freq64 if self.freq64 is not None else self._no_freq(o),
                                 ctx.positions, scale=self.out_scale)
        ctx.set_pending(x, self.out.forward(o, x, accumulate=True, defer=True))

    def _no_freq(self, like):
        if getattr(self, "_empty_freq", None) is None:
            self._empty_freq = torch.zeros(1, dtype=torch.float64, device=like.device)
        return self._empty_freq


register_mixer("gqa_attention", GQAAttention)
