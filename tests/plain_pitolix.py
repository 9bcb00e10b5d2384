"""A plain, slow implementation of the Pitolix decoder: one function per mechanism, whole sequences, no cache.

Everything is computed on the CPU in one dtype (float64 by default) from a configuration dict and a dict of tensors
by name.  It shares no code with the engine: the tests compare the engine's logits with it.

Notation.  x: residual stream [T, width]; h: a sublayer's normed input; p: position (from 0); H query heads over G
key/value heads; D query/key elements and V value elements per head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The stored weight is the factor's distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, heads, D]: of the first `dims` elements, i and i + dims/2 are a pair turned by p * base^(-2i/dims)."""
    if dims == 0:
        return v
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * (base ** (-2.0 * i / dims))[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def query_temperature(positions: torch.Tensor, coef: float, every: int, dtype) -> torch.Tensor:
    """The factor on the query at position p: 1 + coef ln(floor((p + 1) / every) + 1)."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(dtype) + 1.0)


def causal_mask(T: int) -> torch.Tensor:
    return torch.arange(T)[None, :] <= torch.arange(T)[:, None]


def softmax_with_sink(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores [H, T, T].  With a sink the denominator of head h holds exp(sink[h]) once more; nothing is read for it."""
    s = scores.masked_fill(~mask, float("-inf"))
    if sink is None:
        return torch.softmax(s, dim=-1)
    T = s.shape[-1]
    wide = torch.cat([s, sink.to(s.dtype)[:, None, None].expand(-1, T, 1)], dim=-1)
    return torch.softmax(wide, dim=-1)[..., :T]


def _scores_and_values(q, k, v, scale, sink):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]."""
    T, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    a = softmax_with_sink(torch.einsum("ihd,jhd->hij", q, k) * scale, causal_mask(T), sink)
    return torch.einsum("hij,jhv->ihv", a, v)


def attention_sink(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Mixer "attention": no rotation; unit-RMS queries and keys; a query factor that grows with the position; a sink in
    the softmax; a gate per element of the concatenated heads."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = unit_rms((h @ w["q"].T).view(T, H, D), eps)
    k = unit_rms((h @ w["k"].T).view(T, G, D), eps)
    v = (h @ w["v"].T).view(T, G, V)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"], h.dtype)[:, None, None]
    o = _scores_and_values(q, k, v, m["scale"], w["sink"]).reshape(T, H * V)
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def attention_rotary(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Mixer "attention_2": biased projections; a rotation over the first rot.dims elements of each head; plain softmax;
    a gate per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w["q"].T + w["q.b"]).view(T, H, D)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, D)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, V)
    rot = m.get("rot") or {}
    dims, base = rot.get("dims", 0), rot.get("base", 10000.0)
    q, k = rotate_half(q, pos, dims, base), rotate_half(k, pos, dims, base)
    o = _scores_and_values(q, k, v, m["scale"], None)
    o = o * torch.sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (torch.nn.functional.silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


MIXERS = {"attention": attention_sink, "attention_2": attention_rotary}


def _sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer(x: torch.Tensor, tensors: Dict[str, torch.Tensor], i: int, lay: dict, eps: float) -> torch.Tensor:
    """Both sublayers read the same x, each through a norm of its own."""
    p = f"l{i}."
    out = MIXERS[lay["type"]](norm_one_plus(x, tensors[p + "norm1"], eps), _sub(tensors, p + "mix."), lay["mixer"], eps)
    if lay.get("mlp"):
        out = out + dense_ff(norm_one_plus(x, tensors[p + "norm2"], eps), _sub(tensors, p + "mlp."))
    return x + out


def layer_runs(config: dict):
    """(layer, pass number or None, first of its pass) in running order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, None, False) for i in range(b, n)]


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[List] = None):
    """Logits [T, vocab] of one sequence."""
    tensors = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x0 = tensors["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (config.get("embedding") or {}).get("scale", 1.0)
    x = x0
    for i, t, first in layer_runs(config):
        if first:
            if t > 0:
                x = x + x0
            x = x + tensors["loop.step"][t]
        x = layer(x, tensors, i, config["layers"][i], eps)
        if layers_out is not None:
            layers_out.append(x)
    return norm_one_plus(x, tensors["final.norm"], eps) @ tensors["head"].T
