"""A plain, slow implementation of the Buzarax decoder: one function per mechanism, whole sequences, no cache.

Everything is computed on the CPU in one dtype (float64 by default) from a configuration dict and a dict of tensors
by name.  It shares no code with the engine: the tests compare the engine's logits with it.

Notation.  x: residual stream [T, width]; p: position (from 0); X_0 the embedding's output, X_(i+1) what layer i leaves
before the depth average.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def embed(tokens, table: torch.Tensor, bigram: torch.Tensor, e: dict) -> torch.Tensor:
    """Token row plus a row of the pair table chosen by a hash of (previous token, token); the first token of a sequence
    takes the table's last row."""
    buckets = bigram.shape[0] - 1
    b = e["bigram"]
    rows = [buckets] + [(tokens[t - 1] * b["mul_prev"] + tokens[t] * b["mul_cur"]) % buckets for t in range(1, len(tokens))]
    return table[torch.tensor(list(tokens))] + bigram[torch.tensor(rows)]


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict], dtype):
    """(frequency of every pair, factor on cosine and sine)."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, freq: torch.Tensor, mult: float = 1.0) -> torch.Tensor:
    """v [T, heads, D]: of the first `dims` elements, i and i + dims/2 are a pair turned by p * freq[i]; cosine and sine times
    `mult`.  Negative positions turn back."""
    if dims == 0:
        return v
    half = dims // 2
    ang = positions.to(v.dtype)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(ang) * mult, torch.sin(ang) * mult
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


def softmax_plus_one(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """exp(s_j) / (1 + sum exp(s_j)) over the visible j."""
    s = scores.masked_fill(~mask, float("-inf"))
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))


def softmax_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """The left half of the parallel mixer: rotated and then unit-RMS queries and keys, values turned by their position and the
    sum turned back, capped scores, a sink of score zero."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    dims, base = rot.get("dims", 0), rot.get("base", 10000.0)
    q, k, v = (h @ w["q"].T).view(T, H, D), (h @ w["k"].T).view(T, G, D), (h @ w["v"].T).view(T, G, V)
    if dims:
        freq, mult = yarn_frequencies(dims, base, rot.get("scaling"), h.dtype)
        q, k = rotate_half(q, pos, dims, freq, mult), rotate_half(k, pos, dims, freq, mult)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    vfreq = base ** (-2.0 * torch.arange(V // 2, dtype=h.dtype) / V)
    v = rotate_half(v, pos, V, vfreq)
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    mask = pos[None, :] <= pos[:, None]
    p = softmax_plus_one(s, mask[None])
    o = torch.einsum("hij,jhd->ihd", p, v)
    o = rotate_half(o, -pos, V, vfreq)
    return o.reshape(T, H * V) @ w["o"].T


def decayed_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """The right half: S <- decay S + k v^T per head, read out with q; a norm over all heads together, a sigmoid gate."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q, k, v = silu(h @ w["q"].T).view(T, H, D), silu(h @ w["k"].T).view(T, H, D), silu(h @ w["v"].T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1))
    o = unit_rms(torch.stack(out), eps) * w["norm"]
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = softmax_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right = decayed_linear_attention(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def causal_conv(z: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """z [T, C], taps [C, K]: out[t] = bias + sum_j taps[:, K-1-j] z[t-j], zeros before the start."""
    T, K = z.shape[0], taps.shape[1]
    out = bias.expand(T, -1).clone()
    for j in range(min(K, T)):
        out[j:] += taps[:, K - 1 - j] * z[:T - j] if j else taps[:, K - 1] * z
    return out


def gated_recurrence(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """A gated branch beside a short convolution followed by a real-gated linear recurrence per channel."""
    T, R, B = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_conv(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    ub = u.view(T, B, R // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w["ra"], ub) + w["ra.b"]).reshape(T, R)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w["ri"], ub) + w["ri.b"]).reshape(T, R)
    log_a = -8.0 * r * softplus(w["lam"])
    a = torch.exp(log_a)
    inp = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(R, dtype=h.dtype)
    out = []
    for t in range(T):
        S = a[t] * S + inp[t]
        out.append(S)
    return (torch.stack(out) * y) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    lim = f["limit"]
    g = torch.clamp(h @ w["gate"].T, max=lim)
    u = torch.clamp(h @ w["up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def routing(h: torch.Tensor, w: Dict[str, torch.Tensor], top: int):
    """(chosen experts [T, top], their weights): the choice by sigmoid score plus correction, the weight the score alone."""
    s = torch.sigmoid(h @ w["router"].T)
    chosen = torch.topk(s + w["correction"], top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    chosen, weight = routing(h, w, f["router"]["top"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weight[t]):
            a = silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])
            out[t] += c * (w[f"e{e}.down"] @ a)
    return out


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * g


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def sublayer_input(x: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads of the stream: the stream itself.  (A test replaces this to see what a rounding here does.)"""
    return x


def layer(x: torch.Tensor, tensors: Dict[str, torch.Tensor], i: int, lay: dict, eps: float) -> torch.Tensor:
    """x + norm1(mixer(x)), then the same with the feed-forward: the norms act on what the sublayers give."""
    mix = {"rglru": gated_recurrence, "parallel": parallel_mixer}[lay["type"]]
    x = x + scalar_norm(mix(sublayer_input(x), _sub(tensors, f"l{i}.mix."), lay["mixer"], eps), tensors[f"l{i}.norm1"], eps)
    f = lay.get("mlp")
    if f:
        ff = dense_ff if f["kind"] == "dense" else routed_ff
        x = x + scalar_norm(ff(sublayer_input(x), _sub(tensors, f"l{i}.mlp."), f), tensors[f"l{i}.norm2"], eps)
    return x


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[List] = None):
    """Logits [T, vocab] of one sequence.  `layers_out` receives the stream after every layer (after its depth average)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = embed(list(tokens), t["embed"], t["bigram"], config["embedding"])
    history = [x]
    for i, lay in enumerate(config["layers"]):
        history.append(layer(x, t, i, lay, eps))
        x = sum(t[f"l{i}.dwa"][j] * history[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    logits = scalar_norm(x, t["final.norm"], eps) @ t["head"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
