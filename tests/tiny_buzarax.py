"""Small Buzarax configurations with random weights for the tests, as config.json + model.safetensors folders.

The sizes are awkward on purpose: widths that are no multiple of 8, one head, key sizes that differ from value sizes and are no
multiple of 16, as many key heads as heads and fewer, rotations over part, all or none of a head with and without interpolated
frequencies, recurrences wider and narrower than the model with one block or several and one tap or several, experts of which
all or few are chosen, layers without a feed-forward, models of one kind of layer alone, decays near one and near zero.
"""
import json
import math
import os

import numpy as np
import torch


def rot(base, dims, scaling=None):
    d = {"base": base, "dims": dims}
    if scaling is not None:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def parallel(heads, kv_heads, dim, vdim, scale, rotation, softcap, r_heads, r_dim, r_vdim, decay, left_scale=1.0, right_scale=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation}
    if softcap is not None:
        left["softcap"] = softcap
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay)},
                                          "left_scale": left_scale, "right_scale": right_scale}}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def layer(mixer, mlp):
    d = dict(mixer)
    d["mlp"] = mlp
    return d


def model(vocab, width, eps, layers, buckets, mul_prev, mul_cur, logit_softcap=None):
    d = {"architecture": "Buzarax", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}
    if logit_softcap is not None:
        d["logit_softcap"] = logit_softcap
    return d


CONFIGS = {
    # both mixers and both feed-forwards; values longer and shorter than keys; a recurrence wider than the model
    "mix": model(211, 96, 1e-5, [
        layer(parallel(4, 2, 24, 16, 0.21, rot(1000.0, 8, (4.0, 64, 16.0, 2.0)), 20.0, 3, 12, 20, (0.9, 0.5, 0.99), 0.7, 1.3), dense(80, 2.0)),
        layer(rglru(120, 3, 4), moe(5, 2, 24)),
        layer(parallel(3, 3, 16, 20, 0.25, rot(50.0, 16), None, 1, 8, 40, (0.8,), 1.0, 0.5), None),
        layer(rglru(64, 1, 1), moe(3, 3, 16))], 53, 5, 3, logit_softcap=8.0),
    # a width that is no multiple of 8; one head; no rotation of queries and keys; the recurrence first; no cap on the logits
    "odd": model(131, 68, 1e-6, [
        layer(rglru(34, 2, 2), dense(36, 0.5)),
        layer(parallel(1, 1, 18, 6, 0.2, rot(10000.0, 0), 5.0, 2, 10, 6, (0.3, 0.97), 2.0, 0.25), moe(4, 1, 12)),
        layer(parallel(5, 5, 10, 14, 0.4, rot(7.0, 10, (2.0, 16, 4.0, 1.0)), None, 1, 20, 4, (0.999,), 0.5, 1.0), dense(28, 4.0))], 7, 2, 9),
    # sizes that the tensor-core kernels take (heads of 64 and 128, pages of 64)
    "tc": model(160, 128, 1e-5, [
        layer(parallel(4, 2, 64, 64, 0.12, rot(20000.0, 32, (6.0, 128, 24.0, 1.5)), 30.0, 2, 32, 64, (0.95, 0.6), 0.55, 1.25), dense(96, 1.0)),
        layer(rglru(256, 2, 3), moe(8, 2, 64)),
        layer(parallel(2, 1, 128, 128, 0.09, rot(500.0, 64), 40.0, 4, 16, 16, (0.9, 0.8, 0.7, 0.99), 1.0, 1.0), moe(8, 3, 32)),
        layer(parallel(16, 2, 16, 32, 0.25, rot(100.0, 16, (4.0, 32, 8.0, 2.0)), None, 1, 64, 128, (0.98,), 0.8, 0.9), None)], 97, 29, 5,
        logit_softcap=12.0),
    # recurrences alone (no keys are cached at all), slow ones among them
    "rec": model(90, 64, 1e-5, [
        layer(rglru(64, 4, 3), dense(40, 1.5)),
        layer(rglru(96, 2, 5), None)], 31, 3, 11, logit_softcap=30.0),
}
SEEDS = {"mix": 31, "odd": 32, "tc": 33, "rec": 34}


def shapes(cfg):
    """Tensor names and shapes of a configuration."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, W), "final.norm": (), "head": (cfg["vocab"], W)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out.update({p + "norm1": (), p + "norm2": (), p + "dwa": (i + 2,)})
        if lay["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, D, V = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            out.update({p + "mix.left.q": (H * D, W), p + "mix.left.k": (G * D, W), p + "mix.left.v": (G * V, W), p + "mix.left.o": (W, H * V)})
            H, D, V = r["heads"], r["dim"], r["vdim"]
            out.update({p + "mix.right.q": (H * D, W), p + "mix.right.k": (H * D, W), p + "mix.right.v": (H * V, W), p + "mix.right.g": (H * V, W),
                        p + "mix.right.o": (W, H * V), p + "mix.right.norm": (H * V,)})
        else:
            R, B, K = m["width"], m["blocks"], m["conv"]
            out.update({p + "mix.y": (R, W), p + "mix.y.b": (R,), p + "mix.x": (R, W), p + "mix.x.b": (R,), p + "mix.conv": (R, K),
                        p + "mix.conv.b": (R,), p + "mix.ra": (B, R // B, R // B), p + "mix.ra.b": (B, R // B), p + "mix.ri": (B, R // B, R // B),
                        p + "mix.ri.b": (B, R // B), p + "mix.lam": (R,), p + "mix.o": (W, R)})
        f = lay.get("mlp")
        if f and f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        elif f:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            out.update({p + "mlp.router": (E, W), p + "mlp.correction": (E,)})
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
    return out


def draw(cfg, seed, dtype=torch.bfloat16, slow=False):
    """Random tensors: matrices N(0, 1/fan_in) (queries and keys of the linear attention and the dense feed-forward's larger, so
    that states grow and clamps bite), gains around 0.5, biases N(0, 1/4), routers wide enough that choices differ between tokens,
    corrections that change some choices, the average's weights near (0.2, ..., 0.2, 1), recurrence rates over a wide range
    (`slow`: all slow, so that the first tokens still count hundreds of tokens later)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        r = lambda: torch.randn(shape, generator=g)
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.5 + 0.1 * r()
        elif name.endswith("dwa"):
            t = 0.2 + 0.1 * r()
            t[-1] = 1.0 + 0.1 * t[-1]
        elif name.endswith("right.norm"):
            t = 1.0 + 0.1 * r()
        elif name.endswith(".b"):
            t = 0.5 * r()
        elif name.endswith("mix.lam"):
            t = -6.0 + 0.5 * r() if slow else -2.0 + 2.0 * r()
        elif name.endswith("correction"):
            t = 0.2 * r()
        elif name.endswith(("mix.ra", "mix.ri")):
            t = 2.0 * r() / shape[-1] ** 0.5
        elif name.endswith("mix.conv"):
            t = r() / shape[-1] ** 0.5
        elif name.endswith(("router", "mlp.gate", "mlp.up")) and ".e" not in name:
            t = 3.0 * r() / shape[-1] ** 0.5
        elif name in ("embed", "bigram"):
            t = r()
        else:
            t = r() / shape[-1] ** 0.5
        out[name] = t.to(dtype)
    return out


def make_folder(path, name, tensors=None, cfg=None, slow=False):
    """Write config.json + model.safetensors (bfloat16) for configuration `name` (or `cfg`); returns (path, cfg, tensors)."""
    from xyntetik_runner_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    tensors = tensors if tensors is not None else draw(cfg, SEEDS.get(name, 1), slow=slow)
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"), list(tensors.items()), metadata={"format": "pt"})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return path, cfg, tensors


def plain_logits(cfg, tensors, tokens):
    import plain_buzarax
    return plain_buzarax.forward(cfg, tensors, tokens, dtype=torch.float64).to(torch.float32).numpy()


def plain_greedy(cfg, tensors, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]


NEAR_TIE = 0.02        # choice scores closer than this may change places under bfloat16 rounding of what the router reads


def near_tie_sensitivity(cfg, tensors, tokens, ref, most=48):
    """What a change of places between the last chosen expert and the first one left out does to every position's logits, for
    the (layer, position) pairs where their choice scores lie within NEAR_TIE of each other (the `most` closest): the largest
    change per position over these pairs, one pair changed at a time.  A choice that close is made differently by ANY run that
    rounds the router's input, and what follows at that position and, through keys, values and states, at later ones, differs."""
    import plain_buzarax as P
    orig = P.routing
    state = {"call": 0, "swap": None, "margins": []}

    def routing(h, w, top):
        call = state["call"]
        state["call"] += 1
        chosen, weight = orig(h, w, top)
        E = w["router"].shape[0]
        if top == E:
            return chosen, weight
        s = torch.sigmoid(h @ w["router"].T)
        order = torch.argsort(s + w["correction"], dim=-1, descending=True)
        if state["swap"] is None:
            c = s + w["correction"]
            gap = torch.gather(c, 1, order[:, top - 1:top]) - torch.gather(c, 1, order[:, top:top + 1])
            state["margins"] += [(float(gap[p]), call, p) for p in range(h.shape[0])]
        elif state["swap"][0] == call:
            p = state["swap"][1]
            chosen = chosen.clone()
            weight = weight.clone()
            slot = int((chosen[p] == order[p, top - 1]).nonzero()[0])
            chosen[p, slot] = order[p, top]
            weight[p, slot] = s[p, order[p, top]]
        return chosen, weight

    worst = np.zeros(len(tokens))
    scale = float(np.abs(ref).max())
    try:
        P.routing = routing
        plain_logits(cfg, tensors, tokens)
        near = sorted(m for m in state["margins"] if m[0] < NEAR_TIE)[:most]
        for _, call, p in near:
            state["call"], state["swap"] = 0, (call, p)
            worst = np.maximum(worst, np.abs(plain_logits(cfg, tensors, tokens) - ref).max(axis=1) / scale)
    finally:
        P.routing = orig
    return worst


def rounding_sensitivity(cfg, tensors, tokens, draws=3):
    """How far a rounding of every sublayer's input to bfloat16 moves each position's logits in the plain implementation, as a
    fraction of the largest logit: the largest of `draws` runs, the first with the rounding alone, the others with a relative
    nudge of up to 2^-8 before it; and the largest change that a near tie between two experts' choice scores makes when it
    falls the other way (``near_tie_sensitivity``).  Positions where this is large differ by more than the usual rounding in ANY
    bfloat16 run; a bfloat16 comparison allows for it position by position."""
    import plain_buzarax as P
    ref = plain_logits(cfg, tensors, tokens)
    scale = float(np.abs(ref).max())
    orig = P.sublayer_input
    g = torch.Generator().manual_seed(len(tokens))
    worst = near_tie_sensitivity(cfg, tensors, tokens, ref)
    try:
        for d in range(draws):
            def rounded(x, d=d):
                if d:
                    x = x * (1.0 + (torch.rand(x.shape, generator=g, dtype=torch.float64) - 0.5) * 2.0 ** -7)
                return x.to(torch.bfloat16).to(torch.float64)
            P.sublayer_input = rounded
            worst = np.maximum(worst, np.abs(plain_logits(cfg, tensors, tokens) - ref).max(axis=1) / scale)
    finally:
        P.sublayer_input = orig
    return worst


def assert_close_bfloat16(got, ref, sens, what=""):
    """The fixed bfloat16 tolerance of `traces` at every position, except that a position may differ by three times what the
    rounding of the sublayers' inputs alone does to it in the plain implementation (`sens`, from ``rounding_sensitivity``); few
    positions may need that, and the mean over all (of a request of sixteen tokens or more) stays within the fixed mean."""
    import traces
    tol = traces.TOL["bfloat16"]
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    scale = float(np.abs(ref).max())
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    err = diff.max(axis=1) / scale
    allowed = np.maximum(tol["max_rel"], 3.0 * sens)
    bad = np.nonzero(err > allowed)[0]
    assert len(bad) == 0, f"{what}: positions {bad[:10].tolist()} differ by {err[bad[:10]].round(4).tolist()} of the largest logit, allowed {allowed[bad[:10]].round(4).tolist()}"
    over = int((err > tol["max_rel"]).sum())
    assert over <= max(1, len(err) // 10), f"{what}: {over} of {len(err)} positions beyond the fixed tolerance"
    if len(err) >= 16:              # (a mean over a handful of positions is no mean)
        assert diff.mean() <= 1.5 * tol["mean_rel"] * scale, f"{what}: mean |diff| {diff.mean():.3e} > {1.5 * tol['mean_rel']:.1e} * {scale:.3f}"
