"""Small Pitolix configurations with random weights for the tests, as config.json + model.safetensors folders.

The sizes are awkward on purpose: widths that are no multiple of 8, one head, key sizes that differ from value sizes and
are no multiple of 16, as many key heads as heads and fewer, rotations over all, part or none of a head, query factors that
step every few positions (so that prompts and decoded tokens cross several steps), sinks that weigh as much as all the keys,
layers without a feed-forward, loops that start at the first layer or later, run once, twice or three times, and no loop.
"""
import json
import os

import numpy as np
import torch


def sink_attention(heads, kv_heads, dim, vdim, scale, coef=None, every=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def rotary_attention(heads, kv_heads, dim, vdim, scale, base, dims):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "rot": {"base": base, "dims": dims}}}


def layer(mixer, ff):
    d = dict(mixer)
    d["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return d


def model(vocab, width, eps, layers, loop=None, embedding_scale=1.0):
    return {"architecture": "Pitolix", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale}, "norm": {"eps": eps},
            "layers": layers, "loop": None if loop is None else {"start": loop[0], "stop": loop[1], "times": loop[2]}}


CONFIGS = {
    # both mixers; the loop covers the middle layers three times; fewer key heads than heads; values longer and shorter than keys
    "mix": model(211, 96, 1e-5, [
        layer(rotary_attention(4, 2, 24, 16, 0.21, 1000.0, 8), 80),
        layer(sink_attention(6, 2, 12, 20, 0.36, 0.4, 7), 64),
        layer(rotary_attention(3, 3, 16, 16, 0.25, 50.0, 16), None),
        layer(sink_attention(2, 1, 32, 24, 0.22, 0.25, 16), 48)], loop=(1, 3, 3), embedding_scale=4.0),
    # a width that is no multiple of 8; one head; no rotation at all; a loop of one pass from the first layer; no query factor
    "odd": model(131, 68, 1e-6, [
        layer(sink_attention(5, 5, 10, 14, 0.4), 36),
        layer(rotary_attention(1, 1, 18, 6, 0.2, 10000.0, 0), None),
        layer(sink_attention(1, 1, 20, 36, 0.28, 1.5, 3), 28)], loop=(0, 2, 1), embedding_scale=0.5),
    # sizes that the tensor-core kernels take (heads of 64 and 128, pages of 64); no loop
    "tc": model(160, 128, 1e-5, [
        layer(sink_attention(4, 2, 64, 64, 0.16, 0.3, 50), 96),
        layer(rotary_attention(4, 2, 64, 64, 0.12, 20000.0, 32), 64),
        layer(sink_attention(2, 1, 128, 128, 0.11, 0.1, 64), 64),
        layer(rotary_attention(2, 1, 32, 128, 0.15, 500.0, 16), 32),
        layer(rotary_attention(16, 2, 16, 16, 0.25, 100.0, 16), None)], embedding_scale=8.0),
    # the whole model is the loop, twice; heads of 48 and 96 elements (tensor cores without the tcgen05 prompt kernel)
    "loop": model(90, 64, 1e-5, [
        layer(sink_attention(2, 1, 48, 96, 0.18, 0.3, 20), 24),
        layer(rotary_attention(4, 4, 96, 48, 0.1, 10.0, 4), 40)], loop=(0, 2, 2), embedding_scale=2.0),
}
SEEDS = {"mix": 21, "odd": 22, "tc": 23, "loop": 24}


def shapes(cfg):
    """Tensor names and shapes of a configuration."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (W,), p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * V, W), p + "mix.o": (W, H * V)})
        if lay["type"] == "attention":
            out.update({p + "mix.sink": (H,), p + "mix.g": (H * V, W)})
        else:
            out.update({p + "mix.q.b": (H * D,), p + "mix.k.b": (G * D,), p + "mix.v.b": (G * V,), p + "mix.g": (H, W)})
        if lay.get("mlp"):
            ff = lay["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return out


def draw(cfg, seed, dtype=torch.bfloat16):
    """Random tensors: matrices N(0, 1/fan_in) (the gates' larger, so that gates leave one half), norm weights around 0 (they are
    offsets from one), biases N(0, 1/4), sinks N(1, 1) (a sink then weighs about as much as a few keys), the passes' vectors
    N(0, 1)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        r = lambda: torch.randn(shape, generator=g)
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.1 * r()
        elif name.endswith(".b"):
            t = 0.5 * r()
        elif name.endswith("sink"):
            t = 1.0 + r()
        elif name == "loop.step":
            t = r()
        elif name.endswith("mix.g"):
            t = 3.0 * r() / shape[-1] ** 0.5
        else:
            t = r() / shape[-1] ** 0.5
        out[name] = t.to(dtype)
    return out


def make_folder(path, name, tensors=None, cfg=None):
    """Write config.json + model.safetensors (bfloat16) for configuration `name` (or `cfg`); returns (path, cfg, tensors)."""
    from xyntetik_runner_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    tensors = tensors if tensors is not None else draw(cfg, SEEDS.get(name, 1))
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"), list(tensors.items()), metadata={"format": "pt"})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return path, cfg, tensors


def plain_logits(cfg, tensors, tokens):
    import plain_pitolix
    return plain_pitolix.forward(cfg, tensors, tokens, dtype=torch.float64).to(torch.float32).numpy()


def plain_greedy(cfg, tensors, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]


def rounding_sensitivity(cfg, tensors, tokens, draws=3):
    """How far a rounding of every sublayer's input to bfloat16 moves each position's logits in the plain implementation, as a
    fraction of the largest logit: the largest of `draws` runs, the first with the rounding alone, the others with a relative
    nudge of up to 2^-8 before it.  Positions where this is large (two keys whose scores nearly tie under a large score scale)
    differ by more than the usual rounding in ANY bfloat16 run; a bfloat16 comparison allows for it position by position."""
    import plain_pitolix as P
    ref = plain_logits(cfg, tensors, tokens)
    scale = float(np.abs(ref).max())
    orig = P.norm_one_plus
    g = torch.Generator().manual_seed(len(tokens))
    worst = np.zeros(len(tokens))
    try:
        for d in range(draws):
            def rounded(x, w, eps, d=d):
                y = orig(x, w, eps)
                if d:
                    y = y * (1.0 + (torch.rand(y.shape, generator=g, dtype=torch.float64) - 0.5) * 2.0 ** -7)
                return y.to(torch.bfloat16).to(x.dtype)
            P.norm_one_plus = rounded
            worst = np.maximum(worst, np.abs(plain_logits(cfg, tensors, tokens) - ref).max(axis=1) / scale)
    finally:
        P.norm_one_plus = orig
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
    assert over <= max(1, len(err) // 20), f"{what}: {over} of {len(err)} positions beyond the fixed tolerance"
    if len(err) >= 16:              # (a mean over a handful of positions is no mean)
        assert diff.mean() <= tol["mean_rel"] * scale, f"{what}: mean |diff| {diff.mean():.3e} > {tol['mean_rel']:.1e} * {scale:.3f}"
