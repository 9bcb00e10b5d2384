"""Prefill and decode throughput of a Turudra, a Besolix, a Pitolix or a Buzarax model beside a dense Llama of equal size, with the time of
every kernel family inside the steps (``bench.py --designs``).

Sizes resemble real layers; weights are random.  Both models run through the same engine: one prompt of `tokens` tokens
in one step (prefill), and decode steps of `batch` requests that hold `context` tokens each (``Engine.adopt``: the cache
holds whatever the pool holds; the recurrent states start at zero).  Step times are CUDA-event times after warm-up; the
weights of either model exceed the L2 cache, so every step reads them from memory.

Per kernel family, the time inside one step launched kernel by kernel (an event before and after every launch; gaps
between launches count to the family that follows, so small kernels read high), the FLOPs and bytes the family must
move, and the larger of FLOPs / time / measured product peak and bytes / time / measured copy bandwidth: the fraction
of its roofline.
"""
from __future__ import annotations

import time
from typing import Dict, List

import torch

from . import kernels, measure
from .config.besolix import BesolixConfig
from .config.buzarax import BuzaraxConfig
from .config.llama import LlamaConfig
from .config.pitolix import PitolixConfig
from .config.turudra import TurudraConfig
from .engine.engine import EngineParams, StepEntry, random_engine

SIZES = {
    # name: (width, latent attention, mlstm, experts, top, expert ff, shared ff, vocab)
    "w1024": (1024, dict(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256), dict(heads=4, dim=128, vdim=256), 16, 2, 512, 1024, 32000),
    "w2048": (2048, dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512), dict(heads=8, dim=128, vdim=256), 64, 6, 1408, 2816, 32000),
}


def turudra_config(size: str) -> TurudraConfig:
    W, la, ml, E, top, ff, sff, vocab = SIZES[size]
    mlp = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 7.0}, "shared": {"ff": sff, "limit": 7.0}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": dict(la, scale=(la["dim"] + la["rot_dim"]) ** -0.5, rot={"base": 10000.0, "dims": la["rot_dim"]})}
    mlstm = {"type": "mlstm", "mlp": mlp, "mixer": dict(ml, gate_cap=15.0)}
    return TurudraConfig.from_dict({"architecture": "Turudra", "vocab": vocab, "width": W, "embedding": {"scale": 1.0},
                                    "residual_mult": 1.0, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
                                    "layers": [mlstm, latent, mlstm, latent], "loop": {"start": 1, "stop": 3, "times": 2}})


def llama_config(size: str, layers: int, positions: int) -> LlamaConfig:
    """A dense decoder of the same width and number of layer runs whose feed-forward is as wide as the experts a token uses."""
    W, la, ml, E, top, ff, sff, vocab = SIZES[size]
    return LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": W, "num_hidden_layers": layers,
                                  "num_attention_heads": W // 128, "num_key_value_heads": max(1, W // 512), "head_dim": 128,
                                  "intermediate_size": top * ff + sff, "vocab_size": vocab, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                                  "max_position_embeddings": positions, "torch_dtype": "bfloat16"})


BESOLIX_SIZES = {
    # name: (width, attention, delta, latent, feed-forward, vocab); six layers: delta, latent, attention, delta, a latent layer
    # that reads the rows of the first, attention
    "besolix-w1024": (1024, dict(heads=8, kv_heads=2, dim=64, vdim=128, window=1024, rot_dims=32),
                      dict(heads=4, kv_heads=2, dim=128, vdim=128, conv=4),
                      dict(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384, window=1024), 2816, 32000),
    "besolix-w2048": (2048, dict(heads=16, kv_heads=4, dim=128, vdim=128, window=1024, rot_dims=64),
                      dict(heads=8, kv_heads=4, dim=128, vdim=256, conv=4),
                      dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, window=1024), 5632, 32000),
}


def besolix_config(size: str) -> BesolixConfig:
    W, at, dl, la, ff, vocab = BESOLIX_SIZES[size]
    mlp = {"kind": "dense", "ff": ff}
    attention = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": at["heads"], "kv_heads": at["kv_heads"], "dim": at["dim"], "vdim": at["vdim"], "scale": at["dim"] ** -0.5,
                           "rot": {"base": 20000.0, "dims": at["rot_dims"], "scaling": {"factor": 4.0}}, "mask": {"size": at["window"]}}}
    delta = {"type": "delta", "mlp": mlp, "mixer": dict(dl)}
    lm = {k: v for k, v in la.items() if k != "window"}
    lm.update(scale=(la["dim"] + la["rot_dim"]) ** -0.5, rot={"base": 10000.0, "dims": la["rot_dim"]}, mask={"size": la["window"]})
    latent = {"type": "latent_attention", "mlp": mlp, "mixer": lm}
    reader = {"type": "latent_attention", "mlp": mlp, "mixer": dict(lm, kv_from=1)}
    return BesolixConfig.from_dict({"architecture": "Besolix", "vocab": vocab, "width": W, "norm": {"eps": 1e-5},
                                    "layers": [delta, latent, attention, delta, reader, attention]})


def llama_like_besolix(size: str, positions: int) -> LlamaConfig:
    """A dense decoder of the same width, number of layers, feed-forward and attention window."""
    W, at, dl, la, ff, vocab = BESOLIX_SIZES[size]
    return LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": W, "num_hidden_layers": 6,
                                  "num_attention_heads": W // 128, "num_key_value_heads": max(1, W // 512), "head_dim": 128,
                                  "intermediate_size": ff, "vocab_size": vocab, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                                  "max_position_embeddings": positions, "sliding_window": at["window"], "torch_dtype": "bfloat16"})


PITOLIX_SIZES = {
    # name: (width, heads, kv heads, head size, rotated elements, positions per step of the query factor, feed-forward, vocab); four
    # layers (rotary, sink, rotary, sink) of which the middle two run twice: six layer runs
    "pitolix-w1024": (1024, 8, 2, 128, 64, 512, 2816, 32000),
    "pitolix-w2048": (2048, 16, 4, 128, 64, 1024, 5632, 32000),
}


def pitolix_config(size: str) -> PitolixConfig:
    W, H, K, D, rot, every, ff, vocab = PITOLIX_SIZES[size]
    mlp = {"kind": "dense", "ff": ff}
    sizes = {"heads": H, "kv_heads": K, "dim": D, "vdim": D, "scale": D ** -0.5}
    rotary = {"type": "attention_2", "mlp": mlp, "mixer": dict(sizes, rot={"base": 10000.0, "dims": rot})}
    sink = {"type": "attention", "mlp": mlp, "mixer": dict(sizes, q_temp={"coef": 0.1, "every": every})}
    return PitolixConfig.from_dict({"architecture": "Pitolix", "vocab": vocab, "width": W, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
                                    "layers": [rotary, sink, rotary, sink], "loop": {"start": 1, "stop": 3, "times": 2}})


def llama_like_pitolix(size: str, positions: int) -> LlamaConfig:
    """A dense decoder of the same width, number of layer runs, heads and feed-forward."""
    W, H, K, D, rot, every, ff, vocab = PITOLIX_SIZES[size]
    return LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": W, "num_hidden_layers": 6,
                                  "num_attention_heads": H, "num_key_value_heads": K, "head_dim": D,
                                  "intermediate_size": ff, "vocab_size": vocab, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                                  "max_position_embeddings": positions, "torch_dtype": "bfloat16"})


BUZARAX_SIZES = {
    # name: (width, softmax side (heads, kv heads, head size, rotated elements), decay side (heads, key size, value size), recurrence
    # (channels, blocks, taps), dense feed-forward, experts, chosen, expert feed-forward, vocab); six layers: the parallel mixer and
    # the recurrence in turn, dense and routed feed-forwards in turn
    "buzarax-w1024": (1024, (8, 2, 128, 64), (4, 128, 128), (1280, 5, 4), 2816, 16, 2, 1408, 32000),
    "buzarax-w2048": (2048, (16, 4, 128, 64), (8, 128, 128), (2560, 10, 4), 5632, 16, 2, 2816, 32000),
}


def buzarax_config(size: str) -> BuzaraxConfig:
    W, (H, K, D, rot), (rh, rd, rv), (R, B, taps), ff, E, top, eff, vocab = BUZARAX_SIZES[size]
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": eff}}
    par = {"type": "parallel", "mixer": {
        "left": {"heads": H, "kv_heads": K, "dim": D, "vdim": D, "scale": D ** -0.5, "softcap": 30.0,
                 "rot": {"base": 100000.0, "dims": rot, "scaling": {"factor": 16.0, "original": 8192, "fast": 16.0, "slow": 2.0}}},
        "right": {"heads": rh, "dim": rd, "vdim": rv, "decay": [1.0 - 2.0 ** -(3 + 5.0 * h / max(rh - 1, 1)) for h in range(rh)]},
        "left_scale": 0.7, "right_scale": 0.9}}
    rec = {"type": "rglru", "mixer": {"width": R, "blocks": B, "conv": taps}}
    layers = [dict(par, mlp=dense), dict(rec, mlp=moe), dict(par, mlp=moe), dict(rec, mlp=dense), dict(par, mlp=dense), dict(rec, mlp=moe)]
    return BuzaraxConfig.from_dict({"architecture": "Buzarax", "vocab": vocab, "width": W, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
                                    "embedding": {"bigram": {"buckets": 65521, "mul_prev": 257, "mul_cur": 13}}, "layers": layers})


def llama_like_buzarax(size: str, positions: int) -> LlamaConfig:
    """A dense decoder of the same width, number of layers and attention heads, its feed-forward as wide as what a token uses."""
    W, (H, K, D, rot), _, _, ff, E, top, eff, vocab = BUZARAX_SIZES[size]
    return LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": W, "num_hidden_layers": 6,
                                  "num_attention_heads": H, "num_key_value_heads": K, "head_dim": D,
                                  "intermediate_size": (ff + top * eff) // 2, "vocab_size": vocab, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                                  "max_position_embeddings": positions, "torch_dtype": "bfloat16"})


FAMILIES = {
    "gemm_tc": "products (tcgen05)", "gemm_tc_deferred": "products (tcgen05)", "gemm_simt": "products (FMA)",
    "finish_plain": "products (tcgen05)", "finish_add_rmsnorm": "norms", "rmsnorm": "norms", "finish_rope_store": "rotation + cache store",
    "rope_store": "rotation + cache store", "attention_tc": "attention", "attention_mma": "attention", "attention_simt": "attention",
    "latent_prep": "rotation + cache store", "head_matmul": "latent attention: per-head products", "latent_attention": "latent attention: scores and sums",
    "latent_attention_mma": "latent attention: scores and sums", "gemm_tc_grouped": "grouped products (experts, per-head)",
    "moe_gather": "grouped products (experts, per-head)", "heads_gather": "grouped products (experts, per-head)",
    "heads_scatter_gate": "grouped products (experts, per-head)",
    "mlstm": "mlstm recurrence", "route_topk": "routing", "moe_plan": "routing", "moe_gemm": "experts' products", "moe_combine": "experts' sum",
    "delta": "delta recurrence", "head_norm_gate": "delta recurrence", "qk_norm_rope_store": "rotation + cache store",
    "rmsnorm_act": "norms",
    "sigmoid_gate": "output gates", "stream_step": "stream kernels",
    "rglru": "gated linear recurrence", "decay_attention": "decay attention recurrence", "norm_add": "norms", "depth_average": "stream kernels",
    "cast_rows": "stream kernels", "row_norm_gate": "decay attention recurrence", "embed_pair": "stream kernels", "last_token": "stream kernels", "rotate_heads": "rotation + cache store",
    "scaled_add": "stream kernels", "concat_cast": "stream kernels", "softcap": "stream kernels", "embed": "stream kernels", "act_mul": "stream kernels",
}


class _Timed:
    """Events around every launch of the functions in FAMILIES while a step runs."""

    def __init__(self):
        self.marks: List[tuple] = []
        self._orig = {}

    def __enter__(self):
        for name in FAMILIES:
            fn = getattr(kernels, name)
            self._orig[name] = fn

            def wrapped(*a, _fn=fn, _name=name, **k):
                r = _fn(*a, **k)
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                self.marks.append((_name, e))
                return r
            setattr(kernels, name, wrapped)
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        for name, fn in self._orig.items():
            setattr(kernels, name, fn)

    def by_family(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        prev = self.start
        for name, e in self.marks:
            out[FAMILIES[name]] = out.get(FAMILIES[name], 0.0) + prev.elapsed_time(e) * 1e3
            prev = e
        return out


def _work(cfg, tokens: int, keys_per_token: float, decode: bool) -> Dict[str, tuple]:
    """(FLOPs, bytes) that each Turudra-specific family must move in one step of `tokens` tokens."""
    out = {}
    runs = cfg.layer_runs()
    fl_e = by_e = fl_a = by_a = fl_h = by_m = fl_m = 0.0
    for i, _ in runs:
        lay = cfg.layers[i]
        if lay.mlp is not None:
            f = lay.mlp
            fl_e += 2.0 * tokens * f.top * 3 * f.expert.ff * cfg.width
            used = min(f.experts, tokens * f.top)
            by_e += used * 3 * f.expert.ff * cfg.width * 2
        m = lay.mixer
        if m.kind == "latent_attention":
            fl_a += 2.0 * tokens * m.heads * keys_per_token * (2 * m.kv_rank + m.rot_dim)
            by_a += (tokens if decode else 1) * keys_per_token * (m.kv_rank + m.rot_dim) * 2
            fl_h += 2.0 * tokens * m.heads * m.kv_rank * (m.dim + m.vdim)
        else:
            by_m += (tokens if decode else 1) * 2 * m.heads * m.dim * m.vdim * 4
            fl_m += 4.0 * tokens * m.heads * m.dim * m.vdim
    out["experts' products"] = (fl_e, by_e)
    out["grouped products (experts, per-head)"] = (fl_e + fl_h, by_e)
    out["latent attention: scores and sums"] = (fl_a, by_a)
    out["latent attention: per-head products"] = (fl_h, 0.0)
    out["mlstm recurrence"] = (fl_m, by_m)
    return out


def _besolix_work(cfg, tokens: int, keys_per_token: float, decode: bool) -> Dict[str, tuple]:
    """(FLOPs, bytes) that the mixers' own kernel families must move in one step of `tokens` tokens."""
    fl_a = by_a = fl_l = by_l = fl_h = fl_d = by_d = 0.0
    for lay in cfg.layers:
        m = lay.mixer
        keys = min(keys_per_token, getattr(m, "window", None) or keys_per_token)
        span = keys if decode else min(2 * keys_per_token, keys_per_token + (getattr(m, "window", None) or keys_per_token))
        if m.kind == "attention":
            fl_a += 2.0 * tokens * m.heads * keys * (m.dim + m.vdim)
            by_a += (tokens if decode else 1) * span * m.kv_heads * 2 * max(m.dim, m.vdim) * 2
        elif m.kind == "latent_attention":
            fl_l += 2.0 * tokens * m.heads * keys * (2 * m.kv_rank + m.rot_dim)
            by_l += (tokens if decode else 1) * span * (m.kv_rank + m.rot_dim) * 2
            fl_h += 2.0 * tokens * m.heads * m.kv_rank * (m.dim + m.vdim)
        else:
            # per token and state element: the decay, S^T k, the update, S^T q
            fl_d += 7.0 * tokens * m.heads * m.dim * m.vdim
            by_d += (tokens if decode else 1) * 2 * m.heads * m.dim * m.vdim * 4 + tokens * (2 * m.kv_heads * m.dim + 2 * m.heads * m.vdim) * 4
    return {"attention": (fl_a, by_a), "latent attention: scores and sums": (fl_l, by_l), "latent attention: per-head products": (fl_h, 0.0),
            "grouped products (experts, per-head)": (fl_h, 0.0), "delta recurrence": (fl_d, by_d)}


def _llama_work(cfg, tokens, keys_per_token, decode):
    L, W = cfg.num_hidden_layers, cfg.hidden_size
    keys = min(keys_per_token, cfg.sliding_window or keys_per_token)
    span = keys if decode else min(2 * keys_per_token, keys_per_token + (cfg.sliding_window or keys_per_token))
    fl_a = 4.0 * tokens * cfg.num_attention_heads * keys * cfg.head_dim * L
    by_a = (tokens if decode else 1) * span * 2 * cfg.num_key_value_heads * cfg.head_dim * 2 * L
    per_layer = W * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * W + 3 * W * cfg.intermediate_size
    fl_p = 2.0 * tokens * (per_layer * L + cfg.vocab_size * W * (1 if decode else 1.0 / tokens))
    by_p = 2.0 * (per_layer * L + cfg.vocab_size * W)
    # the memory-bound kernels between the products: a norm reads a float32 row and writes an activation row; the rotation
    # reads the projection's rows, writes the queries back and the keys and values into their pages
    by_n = tokens * W * (4 + 2) * (2 * L + 1)
    by_r = tokens * 2.0 * 2 * (cfg.q_dim + 2 * cfg.kv_dim) * L
    return {"attention": (fl_a, by_a), "products (tcgen05)": (fl_p, by_p), "norms": (0.0, by_n), "rotation + cache store": (0.0, by_r)}


def _pitolix_work(cfg, tokens, keys_per_token, decode):
    """(FLOPs, bytes) per kernel family in one step of `tokens` tokens, counted like ``_llama_work``."""
    W = cfg.width
    fl_a = by_a = fl_p = by_p = by_n = by_r = by_g = 0.0
    for i, _ in cfg.layer_runs():
        lay = cfg.layers[i]
        m = lay.mixer
        hd = max(m.dim, m.vdim)
        gate = m.heads * m.vdim if m.kind == "attention" else m.heads
        cols = (m.heads + m.kv_heads) * m.dim + m.kv_heads * m.vdim + gate
        per_layer = W * cols + m.heads * m.vdim * W + (3 * W * lay.mlp.ff if lay.mlp is not None else 0)
        fl_a += 2.0 * tokens * m.heads * keys_per_token * (m.dim + m.vdim)
        by_a += (tokens if decode else 1) * keys_per_token * 2 * m.kv_heads * hd * 2
        fl_p += 2.0 * tokens * per_layer
        by_p += 2.0 * per_layer         # (every run of a looped layer reads its weights again: the layers between exceed the L2 cache)
        by_n += tokens * W * (4 + 2 * (2 if lay.mlp is not None else 1))
        by_r += tokens * 2.0 * ((cols - gate) + (m.heads + 2 * m.kv_heads) * hd)
        by_g += tokens * 2.0 * (2 * m.heads * m.vdim + gate)
    fl_p += 2.0 * cfg.vocab * W * (tokens if decode else 1)
    by_p += 2.0 * cfg.vocab * W
    by_n += tokens * W * (4 + 2)
    return {"attention": (fl_a, by_a), "products (tcgen05)": (fl_p, by_p), "norms": (0.0, by_n), "rotation + cache store": (0.0, by_r),
            "output gates": (0.0, by_g)}


def _buzarax_work(cfg, tokens, keys_per_token, decode):
    """(FLOPs, bytes) per kernel family in one step of `tokens` tokens, counted like ``_llama_work``."""
    W, L = cfg.width, len(cfg.layers)
    fl_a = by_a = fl_p = by_p = by_n = by_r = fl_g = by_g = fl_d = by_d = fl_e = by_e = by_s = 0.0
    once = tokens if decode else 1
    for lay in cfg.layers:
        m = lay.mixer
        if m.kind == "parallel":
            l, r = m.left, m.right
            hd = max(l.dim, l.vdim)
            cols = (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim
            rcols = 2 * r.heads * r.dim + 2 * r.heads * r.vdim
            per = W * (cols + rcols) + (l.heads * l.vdim + r.heads * r.vdim) * W
            fl_a += 2.0 * tokens * l.heads * keys_per_token * (l.dim + l.vdim)
            by_a += once * keys_per_token * 2 * l.kv_heads * hd * 2
            # the values turned in place, the norm/rotation/store kernel, the sums turned back
            by_r += tokens * 2.0 * (2 * l.kv_heads * l.vdim + cols + (l.heads + 2 * l.kv_heads) * hd + 2 * l.heads * hd)
            # per token and state element: decay and update, read-out; the state once per request and step, the rows in float32
            fl_d += 4.0 * tokens * r.heads * r.dim * r.vdim
            by_d += once * 2 * r.heads * r.dim * r.vdim * 4 + tokens * (rcols * 4 + r.heads * r.vdim * (4 + 4 + 2))
        else:
            Bs = m.width // m.blocks
            per = W * 2 * m.width + m.width * W
            fl_g += tokens * (4.0 * m.width * Bs + 40.0 * m.width)
            by_g += tokens * m.width * (2 * 4 + 4 * 4 + 2) + 2 * m.width * Bs * 4
        f = lay.mlp
        if f is not None and f.kind == "dense":
            per += 3 * W * f.ff
        elif f is not None:
            fl_e += 2.0 * tokens * f.top * 3 * f.ff * W
            by_e += min(f.experts, tokens * f.top) * 3 * f.ff * W * 2
            per += f.experts * W
        fl_p += 2.0 * tokens * per
        by_p += 2.0 * per
        # two output norms a layer read a float32 sum and the stream and write the stream (and a rounded copy)
        by_n += tokens * W * (4 + 4 + 4 + 2) * (2 if f is not None else 1)
    fl_p += 2.0 * cfg.vocab * W * (tokens if decode else 1)
    by_p += 2.0 * cfg.vocab * W
    by_n += tokens * W * (4 + 2)
    # the depth averages: layer i reads i + 2 streams and writes two (and a rounded copy); the embedding and its copy
    by_s = tokens * W * 4.0 * (sum(i + 2 + 2 for i in range(L)) + 3) + tokens * W * 2.0 * L
    return {"attention": (fl_a, by_a), "products (tcgen05)": (fl_p, by_p), "norms": (0.0, by_n), "rotation + cache store": (0.0, by_r),
            "gated linear recurrence": (fl_g, by_g), "decay attention recurrence": (fl_d, by_d), "grouped products (experts, per-head)": (fl_e, by_e),
            "stream kernels": (0.0, by_s)}


def _measure(eng, cfg, work_fn, tokens: int, batch: int, context: int, steps: int, warmup: int, pk, phase: str = "both") -> dict:
    vocab = eng.plan.vocab_size
    gen = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, vocab, (tokens,), generator=gen).tolist()

    def prefill_once(timed=None):
        lg = eng.step([StepEntry("p", prompt, [tokens - 1])])
        eng.end("p")
        return lg
    out = {"weight_bytes_per_step": eng.weight_bytes_per_step()}

    def table(fam, work):
        rows = []
        for name, us in sorted(fam.items(), key=lambda kv: -kv[1]):
            row = {"kernels": name, "us": round(us, 1)}
            if name in work and us > 0:
                fl, by = work[name]
                row["tflops"] = round(fl / us / 1e6, 2)
                row["gbs"] = round(by / us / 1e3, 1)
                row["frac"] = round(max(fl / us / 1e6 / pk["bf16_tflops"], by / us / 1e3 / pk["hbm_gbs"]), 4)
            rows.append(row)
        return rows
    if phase in ("both", "prefill"):
        out["prefill"] = _prefill(eng, cfg, work_fn, tokens, warmup, prefill_once, table)
    if phase in ("both", "decode"):
        out["decode"] = _decode(eng, cfg, work_fn, batch, context, steps, warmup, vocab, gen, table)
    eng.check_status()
    return out


def _prefill(eng, cfg, work_fn, tokens, warmup, prefill_once, table):
    for _ in range(max(2, warmup // 2)):
        prefill_once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        prefill_once()
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1) / reps
    with _Timed() as t:
        prefill_once()
    prefill_fam = t.by_family()
    return {"tokens": tokens, "ms": round(prefill_ms, 3), "tok_s": round(tokens / prefill_ms * 1e3),
            "kernels": table(prefill_fam, work_fn(cfg, tokens, (tokens + 1) / 2.0, False))}


def _decode(eng, cfg, work_fn, batch, context, steps, warmup, vocab, gen, table):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ids = [f"d{i}" for i in range(batch)]
    for r in ids:
        eng.adopt(r, context)
    toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()

    def decode_once():
        return eng.step([StepEntry(r, [toks[i]], [0]) for i, r in enumerate(ids)])
    for _ in range(max(3, warmup)):
        decode_once()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        decode_once()
    e1.record()
    torch.cuda.synchronize()
    decode_ms = e0.elapsed_time(e1) / steps
    graphs, eng._graph_ok = eng._graph_ok, False
    decode_once()
    with _Timed() as t:
        decode_once()
    decode_fam = t.by_family()
    eng._graph_ok = graphs
    for r in ids:
        eng.end(r)
    return {"batch": batch, "context": context, "ms": round(decode_ms, 4), "tok_s": round(batch / decode_ms * 1e3),
            "kernels": table(decode_fam, work_fn(cfg, batch, context + steps / 2.0, True))}


def compare(size: str, tokens: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32, warmup: int = 4, root=None,
            models=("turudra", "llama"), phase: str = "both") -> dict:
    pk = measure.peaks(root)
    out = {"size": size, "peaks": pk["source"], "dtype": "bf16", "data": "synthetic: random weights, random tokens"}
    pool = batch * (context + 64 * (2 + (steps + warmup + 8) // 64)) + tokens + 64
    ep = lambda: EngineParams(dtype="bfloat16", max_tokens=pool, page_size=64, max_requests=batch + 1,
                              max_request_tokens=max(tokens, context + steps + warmup + 72), max_step_tokens=tokens)
    if size in BUZARAX_SIZES:
        arms = (("buzarax", buzarax_config(size), _buzarax_work), ("llama", llama_like_buzarax(size, context + tokens), _llama_work))
    elif size in PITOLIX_SIZES:
        arms = (("pitolix", pitolix_config(size), _pitolix_work), ("llama", llama_like_pitolix(size, context + tokens), _llama_work))
    elif size in BESOLIX_SIZES:
        arms = (("besolix", besolix_config(size), _besolix_work), ("llama", llama_like_besolix(size, context + tokens), _llama_work))
    else:
        tcfg = turudra_config(size)
        arms = (("turudra", tcfg, _work), ("llama", llama_config(size, len(tcfg.layer_runs()), context + tokens), _llama_work))
    for name, cfg, work in arms:
        # (`models` names arms to run; "turudra" also stands for the new design's arm of a Besolix size: the default runs both arms)
        if name not in models and not (name in ("besolix", "pitolix", "buzarax") and "turudra" in models):
            continue
        t0 = time.perf_counter()
        eng = random_engine(cfg, 5, ep())
        for kv in eng.kv:
            kv.normal_(0.0, 1.0)
        torch.cuda.synchronize()
        out[name] = _measure(eng, cfg, work, tokens, batch, context, steps, warmup, pk, phase)
        out[name]["load_s"] = round(time.perf_counter() - t0, 1)
        del eng
        torch.cuda.empty_cache()
    return out
