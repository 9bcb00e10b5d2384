"""Buzarax without a GPU: the configuration reader, the plan the builder makes (parts per layer, the average behind every layer,
the embedding's state), and the plain implementation's own consistency (each mechanism written a second way, by hand)."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_buzarax as P
import tiny_buzarax as tb
from xyntetik_runner_b200 import architectures  # noqa: F401
from xyntetik_runner_b200.config import registry
from xyntetik_runner_b200.config.base import ConfigError
from xyntetik_runner_b200.config.buzarax import BuzaraxConfig


@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_config_round_trip_and_tensor_names(name):
    cfg = BuzaraxConfig.from_dict(tb.CONFIGS[name])
    assert BuzaraxConfig.from_dict(cfg.to_dict()) == cfg
    plan = registry.resolve("Buzarax").build_plan(cfg)
    plan.validate()
    want = {n: tuple(s) for n, s in tb.shapes(tb.CONFIGS[name]).items()}
    specs = {n: tuple(s.shape) for n, s in plan.tensor_specs().items() if not s.optional or n in want}
    assert specs == want
    # every layer run is followed by its average, which mixes one stream more than the one before
    assert [(e.layer, e.before, e.after) for e in plan.schedule] == [(i, None, i) for i in range(len(cfg.layers))]
    assert [s.k for s in plan.stream_parts] == list(range(1, len(cfg.layers) + 1)) and plan.keeps_embedding()
    assert plan.embedding.state_need().shape == (1,) and plan.embedding.state_need().dtype == torch.int32


def test_what_each_layer_keeps():
    """The softmax side keeps keys and values in pages, the other side and the recurrence a state per request; a model of
    recurrences alone has no cache group at all."""
    plan = registry.resolve("Buzarax").build_plan(BuzaraxConfig.from_dict(tb.CONFIGS["mix"]))
    needs = [(b.mixer.kv_need(), b.mixer.state_need()) for b in plan.blocks]
    assert needs[0][0].kv_heads == 2 and needs[0][0].head_dim == 32 and needs[0][0].window is None     # max(24, 16) rounded up to 16s
    assert needs[0][1].shape == (3 * 12 * 20,) and needs[1][0] is None and needs[1][1].shape == (120 * 4,)
    assert needs[3][1].shape == (64,)                                                                   # one tap: no tail
    rec = registry.resolve("Buzarax").build_plan(BuzaraxConfig.from_dict(tb.CONFIGS["rec"]))
    assert all(b.mixer.kv_need() is None for b in rec.blocks)


def test_folder_is_resolved_by_its_architecture_key(tmp_path):
    path, cfg, _ = tb.make_folder(str(tmp_path / "m"), "rec")
    arch, typed = registry.load_config(path)
    assert arch.name == "Buzarax" and typed.width == cfg["width"] and len(typed.layers) == 2


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("heads"), "heads"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 26), "dims"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("original"), "original"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("vdim", 15), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("softcap", 0.0), "softcap"),
    (lambda d: d["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda d: d["layers"][0]["mixer"].pop("right"), "right"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("blocks", 7), "blocks"),
    (lambda d: d["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda d: d["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda d: d["embedding"]["bigram"].pop("mul_prev"), "mul_prev"),
    (lambda d: d["embedding"]["bigram"].__setitem__("buckets", 0), "buckets"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d.__setitem__("layers", []), "layers"),
])
def test_config_refusals(edit, word):
    d = copy.deepcopy(tb.CONFIGS["mix"])
    edit(d)
    with pytest.raises(ConfigError, match=word):
        BuzaraxConfig.from_dict(d)


def test_what_a_configuration_may_leave_out():
    d = copy.deepcopy(tb.CONFIGS["mix"])
    d["layers"][0]["mixer"]["left"].pop("rot")
    d["layers"][0]["mixer"]["left"].pop("softcap")
    d["layers"][0]["mixer"]["left"].pop("kv_heads")
    d["layers"][0]["mixer"].pop("left_scale")
    d.pop("logit_softcap")
    cfg = BuzaraxConfig.from_dict(d)
    left = cfg.layers[0].mixer.left
    assert left.rot.dims == 0 and left.softcap is None and left.kv_heads == left.heads and cfg.layers[0].mixer.left_scale == 1.0
    assert cfg.logit_softcap is None
    registry.resolve("Buzarax").build_plan(cfg).validate()


# ---- the plain implementation against hand-worked numbers --------------------------------------------------------------------
def test_interpolated_frequencies_by_hand():
    """dims 8, base 16, original 32: wavelengths 2 pi, 4 pi, 8 pi, 16 pi.  where(t) = 8 ln(32 / (2 pi t)) / (2 ln 16): fast 1 ->
    2.348 -> lo 2; slow 0.25 -> 4.348 -> hi 5; the ramp over pairs 0..3 is 0, 0, 0, 1/3."""
    f, mult = P.yarn_frequencies(8, 16.0, {"factor": 4.0, "original": 32, "fast": 1.0, "slow": 0.25}, torch.float64)
    base = torch.tensor([1.0, 0.5, 0.25, 0.125], dtype=torch.float64)
    want = base.clone()
    want[3] = base[3] / 4.0 / 3.0 + base[3] * 2.0 / 3.0
    assert torch.allclose(f, want, rtol=1e-12) and abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    f2, m2 = P.yarn_frequencies(8, 16.0, None, torch.float64)
    assert torch.equal(f2, base) and m2 == 1.0
    # the engine's position encoding builds the same numbers
    from xyntetik_runner_b200.parts import YarnRope
    r = YarnRope(12, 16.0, 8, factor=4.0, original=32, fast=1.0, slow=0.25)
    assert np.allclose(r.inv_freq64_host, want.numpy(), rtol=1e-12) and abs(r.mscale - mult) < 1e-15
    assert np.array_equal(YarnRope(12, 16.0, 8).inv_freq64_host, base.numpy())


def test_sink_of_score_zero_by_hand():
    s = torch.tensor([[0.0, math.log(3.0)]], dtype=torch.float64)
    p = P.softmax_plus_one(s, torch.tensor([[True, True]]))
    assert torch.allclose(p, torch.tensor([[0.2, 0.6]], dtype=torch.float64))
    p1 = P.softmax_plus_one(s, torch.tensor([[True, False]]))
    assert torch.allclose(p1, torch.tensor([[0.5, 0.0]], dtype=torch.float64))
    big = P.softmax_plus_one(torch.tensor([[800.0, 799.0]], dtype=torch.float64), torch.tensor([[True, True]]))
    assert torch.isfinite(big).all() and abs(float(big.sum()) - 1.0) < 1e-12


def test_rotated_values_see_distances_only():
    """Shifting all positions by a constant changes nothing of what the softmax side gives: queries and keys, and values and the
    sums turned back, only ever meet as differences of positions."""
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 6, "scale": 0.4, "softcap": 3.0, "rot": {"base": 30.0, "dims": 4}}
    g = torch.Generator().manual_seed(1)
    w = {k: torch.randn(s, generator=g, dtype=torch.float64) for k, s in dict(q=(16, 10), k=(8, 10), v=(6, 10), o=(10, 12)).items()}
    h = torch.randn(7, 10, generator=g, dtype=torch.float64)
    a = P.softmax_attention(h, w, m, 1e-6)
    orig = torch.arange
    try:
        # (the function takes its positions from torch.arange(T): shift them)
        torch.arange = lambda *args, **kw: orig(*args, **kw) + (1000 if len(args) == 1 and args[0] == 7 and "dtype" not in kw else 0)
        b = P.softmax_attention(h, w, m, 1e-6)
    finally:
        torch.arange = orig
    assert torch.allclose(a, b, rtol=1e-9, atol=1e-9)


def test_recurrence_by_hand():
    """One channel, one tap, gates fixed by their biases: S_t = a S_(t-1) + sqrt(1 - a^2) i u_t with a = exp(-8 r softplus(lam))."""
    r, i, lam = 0.25, 0.5, 0.3
    w = {"y": torch.zeros(1, 1), "y.b": torch.tensor([10.0]), "x": torch.ones(1, 1), "x.b": torch.zeros(1), "conv": torch.tensor([[2.0]]),
         "conv.b": torch.tensor([1.0]), "ra": torch.zeros(1, 1, 1), "ra.b": torch.tensor([[math.log(r / (1 - r))]]), "ri": torch.zeros(1, 1, 1),
         "ri.b": torch.tensor([[0.0]]), "lam": torch.tensor([lam]), "o": torch.ones(1, 1)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.tensor([[1.0], [-2.0], [0.5]], dtype=torch.float64)
    out = P.gated_recurrence(h, w, {"width": 1, "blocks": 1}, 1e-6)
    a = math.exp(-8.0 * r * math.log1p(math.exp(lam)))
    S, want = 0.0, []
    for x in (1.0, -2.0, 0.5):
        S = a * S + math.sqrt(1 - a * a) * i * (2.0 * x + 1.0)
        want.append(S * 10.0)            # gelu_tanh(10) = 10 to twelve digits
    assert torch.allclose(out.reshape(-1), torch.tensor(want, dtype=torch.float64), rtol=1e-6)   # (the biases above are float32 numbers)


def test_convolution_and_pair_table_by_hand():
    z = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    out = P.causal_conv(z, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert out.reshape(-1).tolist() == [1.5, 12.5, 123.5]
    long_taps = P.causal_conv(z[:2], torch.tensor([[1000.0, 100.0, 10.0, 1.0]], dtype=torch.float64), torch.zeros(1, dtype=torch.float64))
    assert long_taps.reshape(-1).tolist() == [1.0, 12.0]
    table = torch.arange(10, dtype=torch.float64).reshape(10, 1)
    pairs = 100.0 * torch.arange(6, dtype=torch.float64).reshape(6, 1)
    x = P.embed([3, 4, 4], table, pairs, {"bigram": {"buckets": 5, "mul_prev": 2, "mul_cur": 3}})
    assert x.reshape(-1).tolist() == [3.0 + 500.0, 4.0 + 100.0 * ((3 * 2 + 4 * 3) % 5), 4.0 + 100.0 * ((4 * 2 + 4 * 3) % 5)]


def test_experts_by_hand():
    w = {"router": torch.tensor([[1.0], [0.0], [-1.0]], dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.9], dtype=torch.float64)}
    chosen, weight = P.routing(torch.tensor([[2.0]], dtype=torch.float64), w, 2)
    # scores 0.881, 0.5, 0.119; with the correction the third (1.019) comes first and the first (0.881) second; weights stay scores
    assert chosen.tolist() == [[2, 0]]
    assert torch.allclose(weight, torch.sigmoid(torch.tensor([[-2.0, 2.0]], dtype=torch.float64)))


def test_dense_feed_forward_and_depth_average_by_hand():
    w = {"gate": torch.tensor([[1.0]]).double(), "up": torch.tensor([[1.0]]).double(), "down": torch.tensor([[1.0]]).double()}
    out = P.dense_ff(torch.tensor([[5.0], [-5.0], [0.5]], dtype=torch.float64), w, {"limit": 2.0})
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    want = [2.0 * sig(1.702 * 2.0) * 3.0, -5.0 * sig(1.702 * -5.0) * (-2.0 + 1.0), 0.5 * sig(1.702 * 0.5) * 1.5]
    assert torch.allclose(out.reshape(-1), torch.tensor(want, dtype=torch.float64), rtol=1e-12)
    # a model whose layers add nothing (gains of zero): every X_j is what its layer read, a multiple of the embedding's output
    cfg = tb.CONFIGS["rec"]
    t = tb.draw(cfg, 3)
    for n in list(t):
        if n.endswith(("norm1", "norm2")):
            t[n] = torch.zeros_like(t[n])
    streams = []
    P.forward(cfg, t, [1, 2, 3], layers_out=streams)
    x0 = P.embed([1, 2, 3], t["embed"].double(), t["bigram"].double(), cfg["embedding"])
    s0, s1 = t["l0.dwa"].double().sum(), t["l1.dwa"].double()
    assert torch.allclose(streams[0], s0 * x0, rtol=1e-12)
    # X_1 = X_0 (layer 0 read X_0 and added nothing), X_2 = the averaged stream that layer 1 read
    assert torch.allclose(streams[1], (s1[0] + s1[1] + s1[2] * s0) * x0, rtol=1e-12)
