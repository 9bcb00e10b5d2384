"""Pitolix without a GPU: the configuration reader, the plan the builder makes (the order the layers run in, which runs open
a pass of the loop, a norm weight nothing reads), and the plain implementation's own consistency (each mechanism written a
second way, by hand)."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_pitolix as P
import tiny_pitolix as tp
from xyntetik_runner_b200 import architectures  # noqa: F401
from xyntetik_runner_b200.config import registry
from xyntetik_runner_b200.config.base import ConfigError
from xyntetik_runner_b200.config.pitolix import PitolixConfig


@pytest.mark.parametrize("name", list(tp.CONFIGS))
def test_config_round_trip_and_tensor_names(name):
    cfg = PitolixConfig.from_dict(tp.CONFIGS[name])
    assert PitolixConfig.from_dict(cfg.to_dict()) == cfg
    plan = registry.resolve("Pitolix").build_plan(cfg)
    plan.validate()
    specs = {n: tuple(s.shape) for n, s in plan.tensor_specs().items() if not s.optional}
    assert specs == {n: tuple(s) for n, s in tp.shapes(tp.CONFIGS[name]).items()}
    # the order of the runs, and which of them open a pass (and which pass)
    runs = [(e.layer, e.before) for e in plan.schedule]
    assert runs == [(i, t if first else None) for i, t, first in P.layer_runs(tp.CONFIGS[name])]


def test_the_loop_unrolls_into_runs_with_a_cache_of_their_own():
    cfg = PitolixConfig.from_dict(tp.CONFIGS["mix"])
    assert [i for i, _ in cfg.layer_runs()] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [t for _, t in cfg.layer_runs()] == [None, 0, None, 1, None, 2, None, None]
    plan = registry.resolve("Pitolix").build_plan(cfg)
    assert len(plan.stream_parts) == 3 and [s.add_embedding for s in plan.stream_parts] == [False, True, True]
    assert [s.row for s in plan.stream_parts] == [0, 1, 2]
    # a loop of one pass still adds its vector; no loop adds nothing
    one = registry.resolve("Pitolix").build_plan(PitolixConfig.from_dict(tp.CONFIGS["odd"]))
    assert len(one.stream_parts) == 1 and not one.stream_parts[0].add_embedding
    none = registry.resolve("Pitolix").build_plan(PitolixConfig.from_dict(tp.CONFIGS["tc"]))
    assert not none.stream_parts and all(e.before is None for e in none.schedule)


def test_folder_is_resolved_by_its_architecture_key(tmp_path):
    path, cfg, _ = tp.make_folder(str(tmp_path / "m"), "loop")
    arch, typed = registry.load_config(path)
    assert arch.name == "Pitolix" and typed.width == cfg["width"] and len(typed.layers) == 2


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 26), "dims"),
    (lambda d: d["layers"][1]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
    (lambda d: d["layers"][1]["mixer"]["q_temp"].pop("coef"), "coef"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda d: d["loop"].__setitem__("stop", 99), "loop"),
    (lambda d: d["loop"].__setitem__("times", 0), "loop"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d.__setitem__("layers", []), "layers"),
])
def test_config_refusals(edit, word):
    d = copy.deepcopy(tp.CONFIGS["mix"])
    edit(d)
    with pytest.raises(ConfigError, match=word):
        PitolixConfig.from_dict(d)


def test_what_a_configuration_may_leave_out():
    d = copy.deepcopy(tp.CONFIGS["mix"])
    d["layers"][1]["mixer"].pop("q_temp")
    d["layers"][0]["mixer"].pop("rot")
    d.pop("loop")
    d.pop("embedding")
    cfg = PitolixConfig.from_dict(d)
    assert cfg.layers[1].mixer.q_temp is None and cfg.layers[0].mixer.rot_dims == 0 and cfg.loop is None
    assert cfg.embedding_scale == 1.0


def test_a_second_norm_weight_of_a_layer_without_feed_forward_may_be_there_or_not(tmp_path):
    from xyntetik_runner_b200.weights.loader import FolderSource, WeightsError, load_tensors
    cfg = tp.CONFIGS["odd"]
    plan = registry.resolve("Pitolix").build_plan(PitolixConfig.from_dict(cfg))
    specs = plan.tensor_specs()
    assert specs["l1.norm2"].optional and not specs["l0.norm2"].optional
    tensors = tp.draw(cfg, 3)
    path, _, _ = tp.make_folder(str(tmp_path / "without"), None, tensors, cfg)
    assert "l1.norm2" not in load_tensors(specs, FolderSource(path), torch.device("cpu"))
    tensors["l1.norm2"] = torch.zeros(cfg["width"], dtype=torch.bfloat16)
    path, _, _ = tp.make_folder(str(tmp_path / "with"), None, tensors, cfg)
    assert "l1.norm2" in load_tensors(specs, FolderSource(path), torch.device("cpu"))
    del tensors["l0.norm2"]
    path, _, _ = tp.make_folder(str(tmp_path / "lacking"), None, tensors, cfg)
    with pytest.raises(WeightsError, match="l0.norm2"):
        load_tensors(specs, FolderSource(path), torch.device("cpu"))


# ---- the plain implementation, each mechanism a second way ---------------------------------------------------------------
def test_query_factor_steps_where_it_should():
    pos = torch.arange(0, 40)
    f = P.query_temperature(pos, 0.5, 8, torch.float64)
    for p in range(40):
        assert abs(float(f[p]) - (1.0 + 0.5 * math.log((p + 1) // 8 + 1))) < 1e-14
    assert float(f[6]) == 1.0 and float(f[7]) > 1.0            # position 7 is the eighth token: the first step
    assert float(f[14]) == float(f[7]) and float(f[15]) > float(f[14])
    # a step at every position
    g = P.query_temperature(pos, 1.0, 1, torch.float64)
    assert abs(float(g[0]) - (1.0 + math.log(2.0))) < 1e-14 and abs(float(g[9]) - (1.0 + math.log(11.0))) < 1e-14


def test_rotation_by_hand():
    v = torch.arange(1.0, 13.0, dtype=torch.float64).view(1, 1, 12).repeat(3, 1, 1)
    pos = torch.tensor([0, 1, 5])
    out = P.rotate_half(v, pos, 6, 100.0)
    assert torch.equal(out[0], v[0]) and torch.equal(out[..., 6:], v[..., 6:])        # position 0 and the elements past `dims`
    for t, p in enumerate((0, 1, 5)):
        for i in range(3):
            a = p * 100.0 ** (-2.0 * i / 6)
            u, w = float(v[t, 0, i]), float(v[t, 0, i + 3])
            assert abs(float(out[t, 0, i]) - (u * math.cos(a) - w * math.sin(a))) < 1e-12
            assert abs(float(out[t, 0, i + 3]) - (w * math.cos(a) + u * math.sin(a))) < 1e-12
    assert torch.equal(P.rotate_half(v, pos, 0, 100.0), v)


def test_softmax_with_a_sink_by_hand():
    torch.manual_seed(0)
    s = torch.randn(2, 4, 4, dtype=torch.float64)
    sink = torch.tensor([0.3, -2.0], dtype=torch.float64)
    a = P.softmax_with_sink(s, P.causal_mask(4), sink)
    for h in range(2):
        for i in range(4):
            e = [math.exp(float(s[h, i, j])) for j in range(i + 1)]
            den = sum(e) + math.exp(float(sink[h]))
            for j in range(4):
                want = e[j] / den if j <= i else 0.0
                assert abs(float(a[h, i, j]) - want) < 1e-14
    # the weights of a row do not sum to one: the sink takes its share, the more the larger it is
    assert (a.sum(-1) < 1).all()
    big = P.softmax_with_sink(s, P.causal_mask(4), torch.tensor([30.0, 30.0], dtype=torch.float64))
    assert float(big.sum(-1).max()) < 1e-9
    plain = P.softmax_with_sink(s, P.causal_mask(4), None)
    assert torch.allclose(plain.sum(-1), torch.ones(2, 4, dtype=torch.float64))


def _mixer_weights(kind, H, G, D, V, W, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"q": r(H * D, W), "k": r(G * D, W), "v": r(G * V, W), "o": r(W, H * V)}
    if kind == "attention":
        w.update({"sink": r(H), "g": r(H * V, W)})
    else:
        w.update({"q.b": r(H * D), "k.b": r(G * D), "v.b": r(G * V), "g": r(H, W)})
    return w


def test_plain_sink_attention_as_a_loop_over_keys():
    H, G, D, V, W, T, eps = 4, 2, 6, 5, 10, 9, 1e-5
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.37, "q_temp": {"coef": 0.8, "every": 3}}
    w = _mixer_weights("attention", H, G, D, V, W, 1)
    h = torch.randn(T, W, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    got = P.attention_sink(h, w, m, eps)
    unit = lambda x: x / math.sqrt(float((x * x).mean()) + eps)
    for i in (0, 1, 2, 5, 8):
        heads = []
        for hd in range(H):
            kv = hd // (H // G)
            q = unit(w["q"][hd * D:(hd + 1) * D] @ h[i]) * (1.0 + 0.8 * math.log((i + 1) // 3 + 1))
            sc = [float(q @ unit(w["k"][kv * D:(kv + 1) * D] @ h[j])) * 0.37 for j in range(i + 1)]
            den = sum(math.exp(x) for x in sc) + math.exp(float(w["sink"][hd]))
            o = sum(math.exp(sc[j]) / den * (w["v"][kv * V:(kv + 1) * V] @ h[j]) for j in range(i + 1))
            heads.append(o * torch.sigmoid(w["g"][hd * V:(hd + 1) * V] @ h[i]))
        want = w["o"] @ torch.cat(heads)
        assert torch.allclose(got[i], want, rtol=1e-10, atol=1e-12)


def test_plain_rotary_attention_as_a_loop_over_keys():
    H, G, D, V, W, T = 3, 3, 8, 4, 10, 7
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.21, "rot": {"base": 30.0, "dims": 4}}
    w = _mixer_weights("attention_2", H, G, D, V, W, 3)
    h = torch.randn(T, W, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    got = P.attention_rotary(h, w, m, 1e-5)

    def turn(v, p):
        out = v.clone()
        for i in range(2):
            a = p * 30.0 ** (-2.0 * i / 4)
            out[i] = v[i] * math.cos(a) - v[i + 2] * math.sin(a)
            out[i + 2] = v[i + 2] * math.cos(a) + v[i] * math.sin(a)
        return out
    for i in (0, 3, 6):
        heads = []
        for hd in range(H):
            q = turn(w["q"][hd * D:(hd + 1) * D] @ h[i] + w["q.b"][hd * D:(hd + 1) * D], i)
            sc = torch.stack([q @ turn(w["k"][hd * D:(hd + 1) * D] @ h[j] + w["k.b"][hd * D:(hd + 1) * D], j) for j in range(i + 1)]) * 0.21
            a = torch.softmax(sc, 0)
            o = sum(a[j] * (w["v"][hd * V:(hd + 1) * V] @ h[j] + w["v.b"][hd * V:(hd + 1) * V]) for j in range(i + 1))
            heads.append(o * torch.sigmoid(w["g"][hd] @ h[i]))
        assert torch.allclose(got[i], w["o"] @ torch.cat(heads), rtol=1e-10, atol=1e-12)


def test_plain_layer_and_loop_by_hand():
    """Both sublayers read the stream as it enters the layer; the passes of the loop add the embedding's output (not the first)
    and their vector."""
    cfg = tp.CONFIGS["loop"]
    t = {k: v.double() for k, v in tp.draw(cfg, 7).items()}
    toks = [3, 9, 27, 81 % cfg["vocab"], 5]
    outs = []
    got = P.forward(cfg, t, toks, layers_out=outs)
    eps = cfg["norm"]["eps"]
    x0 = t["embed"][toks] * cfg["embedding"]["scale"]
    x = x0
    k = 0
    for pass_no in range(2):
        if pass_no:
            x = x + x0
        x = x + t["loop.step"][pass_no]
        for i, lay in enumerate(cfg["layers"]):
            sub = {n[len(f"l{i}.mix."):]: v for n, v in t.items() if n.startswith(f"l{i}.mix.")}
            ff = {n[len(f"l{i}.mlp."):]: v for n, v in t.items() if n.startswith(f"l{i}.mlp.")}
            a = P.MIXERS[lay["type"]](P.norm_one_plus(x, t[f"l{i}.norm1"], eps), sub, lay["mixer"], eps)
            b = P.dense_ff(P.norm_one_plus(x, t[f"l{i}.norm2"], eps), ff)
            x = x + a + b
            assert torch.allclose(outs[k], x, rtol=1e-12, atol=1e-12)
            k += 1
    assert k == len(outs) == 4
    want = (x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1 + t["final.norm"])) @ t["head"].T
    assert torch.allclose(got, want, rtol=1e-12, atol=1e-12)


def test_plain_prefix_does_not_depend_on_what_follows():
    cfg = tp.CONFIGS["mix"]
    t = tp.draw(cfg, 9)
    toks = [int(x) for x in np.random.RandomState(0).randint(0, cfg["vocab"], size=30)]
    whole = tp.plain_logits(cfg, t, toks)
    assert np.allclose(tp.plain_logits(cfg, t, toks[:11]), whole[:11], rtol=1e-6, atol=1e-6)
