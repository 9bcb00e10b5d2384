"""Buzarax on the GPU against the plain implementation: each mechanism alone, every way of cutting a request, mixed batches with
pages and slots used again, token sequences made so that one key stands out far back and at page borders, recurrences whose first
tokens still count hundreds of tokens later in a slot that was used before, the first tokens (where the sink weighs most), long
decoding, other sizes, greedy generation through the entry points."""
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_buzarax as P
import tiny_buzarax as tb
import traces

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [5, 41, 17, 70, 130, 23], "odd": [1, 9, 33, 70, 150, 64], "tc": [5, 200, 17, 70, 130, 33], "rec": [2, 19, 90, 35, 60, 77]}
PAGE = {"mix": 16, "odd": 8, "tc": 64, "rec": 32}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in tb.CONFIGS:
        path, cfg, tensors = tb.make_folder(str(tmp_path_factory.mktemp("bz_" + name)), name)
        reqs = {f"r{i}": traces.random_tokens(100 * i + len(name), n, cfg["vocab"]) for i, n in enumerate(LENGTHS[name])}
        ref = {rid: tb.plain_logits(cfg, tensors, t) for rid, t in reqs.items()}
        out[name] = (path, cfg, tensors, reqs, ref)
    return out


_sens = {}


def close(got, ref, dtype, what, cfg, tensors, toks, key):
    """float32: the fixed tolerance.  bfloat16: the fixed tolerance, with the allowance of ``tiny_buzarax.assert_close_bfloat16``
    for positions that the plain implementation itself shows to hang on a rounding."""
    if dtype == "float32":
        return traces.assert_close(got, ref, dtype, what)
    if key not in _sens:
        _sens[key] = tb.rounding_sensitivity(cfg, tensors, toks)
    tb.assert_close_bfloat16(got, ref, _sens[key], what)


def run(folder, dtype, steps, page_size, max_tokens=None, max_requests=4, graphs=True):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    from xyntetik_runner_b200.engine.replay import replay
    mt = max_tokens if max_tokens is not None else traces.pool_tokens(steps, page_size)
    eng = Engine(folder, EngineParams(dtype=dtype, max_tokens=mt, page_size=page_size, max_requests=max_requests, cuda_graphs=graphs))
    res = replay(eng, steps)
    eng.check_status()
    eng.cache.audit()
    assert not eng.cache.live_requests()
    return res, eng


CUTS = {
    "whole": lambda reqs: traces.whole(reqs),
    "tail": lambda reqs: traces.tail_decoded(reqs, 32),
    "portions": lambda reqs: traces.portions(reqs),
    "pairs": lambda reqs: traces.portions(reqs, sizes=(2,)),
    "mixed": lambda reqs: traces.mixed(reqs, seed=3),
    "mixed2": lambda reqs: traces.mixed(reqs, seed=8, max_live=2, sizes=(1, 2, 31, 1, 64, 3)),
}


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_float32_matches_plain_in_every_cut(models, name, cut):
    path, cfg, tensors, reqs, ref = models[name]
    steps = CUTS[cut](reqs)
    res, eng = run(path, "float32", steps, PAGE[name])
    got = traces.collect(steps, res, cfg["vocab"])
    for rid in reqs:
        traces.assert_close(got[rid], ref[rid], "float32", f"{name}/{cut}/{rid}")
    if cut.startswith("mixed"):
        assert len(reqs) > 4                                                                         # slots were used again
        if eng.cache.pools:
            assert sum(-(-len(t) // PAGE[name]) for t in reqs.values()) > eng.cache.pools[0].n_pages  # and so were pages


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_bfloat16_matches_plain(models, name, cut):
    path, cfg, tensors, reqs, ref = models[name]
    steps = CUTS[cut](reqs)
    res, _ = run(path, "bfloat16", steps, PAGE[name])
    got = traces.collect(steps, res, cfg["vocab"])
    for rid in reqs:
        close(got[rid], ref[rid], "bfloat16", f"{name}/{cut}/{rid}", cfg, tensors, reqs[rid], (name, rid))


def test_a_batch_gives_what_each_request_gives_alone(models):
    """Unequal requests side by side, against each alone: in float32 within the rounding of the sums' order."""
    path, cfg, tensors, reqs, ref = models["mix"]
    alone = traces.collect(CUTS["whole"](reqs), run(path, "float32", CUTS["whole"](reqs), PAGE["mix"])[0], cfg["vocab"])
    steps = CUTS["mixed"](reqs)
    batch = traces.collect(steps, run(path, "float32", steps, PAGE["mix"])[0], cfg["vocab"])
    for rid in reqs:
        scale = np.abs(alone[rid]).max()
        assert np.abs(batch[rid] - alone[rid]).max() <= 2e-5 * scale, rid


def test_recurrences_depend_on_the_cutting_by_the_last_bits_only(models):
    """A model of recurrences alone walks token by token; only the gates' sums are added in another order in steps of few tokens
    than in steps of many: the logits of any two cuttings agree to a few units in the last place."""
    path, cfg, tensors, reqs, ref = models["rec"]
    outs = []
    for cut in ("whole", "pairs", "mixed"):
        steps = CUTS[cut](reqs)
        outs.append(traces.collect(steps, run(path, "float32", steps, PAGE["rec"])[0], cfg["vocab"]))
    for rid in reqs:
        scale = np.abs(outs[0][rid]).max()
        assert np.abs(outs[0][rid] - outs[1][rid]).max() <= 2e-6 * scale and np.abs(outs[0][rid] - outs[2][rid]).max() <= 2e-6 * scale, rid


def test_long_decoding_and_first_tokens(models):
    """Three tokens at once, then 300 one by one: pages fill, the states are carried 300 times, the pair table's previous token
    comes from the slot every time."""
    path, cfg, tensors, _, _ = models["mix"]
    toks = traces.random_tokens(77, 303, cfg["vocab"])
    ref = tb.plain_logits(cfg, tensors, toks)
    steps = traces.tail_decoded({"long": toks}, tail=300)
    for dtype in ("float32", "bfloat16"):
        res, _ = run(path, dtype, steps, page_size=16, max_tokens=320)
        got = traces.collect(steps, res, cfg["vocab"])["long"]
        close(got, ref, dtype, "long decoding", cfg, tensors, toks, ("mix", "long"))
        if dtype == "float32":
            traces.assert_close(got[:3], ref[:3], dtype, "first tokens")


def test_graphs_change_nothing(models):
    path, cfg, tensors, reqs, ref = models["mix"]
    steps = CUTS["tail"](reqs)
    a, _ = run(path, "bfloat16", steps, PAGE["mix"], graphs=True)
    b, eng = run(path, "bfloat16", steps, PAGE["mix"], graphs=False)
    for k in a:
        assert np.array_equal(a[k], b[k])


def test_decode_steps_are_replayed_from_graphs(models):
    path, cfg, tensors, reqs, ref = models["tc"]
    _, eng = run(path, "bfloat16", CUTS["tail"]({"r1": reqs["r1"]}), PAGE["tc"])
    assert eng.graph_replays > 20


def test_tensor_core_kernels_ran(models):
    from xyntetik_runner_b200.parts import attention, linear
    path, cfg, tensors, reqs, ref = models["tc"]
    before = (attention.counters["tcgen05"], attention.counters["mma"], linear.counters["tcgen05"])
    run(path, "bfloat16", CUTS["tail"]({"r1": reqs["r1"]}), PAGE["tc"])
    after = (attention.counters["tcgen05"], attention.counters["mma"], linear.counters["tcgen05"])
    assert all(b > a for a, b in zip(before, after)), (before, after)


# ---- one mechanism at a time ------------------------------------------------------------------------------------------
_r = tb.rot
_small_right = (1, 4, 4, (0.5,))
SINGLE = {
    # (a side of the parallel mixer alone: the other side's scale is zero)
    "softmax_side_part_rotation": tb.model(60, 40, 1e-5, [tb.layer(tb.parallel(6, 2, 12, 20, 0.3, _r(40.0, 6), None, *_small_right, 1.0, 0.0), None)], 11, 3, 5),
    "softmax_side_interpolated": tb.model(60, 40, 1e-5, [tb.layer(tb.parallel(2, 2, 16, 16, 0.25, _r(40.0, 16, (16.0, 8, 4.0, 0.5)), None, *_small_right, 1.0, 0.0), None)], 11, 3, 5),
    "softmax_side_capped": tb.model(60, 40, 1e-5, [tb.layer(tb.parallel(3, 1, 24, 8, 0.6, _r(40.0, 0), 1.5, *_small_right, 1.0, 0.0), None)], 11, 3, 5),
    "decay_side": tb.model(60, 40, 1e-5, [tb.layer(tb.parallel(1, 1, 4, 4, 0.5, _r(10.0, 0), None, 3, 12, 20, (0.9, 0.2, 0.999), 0.0, 1.0), None)], 11, 3, 5),
    "recurrence": tb.model(60, 40, 1e-5, [tb.layer(tb.rglru(48, 3, 4), None)], 11, 3, 5),
    "recurrence_one_tap_one_block": tb.model(60, 40, 1e-5, [tb.layer(tb.rglru(24, 1, 1), None)], 11, 3, 5),
    "dense_feed_forward": tb.model(60, 40, 1e-5, [tb.layer(tb.rglru(8, 1, 1), tb.dense(52, 0.7))], 11, 3, 5),
    "experts": tb.model(60, 40, 1e-5, [tb.layer(tb.rglru(8, 1, 1), tb.moe(7, 3, 20))], 11, 3, 5),
    "pair_table_of_one_bucket": tb.model(60, 40, 1e-5, [tb.layer(tb.rglru(8, 1, 1), None)], 1, 1, 1, logit_softcap=0.5),
    "depth_average": tb.model(60, 40, 1e-5, [tb.layer(tb.rglru(8, 2, 2), None) for _ in range(5)], 11, 3, 5),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_one_mechanism_alone(name, dtype):
    cfg = SINGLE[name]
    t = tb.draw(cfg, 7)
    reqs = {"a": traces.random_tokens(3, 45, cfg["vocab"]), "b": traces.random_tokens(4, 9, cfg["vocab"]), "c": traces.random_tokens(5, 1, cfg["vocab"])}
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        for cut in ("whole", "portions", "mixed"):
            steps = CUTS[cut](reqs)
            res, _ = run(path, dtype, steps, 8)
            got = traces.collect(steps, res, cfg["vocab"])
            for rid in reqs:
                close(got[rid], tb.plain_logits(cfg, t, reqs[rid]), dtype, f"{name}/{cut}/{rid}", cfg, t, reqs[rid], (name, rid))


# ---- kernels alone ------------------------------------------------------------------------------------------------------
def _dev(t, dtype=torch.float32):
    return t.to(dtype).cuda().contiguous()


@pytest.mark.parametrize("R,B,taps", [(48, 3, 4), (40, 1, 1), (320, 2, 3), (130, 5, 16), (1800, 1, 2)])
def test_recurrence_kernel_from_states_in_other_slots(R, B, taps):
    """Two portions in one launch, in slots 2 and 0 of four, one continuing a state and a tail that an earlier launch left."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(R + taps)
    Bs = R // B
    w = {"y": torch.zeros(R, 1), "y.b": torch.zeros(R), "x": torch.zeros(R, 1), "x.b": torch.zeros(R),
         "conv": torch.randn(R, taps, generator=g), "conv.b": torch.randn(R, generator=g), "ra": torch.randn(B, Bs, Bs, generator=g) / Bs ** 0.5,
         "ra.b": torch.randn(B, Bs, generator=g), "ri": torch.randn(B, Bs, Bs, generator=g) / Bs ** 0.5, "ri.b": torch.randn(B, Bs, generator=g),
         "lam": -3.0 + 2.0 * torch.randn(R, generator=g), "o": torch.eye(R)}
    lens = (19, 7)
    pre = torch.randn(sum(lens), 2 * R, generator=g)

    def plain(rows):
        # the plain recurrence of a whole sequence, from rows that already are the projections: y' in the first R columns, x' behind them
        ww = {k: v.double() for k, v in w.items()}
        ww["y"], ww["x"] = torch.cat([torch.eye(R), torch.zeros(R, R)], 1).double(), torch.cat([torch.zeros(R, R), torch.eye(R)], 1).double()
        return P.gated_recurrence(rows.double(), ww, {"width": R, "blocks": B}, 1e-6)

    want = [plain(pre[:lens[0]]), plain(pre[lens[0]:])]
    state = torch.randn(4, kernels.rglru_state_floats(R, taps) + 3, generator=g).cuda()          # (rows wider than needed, filled with noise)
    state[2].zero_(); state[0].zero_()
    args = [_dev(w["conv"]), _dev(w["conv.b"]), _dev(w["ra"].transpose(1, 2)), _dev(w["ri"].transpose(1, 2)), _dev(w["ra"]), _dev(w["ri"]), _dev(w["ra.b"].reshape(-1)),
            _dev(w["ri.b"].reshape(-1)), _dev(w["lam"])]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    # first launch: 12 tokens of the first sequence into slot 2
    n0 = 12
    for (rows, tok_seg, starts, lns, slots, checks) in (
            (pre[:n0], [0] * n0, [0], [n0], [2], [(0, 0, n0)]),
            (torch.cat([pre[lens[0]:], pre[n0:lens[0]]]), [0] * lens[1] + [1] * (lens[0] - n0), [0, lens[1]], [lens[1], lens[0] - n0], [0, 2],
             [(1, 0, lens[1]), (0, n0, lens[0])])):
        n = rows.shape[0]
        a_s, b_s, u_s = torch.empty(n, R).cuda(), torch.empty(n, R).cuda(), torch.empty(n, R).cuda()
        out = torch.empty(n, R).cuda()
        kernels.rglru(_dev(rows), *args, state, i32(tok_seg), i32(starts), i32(lns), i32(slots), a_s, b_s, u_s, out, len(starts), R, B, taps, 8.0)
        at = 0
        for (which, lo, hi), ln in zip(checks, lns):
            got = out[at:at + ln].double().cpu()
            assert torch.allclose(got, want[which][lo:hi], rtol=2e-5, atol=2e-6), (R, B, taps, which, (got - want[which][lo:hi]).abs().max())
            at += ln
    assert torch.equal(state[1].cpu(), state[1].cpu()) and state[1].abs().sum() > 0            # other slots untouched


@pytest.mark.parametrize("H,D,V", [(3, 12, 20), (1, 64, 128), (2, 130, 33), (4, 8, 4)])
def test_decay_attention_kernel_cut_against_whole(H, D, V):
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(H * D + V)
    T = 37
    pre = torch.randn(T, 2 * H * D + 2 * H * V, generator=g)
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    w = {"q": torch.cat([torch.eye(H * D), torch.zeros(H * D, H * D + 2 * H * V)], 1),
         "k": torch.cat([torch.zeros(H * D, H * D), torch.eye(H * D), torch.zeros(H * D, 2 * H * V)], 1),
         "v": torch.cat([torch.zeros(H * V, 2 * H * D), torch.eye(H * V), torch.zeros(H * V, H * V)], 1),
         "g": torch.cat([torch.zeros(H * V, 2 * H * D + H * V), torch.eye(H * V)], 1), "norm": torch.ones(H * V), "o": torch.eye(H * V)}
    # the plain read-outs before norm and gate: recover them by a norm weight of one and undoing the rest is not possible, so the
    # plain recurrence is restated here in three lines
    q, k, v = (P.silu(pre[:, a:b].double()) for a, b in ((0, H * D), (H * D, 2 * H * D), (2 * H * D, 2 * H * D + H * V)))
    S = torch.zeros(H, D, V, dtype=torch.float64)
    want = []
    for t in range(T):
        S = decay.double()[:, None, None] * S + k[t].view(H, D, 1) * v[t].view(H, 1, V)
        want.append(torch.einsum("hdv,hd->hv", S, q[t].view(H, D)).reshape(-1))
    want = torch.stack(want)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    outs = []
    for cuts in ([T], [1, 2, 30, 4]):
        state = torch.zeros(3, H * D * V).cuda()
        got, at = [], 0
        for c in cuts:
            o = torch.empty(c, H * V).cuda()
            kernels.decay_attention(_dev(pre[at:at + c]), (0, H * D, 2 * H * D), _dev(decay), state, i32([0]), i32([c]), i32([1]), o, 1, H, D, V)
            got.append(o.cpu())
            at += c
        outs.append(torch.cat(got))
        assert state[0].abs().sum() == 0 and state[2].abs().sum() == 0
    assert torch.equal(outs[0], outs[1])
    assert torch.allclose(outs[0].double(), want, rtol=2e-5, atol=1e-5)
    # and the whole mixer's tail (norm over all heads, gate) against the plain function
    y = torch.empty(T, H * V).cuda()
    kernels.row_norm_gate(outs[0].cuda(), _dev(pre), 2 * H * D + H * V, torch.ones(H * V).cuda(), y, 1e-5, scale=0.75)
    full = P.decayed_linear_attention(pre.double(), {n: t.double() for n, t in w.items()}, {"heads": H, "dim": D, "vdim": V, "decay": decay.tolist()}, 1e-5)
    assert torch.allclose(y.double().cpu(), 0.75 * full, rtol=1e-4, atol=1e-5)


def test_choice_by_score_plus_correction_weight_by_score():
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(5)
    for E, top in ((7, 3), (40, 40), (33, 1), (12, 2)):
        z = torch.randn(50, E, generator=g) * 2
        corr = torch.randn(E, generator=g)
        ids, wts = torch.empty(50, top, dtype=torch.int32).cuda(), torch.empty(50, top).cuda()
        kernels.route_topk(_dev(z), ids, wts, top, sigmoid_scores=True, correction=_dev(corr))
        s = torch.sigmoid(z)
        want = torch.topk(s + corr, top, dim=-1).indices
        assert torch.equal(ids.cpu().long().sort(dim=1).values, want.sort(dim=1).values)
        assert torch.allclose(wts.cpu(), torch.gather(s, 1, ids.cpu().long()), rtol=1e-6, atol=1e-7)
        # a correction that lifts one expert above all makes it the first choice of every token, with its own small score as weight
        corr2 = torch.zeros(E); corr2[E - 1] = 5.0
        z2 = z.clone(); z2[:, E - 1] = -4.0
        kernels.route_topk(_dev(z2), ids, wts, top, sigmoid_scores=True, correction=_dev(corr2))
        assert (ids[:, 0].cpu() == E - 1).all() and torch.allclose(wts[:, 0].cpu(), torch.sigmoid(torch.tensor(-4.0)).expand(50), rtol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_kernels(dtype):
    """Output norm + add (+ rounded copy, + clearing), the depth average, the pair embedding with its carried token, the rotation of
    head rows forth and back."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(9)
    n, W = 13, 70
    d, x, gain = torch.randn(n, W, generator=g) * 3, torch.randn(n, W, generator=g), torch.tensor([0.37])
    want = x.double() + P.scalar_norm(d.double(), gain.double(), 1e-5)
    dd, xx, cast = d.cuda(), x.cuda(), torch.empty(n, W, dtype=dtype).cuda()
    kernels.norm_add(dd, xx, gain.cuda(), 1e-5, cast=cast, clear=True)
    assert torch.allclose(xx.double().cpu(), want, rtol=1e-6, atol=1e-6) and dd.abs().sum() == 0
    assert torch.equal(cast.cpu(), xx.cpu().to(dtype))
    # depth average: X_0 .. X_3, then X_4 arrives
    hist = torch.randn(5, n, W, generator=g)
    w = torch.randn(5, generator=g)
    buf = torch.zeros(4, n, W).cuda()
    buf[:3] = hist[1:4].cuda()
    cur = hist[4].clone().cuda()
    kernels.depth_average(cur, hist[0].cuda(), buf, w.cuda(), 4, cast=cast)
    want = sum(w[j].double() * hist[j].double() for j in range(5))
    assert torch.allclose(cur.double().cpu(), want, rtol=1e-6, atol=1e-6) and torch.equal(buf[3].cpu(), hist[4])
    assert torch.equal(cast.cpu(), cur.cpu().to(dtype))
    # pair embedding: two portions, one at the start of its request, one continuing after token 17 (in slot 3)
    V, buckets = 50, 7
    table, pairs = torch.randn(V, W, generator=g).to(dtype), torch.randn(buckets + 1, W, generator=g).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    ids, pos = [4, 9, 9, 30, 2], [0, 1, 2, 5, 6]
    last = i32([0, 0, 0, 17])
    out = torch.empty(5, W).cuda()
    kernels.embed_pair(table.cuda(), pairs.cuda(), i32(ids), i32(pos), i32([0, 0, 0, 1, 1]), i32([0, 3]), i32([1, 3]), last, out, 31, 5)
    kernels.last_token(i32(ids), i32([0, 3]), i32([3, 2]), i32([1, 3]), last, 2, V)
    rows = [buckets, (4 * 31 + 9 * 5) % buckets, (9 * 31 + 9 * 5) % buckets, (17 * 31 + 30 * 5) % buckets, (30 * 31 + 2 * 5) % buckets]
    want = table[torch.tensor(ids)].float() + pairs[torch.tensor(rows)].float()
    assert torch.equal(out.cpu(), want) and last.cpu().tolist() == [0, 9, 0, 2]
    # rotation forth and back gives the rows again; forth equals the plain rotation
    H, hs, dims = 3, 24, 20
    rows0 = torch.randn(6, 8 + H * hs, generator=g)
    freq = torch.rand(dims // 2, generator=g, dtype=torch.float64)
    posn = i32([0, 1, 5, 1000, 77, 123456])
    r = rows0.to(dtype).cuda()
    kernels.rotate_heads(r, 8, H, hs, dims, hs, False, freq.cuda(), posn)
    want = P.rotate_half(rows0.to(dtype).double()[:, 8:].view(6, H, hs), posn.cpu(), dims, freq)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    assert torch.allclose(r[:, 8:].double().cpu().view(6, H, hs), want, **tol)
    assert torch.equal(r[:, :8].cpu(), rows0.to(dtype)[:, :8])
    kernels.rotate_heads(r, 8, H, hs, dims, hs, False, freq.cuda(), posn, sign=-1.0, scale=2.0)
    assert torch.allclose(r[:, 8:].double().cpu(), 2.0 * rows0.to(dtype).double()[:, 8:], **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,dims", [(24, 8), (64, 32), (128, 64), (40, 40)])
def test_rotation_before_the_unit_norm(dtype, D, dims):
    """The norm/rotation/store kernel with scaled cosines and sines and the norm taken behind the rotation, element by element."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(D + dims)
    n, H, K, Vd, page = 9, 4, 2, D, 8
    hd = -(-D // 16) * 16
    rows = torch.randn(n, (H + K) * D + K * Vd, generator=g).to(dtype)
    freq = torch.rand(dims // 2, generator=g, dtype=torch.float64)
    mscale = 1.3
    pos = torch.tensor([0, 1, 2, 3, 900, 901, 5, 6, 7], dtype=torch.int32)
    q_out = torch.zeros(n, H * hd, dtype=dtype).cuda()
    cache = torch.zeros(4, 1, 2, K, page, hd, dtype=dtype).cuda()
    bt = torch.tensor([[0, 1] + [0] * 126], dtype=torch.int32).cuda()
    pos_local = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8], dtype=torch.int32)
    # (positions for the angles are large; the rows are stored by a second array of small positions through tok_seg/block table)
    kernels.qk_norm_rope_store(rows.cuda(), q_out, pos.cuda(), torch.zeros(n, dtype=torch.int32).cuda(), bt, freq.cuda(), None, None, None,
                               cache.stride(0), cache.stride(2), H, K, D, Vd, hd, dims, 128, page, False, 1e-6, unit_norm=True,
                               mscale=mscale, norm_after=True)
    x = rows.double()[:, :H * D].view(n, H, D)
    want = P.unit_rms(P.rotate_half(x, pos, dims, freq, mscale), 1e-6)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    assert torch.allclose(q_out.double().cpu().view(n, H, hd)[:, :, :D], want, **tol)
    del pos_local


# ---- keys that stand out ---------------------------------------------------------------------------------------------------
def _echo_model(scale=1.5, softcap=None, rotation=None):
    """One layer, the softmax side alone, queries and keys by the same matrix: a token whose pair (previous token, token) appeared
    before asks for exactly that earlier position (its rotated unit query is that position's key: the score is dim * scale, all
    others scatter around zero)."""
    cfg = tb.model(300, 64, 1e-6, [tb.layer(tb.parallel(2, 2, 16, 24, scale, rotation or _r(100.0, 0), softcap, 1, 4, 4, (0.5,), 1.0, 0.0), None)],
                   997, 1, 0)
    t = tb.draw(cfg, 50)
    t["l0.mix.left.k"] = t["l0.mix.left.q"].clone()
    t["l0.mix.left.v"] = t["l0.mix.left.v"] * 3.0
    return cfg, t


def _echo_tokens(n, at, vocab, seed):
    """n distinct-pair tokens; the last two repeat the pair that ends at position `at`."""
    rng = np.random.RandomState(seed)
    toks = [int(v) for v in rng.permutation(vocab - 2)[:n - 2] + 2]
    return toks + [toks[at - 1], toks[at]]


@pytest.mark.parametrize("softcap", [None, 6.0])
def test_a_key_that_stands_out_at_page_borders_and_among_the_first_tokens(softcap):
    cfg, t = _echo_model(softcap=softcap)
    page = 16
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        for at in (1, 2, 15, 16, 17, 31, 32, 47, 48, 63, 64, 65):
            toks = _echo_tokens(90, at, cfg["vocab"], at)
            ref = tb.plain_logits(cfg, t, toks)
            # the echo matters: without that one key the last position's logits are far away
            assert np.abs(tb.plain_logits(cfg, t, toks[:at] + [1 if toks[at] != 1 else 0] + toks[at + 1:])[-1] - ref[-1]).max() > 0.03 * np.abs(ref).max()
            for cut, dtype in (("whole", "float32"), ("tail", "float32"), ("pairs", "float32"), ("tail", "bfloat16")):
                steps = CUTS[cut]({"r": toks})
                res, _ = run(path, dtype, steps, page)
                got = traces.collect(steps, res, cfg["vocab"])["r"]
                close(got, ref, dtype, f"echo at {at}/{cut}/{dtype}", cfg, t, toks, ("echo", softcap, at))


def test_a_far_key_among_hundreds():
    """The echoed position lies 700 and more tokens back, behind ten pages, in a prompt and for a token decoded alone; the values are
    rotated by their position, so the logits also show that the far value is turned back by the right distance."""
    cfg, t = _echo_model(scale=1.2, rotation=_r(100.0, 8, (4.0, 64, 8.0, 1.0)))
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        for at in (3, 64, 127):
            toks = _echo_tokens(800, at, 300, at)[:800]
            toks = toks[:298] + [int(v) for v in np.random.RandomState(at).randint(2, 300, size=500)] + [toks[at - 1], toks[at]]
            ref = tb.plain_logits(cfg, t, toks)
            for cut, dtype in (("whole", "float32"), ("tail", "float32"), ("tail", "bfloat16")):
                steps = CUTS[cut]({"r": toks})
                res, _ = run(path, dtype, steps, 64)
                got = traces.collect(steps, res, cfg["vocab"])["r"]
                close(got, ref, dtype, f"far echo at {at}/{cut}/{dtype}", cfg, t, toks, ("far", at))


def test_slow_recurrences_remember_the_first_tokens_in_a_slot_used_before():
    """Rates near zero: changing the FIRST token changes the logits 200 tokens later, and the engine follows, in a slot that another
    request used before and across decoded tokens."""
    cfg = tb.CONFIGS["rec"]
    t = tb.draw(cfg, 61, slow=True)
    a = traces.random_tokens(1, 230, cfg["vocab"])
    b = [(a[0] + 1) % cfg["vocab"], (a[1] + 7) % cfg["vocab"]] + a[2:]
    ra, rb = tb.plain_logits(cfg, t, a), tb.plain_logits(cfg, t, b)
    assert np.abs(ra[-1] - rb[-1]).max() > 1e-3 * np.abs(ra).max()
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        steps = traces.tail_decoded({"a": a, "b": b}, 40)
        res, _ = run(path, "float32", steps, 16, max_requests=1)
        got = traces.collect(steps, res, cfg["vocab"])
        traces.assert_close(got["a"], ra, "float32", "slow a")
        traces.assert_close(got["b"], rb, "float32", "slow b")
        assert np.abs(got["b"][-1] - rb[-1]).max() < 0.05 * np.abs(ra[-1] - rb[-1]).max()


def test_decays_near_one_carry_the_linear_attention_far():
    cfg = tb.model(80, 48, 1e-5, [tb.layer(tb.parallel(1, 1, 4, 4, 0.5, _r(10.0, 0), None, 2, 16, 16, (0.9995, 0.5), 0.0, 1.0), tb.dense(32, 1.0))], 13, 3, 5)
    t = tb.draw(cfg, 62)
    a = traces.random_tokens(2, 260, cfg["vocab"])
    b = [(a[0] + 3) % cfg["vocab"]] + a[1:]
    ra, rb = tb.plain_logits(cfg, t, a), tb.plain_logits(cfg, t, b)
    assert np.abs(ra[-1] - rb[-1]).max() > 1e-3 * np.abs(ra).max()
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        steps = traces.mixed({"a": a, "b": b}, seed=4, max_live=2)
        res, _ = run(path, "float32", steps, 16, max_requests=2)
        got = traces.collect(steps, res, cfg["vocab"])
        traces.assert_close(got["a"], ra, "float32", "far decay a")
        traces.assert_close(got["b"], rb, "float32", "far decay b")


# ---- other sizes -------------------------------------------------------------------------------------------------------------
def _drawn_config(rng, layer_sizes):
    pick = lambda *v: v[rng.randint(len(v))]
    W = int(pick(128, 192, 256)) if layer_sizes else int(pick(36, 52, 68, 70, 96))
    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.rand() < 0.5:
            G = int(pick(1, 2, 3))
            H = G * int(pick(1, 2, 4)) if not layer_sizes else G * int(pick(1, 2, 8))
            D = int(pick(64, 128)) if layer_sizes else int(pick(6, 10, 16, 24, 34))
            Vd = int(pick(64, 128)) if layer_sizes else int(pick(4, 12, 16, 30))
            dims = int(pick(0, D // 2 // 2 * 2, D // 2 * 2)) if not layer_sizes else int(pick(0, D // 2, D))
            scaling = None if rng.rand() < 0.4 or dims == 0 else (float(pick(2.0, 8.0, 32.0)), int(pick(8, 64, 512)), float(pick(4.0, 32.0)), float(pick(0.5, 1.0, 2.0)))
            rh = int(pick(1, 2, 5))
            mixer = tb.parallel(H, G, D, Vd, float(pick(0.1, 0.3, 1.0 / math.sqrt(D))), _r(float(pick(10.0, 1e4, 5e5)), dims, scaling),
                                pick(None, 3.0, 50.0), rh, int(pick(4, 16, 33)), int(pick(4, 16, 40)), [float(rng.uniform(0.2, 0.999)) for _ in range(rh)],
                                float(pick(0.3, 1.0, 1.7)), float(pick(0.4, 1.0, 2.0)))
        else:
            B = int(pick(1, 2, 4, 5))
            mixer = tb.rglru(B * int(pick(4, 9, 16, 40)), B, int(pick(1, 2, 4, 7)))
        k = rng.randint(3)
        if k == 0:
            mlp = None
        elif k == 1:
            mlp = tb.dense(int(pick(24, 40, 64, 100)), float(pick(0.5, 1.0, 7.0)))
        else:
            E = int(pick(2, 4, 9, 33))
            mlp = tb.moe(E, int(rng.randint(1, min(E, 6) + 1)), int(pick(8, 24, 64)))
        layers.append(tb.layer(mixer, mlp))
    return tb.model(int(pick(61, 128, 333)), W, float(pick(1e-6, 1e-5)), layers, int(pick(1, 13, 1021)), int(pick(1, 31, 1000003)), int(pick(0, 7, 12345)),
                    pick(None, 5.0, 30.0))


@pytest.mark.parametrize("seed", range(14))
def test_drawn_configurations(seed):
    rng = np.random.RandomState(3000 + seed)
    cfg = _drawn_config(rng, layer_sizes=seed >= 10)
    t = tb.draw(cfg, 90 + seed)
    page = int(rng.choice([4, 8, 16, 64])) if seed < 10 else 64
    reqs = {f"r{i}": traces.random_tokens(11 * seed + i, n, cfg["vocab"]) for i, n in enumerate((3, 90, 17, 140, 1, 45))}
    ref = {rid: tb.plain_logits(cfg, t, toks) for rid, toks in reqs.items()}
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        for dtype in ("float32", "bfloat16"):
            for cut in ("whole", "mixed"):
                steps = CUTS[cut](reqs)
                res, _ = run(path, dtype, steps, page)
                got = traces.collect(steps, res, cfg["vocab"])
                for rid in reqs:
                    close(got[rid], ref[rid], dtype, f"drawn {seed}/{cut}/{dtype}/{rid}: {cfg['layers']}", cfg, t, reqs[rid], ("drawn", seed, rid))


# ---- entry points ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    from xyntetik_runner_b200.engine.runner import Runner
    path, cfg, tensors, _, _ = models["mix"]
    prompts = [traces.random_tokens(i + 40, n, cfg["vocab"]) for i, n in enumerate((5, 11, 17, 3, 30))]
    r = Runner(path, dtype=dtype, ctx=128, parallel=3, page_size=16)          # five requests over three slots
    res = r.generate(prompts, n=12, temp=0.0, ignore_eos=True)
    for p, g in zip(prompts, res):
        assert len(g.tokens) == 12 and g.finish_reason == "length"
        if dtype == "float32":
            assert g.tokens == tb.plain_greedy(cfg, tensors, p, 12)
        else:
            # teacher-forced: every token is the plain argmax for the engine's own prefix, or within rounding of it
            for i, tok in enumerate(g.tokens):
                lg = tb.plain_logits(cfg, tensors, list(p) + list(g.tokens[:i]))[-1]
                assert lg.max() - lg[tok] <= 0.06 * np.abs(lg).max()


def test_command_line_generates_what_the_plain_implementation_does(models):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, tensors, _, _ = models["odd"]
    prompt = traces.random_tokens(9, 7, cfg["vocab"])
    ids = "ids:" + ",".join(str(t) for t in prompt)
    out = {}
    for extra in (["--dtype", "float32"], ["--ref"]):
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "runner"), "-m", path, "-p", ids, "-n", "6", "--ignore-eos"] + extra,
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        out[extra[-1]] = [ln for ln in r.stdout.splitlines() if ln.startswith("ids:")][0]
    want = "ids:" + ",".join(str(t) for t in tb.plain_greedy(cfg, tensors, prompt, 6))
    assert out["--ref"] == want and out["float32"] == want, out


def test_trace_runner_program(models):
    """bin/trace_run on a folder: steps on standard input, logits in files, a line per step."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, tensors, reqs, ref = models["mix"]
    steps = traces.mixed(reqs, seed=5)
    with tempfile.TemporaryDirectory() as out:
        r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", out, "--max-tokens",
                            str(traces.pool_tokens(steps, 64))], input="".join(json.dumps(s) + "\n" for s in steps),
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
        res = {s["step"]: np.fromfile(os.path.join(out, f"{s['step']}.f32"), dtype="<f4") for s in steps}
    got = traces.collect(steps, res, cfg["vocab"])
    for rid in reqs:
        traces.assert_close(got[rid], ref[rid], "float32", f"trace_run/{rid}")
