"""Besolix on the GPU against the plain implementation: each mechanism alone, every way of cutting a request, mixed
batches with pages and state slots used again, tokens crafted so that one key stands out just inside and just outside
a window, at page borders and far back, long decoding, other sizes, greedy generation through the entry points."""
import copy
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_besolix as P
import tiny_besolix as tb
import traces

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [5, 41, 17, 70, 130, 23], "odd": [1, 9, 33, 70, 150, 64], "tc": [5, 200, 17, 70, 130, 33],
           "rec": [2, 19, 90, 35, 60, 77], "win": [3, 29, 66, 100, 9, 48]}
PAGE = {"mix": 16, "odd": 8, "tc": 64, "rec": 32, "win": 4}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in tb.CONFIGS:
        path, cfg, tensors = tb.make_folder(str(tmp_path_factory.mktemp("be_" + name)), name)
        reqs = {f"r{i}": traces.random_tokens(100 * i + len(name), n, cfg["vocab"]) for i, n in enumerate(LENGTHS[name])}
        ref = {rid: tb.plain_logits(cfg, tensors, t) for rid, t in reqs.items()}
        out[name] = (path, cfg, tensors, reqs, ref)
    return out


_sens = {}


def close(got, ref, dtype, what, cfg, tensors, toks, key):
    """float32: the fixed tolerance.  bfloat16: the fixed tolerance, with the allowance of ``tiny_besolix.assert_close_bfloat16``
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


class Session:
    """One engine for several traces (every trace ends all of its requests)."""

    def __init__(self, folder, dtype, page_size, max_tokens, max_requests=4):
        from xyntetik_runner_b200.engine.engine import Engine, EngineParams
        self.eng = Engine(folder, EngineParams(dtype=dtype, max_tokens=max_tokens, page_size=page_size, max_requests=max_requests))

    def play(self, steps):
        from xyntetik_runner_b200.engine.replay import replay
        res = replay(self.eng, steps)
        self.eng.check_status()
        self.eng.cache.audit()
        assert not self.eng.cache.live_requests()
        return res


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
    if cut.startswith("mixed") and eng.cache.pools:
        assert sum(-(-len(t) // PAGE[name]) for t in reqs.values()) > eng.cache.pools[0].n_pages      # pages were used again
    if cut.startswith("mixed"):
        assert len(reqs) > 4            # and so were the state slots


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_bfloat16_matches_plain(models, name, cut):
    path, cfg, tensors, reqs, ref = models[name]
    steps = CUTS[cut](reqs)
    res, _ = run(path, "bfloat16", steps, PAGE[name])
    got = traces.collect(steps, res, cfg["vocab"])
    for rid in reqs:
        close(got[rid], ref[rid], "bfloat16", f"{name}/{cut}/{rid}", cfg, tensors, reqs[rid], (name, rid))


def test_float32_cuts_agree_bit_for_bit_where_the_kernels_fix_their_order(models):
    """The recurrence walks token by token and the float32 products add in a fixed order: a model of recurrences alone gives the
    same bits however its requests are cut."""
    path, cfg, tensors, reqs, ref = models["rec"]
    base = None
    for cut in ("whole", "portions", "pairs", "mixed"):
        steps = CUTS[cut](reqs)
        res, _ = run(path, "float32", steps, PAGE["rec"])
        got = traces.collect(steps, res, cfg["vocab"])
        if base is None:
            base = got
        for rid in reqs:
            assert np.array_equal(got[rid], base[rid]), (cut, rid)


def test_long_decoding_and_first_tokens(models):
    """Three tokens at once, then 300 one by one: the state is carried 300 times, windows slide over decoded tokens, pages fill,
    are let go behind the windows and taken again."""
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
    b, _ = run(path, "bfloat16", steps, PAGE["mix"], graphs=False)
    for k in a:
        assert np.array_equal(a[k], b[k])


def test_tensor_core_kernels_ran(models):
    from xyntetik_runner_b200.parts import attention, latent_attention, linear
    path, cfg, tensors, reqs, ref = models["tc"]
    before = (attention.counters["tcgen05"], attention.counters["mma"], latent_attention.counters["mma"], linear.counters["tcgen05"])
    run(path, "bfloat16", CUTS["tail"]({"r1": reqs["r1"]}), PAGE["tc"])
    after = (attention.counters["tcgen05"], attention.counters["mma"], latent_attention.counters["mma"], linear.counters["tcgen05"])
    assert all(b > a for a, b in zip(before, after)), (before, after)


# ---- one mechanism at a time ------------------------------------------------------------------------------------------
SINGLE = {
    "attention": tb.model(60, 40, 1e-5, [tb.layer(tb.attention(3, 1, 12, 20, 0.3, tb._rot(40.0, 6, 3.0), window=11), None)]),
    "attention_all_keys": tb.model(60, 40, 1e-5, [tb.layer(tb.attention(2, 2, 16, 16, 0.25, tb._rot(40.0, 16)), None)]),
    "delta": tb.model(60, 40, 1e-5, [tb.layer(tb.delta(3, 1, 12, 20, 4), None)]),
    "delta_one_tap": tb.model(60, 40, 1e-5, [tb.layer(tb.delta(2, 2, 36, 6, 1), None)]),
    "latent": tb.model(60, 40, 1e-5, [tb.layer(tb.latent(3, 8, 4, 6, 12, 10, 0.3, base=40.0, window=9), None)]),
    "latent_no_plain_part": tb.model(60, 40, 1e-5, [tb.layer(tb.latent(2, 0, 8, 6, 12, 10, 0.3, base=40.0), None)]),
    "latent_shared": tb.model(60, 40, 1e-5, [tb.layer(tb.latent(3, 8, 4, 6, 12, 10, 0.3, base=40.0, window=9), None),
                                             tb.layer(tb.latent(2, 4, 4, 10, 12, 6, 0.3, base=40.0, window=14, kv_from=0), None)]),
    "feed_forward": tb.model(60, 40, 1e-5, [tb.layer(tb.delta(1, 1, 4, 4, 1), 52)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_one_mechanism_alone(name, dtype):
    cfg = SINGLE[name]
    tensors = tb.draw(cfg, 31)
    reqs = {"a": traces.random_tokens(1, 50, 60), "b": traces.random_tokens(2, 21, 60), "c": traces.random_tokens(3, 2, 60)}
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, tensors, cfg)
        for cut in ("whole", "portions", "mixed"):
            steps = CUTS[cut](reqs)
            res, _ = run(path, dtype, steps, page_size=8)
            got = traces.collect(steps, res, 60)
            for rid, toks in reqs.items():
                close(got[rid], tb.plain_logits(cfg, tensors, toks), dtype, f"{name}/{cut}/{rid}", cfg, tensors, toks, (name, rid))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("adjacent", [True, False])
def test_norm_rotation_and_store_kernel(dtype, adjacent):
    """Query and key heads normed, rotated and stored with values of another size: against the formulas, element by element."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(5)
    dev = "cuda"
    # (the later sizes fall on 16-byte borders, which bfloat16 rows take eight elements a lane: 4, 8, 16 and 32 lanes a head, heads
    # that do not fill the last warp, values longer and shorter than keys, a rotation over part of a head and over all of it)
    for H, K, D, Vd, rot in ((3, 1, 12, 20, 6), (2, 2, 16, 16, 16), (4, 2, 40, 8, 0), (1, 1, 6, 70, 4), (9, 3, 24, 8, 16), (5, 2, 64, 128, 32),
                             (3, 1, 128, 64, 128), (4, 4, 48, 96, 16), (2, 1, 256, 8, 64), (7, 1, 32, 32, 0), (16, 4, 128, 128, 64)):
        hd = -(-max(D, Vd) // 16) * 16
        n, page, max_pages = 9, 4, 8
        cols = (H + K) * D + K * Vd
        inp = torch.randn(n, cols).to(dtype)
        qw, kw = torch.rand(D) + 0.5, torch.rand(D) + 0.5
        freq = torch.tensor([37.0 ** (-2.0 * i / rot) / 1.5 for i in range(rot // 2)], dtype=torch.float64) if rot else None
        positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 29], dtype=torch.int32)
        bt = torch.tensor([[5, 2, 7, 0, 1, 3, 6, 4]], dtype=torch.int32)
        cache = torch.full((8, 2, K, page, hd), 7.0, dtype=dtype, device=dev)               # [page][K|V][kv head][token][hd]
        q_out = torch.full((n, (H + 2 * K) * hd), 7.0, dtype=dtype, device=dev)
        kernels.qk_norm_rope_store(inp.to(dev), q_out, positions.to(dev), torch.zeros(n, dtype=torch.int32, device=dev), bt.to(dev),
                                   None if freq is None else freq.to(dev), qw.to(dev), kw.to(dev), cache.data_ptr(), cache.stride(0),
                                   cache.stride(1), H, K, D, Vd, hd, rot, max_pages, page, adjacent, 1e-5)
        x = inp.double()

        def turn(v, pos):
            out = v.clone()
            for i in range(rot // 2):
                a, b = (2 * i, 2 * i + 1) if adjacent else (i, i + rot // 2)
                ang = float(pos) * float(freq[i])
                out[..., a] = v[..., a] * np.cos(ang) - v[..., b] * np.sin(ang)
                out[..., b] = v[..., b] * np.cos(ang) + v[..., a] * np.sin(ang)
            return out
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        q_got, cache_h = q_out.cpu().double(), cache.cpu().double()
        for t in range(n):
            pos = int(positions[t])
            q = turn(P.norm_plain(x[t, :H * D].view(H, D), qw.double(), 1e-5), pos)
            k = turn(P.norm_plain(x[t, H * D:(H + K) * D].view(K, D), kw.double(), 1e-5), pos)
            v = x[t, (H + K) * D:].view(K, Vd)
            got_q = q_got[t, :H * hd].view(H, hd)
            assert (got_q[:, :D] - q).abs().max() < tol and (got_q[:, D:] == 0).all()
            pg, at = int(bt[0, pos // page]), pos % page
            assert (cache_h[pg, 0, :, at, :D] - k).abs().max() < tol and (cache_h[pg, 0, :, at, D:] == 0).all()
            assert (cache_h[pg, 1, :, at, :Vd] - v).abs().max() < tol and (cache_h[pg, 1, :, at, Vd:] == 0).all()
        written = {(int(bt[0, int(p) // page]), int(p) % page) for p in positions}
        for pg in range(8):
            for at in range(page):
                if (pg, at) not in written:
                    assert (cache_h[pg, :, :, at] == 7.0).all()                  # no other row was touched


def test_delta_kernels_from_states_in_other_slots():
    """Two requests in slots 3 and 1, cut differently, beside the plain recurrence; the slots that are not named stay as they
    were; a walk cut in portions leaves the same bits as one walk."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(6)
    dev = "cuda"
    for H, G, D, V, taps in ((4, 2, 12, 20, 3), (1, 1, 70, 5, 1), (2, 2, 130, 33, 5), (6, 3, 32, 64, 4)):
        CH = 2 * G * D + H * V
        W = 24
        lens = {3: 23, 1: 9}
        w = {"q": torch.randn(G * D, W), "k": torch.randn(G * D, W), "v": torch.randn(H * V, W), "g": torch.randn(H * V, W),
             "o": torch.eye(H * V), "norm": torch.ones(V), "b": torch.randn(H, W), "a": torch.randn(H, W), "A_log": torch.randn(H) - 1,
             "dt_bias": torch.randn(H), "q.conv": torch.randn(G * D, taps), "k.conv": torch.randn(G * D, taps), "v.conv": torch.randn(H * V, taps)}
        w = {k: v.double() for k, v in w.items()}
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "conv": taps}
        hs = {s: torch.randn(n, W, dtype=torch.float64) * 0.5 for s, n in lens.items()}
        conv_w = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]]).float().to(dev)
        neg_a, dtb = (-torch.exp(w["A_log"])).float().to(dev), w["dt_bias"].float().to(dev)
        floats = kernels.delta_state_floats(H, G, D, V, taps)

        def walk(cuts):
            """cuts: per step, {slot: tokens}."""
            state = torch.zeros(5, floats + 3, device=dev)
            state[[0, 2, 4]] = 9.0
            at = {s: 0 for s in lens}
            outs = {s: [] for s in lens}
            for step in cuts:
                rows, seg_start, seg_len, seg_slot, tok_seg = [], [], [], [], []
                for i, (s, cnt) in enumerate(step.items()):
                    seg_start.append(sum(seg_len)); seg_len.append(cnt); seg_slot.append(s); tok_seg += [i] * cnt
                    hh = hs[s][at[s]:at[s] + cnt]
                    rows.append(torch.cat([hh @ w["q"].T, hh @ w["k"].T, hh @ w["v"].T, hh @ w["b"].T, hh @ w["a"].T], dim=1))
                rows = torch.cat(rows).float()
                n = rows.shape[0]
                proj = torch.zeros(n, CH + 5, device=dev)                      # (a row stride that is not the width)
                proj[:, :CH] = rows[:, :CH].to(dev)
                gates = rows[:, CH:].contiguous().to(dev)
                i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
                qkv, coef, o = torch.empty(n, CH, device=dev), torch.empty(n, 2 * H, device=dev), torch.empty(n, H * V, device=dev)
                kernels.delta(proj[:, :CH], conv_w, gates, neg_a, dtb, state, qkv, coef, o, i32(tok_seg), i32(seg_start), i32(seg_len),
                              i32(seg_slot), len(seg_len), H, G, D, V, taps)
                o = o.cpu()
                for i, (s, cnt) in enumerate(step.items()):
                    outs[s].append(o[seg_start[i]:seg_start[i] + cnt])
                    at[s] += cnt
            return {s: torch.cat(v) for s, v in outs.items()}, state.cpu()
        whole, st_whole = walk([{3: 23, 1: 9}])
        cut, st_cut = walk([{3: 2}, {1: 1, 3: 1}, {3: 7, 1: 6}, {1: 2}, {3: 13}])
        assert (st_whole[[0, 2, 4]] == 9.0).all() and (st_whole[:, floats:][[1, 3]] == 0).all()
        for s in lens:
            assert torch.equal(whole[s], cut[s]), (H, D, V, taps, s)
            # the plain read-outs: undo the output norm's division by taking the plain function apart
            T = lens[s]
            silu = torch.nn.functional.silu
            q = silu(P.short_conv(hs[s] @ w["q"].T, w["q.conv"])).view(T, G, D)
            k = silu(P.short_conv(hs[s] @ w["k"].T, w["k.conv"])).view(T, G, D)
            v = silu(P.short_conv(hs[s] @ w["v"].T, w["v.conv"])).view(T, H, V)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
            beta = torch.sigmoid(hs[s] @ w["b"].T)
            decay = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(hs[s] @ w["a"].T + w["dt_bias"]))
            S = torch.zeros(H, D, V, dtype=torch.float64)
            for t in range(T):
                S = S * decay[t][:, None, None]
                u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
                S = S + k[t][:, :, None] * u[:, None, :]
                want = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
                assert (whole[s][t].double() - want).abs().max() < 2e-5 * max(1.0, float(want.abs().max())), (H, D, V, taps, s, t)
        assert torch.equal(st_whole, st_cut)
        # the state's matrix is S transposed, per head [V][D]
        assert (st_whole[1, :H * V * D].view(H, V, D).double() - 0).abs().max() > 0


def test_latent_attention_kernels_with_a_window():
    """Both kernels with windows that end inside a tile, at a page border and beyond the start, one range of keys and many:
    against softmax over the visible rows, with one row made to stand out just inside the window and one just outside."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(7)
    dev = "cuda"
    H, C, R, page, n_ctx = 5, 64, 8, 16, 300
    n_pages = -(-n_ctx // page) + 5
    rows = (torch.randn(n_ctx, C + R) * 0.3).to(torch.bfloat16)
    perm = torch.randperm(n_pages)[: -(-n_ctx // page)].to(torch.int32)
    cache = torch.zeros(n_pages, page, C + R, dtype=torch.bfloat16)
    for p in range(n_ctx):
        cache[perm[p // page], p % page] = rows[p]
    mp = len(perm) + 2
    bt = torch.full((1, mp), -1, dtype=torch.int32)
    bt[0, : len(perm)] = perm
    bt, cache_d = bt.to(dev), cache.to(dev)
    positions = [299, 0, 31, 32, 47, 48, 150, 64]
    n = len(positions)
    seg = torch.zeros(n, dtype=torch.int32, device=dev)
    pos_d = torch.tensor(positions, dtype=torch.int32, device=dev)
    for window in (1, 2, 16, 17, 33, 48, 100, 299, 300, 301):
        ql = torch.randn(n, H, C) * 0.2
        qr = torch.randn(n, H, R) * 0.2
        for i, pos in enumerate(positions):
            inside, outside = pos - window + 1, pos - window
            if inside >= 0:
                ql[i, 1] = rows[inside, :C].float() * 12          # head 1 looks for the oldest row it may see
            if outside >= 0:
                ql[i, 2] = rows[outside, :C].float() * 12         # head 2 for the newest it may not
        ql16, qr16 = ql.reshape(n, H * C).to(torch.bfloat16).to(dev), qr.reshape(n, H * R).to(torch.bfloat16).to(dev)
        want = torch.zeros(n, H, C, dtype=torch.float64)
        for i, pos in enumerate(positions):
            lo = max(0, pos - window + 1)
            k = rows[lo: pos + 1].double()
            q = torch.cat([ql16[i].cpu().double().view(H, C), qr16[i].cpu().double().view(H, R)], dim=1)
            a = torch.softmax(q @ k.T * 0.7, dim=-1)
            want[i] = a @ k[:, :C]
            if pos - window + 1 >= 0 and window > 1:
                assert a[1, 0] > 0.5
        want = want.view(n, H * C)
        got = torch.empty(n, H * C, device=dev)
        kernels.latent_attention(ql16.float(), qr16, 0, R, got, cache_d.data_ptr(), page * (C + R), pos_d, seg, bt, H, C, R, mp, page, 0.7,
                                 window=window)
        assert (got.cpu().double() - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max())), window
        reach = min(n_ctx, window)
        mt = -(-H // 16)
        for chunk, splits in ((-(-reach // 32) * 32, 1), (32, -(-reach // 32)), (64, -(-reach // 64) + 1)):
            got = torch.full((n, H * C), float("nan"), device=dev)
            po = torch.full((n * mt * splits * 16 * C,), float("nan"), device=dev)
            pm = torch.full((n * mt * splits * 32,), float("nan"), device=dev)
            kernels.latent_attention_mma(ql16, qr16, 0, R, got, po, pm, cache_d.data_ptr(), page * (C + R), pos_d, seg, bt, H, C, R, mp,
                                         page, 0.7, chunk, splits, window=window)
            err = (got.cpu().double() - want).abs().max().item()
            assert err < 1.5e-2 * float(want.abs().max()), (window, chunk, splits, err)


# ---- tokens crafted so that one key stands out ----------------------------------------------------------------------------
def _seeker_attention(window, score=12.0):
    """A one-layer attention model with two special tokens: `B` (id 1) and `A` (id 0), A's embedding solved so that the query of
    every head of A points along B's key; the score scale is set so that this one score is 12 (the others scatter around 0 with a
    spread of 3): A's output is B's value whenever B is visible."""
    cfg = tb.model(40, 64, 1e-5, [tb.layer(tb.attention(2, 1, 16, 24, 1.0, tb._rot(10000.0, 2), window=window), None)])
    t = tb.draw(cfg, 41)
    w = {k: v.double() for k, v in t.items()}
    h_b = P.norm_one_plus(w["embed"][1][None], w["l0.norm1"], 1e-5)[0]
    k_b = P.norm_plain((w["l0.mix.k"] @ h_b)[None], w["l0.mix.k.norm"], 1e-5)[0]     # [16]: the one key head, normed
    k_dir = k_b / w["l0.mix.q.norm"]                                                 # undo the query norm's weight
    k_dir[:2] = 0                                                                    # leave the rotated pair out of it
    y = torch.linalg.pinv(w["l0.mix.q"]) @ torch.cat([k_dir, k_dir])                 # W_q y = the wanted direction, both heads
    t["embed"][0] = (y / (1.0 + w["l0.norm1"]) * 3.0 / y.abs().max()).to(torch.bfloat16)
    h_a = P.norm_one_plus(t["embed"][0].double()[None], w["l0.norm1"], 1e-5)[0]
    q_a = P.norm_plain((w["l0.mix.q"] @ h_a).view(2, 16), w["l0.mix.q.norm"], 1e-5)
    cfg["layers"][0]["mixer"]["scale"] = float(score / (q_a[:, 2:] @ k_b[2:]).min())
    return cfg, t


def _seeker_latent(window, kv_from=False, score=12.0):
    """The same for latent attention (alone, or reading the rows that a layer before it caches): the unrotated part of A's
    queries, which passes the queries' latent and its norm, points along the unrotated key that B's latent expands to."""
    layers = [tb.layer(tb.latent(2, 16, 2, 12, 16, 40, 1.0, base=10000.0, window=window), None)]
    if kv_from:
        layers = [tb.layer(tb.latent(1, 4, 2, 4, 16, 8, 0.1, base=10000.0, window=3), None),
                  tb.layer(tb.latent(2, 16, 2, 12, 16, 40, 1.0, base=10000.0, window=window, kv_from=0), None)]
    cfg = tb.model(40, 64, 1e-5, layers)
    t = tb.draw(cfg, 43)
    if kv_from:
        t["l0.mix.o"] = torch.zeros_like(t["l0.mix.o"])        # layer 0 only fills the cache: layer 1 reads the embeddings
    t["l0.mix.dkv"][16:] *= 0.1                                # the rotated key part stays small beside the crafted score
    w = {k: v.double() for k, v in t.items()}
    own, rd, n1_own, n1_rd = ("l0.mix.", "l1.mix.", "l0.norm1", "l1.norm1") if kv_from else ("l0.mix.", "l0.mix.", "l0.norm1", "l0.norm1")
    h_b = P.norm_one_plus(w["embed"][1][None], w[n1_own], 1e-5)[0]
    c_b = P.norm_plain((w[own + "dkv"] @ h_b)[None, :16], w[own + "dkv.norm"], 1e-5)[0]
    k_b = w[rd + "uk"] @ c_b                                                         # [2 heads x 16]
    # q_plain = W_uq[plain rows] (w_dq * W_dq y) / rms: linear in y up to a positive factor
    rows = torch.cat([torch.arange(0, 16), torch.arange(18, 34)])
    M = w[rd + "uq"][rows] @ (w[rd + "dq.norm"][:, None] * w[rd + "dq"])
    y = torch.linalg.pinv(M) @ k_b
    t["embed"][0] = (y / (1.0 + w[n1_rd]) * 3.0 / y.abs().max()).to(torch.bfloat16)
    h_a = P.norm_one_plus(t["embed"][0].double()[None], w[n1_rd], 1e-5)[0]
    q_a = (w[rd + "uq"] @ P.norm_plain((w[rd + "dq"] @ h_a)[None], w[rd + "dq.norm"], 1e-5)[0])[rows].view(2, 16)
    cfg["layers"][-1]["mixer"]["scale"] = float(score / (q_a * k_b.view(2, 16)).sum(-1).min())
    return cfg, t


def _standout_cases(cfg, t, window, page):
    """(tokens, place of A, is B visible) with B just inside and just outside the window of A, A and B on either side of page
    borders, A in the prompt; fillers are ids >= 2."""
    rng = np.random.RandomState(window)
    cases = []
    for pa in (window + page, 2 * page - 1, 2 * page, 5 * page + 3):
        for dist, seen in ((window - 1, True), (window, False), (1, True), (window // 2, True)):
            pb = pa - dist
            if pb < 0 or dist < 1 or (dist >= window) == seen:
                continue
            toks = [int(x) for x in rng.randint(2, cfg["vocab"], size=pa + 6)]
            toks[pb], toks[pa] = 1, 0
            cases.append((toks, pa, seen))
    return cases


@pytest.mark.parametrize("kind", ["attention", "latent", "latent_shared"])
def test_a_key_just_inside_and_just_outside_the_window(kind):
    window, page = 21, 8
    cfg, t = {"attention": _seeker_attention, "latent": _seeker_latent, "latent_shared": lambda w: _seeker_latent(w, True)}[kind](window)
    cases = _standout_cases(cfg, t, window, page)
    assert len(cases) >= 8
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        sessions = {dtype: Session(path, dtype, page, 128) for dtype in ("float32", "bfloat16")}
        for toks, pa, seen in cases:
            ref = tb.plain_logits(cfg, t, toks)
            # the crafted token does what it is made for: with B out of the way A's logits are quite other ones
            moved = list(toks)
            moved[toks.index(1)] = 2
            far = np.abs(tb.plain_logits(cfg, t, moved)[pa] - ref[pa]).max() / np.abs(ref[pa]).max()
            assert (far > 0.05) == seen, (kind, pa, seen, far)
            for dtype in ("float32", "bfloat16"):
                for steps in (traces.whole({"a": toks}),                                             # A inside a prompt
                              traces.tail_decoded({"a": toks}, len(toks) - pa + 2),                  # A decoded alone
                              traces.portions({"a": toks}, sizes=(pa, 2, 1, 3)),                     # A first of a portion of two
                              traces.portions({"a": toks}, sizes=(3, 2))):
                    got = traces.collect(steps, sessions[dtype].play(steps), cfg["vocab"])["a"]
                    close(got, ref, dtype, f"{kind}: A at {pa}, B {'inside' if seen else 'outside'}", cfg, t, toks, (kind, pa, seen))


def test_a_far_key_among_hundreds():
    """B at place 5, A 500 tokens later, no window: A's logits hang on B across dozens of pages, in a prompt and decoded."""
    for make in (_seeker_attention, _seeker_latent):
        cfg, t = make(None, score=18.0)
        toks = [int(x) for x in np.random.RandomState(9).randint(2, cfg["vocab"], size=520)]
        toks[5], toks[505] = 1, 0
        ref = tb.plain_logits(cfg, t, toks)
        moved = list(toks)
        moved[5] = 2
        assert np.abs(tb.plain_logits(cfg, t, moved)[505] - ref[505]).max() > 0.05 * np.abs(ref[505]).max()
        with tempfile.TemporaryDirectory() as tmp:
            path, _, _ = tb.make_folder(tmp, None, t, cfg)
            for dtype in ("float32", "bfloat16"):
                for steps in (traces.whole({"a": toks}), traces.tail_decoded({"a": toks}, 40), traces.portions({"a": toks}, sizes=(97, 2, 150))):
                    res, _ = run(path, dtype, steps, page_size=16)
                    close(traces.collect(steps, res, cfg["vocab"])["a"], ref, dtype, "far key", cfg, t, toks, ("far", make.__name__))


def test_the_recurrence_remembers_a_far_token(models):
    """Slow decays: the first tokens still move the logits 200 tokens later, in every cut and with the slot used before."""
    path0, cfg, _, _, _ = models["rec"]
    t = tb.draw(cfg, 5, slow_decay=True)
    toks = traces.random_tokens(4, 220, cfg["vocab"])
    other = list(toks)
    other[1] = (toks[1] + 1) % cfg["vocab"]
    ref = tb.plain_logits(cfg, t, toks)
    assert np.abs(tb.plain_logits(cfg, t, other)[219] - ref[219]).max() > 1e-3 * np.abs(ref[219]).max()
    reqs = {"first": other, "a": toks}                     # "first" leaves its state in the slot that "a" gets
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tb.make_folder(tmp, None, t, cfg)
        for dtype in ("float32", "bfloat16"):
            for cut in ("whole", "tail", "portions"):
                steps = CUTS[cut](reqs)
                res, _ = run(path, dtype, steps, page_size=16, max_requests=1)
                close(traces.collect(steps, res, cfg["vocab"])["a"], ref, dtype, f"far token/{cut}", cfg, t, toks, ("far token",))


# ---- other sizes -----------------------------------------------------------------------------------------------------------
def _drawn_config(rng):
    """A configuration drawn at random: any order of the mixers, sizes that are and are not multiples of 8 and 16."""
    pick = lambda *xs: xs[rng.randint(len(xs))]
    width = pick(40, 52, 64, 72, 128)
    layers, owners = [], []
    for i in range(rng.randint(1, 5)):
        kind = pick("attention", "delta", "latent", "latent")
        ff = pick(None, 24, 40, 64)
        if kind == "attention":
            kv = pick(1, 2, 3)
            D = pick(8, 12, 16, 32, 48, 64)
            dims = pick(0, 2, D // 2 // 2 * 2, D)
            layers.append(tb.layer(tb.attention(kv * pick(1, 2, 4), kv, D, pick(D, D, 8, 24, 64), pick(0.1, 0.25, D ** -0.5),
                                                tb._rot(pick(50.0, 1e4, 1e5), dims, pick(None, 2.0, 16.0)), pick(None, 1, 7, 32, 100)), ff))
        elif kind == "delta":
            G = pick(1, 2)
            layers.append(tb.layer(tb.delta(G * pick(1, 2, 3), G, pick(4, 8, 24, 64, 72), pick(4, 16, 40, 64), pick(1, 2, 3, 4, 6)), ff))
        else:
            reuse = owners and rng.rand() < 0.5
            if reuse:
                o = owners[rng.randint(len(owners))]
                mo = layers[o]["mixer"]
                C, R, base = mo["kv_rank"], mo["rot_dim"], mo["rot"]["base"]
            else:
                C, R, base = pick(8, 20, 64, 128), pick(2, 4, 8, 16), pick(50.0, 1e4)
            layers.append(tb.layer(tb.latent(pick(1, 2, 5, 17), pick(0, 4, 8, 16), R, pick(4, 8, 24), C, pick(6, 8, 24, 40), pick(0.1, 0.3),
                                             base=base, window=pick(None, 1, 5, 40, 64), kv_from=o if reuse else None), ff))
            if not reuse:
                owners.append(i)
    return tb.model(pick(50, 97, 128), width, pick(1e-5, 1e-6), layers)


def _drawn_config_of_layer_sizes(rng):
    """The same with sizes like real layers': multiples of 16, several heads, latents of 64 to 256, windows of 40 to 200."""
    pick = lambda *xs: xs[rng.randint(len(xs))]
    layers, owners = [], []
    for i in range(rng.randint(3, 6)):
        kind = pick("attention", "delta", "latent", "latent")
        ff = pick(None, 128, 256)
        if kind == "attention":
            kv = pick(1, 2, 4)
            D = pick(32, 64, 96, 128)
            layers.append(tb.layer(tb.attention(kv * pick(1, 2, 3), kv, D, pick(32, 64, 96, 128), D ** -0.5,
                                                tb._rot(pick(1e4, 2e4, 5e5), pick(8, 16, 32, D), pick(None, 2.0, 4.0)), pick(None, 48, 64, 96, 200)), ff))
        elif kind == "delta":
            G = pick(1, 2, 4)
            layers.append(tb.layer(tb.delta(G * pick(1, 2), G, pick(32, 64, 128), pick(32, 64, 128), pick(2, 3, 4)), ff))
        else:
            reuse = owners and rng.rand() < 0.5
            if reuse:
                o = owners[rng.randint(len(owners))]
                mo = layers[o]["mixer"]
                C, R, base = mo["kv_rank"], mo["rot_dim"], mo["rot"]["base"]
            else:
                C, R, base = pick(64, 96, 128, 192, 256), pick(8, 16, 32), pick(1e4, 5e4)
            D = pick(16, 32, 64)
            layers.append(tb.layer(tb.latent(pick(2, 4, 6, 8, 12), D, R, pick(16, 32, 64), C, pick(64, 96, 128), (D + R) ** -0.5,
                                             base=base, window=pick(None, 40, 72, 100, 128), kv_from=o if reuse else None), ff))
            if not reuse:
                owners.append(i)
    return tb.model(pick(320, 512), pick(128, 192, 256), pick(1e-5, 1e-6), layers)


@pytest.mark.parametrize("seed", range(16))
def test_drawn_configurations(seed):
    rng = np.random.RandomState(1000 + seed)
    cfg = _drawn_config(rng) if seed < 12 else _drawn_config_of_layer_sizes(rng)
    t = tb.draw(cfg, 50 + seed)
    page = int(rng.choice([4, 8, 16, 64])) if seed < 12 else 64
    reqs = {f"r{i}": traces.random_tokens(7 * seed + i, n, cfg["vocab"]) for i, n in enumerate((3, 90, 17, 140, 1, 45) if seed < 12 else (3, 90, 17, 240, 1, 45))}
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


# ---- through the entry points --------------------------------------------------------------------------------------------
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
    path, cfg, tensors, _, _ = models["win"]
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
    import json
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, tensors, reqs, ref = models["odd"]
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
