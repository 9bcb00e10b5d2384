"""Pitolix on the GPU against the plain implementation: each mechanism alone, every way of cutting a request, mixed batches
with pages and slots used again, tokens crafted so that one key stands out far back and at page borders, sinks that take most
of a softmax, query factors that step inside prompts and between decoded tokens, the first tokens, long decoding, other sizes,
greedy generation through the entry points."""
import copy
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_pitolix as P
import tiny_pitolix as tp
import traces

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [5, 41, 17, 70, 130, 23], "odd": [1, 9, 33, 70, 150, 64], "tc": [5, 200, 17, 70, 130, 33], "loop": [2, 19, 90, 35, 60, 77]}
PAGE = {"mix": 16, "odd": 8, "tc": 64, "loop": 32}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in tp.CONFIGS:
        path, cfg, tensors = tp.make_folder(str(tmp_path_factory.mktemp("pi_" + name)), name)
        reqs = {f"r{i}": traces.random_tokens(100 * i + len(name), n, cfg["vocab"]) for i, n in enumerate(LENGTHS[name])}
        ref = {rid: tp.plain_logits(cfg, tensors, t) for rid, t in reqs.items()}
        out[name] = (path, cfg, tensors, reqs, ref)
    return out


_sens = {}


def close(got, ref, dtype, what, cfg, tensors, toks, key):
    """float32: the fixed tolerance.  bfloat16: the fixed tolerance, with the allowance of ``tiny_pitolix.assert_close_bfloat16``
    for positions that the plain implementation itself shows to hang on a rounding."""
    if dtype == "float32":
        return traces.assert_close(got, ref, dtype, what)
    if key not in _sens:
        _sens[key] = tp.rounding_sensitivity(cfg, tensors, toks)
    tp.assert_close_bfloat16(got, ref, _sens[key], what)


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
@pytest.mark.parametrize("name", list(tp.CONFIGS))
def test_float32_matches_plain_in_every_cut(models, name, cut):
    path, cfg, tensors, reqs, ref = models[name]
    steps = CUTS[cut](reqs)
    res, eng = run(path, "float32", steps, PAGE[name])
    got = traces.collect(steps, res, cfg["vocab"])
    for rid in reqs:
        traces.assert_close(got[rid], ref[rid], "float32", f"{name}/{cut}/{rid}")
    if cut.startswith("mixed"):
        assert sum(-(-len(t) // PAGE[name]) for t in reqs.values()) > eng.cache.pools[0].n_pages      # pages were used again
        assert len(reqs) > 4                                                                         # and so were the slots


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", list(tp.CONFIGS))
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


def test_long_decoding_and_first_tokens(models):
    """Three tokens at once, then 300 one by one: the query factor steps dozens of times between decoded tokens, pages fill
    and the loop's passes each keep rows of their own."""
    path, cfg, tensors, _, _ = models["mix"]
    toks = traces.random_tokens(77, 303, cfg["vocab"])
    ref = tp.plain_logits(cfg, tensors, toks)
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
    from xyntetik_runner_b200.parts import attention, linear
    path, cfg, tensors, reqs, ref = models["tc"]
    before = (attention.counters["tcgen05"], attention.counters["mma"], linear.counters["tcgen05"])
    run(path, "bfloat16", CUTS["tail"]({"r1": reqs["r1"]}), PAGE["tc"])
    after = (attention.counters["tcgen05"], attention.counters["mma"], linear.counters["tcgen05"])
    assert all(b > a for a, b in zip(before, after)), (before, after)


# ---- one mechanism at a time ------------------------------------------------------------------------------------------
_tiny_sink = tp.sink_attention(1, 1, 4, 4, 0.5)
SINGLE = {
    "sink_attention": tp.model(60, 40, 1e-5, [tp.layer(tp.sink_attention(3, 1, 12, 20, 0.3), None)]),
    "sink_attention_query_factor": tp.model(60, 40, 1e-5, [tp.layer(tp.sink_attention(4, 2, 16, 16, 0.25, 1.2, 5), None)]),
    "sink_attention_factor_every_position": tp.model(60, 40, 1e-5, [tp.layer(tp.sink_attention(2, 2, 20, 8, 0.2, 0.6, 1), None)]),
    "rotary_attention_all": tp.model(60, 40, 1e-5, [tp.layer(tp.rotary_attention(2, 2, 16, 16, 0.25, 40.0, 16), None)]),
    "rotary_attention_part": tp.model(60, 40, 1e-5, [tp.layer(tp.rotary_attention(6, 2, 12, 20, 0.3, 40.0, 6), None)]),
    "rotary_attention_none": tp.model(60, 40, 1e-5, [tp.layer(tp.rotary_attention(3, 1, 24, 8, 0.2, 40.0, 0), None)]),
    "feed_forward": tp.model(60, 40, 1e-5, [tp.layer(_tiny_sink, 52)]),
    "loop_of_one_layer": tp.model(60, 40, 1e-5, [tp.layer(_tiny_sink, 24)], loop=(0, 1, 3), embedding_scale=3.0),
    "loop_after_a_layer": tp.model(60, 40, 1e-5, [tp.layer(_tiny_sink, 24), tp.layer(_tiny_sink, None)], loop=(1, 2, 2), embedding_scale=0.25),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_one_mechanism_alone(name, dtype):
    cfg = SINGLE[name]
    tensors = tp.draw(cfg, 31)
    reqs = {"a": traces.random_tokens(1, 50, 60), "b": traces.random_tokens(2, 21, 60), "c": traces.random_tokens(3, 2, 60)}
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tp.make_folder(tmp, None, tensors, cfg)
        for cut in ("whole", "portions", "mixed"):
            steps = CUTS[cut](reqs)
            res, _ = run(path, dtype, steps, page_size=8)
            got = traces.collect(steps, res, 60)
            for rid, toks in reqs.items():
                close(got[rid], tp.plain_logits(cfg, tensors, toks), dtype, f"{name}/{cut}/{rid}", cfg, tensors, toks, (name, rid))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unit_heads_query_factor_and_store_kernel(dtype):
    """Query and key heads divided by their root mean square, the queries times the factor of their position, keys and values of
    another size stored in their pages: against the formulas, element by element; positions on both sides of the factor's steps."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(5)
    dev = "cuda"
    # (the later sizes fall on 16-byte borders, which bfloat16 rows take eight elements a lane: 4, 8, 16 and 32 lanes a head)
    for H, K, D, Vd, coef, every in ((3, 1, 12, 20, 0.7, 4), (2, 2, 16, 16, 0.3, 1), (4, 2, 40, 8, 0.0, 0), (1, 1, 6, 70, 2.0, 29), (14, 7, 36, 16, 0.3, 8),
                                     (9, 3, 24, 8, 0.5, 2), (5, 2, 64, 128, 0.3, 5), (3, 3, 96, 96, 1.0, 3), (2, 1, 256, 8, 0.2, 28), (16, 4, 128, 128, 0.1, 6)):
        hd = -(-max(D, Vd) // 16) * 16
        n, page, max_pages = 9, 4, 8
        cols = (H + K) * D + K * Vd
        inp = torch.randn(n, cols).to(dtype)
        positions = torch.tensor([0, 1, 2, 3, 4, 6, 7, 27, 28], dtype=torch.int32)
        bt = torch.tensor([[5, 2, 7, 0, 1, 3, 6, 4]], dtype=torch.int32)
        cache = torch.full((8, 2, K, page, hd), 7.0, dtype=dtype, device=dev)               # [page][K|V][kv head][token][hd]
        q_out = torch.full((n, (H + 2 * K) * hd), 7.0, dtype=dtype, device=dev)
        kernels.qk_norm_rope_store(inp.to(dev), q_out, positions.to(dev), torch.zeros(n, dtype=torch.int32, device=dev), bt.to(dev),
                                   None, None, None, cache.data_ptr(), cache.stride(0), cache.stride(1), H, K, D, Vd, hd, 0, max_pages,
                                   page, False, 1e-5, True, coef, every)
        x = inp.double()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        q_got, cache_h = q_out.cpu().double(), cache.cpu().double()
        for t in range(n):
            pos = int(positions[t])
            f = 1.0 + coef * math.log((pos + 1) // every + 1) if every else 1.0
            q = P.unit_rms(x[t, :H * D].view(H, D), 1e-5) * f
            k = P.unit_rms(x[t, H * D:(H + K) * D].view(K, D), 1e-5)
            v = x[t, (H + K) * D:].view(K, Vd)
            got_q = q_got[t, :H * hd].view(H, hd)
            assert (got_q[:, :D] - q).abs().max() < tol * max(1.0, f) and (got_q[:, D:] == 0).all()
            pg, at = int(bt[0, pos // page]), pos % page
            assert (cache_h[pg, 0, :, at, :D] - k).abs().max() < tol and (cache_h[pg, 0, :, at, D:] == 0).all()
            assert (cache_h[pg, 1, :, at, :Vd] - v).abs().max() < tol and (cache_h[pg, 1, :, at, Vd:] == 0).all()
        written = {(int(bt[0, int(p) // page]), int(p) % page) for p in positions}
        for pg in range(8):
            for at in range(page):
                if (pg, at) not in written:
                    assert (cache_h[pg, :, :, at] == 7.0).all()                  # no other row was touched
        # the same rows as the partial sums of a product that was cut in three, with a bias and columns of gates behind the values:
        # the kernel sums them into the rows (gates included) and gives what it gives for the finished rows
        extra = 5
        parts = torch.randn(3, n, cols + extra)
        bias = torch.randn(cols + extra)
        done = (((parts[0] + parts[1]) + parts[2]) + bias).to(dtype)          # (the kernel's own order, so that the rows are equal bit for bit)
        wide = torch.full((n, cols + extra + 3), 7.0, dtype=dtype, device=dev)
        cache_a, cache_b = (torch.full((8, 2, K, page, hd), 7.0, dtype=dtype, device=dev) for _ in range(2))
        q_a, q_b = (torch.full((n, (H + 2 * K) * hd), 7.0, dtype=dtype, device=dev) for _ in range(2))
        common = (positions.to(dev), torch.zeros(n, dtype=torch.int32, device=dev), bt.to(dev), None, None, None)
        sizes = (H, K, D, Vd, hd, 0, max_pages, page, False, 1e-5, True, coef, every)
        kernels.qk_norm_rope_store(wide[:, :cols + extra], q_a, *common, cache_a.data_ptr(), cache_a.stride(0), cache_a.stride(1), *sizes,
                                   partial=parts.to(dev), splits=3, bias=bias.to(dev))
        kernels.qk_norm_rope_store(done.to(dev), q_b, *common, cache_b.data_ptr(), cache_b.stride(0), cache_b.stride(1), *sizes)
        assert torch.equal(wide[:, :cols + extra].cpu(), done) and (wide[:, cols + extra:] == 7.0).all()
        assert torch.equal(q_a[:, :H * hd], q_b[:, :H * hd]) and torch.equal(cache_a, cache_b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_gate_kernel(dtype):
    """A gate per element and a gate per head, on heads whose rows are wider than their values; the gates are columns of a
    wider array."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(6)
    # (gates that start at column 16 of rows of a multiple of eight elements are on 16-byte borders: eight elements a thread)
    for H, hd, Vd, at, behind in ((3, 32, 20, 11, 3), (8, 96, 96, 11, 3), (1, 16, 5, 11, 3), (5, 64, 64, 11, 3), (8, 96, 96, 16, 0), (5, 64, 64, 16, 8),
                                  (4, 128, 64, 16, 0), (3, 32, 24, 8, 0)):
        n = 7
        for each in (True, False):
            o = torch.randn(n, H * hd).to(dtype)
            wide = torch.randn(n, at + (H * Vd if each else H) + behind).to(dtype)
            g = wide[:, at:at + (H * Vd if each else H)]
            od, wd = o.cuda(), wide.cuda()
            kernels.sigmoid_gate(od, wd[:, at:at + g.shape[1]], H, hd, Vd, each)
            s = torch.sigmoid(g.double())
            want = o.double().view(n, H, hd).clone()
            want[:, :, :Vd] *= s.view(n, H, Vd) if each else s.view(n, H, 1)
            got = od.cpu().double().view(n, H, hd)
            tol = 1e-6 if dtype == torch.float32 else 1e-2
            assert (got[:, :, :Vd] - want[:, :, :Vd]).abs().max() < tol * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_norms_of_one_row_in_one_kernel(dtype):
    """A second weight and a second output in the norm kernels, alone and behind the sum of a product's partial sums: every width
    and row count that chooses another kernel (scalar and 16-byte, one block a row and a cluster of blocks a row)."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(8)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for n, d in ((1, 68), (3, 250), (9, 256), (5, 1024), (40, 1024), (100, 1024), (70, 2048), (8, 2048), (20, 4096), (2, 9000)):
        x = torch.randn(n, d) * 3.0
        w1, w2 = 1.0 + 0.1 * torch.randn(d), 1.0 + 0.1 * torch.randn(d)
        unit = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5)
        o1, o2 = (torch.full((n, d), 7.0, dtype=dtype, device="cuda") for _ in range(2))
        kernels.rmsnorm(x.cuda(), w1.cuda(), o1, 1e-5, None, w2.cuda(), o2)
        for o, w in ((o1, w1), (o2, w2)):
            assert (o.cpu().double() - unit * w.double()).abs().max() < tol * 8, (n, d)
        # behind a sum: x += the splits' partial sums + bias, then both norms of the new row
        for splits in (1, 3, 17):
            part = torch.randn(splits, n, d)
            bias = torch.randn(d)
            xd = x.cuda()
            o1.fill_(7.0), o2.fill_(7.0)
            kernels.finish_add_rmsnorm(part.cuda(), splits, bias.cuda(), xd, w1.cuda(), o1, 1e-5, w2.cuda(), o2)
            new = x.double() + part.double().sum(0) + bias.double()
            assert (xd.cpu().double() - new).abs().max() < 1e-4
            unit = new / torch.sqrt((new ** 2).mean(-1, keepdim=True) + 1e-5)
            for o, w in ((o1, w1), (o2, w2)):
                assert (o.cpu().double() - unit * w.double()).abs().max() < tol * 8, (n, d, splits)
            # without the second norm the first is what it was
            xd, alone = x.cuda(), torch.empty_like(o1)
            kernels.finish_add_rmsnorm(part.cuda(), splits, bias.cuda(), xd, w1.cuda(), alone, 1e-5)
            assert torch.equal(alone, o1)


def test_stream_step_kernel():
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(7)
    for n, W in ((1, 68), (9, 256), (130, 40)):
        x, x0, v = torch.randn(n, W), torch.randn(n, W), torch.randn(W)
        for use0, usev in ((True, True), (False, True), (True, False)):
            xd = x.cuda()
            kernels.stream_step(xd, x0.cuda() if use0 else None, v.cuda() if usev else None)
            want = x + (x0 if use0 else 0) + (v if usev else 0)
            assert torch.equal(xd.cpu(), want) or (xd.cpu() - want).abs().max() < 1e-6


# ---- tokens crafted so that one key stands out ----------------------------------------------------------------------------
def _seeker(kind, score=14.0, sink=None):
    """A one-layer model with two special tokens: `B` (id 1) and `A` (id 0).  A's embedding is solved so that the query of every
    head of A points along B's key, and the score scale is set so that this one score is `score` (the others scatter around 0
    with a spread of about 3): A's output is B's value wherever B stands before it.  `sink`: the value of every head's sink."""
    if kind == "sink":
        cfg = tp.model(40, 64, 1e-5, [tp.layer(tp.sink_attention(2, 1, 16, 24, 1.0, 0.5, 64), None)])
    else:
        cfg = tp.model(40, 64, 1e-5, [tp.layer(tp.rotary_attention(2, 1, 16, 24, 1.0, 10000.0, 2), None)])
    t = tp.draw(cfg, 41)
    if kind == "sink":
        t["l0.mix.sink"] = torch.full((2,), 0.0 if sink is None else float(sink)).to(torch.bfloat16)
    else:
        t["l0.mix.q.b"] = torch.zeros_like(t["l0.mix.q.b"])           # (the keys keep their bias)
    w = {k: v.double() for k, v in t.items()}
    h_b = P.norm_one_plus(w["embed"][1][None], w["l0.norm1"], 1e-5)[0]
    k_b = w["l0.mix.k"] @ h_b
    if kind == "sink":
        k_b = P.unit_rms(k_b[None], 1e-5)[0]
    else:
        k_b = k_b + w["l0.mix.k.b"]
    k_dir = k_b.clone()
    if kind != "sink":
        k_dir[0] = k_dir[1] = 0                                       # leave the rotated pair out of it
    y = torch.linalg.pinv(w["l0.mix.q"]) @ torch.cat([k_dir, k_dir])  # W_q y = the wanted direction, both heads
    t["embed"][0] = (y / (1.0 + w["l0.norm1"]) * 3.0 / y.abs().max()).to(torch.bfloat16)
    h_a = P.norm_one_plus(t["embed"][0].double()[None], w["l0.norm1"], 1e-5)[0]
    q_a = (w["l0.mix.q"] @ h_a).view(2, 16)
    if kind == "sink":
        q_a = P.unit_rms(q_a, 1e-5)
        dots = q_a @ k_b
    else:
        dots = q_a[:, 2:] @ k_b[2:]
    cfg["layers"][0]["mixer"]["scale"] = float(score / dots.min())
    return cfg, t


def _standout_cases(cfg, page):
    """(tokens, place of A) with B one token, half a page, a page and several pages before A, A and B on either side of page
    borders and among the very first tokens; fillers are ids >= 2."""
    rng = np.random.RandomState(page)
    cases = []
    for pa, dist in ((1, 1), (2, 2), (page - 1, page - 1), (page, 1), (page, page), (2 * page - 1, page // 2), (2 * page, page + 1),
                     (5 * page + 3, 5 * page + 3), (5 * page + 3, 4 * page + 4), (7 * page, 6 * page), (7 * page - 1, 7 * page - 2)):
        toks = [int(x) for x in rng.randint(2, cfg["vocab"], size=pa + 4)]
        toks[pa - dist], toks[pa] = 1, 0
        cases.append((toks, pa))
    return cases


@pytest.mark.parametrize("kind", ["sink", "rotary"])
def test_a_key_that_stands_out_at_page_borders_and_among_the_first_tokens(kind):
    page = 8
    cfg, t = _seeker(kind)
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tp.make_folder(tmp, None, t, cfg)
        sessions = {dtype: Session(path, dtype, page, 128) for dtype in ("float32", "bfloat16")}
        for toks, pa in _standout_cases(cfg, page):
            ref = tp.plain_logits(cfg, t, toks)
            # the crafted token does what it is made for: with B out of the way A's logits are quite other ones
            moved = list(toks)
            moved[toks.index(1)] = 2
            assert np.abs(tp.plain_logits(cfg, t, moved)[pa] - ref[pa]).max() > 0.05 * np.abs(ref[pa]).max(), (kind, pa)
            for dtype in ("float32", "bfloat16"):
                for steps in (traces.whole({"a": toks}),                                             # A inside a prompt
                              traces.tail_decoded({"a": toks}, len(toks) - pa + 1),                  # A decoded alone
                              traces.portions({"a": toks}, sizes=(pa, 2, 1, 3)),                     # A first of a portion of two
                              traces.portions({"a": toks}, sizes=(3, 2))):
                    got = traces.collect(steps, sessions[dtype].play(steps), cfg["vocab"])["a"]
                    close(got, ref, dtype, f"{kind}: A at {pa}", cfg, t, toks, (kind, pa, toks.index(1)))


def test_a_far_key_among_hundreds():
    """B at place 5, A 500 tokens later: A's logits hang on B across dozens of pages, in a prompt and decoded."""
    for kind in ("sink", "rotary"):
        cfg, t = _seeker(kind, score=18.0)
        toks = [int(x) for x in np.random.RandomState(9).randint(2, cfg["vocab"], size=520)]
        toks[5], toks[505] = 1, 0
        ref = tp.plain_logits(cfg, t, toks)
        moved = list(toks)
        moved[5] = 2
        assert np.abs(tp.plain_logits(cfg, t, moved)[505] - ref[505]).max() > 0.05 * np.abs(ref[505]).max()
        with tempfile.TemporaryDirectory() as tmp:
            path, _, _ = tp.make_folder(tmp, None, t, cfg)
            for dtype in ("float32", "bfloat16"):
                for steps in (traces.whole({"a": toks}), traces.tail_decoded({"a": toks}, 40), traces.portions({"a": toks}, sizes=(97, 2, 150))):
                    res, _ = run(path, dtype, steps, page_size=16)
                    close(traces.collect(steps, res, cfg["vocab"])["a"], ref, dtype, "far key", cfg, t, toks, ("far", kind))


@pytest.mark.parametrize("offset", [-30.0, -1.0, 3.0])
def test_a_sink_beside_a_key_that_stands_out(offset):
    """One score that stands out and a sink far below it, within reach of it, and above it: the sink takes nothing, a part, or nearly
    all of A's softmax.  A sink that is left out, counted per key range or scaled shows at once."""
    factor = 1.0 + 0.5 * math.log(401 // 64 + 1)               # the query factor at A's place: it scales the crafted score of 14
    sink = 14.0 * factor + offset
    cfg, t = _seeker("sink", sink=sink)
    toks = [int(x) for x in np.random.RandomState(3).randint(2, cfg["vocab"], size=420)]
    toks[7], toks[400], toks[2] = 1, 0, 0
    ref = tp.plain_logits(cfg, t, toks)
    without = copy.deepcopy(t)
    without["l0.mix.sink"] = torch.full((2,), -30.0).to(torch.bfloat16)
    moved = np.abs(tp.plain_logits(cfg, without, toks)[400] - ref[400]).max() / np.abs(ref[400]).max()
    assert (moved > 0.02) == (offset > -10), moved
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tp.make_folder(tmp, None, t, cfg)
        for dtype in ("float32", "bfloat16"):
            for page, steps in ((16, traces.whole({"a": toks})), (16, traces.tail_decoded({"a": toks}, 30)), (64, traces.tail_decoded({"a": toks}, 30)),
                                (8, traces.portions({"a": toks}, sizes=(399, 2, 1, 5))), (64, traces.portions({"a": toks}, sizes=(130, 2)))):
                res, _ = run(path, dtype, steps, page_size=page)
                close(traces.collect(steps, res, cfg["vocab"])["a"], ref, dtype, f"sink {offset:+}", cfg, t, toks, ("sinkcase", offset))


def test_sinks_in_kernels_of_every_head_size():
    """Sinks that outweigh the keys on some heads and vanish on others, with head sizes that go to the tcgen05 prompt kernel (64,
    128), to the mma kernels alone (48, 96) and, in float32, to the plain-arithmetic kernel; long enough for several key ranges."""
    for D, V, page in ((64, 64, 64), (128, 128, 64), (48, 96, 32), (32, 16, 16), (24, 200, 16)):
        cfg = tp.model(50, 64, 1e-5, [tp.layer(tp.sink_attention(4, 2, D, V, 2.0 / D, 0.4, 100), None)])
        t = tp.draw(cfg, D)
        t["l0.mix.sink"] = torch.tensor([6.0, -6.0, 2.0, 0.0]).to(torch.bfloat16)
        toks = traces.random_tokens(D, 700, 50)
        ref = tp.plain_logits(cfg, t, toks)
        with tempfile.TemporaryDirectory() as tmp:
            path, _, _ = tp.make_folder(tmp, None, t, cfg)
            for dtype in ("float32", "bfloat16"):
                for steps in (traces.whole({"a": toks}), traces.tail_decoded({"a": toks}, 20), traces.portions({"a": toks}, sizes=(300, 2, 250, 1, 40))):
                    res, _ = run(path, dtype, steps, page_size=page)
                    close(traces.collect(steps, res, 50)["a"], ref, dtype, f"sinks D={D} V={V}", cfg, t, toks, ("sinks", D))


@pytest.mark.parametrize("every", [16, 5])
def test_the_query_factor_steps_at_the_right_token(every):
    """A large coefficient: the factor doubles the queries at the token whose number (from one) reaches `every`, at a page's last
    row (every = page) and inside one; in prompts, between decoded tokens and at the start of a portion."""
    cfg = tp.model(50, 48, 1e-5, [tp.layer(tp.sink_attention(2, 1, 16, 16, 0.5, 1.5, every), 32)])
    t = tp.draw(cfg, 77)
    toks = traces.random_tokens(every, 3 * every + 4, 50)
    ref = tp.plain_logits(cfg, t, toks)
    late = copy.deepcopy(cfg)
    late["layers"][0]["mixer"]["q_temp"]["every"] = every + 1
    other = tp.plain_logits(late, t, toks)
    assert np.abs(other[every - 1] - ref[every - 1]).max() > 0.02 * np.abs(ref).max()      # a step one token late shows
    assert np.abs(other[every - 2] - ref[every - 2]).max() < 1e-6
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tp.make_folder(tmp, None, t, cfg)
        for dtype in ("float32", "bfloat16"):
            for steps in (traces.whole({"a": toks}), traces.tail_decoded({"a": toks}, 2 * every + 6), traces.portions({"a": toks}, sizes=(every - 1, 2, every - 2, 1, 2)),
                          traces.portions({"a": toks}, sizes=(2,))):
                res, _ = run(path, dtype, steps, page_size=16)
                close(traces.collect(steps, res, 50)["a"], ref, dtype, f"query factor every {every}", cfg, t, toks, ("qtemp", every))


# ---- other sizes, drawn -----------------------------------------------------------------------------------------------------
def _drawn_config(rng, layer_sizes=False):
    pick = lambda *xs: xs[rng.randint(len(xs))]
    layers = []
    L = int(rng.randint(1, 6))
    for i in range(L):
        ff = pick(None, 24, 40, 72) if not layer_sizes else pick(None, 128, 320)
        kv = pick(1, 2, 3) if not layer_sizes else pick(1, 2, 4)
        if layer_sizes:
            D, V = pick(32, 64, 80, 128), pick(32, 64, 128)
        else:
            D, V = pick(4, 10, 16, 24, 36), pick(4, 12, 16, 30, 40)
        H = kv * pick(1, 2, 4)
        scale = pick(0.5, 1.0, 2.0) / math.sqrt(D)
        if rng.rand() < 0.5:
            qt = pick(None, (0.2, 1), (0.9, 6), (0.4, 33), (0.1, 1000))
            layers.append(tp.layer(tp.sink_attention(H, kv, D, V, scale, *(qt or ())), ff))
        else:
            dims = pick(0, 2, D // 2 * 2, (D // 4) * 2)
            layers.append(tp.layer(tp.rotary_attention(H, kv, D, V, scale, pick(10.0, 1e4, 5e5), dims), ff))
    loop = None
    if rng.rand() < 0.7:
        a = int(rng.randint(0, L))
        loop = (a, int(rng.randint(a + 1, L + 1)), int(rng.randint(1, 4)))
    return tp.model(pick(70, 130, 300), pick(36, 64, 100) if not layer_sizes else pick(128, 192), pick(1e-5, 1e-6, 1e-3), layers, loop=loop,
                    embedding_scale=pick(1.0, 0.3, 6.0))


@pytest.mark.parametrize("seed", range(12))
def test_drawn_configurations(seed):
    rng = np.random.RandomState(2000 + seed)
    cfg = _drawn_config(rng, layer_sizes=seed >= 8)
    t = tp.draw(cfg, 90 + seed)
    page = int(rng.choice([4, 8, 16, 64])) if seed < 8 else 64
    reqs = {f"r{i}": traces.random_tokens(11 * seed + i, n, cfg["vocab"]) for i, n in enumerate((3, 90, 17, 140, 1, 45))}
    ref = {rid: tp.plain_logits(cfg, t, toks) for rid, toks in reqs.items()}
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tp.make_folder(tmp, None, t, cfg)
        for dtype in ("float32", "bfloat16"):
            for cut in ("whole", "mixed"):
                steps = CUTS[cut](reqs)
                res, _ = run(path, dtype, steps, page)
                got = traces.collect(steps, res, cfg["vocab"])
                for rid in reqs:
                    close(got[rid], ref[rid], dtype, f"drawn {seed}/{cut}/{dtype}/{rid}: {cfg['layers']} {cfg['loop']}", cfg, t, reqs[rid],
                          ("drawn", seed, rid))


def test_wide_heads_and_long_prompts():
    """Heads of 80 to 256 elements (values of 48 to 256), 20 heads over one key head, a rotation over the whole head, a loop over three
    layers, prompts of several hundred tokens: whole, with a decoded tail and in mixed batches, in both precisions."""
    cfg = tp.model(1000, 320, 1e-5, [
        tp.layer(tp.sink_attention(10, 5, 80, 112, 0.11, 0.3, 256), 640),
        tp.layer(tp.rotary_attention(12, 3, 160, 64, 0.08, 10000.0, 80), 512),
        tp.layer(tp.sink_attention(6, 6, 192, 192, 0.07, 0.5, 100), None),
        tp.layer(tp.rotary_attention(4, 1, 256, 256, 0.0625, 500000.0, 256), 256),
        tp.layer(tp.rotary_attention(20, 1, 32, 48, 0.17, 100.0, 16), 384)], loop=(1, 4, 2), embedding_scale=16.0)
    t = tp.draw(cfg, 77)
    reqs = {f"r{i}": traces.random_tokens(31 * i + 5, n, cfg["vocab"]) for i, n in enumerate((700, 3, 260, 129))}
    ref = {rid: tp.plain_logits(cfg, t, toks) for rid, toks in reqs.items()}
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tp.make_folder(tmp, None, t, cfg)
        for dtype in ("float32", "bfloat16"):
            for cut in ("whole", "tail", "mixed"):
                steps = CUTS[cut](reqs)
                res, _ = run(path, dtype, steps, 64)
                got = traces.collect(steps, res, cfg["vocab"])
                for rid in reqs:
                    close(got[rid], ref[rid], dtype, f"wide/{cut}/{dtype}/{rid}", cfg, t, reqs[rid], ("wide", rid))


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
            assert g.tokens == tp.plain_greedy(cfg, tensors, p, 12)
        else:
            # teacher-forced: every token is the plain argmax for the engine's own prefix, or within rounding of it
            for i, tok in enumerate(g.tokens):
                lg = tp.plain_logits(cfg, tensors, list(p) + list(g.tokens[:i]))[-1]
                assert lg.max() - lg[tok] <= 0.06 * np.abs(lg).max()


def test_command_line_generates_what_the_plain_implementation_does(models):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, tensors, _, _ = models["loop"]
    prompt = traces.random_tokens(9, 7, cfg["vocab"])
    ids = "ids:" + ",".join(str(t) for t in prompt)
    out = {}
    for extra in (["--dtype", "float32"], ["--ref"]):
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "runner"), "-m", path, "-p", ids, "-n", "6", "--ignore-eos"] + extra,
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        out[extra[-1]] = [ln for ln in r.stdout.splitlines() if ln.startswith("ids:")][0]
    want = "ids:" + ",".join(str(t) for t in tp.plain_greedy(cfg, tensors, prompt, 6))
    assert out["--ref"] == want and out["float32"] == want, out


def test_trace_runner_program(models):
    """bin/trace_run on a folder: steps on standard input, logits in files, a line per step."""
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
