"""Mokatar on the GPU against the plain implementation: each kernel and each mechanism alone, whole prompts against
token-by-token decoding, prompts fed in portions, unequal batches, pages, slots and state rows used again, keys far
back, on the pages' borders and on either side of the window's and the kept tokens' edges, the sink's share, state
carried from the first token, the token in front across a step's border, long decoding, looped layers with a cache per
pass, generation through the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TOL
from plain import mokatar_plain as M
from mokatar_helpers import (assert_rows_close as assert_close, biased, clear_tokens, config, dense, gla, layer, make,
                             moe, plain_logits, windowed)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _engine(path, dtype, max_tokens=1024):
    from stratum_b200.engine import Engine, load_model
    model, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    return Engine(model, max_tokens=max_tokens)


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "TC") for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    path, cfg, w = make(str(tmp_path_factory.mktemp(f"mok{name}_{dtype}")), name, dtype, seed=len(name) + 1)
    return name, dtype, cfg, w, _engine(path, dtype), path


def _dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()


def _i32(a):
    return _dev(np.asarray(a), torch.int32)


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("heads,dim,vdim,rank", [(3, 12, 20, 10), (2, 40, 8, 4), (1, 9, 7, 3), (4, 64, 32, 16),
                                                 (2, 130, 70, 5), (1, 260, 8, 2), (5, 16, 16, 1), (2, 8, 4, 8)])
@pytest.mark.parametrize("long", [77, 520])
def test_gla_kernels(heads, dim, vdim, rank, long):
    """The three kernels of gated linear attention on projections made here: two sequences of unequal lengths whose
    tokens come in three steps (many, three and two, one), states in slots that lie apart, against the plain loop over
    whole sequences."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(dim + vdim)
    HD, HV = heads * dim, heads * vdim
    width = 2 * HD + 2 * HV + rank
    lens = (long, 9)
    proj = [rng.standard_normal((n, width)) for n in lens]
    w_a2, b_a2 = rng.standard_normal((HD, rank)) * 0.5, rng.uniform(0.0, 5.0, HD)
    gain, tau = rng.uniform(0.5, 1.5, vdim), 3.0
    # the plain mixer, fed the projections directly: pieces of the identity in place of the weights
    eye = np.eye(width)
    w = {"q": eye[:HD], "k": eye[HD:2 * HD], "v": eye[2 * HD:2 * HD + HV], "g": eye[2 * HD + HV:2 * HD + 2 * HV],
         "a1": eye[2 * HD + 2 * HV:], "a2": w_a2, "a2.b": b_a2, "norm": gain, "o": np.eye(HV)}
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    want = [M.gla(m, w, "", p, 1e-5) for p in proj]
    st = torch.zeros(6, HD * vdim + 3, device="cuda")
    slots = (4, 1)
    done = [0, 0]
    got = [[], []]
    for cut in ((long - 4, 6), (3, 2), (1, 1)):
        rows_ = np.concatenate([proj[i][done[i]:done[i] + cut[i]] for i in range(2)])
        T = rows_.shape[0]
        seq = np.concatenate([np.full(cut[i], i) for i in range(2)])
        g = K.GlaStep(_dev(rows_), heads, dim, vdim, rank, tau, dim ** -0.5, 1e-5)
        inner = torch.empty(T, rank + 3, device="cuda")
        g.cast(inner)
        assert torch.equal(inner[:, :rank], _dev(rows_)[:, width - rank:])
        z = (inner[:, :rank].double() @ _dev(w_a2, torch.float64).T + _dev(b_a2, torch.float64)).float().contiguous()
        g.decay(z)                                            # the second projection is the caller's product
        o_raw = torch.empty(T, HV, device="cuda")
        out = torch.empty(T, HV + 5, device="cuda")
        g.recur(o_raw, st, _i32(seq), _i32([0, cut[0], T]), _i32(slots), True)
        g.finish(_dev(gain), out)
        o = out[:, :HV].cpu().numpy()
        got[0].append(o[:cut[0]]); got[1].append(o[cut[0]:])
        done = [done[i] + cut[i] for i in range(2)]
    for i in range(2):
        g = np.concatenate(got[i])
        assert np.isfinite(g).all()
        assert np.max(np.abs(g - want[i])) <= 3e-5 * np.max(np.abs(want[i])), (i, np.max(np.abs(g - want[i])))
    assert float(st[0].abs().max()) == 0.0 and float(st[5].abs().max()) == 0.0            # rows of nobody stay clean
    assert float(st[:, HD * vdim:].abs().max()) == 0.0                                    # nothing beyond a state


def test_gla_kernel_leaves_the_state_alone_when_told_to():
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(3)
    heads, dim, vdim, rank, T = 2, 8, 16, 3, 5
    HD, HV = heads * dim, heads * vdim
    st = _dev(rng.standard_normal((2, HD * vdim)))
    before = st.clone()
    out = torch.empty(T, HV, device="cuda")
    g = K.GlaStep(_dev(rng.standard_normal((T, 2 * HD + 2 * HV + rank))), heads, dim, vdim, rank, 2.0, 1.0, 1e-5)
    g.decay(_dev(rng.standard_normal((T, HD))))
    g.recur(torch.empty(T, HV, device="cuda"), st, torch.zeros(T, dtype=torch.int32, device="cuda"), _i32([0, T]),
            _i32([1]), False)
    g.finish(torch.ones(vdim, device="cuda"), out)
    assert torch.equal(st, before) and bool(torch.isfinite(out).all())


def _paged(k, pages_of, n_pages, page=64):
    """k [T, G, D] of one sequence -> cache [n_pages, G, page, D] filled through the page list `pages_of`."""
    T, G, D = k.shape
    cache = np.zeros((n_pages, G, page, D))
    for t in range(T):
        cache[pages_of[t // page], :, t % page] = k[t]
    return cache


@pytest.mark.parametrize("per_head,half,own_values", [(True, False, True), (False, True, True), (False, False, False),
                                                      (True, True, True)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_qk_norm_rope_forms(per_head, half, own_values, dtype):
    """Norm over a head or over the whole projection, neighbouring pairs or halves, a magnitude on cos and sin, values
    of their own size or the keys as projected; tokens of two sequences at positions that lie in pages used before."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(7)
    H, G, D, Dv, pairs = 4, 2, 12, 20, 4
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    pos = np.array([0, 1, 2, 64, 65, 130], dtype=np.int64)
    seq = np.array([0, 0, 0, 1, 1, 1])
    T = len(pos)
    width = H * D + G * D + (G * Dv if own_values else 0)
    proj = rng.standard_normal((T, width)) * 2
    qg = rng.uniform(0.5, 1.5, D if per_head else H * D)
    kg = rng.uniform(0.5, 1.5, D if per_head else G * D)
    f, mag = rng.uniform(0.01, 1.0, pairs), 1.3
    table = np.array([[5, 2, -1], [3, 0, 7]])                 # sequence 1 holds pages 3, 0, 7
    kc = torch.full((8, G, 64, D), 9.0, dtype=td, device="cuda")
    vc = torch.full((8, G, 64, Dv if own_values else D), 9.0, dtype=td, device="cuda")
    q_out = torch.empty(T, H * D + 8, dtype=td, device="cuda")
    K.qk_norm_rope(_dev(proj), _i32(pos), _i32(seq), _i32(table), _dev(qg), _dev(kg), _dev(f), 1e-5, q_out, kc, vc, H, G,
                   D, 64, True, v_dim=Dv if own_values else 0, per_head=per_head, half=half, magnitude=mag)
    q, k = proj[:, :H * D], proj[:, H * D:(H + G) * D]
    if per_head:
        qn = M.rms_norm(q.reshape(T, H, D), qg, 1e-5)
        kn = M.rms_norm(k.reshape(T, G, D), kg, 1e-5)
    else:
        qn, kn = M.rms_norm(q, qg, 1e-5).reshape(T, H, D), M.rms_norm(k, kg, 1e-5).reshape(T, G, D)
    qn, kn = M.rotate(qn, pos, f, mag, not half), M.rotate(kn, pos, f, mag, not half)
    tol = 1e-5 if dtype == "float32" else 5e-3                # float32: the angle position * f is a float32 product
    assert np.max(np.abs(q_out[:, :H * D].float().cpu().numpy() - qn.reshape(T, -1))) <= tol * np.max(np.abs(qn))
    vals = proj[:, (H + G) * D:].reshape(T, G, Dv) if own_values else k.reshape(T, G, D)
    for t in range(T):
        page = table[seq[t], pos[t] // 64]
        got_k = kc[page, :, pos[t] % 64].float().cpu().numpy()
        got_v = vc[page, :, pos[t] % 64].float().cpu().numpy()
        assert np.max(np.abs(got_k - kn[t])) <= tol * np.max(np.abs(kn))
        assert np.max(np.abs(got_v - vals[t])) <= tol * np.max(np.abs(vals))
    assert float((kc != 9.0).sum()) == T * G * D             # nothing else was written


@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 12, 20), (3, 3, 20, 22), (8, 1, 64, 64), (2, 2, 33, 5)])
def test_windowed_attention_kernel_with_kept_first_keys_and_sink(H, G, D, Dv):
    """The float32 attention kernel over the paged cache: a window, first keys that stay visible, a sink per head;
    every position of a prompt and of tokens decoded alone, keys in pages that lie anywhere."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(D)
    T = 330
    q, k, v = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, G, Dv))
    sink = rng.uniform(-1.0, 3.0, H)
    pages_of = [6, 2, 9, 0, 4, 7]
    kc, vc = _dev(_paged(k, pages_of, 10)), _dev(_paged(v, pages_of, 10))
    table = _i32([pages_of])
    for window, keep in ((40, 5), (130, 70), (5, 0), (64, 64), (33, 200), (0, 0)):
        want = M.masked_softmax_attention(q, k, v, 0.3, sink, window, keep)
        shape = K.AttentionShape(H, H // G, 1, D, Dv, False, 0.3, window=window, sink=_dev(sink), keep_first=keep)
        out = torch.empty(T, H * Dv, device="cuda")
        K.attention_general(shape, _dev(q.reshape(T, -1)), kc, vc, _i32(np.arange(T)), _i32(np.zeros(T)), table, out, 64)
        err = np.max(np.abs(out.cpu().numpy().reshape(T, H, Dv) - want))
        assert err <= 2e-5 * np.max(np.abs(want)), (window, keep, err)
        rows = [0, 1, keep, max(keep - 1, 0), window + keep, 255, 256, T - 1]
        rows = sorted({min(max(r, 0), T - 1) for r in rows})
        one = torch.empty(len(rows), H * Dv, device="cuda")
        K.attention_general(shape, _dev(q[rows].reshape(len(rows), -1)), kc, vc, _i32(rows),
                            _i32(np.zeros(len(rows))), table, one, 64)
        assert np.max(np.abs(one.cpu().numpy().reshape(-1, H, Dv) - want[rows])) <= 2e-5 * np.max(np.abs(want))


def test_pair_embedding_kernel_and_its_state():
    """Rows chosen by the token and the one in front: inside a step, across two steps of the same slot (from the
    state), and for a sequence's first token; a slot that is not in a step keeps its entry."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    vocab, width, buckets, mp, mc, scale = 50, 24, 17, 7, 13, 2.5
    table, pairs = rng.standard_normal((vocab, width)), rng.standard_normal((buckets + 1, width))
    last = torch.full((5, 1), 41, dtype=torch.int32, device="cuda")
    row = lambda prev, tok: buckets if prev is None else (prev * mp + tok * mc) % buckets      # noqa: E731
    want = lambda prev, tok: table[tok] * scale + pairs[row(prev, tok)]                        # noqa: E731

    def run(ids, pos, seq, start, slots, keep=False):
        out = torch.empty(len(ids), width, device="cuda")
        out2 = torch.empty(len(ids), width, device="cuda") if keep else None
        K.embed_pairs(_dev(table), _dev(pairs), _i32(ids), _i32(pos), _i32(seq), _i32(start), _i32(slots), last, out,
                      out2, scale, mp, mc, True)
        if keep:
            assert torch.equal(out, out2)
        return out.cpu().numpy()
    # step 1: sequence A (slot 3) brings 3 tokens from its start, sequence B (slot 0) one token at position 9
    got = run([4, 5, 6, 7], [0, 1, 2, 9], [0, 0, 0, 1], [0, 3, 4], [3, 0], keep=True)
    ref = np.stack([want(None, 4), want(4, 5), want(5, 6), want(41, 7)])
    assert np.max(np.abs(got - ref)) <= 1e-6 * np.max(np.abs(ref))
    assert last.flatten().tolist() == [7, 41, 41, 6, 41]
    # step 2: one token each (the sequences in the other order), and a row of no sequence
    got = run([8, 9, 3], [10, 3, 0], [0, 1, -1], [0, 1, 2, 3], [0, 3, 4])
    ref = np.stack([want(7, 8), want(6, 9), want(None, 3)])
    assert np.max(np.abs(got - ref)) <= 1e-6 * np.max(np.abs(ref))
    assert last.flatten().tolist() == [8, 41, 41, 9, 41]
    bf = torch.empty(1, width, device="cuda")
    K.embed_pairs(_dev(table, torch.bfloat16), _dev(pairs, torch.bfloat16), _i32([2]), _i32([11]), _i32([0]),
                  _i32([0, 1]), _i32([0]), last, bf, None, scale, mp, mc, False)
    assert last[0, 0].item() == 8                             # told to leave the state alone
    t16, p16 = _dev(table, torch.bfloat16).float().cpu().numpy(), _dev(pairs, torch.bfloat16).float().cpu().numpy()
    assert np.allclose(bf.cpu().numpy()[0], t16[2] * scale + p16[row(8, 2)], atol=1e-5)


@pytest.mark.parametrize("experts,top", [(6, 2), (8, 3), (12, 4), (5, 1), (4, 4), (40, 6)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_router_with_a_bias_and_weights_over_the_chosen(experts, top, dtype):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(experts)
    T, width = 33, 72
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    x = _dev(rng.standard_normal((T, width)), td)
    wr, b = rng.standard_normal((experts, width)) * 0.7, rng.uniform(-2, 2, experts)
    dense_w = torch.empty(T, experts, device="cuda")
    chosen = torch.empty(T, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(T, top, device="cuda")
    K.moe_route(x, _dev(wr), None, dense_w, chosen, weights, top, 1, 1, 1.0, softmax=True, renorm=True, bias=_dev(b))
    f = {"router": {"experts": experts, "top": top}}
    margins = []
    c_ref, w_ref = M.route(f, {"router": wr.astype(np.float32), "router.b": b.astype(np.float32)}, "",
                           x.float().cpu().numpy(), margins)
    for t in range(T):
        if margins and margins[t] < 1e-4:
            continue
        assert sorted(chosen[t].tolist()) == sorted(c_ref[t].tolist())
        by_expert = dict(zip(c_ref[t].tolist(), w_ref[t]))
        for e, wgt in zip(chosen[t].tolist(), weights[t].tolist()):
            assert abs(wgt - by_expert[e]) <= 2e-5
            assert abs(dense_w[t, e].item() - wgt) == 0.0
        assert abs(float(dense_w[t].sum()) - 1.0) <= 1e-5


def test_add_rows_kernel():
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    x, a, r = rng.standard_normal((37, 70)), rng.standard_normal((37, 70)), rng.standard_normal(70)
    xd = _dev(x)
    K.add_rows(xd, _dev(a), _dev(r))
    assert np.allclose(xd.cpu().numpy(), x + a + r, atol=1e-6)
    xd = _dev(x)
    K.add_rows(xd, None, _dev(r))
    assert np.allclose(xd.cpu().numpy(), x + r, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_norms_from_one_pass(dtype):
    """Both sublayers' norms of the same rows: the plain norm twice, and the bits of the one-output kernel."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    for rows, width in ((1, 72), (5, 70), (300, 512), (3, 4100), (260, 2048)):
        x = rng.standard_normal((rows, width)) * 3
        ga, gb = rng.uniform(0.5, 1.5, width), rng.uniform(-0.5, 2.0, width)
        a, b = torch.empty(rows, width, dtype=td, device="cuda"), torch.empty(rows, width, dtype=td, device="cuda")
        K.rmsnorm_pair(_dev(x), _dev(ga), _dev(gb), 1e-5, a, b)
        tol = 3e-6 if dtype == "float32" else 5e-3
        for got, g in ((a, ga), (b, gb)):
            want = M.rms_norm(x, g, 1e-5)
            assert np.max(np.abs(got.float().cpu().numpy() - want)) <= tol * np.max(np.abs(want))
            one = torch.empty(rows, width, dtype=td, device="cuda")
            K.rmsnorm(_dev(x), _dev(g), 1e-5, one)
            assert torch.equal(one, got)


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["windowed", "biased", "gla", "moe", "dense", "loop"])
def test_each_mechanism_alone(name, dtype, tmp_path):
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / name), name, dtype, seed=3)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(1)
    for n in (1, 2, 7, 100):
        toks = clear_tokens(rng, n, cfg, w, dtype)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        engine.release(slot)
        assert_close(got, plain_logits(cfg, w, toks), dtype, f"{name} n={n}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_model_without_pair_table_rotation_window_and_loop(dtype, tmp_path):
    """What a file does not mention does not exist: the same layers with those keys left out."""
    import copy
    from mokatar_helpers import MOK_A
    from stratum_b200.engine import StepEntry
    raw = copy.deepcopy(MOK_A)
    del raw["embedding"]["bigram"]
    del raw["layers"][0]["mixer"]["rot"]
    del raw["layers"][0]["mixer"]["mask"]
    del raw["layers"][2]["mixer"]["rot"]["scaling"]
    del raw["loop"]
    path, cfg, w = make(str(tmp_path / "bare"), None, dtype, seed=12, cfg=raw)
    assert "bigram" not in w
    engine = _engine(path, dtype)
    toks = clear_tokens(np.random.default_rng(0), 90, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks[:70], list(range(70)))]).cpu().numpy()
    got = np.concatenate([got] + [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks[70:]])
    engine.release(slot)
    assert_close(got, ref, dtype, "a bare model")


def test_the_stream_after_every_layer_run(tmp_path):
    """float32: the residual stream behind every stop of the schedule that is a layer, looped passes included."""
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / "streams"), "A", "float32", seed=5)
    engine = _engine(path, "float32")
    seen = []
    for lay in engine.model.layers:
        arr = lay.arrangement
        if arr.kind == "stream_op":
            continue

        def wrapped(layer_, x, step, cache, _f=arr.forward):
            _f(layer_, x, step, cache)
            seen.append(x.cpu().numpy().copy())
        arr.forward = wrapped
    toks = clear_tokens(np.random.default_rng(0), 40, cfg, w, "float32")
    slot = engine.acquire()
    engine.step([StepEntry(slot, toks, [39])])
    engine.release(slot)
    want = []
    M.forward(cfg, w, toks, want)
    assert len(seen) == len(want) == 8
    for i, (a, b) in enumerate(zip(seen, want)):
        assert np.max(np.abs(a - b)) <= 2e-5 * np.max(np.abs(b)), f"layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_both_ways(dtype, tmp_path, monkeypatch):
    """All experts' matrices stacked into two products, and tokens gathered by expert: the same logits."""
    from stratum_b200.engine import StepEntry
    from stratum_b200.parts import moe as moe_part
    path, cfg, w = make(str(tmp_path / "moe"), "moe", dtype, seed=2)
    toks = clear_tokens(np.random.default_rng(0), 90, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    for rows in (10 ** 9, 0):
        monkeypatch.setattr(moe_part, "GROUPED_MIN_ROWS", rows)
        engine = _engine(path, dtype)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(90)))]).cpu().numpy()
        engine.release(slot)
        assert_close(got, ref, dtype, f"experts, grouped from {rows} rows on")


# ------------------------------------------------------------------------------------------ whole models
def test_whole_prompt_all_positions(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(1)
    for n in (1, 2, 3, 5, 6, 63, 64, 65, 200):
        toks = clear_tokens(rng, n, cfg, w, dtype)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        engine.release(slot)
        assert_close(got, plain_logits(cfg, w, toks), dtype, f"{name} whole n={n}")
    engine.cache.check()


def test_prefill_against_token_by_token(setup):
    """The same tokens whole, and one by one from the first: the same logits (float32: to rounding)."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    n = 150
    toks = clear_tokens(np.random.default_rng(2), n, cfg, w, dtype)
    a, b = engine.acquire(), engine.acquire()
    whole = engine.step([StepEntry(a, toks, list(range(n)))]).cpu().numpy()
    single = np.concatenate([engine.step([StepEntry(b, [t], [0])]).cpu().numpy() for t in toks])
    engine.release(a); engine.release(b)
    ref = plain_logits(cfg, w, toks)
    assert_close(whole, ref, dtype, f"{name} whole")
    assert_close(single, ref, dtype, f"{name} one by one")
    if dtype == "float32":
        assert np.max(np.abs(whole - single)) <= 2e-5 * np.max(np.abs(ref))


def test_the_same_bits_every_run(setup):
    """A batch of prompts and some decoded tokens, three times over in slots, pages and state rows that were just given
    back: every run's logits are the same bits."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(17)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (90, 7, 64, 33)]
    more = [[int(t) for t in rng.integers(0, cfg["vocab"], 6)] for _ in prompts]
    runs = []
    for _ in range(3):
        slots = [engine.acquire() for _ in prompts]
        got = [engine.step([StepEntry(s, p, list(range(len(p)))) for s, p in zip(slots, prompts)]).cpu().numpy()]
        for i in range(6):
            got.append(engine.step([StepEntry(s, [m[i]], [0]) for s, m in zip(slots, more)]).cpu().numpy())
        for s in slots:
            engine.release(s)
        runs.append(np.concatenate(got))
    assert np.isfinite(runs[0]).all()
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2]), f"{name} {dtype}: runs differ"


@pytest.mark.parametrize("portion", [2, 3, 31, 64, 100])
def test_prompt_in_portions(setup, portion):
    """A prompt cut into portions of a few sizes, down to two tokens; portions start inside pages and on their
    borders, and the first token of every portion reads the token in front of it from the sequence's state."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    n = 150 if portion > 3 else 80
    toks = clear_tokens(np.random.default_rng(portion), n, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([StepEntry(slot, toks[i:i + portion], list(range(len(toks[i:i + portion]))))]).cpu().numpy()
           for i in range(0, n, portion)]
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, f"{name} portions of {portion}")


def test_unequal_batches_against_each_alone_slots_reused(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(3)
    for batch_no, lens in enumerate([(5, 9, 12), (1, 67), (70, 3, 33, 64)]):
        extra_n = [3 + 2 * i for i in range(len(lens))]
        full = [clear_tokens(rng, n + k, cfg, w, dtype) for n, k in zip(lens, extra_n)]
        prompts = [f[:n] for f, n in zip(full, lens)]
        extra = [f[n:] for f, n in zip(full, lens)]
        refs = [plain_logits(cfg, w, f) for f in full]
        slots = [engine.acquire() for _ in lens]
        out = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
        alone = []
        for p in prompts:                                   # each alone, in a slot and pages of its own
            s = engine.acquire()
            alone.append(engine.step([StepEntry(s, p, [len(p) - 1])]).cpu().numpy()[0])
            engine.release(s)
        for i, p in enumerate(prompts):
            assert_close(out[i], refs[i][len(p) - 1], dtype, f"{name} batch {batch_no} prompt {i}")
            if dtype == "float32":
                assert np.max(np.abs(out[i] - alone[i])) <= 2e-5 * np.max(np.abs(refs[i]))
        live, step = list(range(len(lens))), 0
        while live:
            out = engine.step([StepEntry(slots[i], [extra[i][step]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                assert_close(out[row], refs[i][len(prompts[i]) + step], dtype, f"{name} batch {batch_no} seq {i} +{step}")
            step += 1
            for i in list(live):
                if step >= len(extra[i]):
                    engine.release(slots[i])
                    live.remove(i)
        engine.cache.check()
    assert engine.cache.tokens_held() == 0


def test_pages_and_slots_used_again(setup):
    """A cache of four pages and few slots: every request takes pages and state rows (one per pass of every looped
    layer, and the embedding's) that another one has just given back."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, _, path = setup
    engine = _engine(path, dtype, max_tokens=256)
    rng = np.random.default_rng(4)
    held = []
    for n in (130, 60, 190, 64, 129):
        while held and engine.cache.tokens_held() + ((n + 63) // 64) * 64 > 256:
            engine.release(held.pop(0))
        toks = clear_tokens(rng, n, cfg, w, dtype)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks[:-1], [n - 2])]).cpu().numpy()
        got = np.concatenate([got, engine.step([StepEntry(slot, toks[-1:], [0])]).cpu().numpy()])
        assert_close(got, plain_logits(cfg, w, toks)[-2:], dtype, f"{name} reuse n={n}")
        held.append(slot)
        engine.cache.check()


def test_first_tokens_and_long_decoding(setup):
    """Positions 0, 1, 2 one by one, then on across several pages and several windows' lengths; a windowed layer
    gives back the pages that fall behind its window and keeps those of its first tokens."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    n = 270
    toks = clear_tokens(np.random.default_rng(5), n, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    check = {0, 1, 2, 3, 4, 5, 6} | set(range(7, n, 29)) | {63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257, n - 1}
    got = []
    for i in range(n):
        out = engine.step([StepEntry(slot, [toks[i]], [0] if i in check else [])])
        if i in check:
            got.append(out.cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref[sorted(check)], dtype, f"{name} long decode")
    engine.cache.check()
    assert engine.cache.tokens_held() == 0


# ------------------------------------------------------------------------------------------ one key decides
def _marked_key_model(path, dtype, kind, big=False):
    """One attention layer in which token 7 is the only one with anything in the embedding's first dimension, and token
    8 the only one with anything in the second.  The last dimension of every key head (which is not rotated) reads the
    first dimension and nothing else, the last dimension of every query head reads the second; with gains of 3 on the
    normalised queries and keys the marked key's score stands far above the hundreds of others when token 8 asks,
    wherever the key lies, and the heads' outputs are its value."""
    if kind == "attention":
        mixer = (windowed(heads=8, kv=1, dim=64, vdim=64, rot=32, size=130, keep=70, scale=0.1, original=32) if big
                 else windowed(heads=4, kv=2, dim=16, vdim=24, rot=8, size=40, keep=5, scale=0.25))
    else:
        mixer = (biased(heads=4, kv=4, dim=32, vdim=48, rot=16, scale=0.15) if big
                 else biased(heads=4, kv=2, dim=16, vdim=24, rot=8, scale=0.25))
    cfg_raw = config([layer(kind, mixer)], vocab=120, width=64, emb_scale=1.0)
    H, G, D = mixer["heads"], mixer["kv_heads"], mixer["dim"]

    def edit(t):
        e = t["embed"].float()
        e[:, :2] = 0.0
        e[7, 0] = e[8, 1] = 24.0
        t["embed"] = e.to(t["embed"].dtype)
        b = t["bigram"].float()
        b[:, :2] = 0.0
        t["bigram"] = b.to(t["bigram"].dtype)
        t["l0.norm1"] = torch.zeros_like(t["l0.norm1"])
        for name, heads, col in (("l0.mix.k", G, 0), ("l0.mix.q", H, 1)):
            m = t[name].float()
            m[:, :2] = 0.0
            for h in range(heads):
                m[h * D + D - 1] = 0.0
                m[h * D + D - 1, col] = 4.0
            t[name] = m.to(t[name].dtype)
        for name in ("l0.mix.q.norm", "l0.mix.k.norm"):
            t[name] = torch.full_like(t[name], 3.0)
        for name in ("l0.mix.q.b", "l0.mix.k.b"):
            if name in t:
                t[name] = torch.zeros_like(t[name])
    return make(path, None, dtype, seed=9, edit=edit, cfg=cfg_raw)


def _three_forms(engine, toks, dtype, ref, what):
    """The last token's logits as a whole prompt, as the last token of a prompt's second portion, and decoded alone
    after a few decoded tokens."""
    from stratum_b200.engine import StepEntry
    n = len(toks)
    slot = engine.acquire()
    whole = engine.step([StepEntry(slot, toks, [n - 1])]).cpu().numpy()[0]
    engine.release(slot)
    slot = engine.acquire()
    first = min(201, n - 2)
    engine.step([StepEntry(slot, toks[:first], [])])
    cut = engine.step([StepEntry(slot, toks[first:], [n - first - 1])]).cpu().numpy()[0]
    engine.release(slot)
    slot = engine.acquire()
    engine.step([StepEntry(slot, toks[:n - 4], [])])
    for t in toks[n - 4:n - 1]:
        engine.step([StepEntry(slot, [t], [])])
    decoded = engine.step([StepEntry(slot, toks[n - 1:], [0])]).cpu().numpy()[0]
    engine.release(slot)
    assert_close(whole, ref, dtype, f"{what}, whole")
    assert_close(cut, ref, dtype, f"{what}, second portion")
    assert_close(decoded, ref, dtype, f"{what}, decoded")


@pytest.mark.parametrize("big", [False, True], ids=["small", "tensor-core sizes"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_decides(dtype, big, tmp_path):
    """Causal attention over every key: the marked key 1, 63, 64, 65, 128, 300 places back and at position 0, among
    520 keys: the asking token's logits are the marked key's (moving it away changes them wholesale, shown on the plain
    implementation)."""
    path, cfg, w = _marked_key_model(str(tmp_path / "far"), dtype, "attention_2", big)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(0)
    n = 520
    for back in (1, 63, 64, 65, 128, 300, n - 1):
        toks = [int(x) for x in rng.integers(9, cfg["vocab"], n)]
        toks[-1] = 8
        toks[n - 1 - back] = 7
        ref = plain_logits(cfg, w, toks)[-1]
        moved = list(toks)
        moved[n - 1 - back] = 9
        assert np.max(np.abs(plain_logits(cfg, w, moved)[-1] - ref)) > 0.15 * np.max(np.abs(ref))
        _three_forms(engine, toks, dtype, ref, f"marked key {back} back")


@pytest.mark.parametrize("big", [False, True], ids=["small", "tensor-core sizes"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_on_either_side_of_the_windows_and_the_kept_tokens_edges(dtype, big, tmp_path):
    """A window of `size` keys that keeps the first `keep` tokens: a marked key size - 1 places back decides the
    logits, one place further out it changes next to nothing (the token behind it, which is inside the window, has
    another row of the pair table); at position keep - 1 it decides them from hundreds of places away, at position keep
    it changes nothing (all shown on the plain implementation).  Sequence lengths put the window's first key on a
    page's first and last place."""
    path, cfg, w = _marked_key_model(str(tmp_path / "edge"), dtype, "attention", big)
    mask = cfg["layers"][0]["mixer"]["mask"]
    size, keep = mask["size"], mask["keep_first"]
    engine = _engine(path, dtype)
    rng = np.random.default_rng(1)
    border = 64 * (1 + (keep + size) // 128)                  # a page's border behind the kept tokens
    for n in (size + border, size + border - 1, 300, 333):
        for at, seen in ((n - size, True), (n - size - 1, False), (keep - 1, True), (keep, False), (0, True)):
            toks = [int(x) for x in rng.integers(9, cfg["vocab"], n)]
            toks[-1] = 8
            toks[at] = 7
            ref = plain_logits(cfg, w, toks)[-1]
            moved = list(toks)
            moved[at] = 9
            changed = np.max(np.abs(plain_logits(cfg, w, moved)[-1] - ref)) / np.max(np.abs(ref))
            assert changed > 0.15 if seen else changed < 0.03, f"n={n}: the marked key at {at} changes the logits by {changed}"
            _three_forms(engine, toks, dtype, ref, f"n={n}, marked key at {at}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_the_sinks_share(kind, dtype, tmp_path):
    """Few keys and a sink that outweighs them: leaving the sink out, scaling it or counting it twice would all show.
    The learned sink is made large; the biased attention's sink is the constant zero beside small scores."""
    from stratum_b200.engine import StepEntry
    mixer = windowed(heads=4, kv=2, dim=16, vdim=24, rot=8, size=40, keep=5, scale=0.05) if kind == "attention" \
        else biased(heads=4, kv=2, dim=16, vdim=24, rot=8, scale=0.02)
    cfg_raw = config([layer(kind, mixer)], vocab=120, width=64)

    def edit(t):
        if "l0.mix.sink" in t:
            t["l0.mix.sink"] = torch.tensor([2.0, 3.0, 4.0, 1.0]).to(t["l0.mix.sink"].dtype)
    path, cfg, w = make(str(tmp_path / "sink"), None, dtype, seed=6, edit=edit, cfg=cfg_raw)
    toks = [int(x) for x in np.random.default_rng(0).integers(0, 120, 12)]
    ref = plain_logits(cfg, w, toks)
    # what the logits would be without a sink (a model of the other kind has none to remove: compare the first token,
    # whose only key would get all the weight)
    no_sink = dict(w)
    if kind == "attention":
        no_sink["l0.mix.sink"] = np.full(4, -60.0)
        assert np.max(np.abs(plain_logits(cfg, no_sink, toks) - ref)) > 0.1 * np.max(np.abs(ref))
    engine = _engine(path, dtype)
    slot = engine.acquire()
    whole = engine.step([StepEntry(slot, toks, list(range(12)))]).cpu().numpy()
    engine.release(slot)
    slot = engine.acquire()
    single = np.concatenate([engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks])
    engine.release(slot)
    assert_close(whole, ref, dtype, f"{kind} sink, whole")
    assert_close(single, ref, dtype, f"{kind} sink, one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("at", [0, 5, 63, 64])
def test_the_state_carries_a_token_from_far_back(at, dtype, tmp_path):
    """One gated-linear-attention layer that hardly decays: hundreds of tokens later the output is still shaped by one
    marked token's large key, which every later query asks for (shown on the plain implementation), through a prompt cut in two, a state row used before,
    and decoded tokens."""
    from stratum_b200.engine import StepEntry
    heads, dim = 2, 8
    cfg_raw = config([layer("gla", gla(heads=heads, dim=dim, vdim=12, tau=4.0, rank=3))], vocab=90, width=48, emb_scale=1.0)

    def edit(t):
        t["l0.mix.a2.b"] = torch.full_like(t["l0.mix.a2.b"], 9.0)
        t["l0.mix.a2"] = (t["l0.mix.a2"].float() * 0.01).to(t["l0.mix.a2"].dtype)
        t["l0.norm1"] = torch.zeros_like(t["l0.norm1"])
        e = t["embed"].float()
        e[:, 0] = 0.0
        e[1, 0] = 24.0                                       # the marked token alone has a first dimension
        e[:, 1] = 8.0                                        # every token has the same second one
        t["embed"] = e.to(t["embed"].dtype)
        b = t["bigram"].float()
        b[:, :2] = 0.0
        t["bigram"] = b.to(t["bigram"].dtype)
        for name, col in (("l0.mix.k", 0), ("l0.mix.q", 1)):  # keys read the first into every head's first channel,
            m = t[name].float()                              # queries the second: every later token asks for the mark
            m[:, :2] = 0.0
            for h in range(heads):
                m[h * dim, col] = 6.0
            t[name] = m.to(t[name].dtype)
        t["l0.mix.o"] = (t["l0.mix.o"].float() * 10).to(t["l0.mix.o"].dtype)       # the mixer outweighs the stream
        t["l0.mix.g"] = (t["l0.mix.g"].float() * 3).to(t["l0.mix.g"].dtype)
    path, cfg, w = make(str(tmp_path / "state"), None, dtype, seed=4, edit=edit, cfg=cfg_raw)
    toks = [int(t) for t in np.random.default_rng(1).integers(2, 90, 400)]
    toks[at] = 1
    ref = plain_logits(cfg, w, toks)
    other = list(toks)
    other[at] = 2
    assert np.max(np.abs(plain_logits(cfg, w, other)[-1] - ref[-1])) > 0.1 * np.max(np.abs(ref[-1]))
    engine = _engine(path, dtype)
    slot = engine.acquire()                                  # somebody else's state in the row first
    engine.step([StepEntry(slot, other[:90], [])])
    engine.release(slot)
    slot = engine.acquire()
    engine.step([StepEntry(slot, toks[:131], [])])
    got = engine.step([StepEntry(slot, toks[131:390], [258])]).cpu().numpy()
    got = np.concatenate([got] + [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks[390:]])
    engine.release(slot)
    assert_close(got, ref[389:], dtype, "state from far back")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_token_in_front_across_a_steps_border(dtype, tmp_path):
    """A model whose pair table dwarfs its token table: the logits at a position are decided by the pair (token in
    front, token).  Changing the last token of one step changes the logits of the next step's first token exactly as
    the plain implementation says, in a batch of two requests and in a slot used before."""
    from stratum_b200.engine import StepEntry
    cfg_raw = config([layer("gla", gla(heads=1, dim=8, vdim=8, tau=4.0, rank=2), dense(40))], vocab=60, width=48,
                     emb_scale=0.05, buckets=997, mul_prev=29, mul_cur=19)
    path, cfg, w = make(str(tmp_path / "pairs"), None, dtype, seed=8, cfg=cfg_raw)
    a, b = [3, 9, 27, 21, 5, 11], [3, 9, 28, 21, 5, 11]
    other = [40, 41, 42, 43]
    ra, rb, ro = plain_logits(cfg, w, a), plain_logits(cfg, w, b), plain_logits(cfg, w, other)
    assert np.max(np.abs(ra[3] - rb[3])) > 0.2 * np.max(np.abs(ra[3]))
    engine = _engine(path, dtype)
    slot = engine.acquire()
    engine.step([StepEntry(slot, [50, 51, 52], [])])         # leaves a token in this slot's entry
    engine.release(slot)
    for toks, ref in ((a, ra), (b, rb)):
        s1, s2 = engine.acquire(), engine.acquire()
        first = engine.step([StepEntry(s1, toks[:3], [0, 2]), StepEntry(s2, other[:1], [0])]).cpu().numpy()
        assert_close(first, np.stack([ref[0], ref[2], ro[0]]), dtype, "first step")
        nxt = engine.step([StepEntry(s2, other[1:2], [0]), StepEntry(s1, toks[3:4], [0])]).cpu().numpy()
        assert_close(nxt, np.stack([ro[1], ref[3]]), dtype, "the step after")
        last = engine.step([StepEntry(s1, toks[4:], [0, 1]), StepEntry(s2, other[2:], [1])]).cpu().numpy()
        assert_close(last, np.stack([ref[4], ref[5], ro[3]]), dtype, "a portion of two")
        engine.release(s1); engine.release(s2)


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, tmp_path):
    """Stratum.generate: the scheduler's batches, replayed decode graphs (token ids fed on the device, so the token in
    front comes from the state), slots given back; every picked token is the plain implementation's best (or within
    rounding of it)."""
    from stratum_b200 import Stratum
    path, cfg, w = make(str(tmp_path / "gen"), "A", dtype, seed=11)
    rng = np.random.default_rng(0)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (5, 70, 12, 1)]
    llm = Stratum(path, dtype=dtype, max_tokens=1024)
    res = llm.generate(prompts, max_new_tokens=10, stop_ids=())
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 10
        seq = list(p)
        for tok in r.tokens:
            margins = []
            ref = M.forward(cfg, w, seq, margins=margins)[-1]
            if margins and min(margins) < (1e-4 if dtype == "float32" else 0.1):
                break                                    # a router near a tie: what follows is no test
            ref = ref - ref.mean()
            assert ref[tok] >= ref.max() - 2 * TOL[dtype] * float(np.max(np.abs(ref))), (p, r.tokens, tok)
            seq.append(tok)
    serial = llm.generate(prompts, max_new_tokens=10, stop_ids=(), max_batch=2)
    if dtype == "float32":
        assert [r.tokens for r in serial] == [r.tokens for r in res]
    llm.engine.cache.check()
    assert llm.engine.cache.tokens_held() == 0


def test_trace_replay_program(tmp_path):
    """`bin/trace_run` fed steps on standard input: a batch of two requests, then single tokens, one request ending
    earlier, then a request that takes the pages and the state rows given back."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, w = make(str(tmp_path / "replay"), "A", "float32", seed=21)
    rng = np.random.default_rng(8)
    vocab = cfg["vocab"]
    a, b, c = (clear_tokens(rng, n, cfg, w, "float32") for n in (70, 9, 33))
    ra, rb, rc = (plain_logits(cfg, w, t) for t in (a, b, c))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]},
                                     {"id": "b", "tokens": b[:5], "want": []}], "end": []}]
    for i in range(10):
        ents = [{"id": "a", "tokens": [a[60 + i]], "want": [0]}]
        end = ["a"] if i == 9 else []
        if i < 4:
            ents.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
            if i == 3:
                end.append("b")
        steps.append({"step": 1 + i, "entries": ents, "end": end})
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": c, "want": list(range(33))}], "end": ["c"]})
    out = str(tmp_path / "out")
    p = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32",
                          "--out", out, "--max-tokens", "192"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {s['step']}"
    p.stdin.close()
    assert p.wait(timeout=600) == 0
    read = lambda n: np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, vocab)   # noqa: E731
    assert_close(read(0), ra[[0, 59]], "float32", "trace step 0")
    for i in range(10):
        got = read(1 + i)
        assert_close(got[0], ra[60 + i], "float32", f"trace a {i}")
        if i < 4:
            assert_close(got[1], rb[5 + i], "float32", f"trace b {i}")
    assert_close(read(11), rc, "float32", "trace c")
