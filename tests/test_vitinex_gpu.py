"""Vitinex on the GPU against the plain implementation: each kernel and each mechanism alone, whole prompts against
token-by-token decoding, prompts fed in portions, unequal batches, pages, slots and state rows used again, keys far
back and on the pages' borders, state carried from the first token, the first tokens, long decoding, looped layers
with a cache per pass, generation through the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TOL
from plain import vitinex_plain as V
from vitinex_helpers import (assert_rows_close as assert_close, clear_tokens, config, dense, latent, layer, make, moe,
                             plain_logits, ssm)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _engine(path, dtype, max_tokens=1024):
    from stratum_b200.engine import Engine, load_model
    model, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    return Engine(model, max_tokens=max_tokens)


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "TC") for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    path, cfg, w = make(str(tmp_path_factory.mktemp(f"vit{name}_{dtype}")), name, dtype, seed=len(name) + 1)
    return name, dtype, cfg, w, _engine(path, dtype), path


def _dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()


# ------------------------------------------------------------------------------------------ kernels alone
def test_layer_norm_kernels():
    """The norm in front of a sublayer (also on chosen rows), and the norm behind it that adds into the stream and
    makes the next sublayer's input from the row it has just written."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    for rows, width in ((1, 72), (5, 70), (300, 512), (3, 4100)):
        x = rng.standard_normal((rows, width)) * 3 + rng.uniform(-5, 5, (rows, 1))       # means far from zero
        y = rng.standard_normal((rows, width)) * 2 - 1.0
        w, w2 = rng.uniform(0.3, 1.5, width), rng.uniform(0.5, 1.5, width)
        out = torch.empty(rows, width, device="cuda")
        K.layernorm(_dev(x), _dev(w), 1e-5, out)
        want = V.layer_norm(x, w, 1e-5)
        assert np.max(np.abs(out.cpu().numpy() - want)) <= 3e-6 * np.max(np.abs(want))
        pick = np.array([rows - 1, 0], dtype=np.int32)
        some = torch.empty(2, width, dtype=torch.bfloat16, device="cuda")
        K.layernorm(_dev(x), _dev(w), 1e-5, some, _dev(pick, torch.int32))
        assert np.max(np.abs(some.float().cpu().numpy() - want[pick])) <= 5e-3 * np.max(np.abs(want))
        xd, nxt = _dev(x), torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
        K.layernorm_into_residual(_dev(y), _dev(0.7 * w), 1e-5, xd, True, _dev(w2), 1e-6, nxt)
        new = x.astype(np.float32).astype(np.float64) + 0.7 * V.layer_norm(y, w, 1e-5)
        assert np.max(np.abs(xd.cpu().numpy() - new)) <= 3e-6 * np.max(np.abs(new))
        want2 = V.layer_norm(new, w2, 1e-6)
        assert np.max(np.abs(nxt.float().cpu().numpy() - want2)) <= 5e-3 * np.max(np.abs(want2))
        yd = _dev(y)
        K.layernorm_into_residual(yd, _dev(w), 1e-5, yd, False)                           # in place, nothing added
        assert np.max(np.abs(yd.cpu().numpy() - V.layer_norm(y, w, 1e-5))) <= 3e-6 * np.max(np.abs(want))


@pytest.mark.parametrize("heads,vdim,state,groups,taps,parts", [
    (4, 12, 24, 2, 3, 3), (3, 20, 40, 3, 5, 2), (2, 9, 10, 1, 2, 1), (4, 32, 64, 2, 4, 2), (8, 16, 128, 1, 4, 4),
    (1, 8, 8, 1, 1, 1), (2, 70, 130, 2, 2, 5), (6, 4, 16, 6, 4, 24), (2, 40, 260, 1, 3, 1)])
@pytest.mark.parametrize("long", [77, 520])
def test_state_space_kernels(heads, vdim, state, groups, taps, parts, long):
    """The three kernels of the state-space mixer on projections made here: two sequences of unequal lengths whose
    tokens come in three steps (many, three and two, one), states in slots that lie apart, against the plain loop over
    whole sequences."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(state + vdim)
    inner, gn = heads * vdim, groups * state
    C = inner + 2 * gn
    width = inner + C + heads
    lens = (long, 9)               # 520: dozens of staged token groups in the recurrence
    proj = [rng.standard_normal((n, width)) for n in lens]
    conv, conv_b = rng.uniform(-0.8, 0.8, (C, taps)), rng.uniform(-0.3, 0.3, C)
    a_log, dt_bias = rng.uniform(-2, 0.5, heads), rng.uniform(-1, 1, heads)
    d_skip, gain = rng.uniform(-1, 1.5, heads), rng.uniform(0.5, 1.5, inner)
    # the plain mixer, fed the projections directly: identity matrices in place of the weights
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": taps, "norm_groups": parts}
    w = {"in": np.eye(width), "conv": conv, "conv.b": conv_b, "A_log": a_log, "dt_bias": dt_bias, "D": d_skip,
         "norm": gain, "o": np.eye(inner)}
    want = [V.state_space_mixer(p, w, m, 1e-5) for p in proj]
    n_state = inner * state + (taps - 1) * C
    slots_total = 6
    st = torch.zeros(slots_total, n_state, device="cuda")
    slots = (4, 1)
    done = [0, 0]
    got = [[], []]
    for cut in ((long - 4, 6), (3, 2), (1, 1)):
        rows_ = np.concatenate([proj[i][done[i]:done[i] + cut[i]] for i in range(2)])
        T = rows_.shape[0]
        pos = np.concatenate([np.arange(done[i], done[i] + cut[i]) for i in range(2)])
        seq = np.concatenate([np.full(cut[i], i) for i in range(2)])
        start = np.array([0, cut[0], T])
        act = torch.empty(T, C + 2 * heads + 3, device="cuda")
        y_raw = torch.empty(T, inner, device="cuda")
        out = torch.empty(T, inner + 5, device="cuda")
        K.ssm_scan(_dev(rows_), _dev(conv), _dev(conv_b), _dev(a_log), _dev(dt_bias), _dev(d_skip), _dev(gain), act,
                   y_raw, out, st, _dev(pos, torch.int32), _dev(seq, torch.int32), _dev(start, torch.int32),
                   _dev(np.array(slots), torch.int32), heads, vdim, state, groups, parts, 1e-5, True)
        o = out[:, :inner].cpu().numpy()
        got[0].append(o[:cut[0]]); got[1].append(o[cut[0]:])
        done = [done[i] + cut[i] for i in range(2)]
    for i in range(2):
        g = np.concatenate(got[i])
        assert np.isfinite(g).all()
        assert np.max(np.abs(g - want[i])) <= 3e-5 * np.max(np.abs(want[i])), (i, np.max(np.abs(g - want[i])))
    assert float(st[0].abs().max()) == 0.0 and float(st[5].abs().max()) == 0.0            # rows of nobody stay clean


def test_state_space_kernel_leaves_the_state_alone_when_told_to():
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(3)
    heads, vdim, state, groups, taps = 2, 8, 16, 1, 3
    inner, C = heads * vdim, heads * vdim + 2 * groups * state
    T = 5
    st = _dev(rng.standard_normal((2, inner * state + (taps - 1) * C)))
    before = st.clone()
    out = torch.empty(T, inner, device="cuda")
    K.ssm_scan(_dev(rng.standard_normal((T, inner + C + heads))), _dev(rng.standard_normal((C, taps))),
               torch.zeros(C, device="cuda"), torch.zeros(heads, device="cuda"), torch.zeros(heads, device="cuda"),
               torch.ones(heads, device="cuda"), torch.ones(inner, device="cuda"),
               torch.empty(T, C + 2 * heads, device="cuda"), torch.empty(T, inner, device="cuda"), out, st,
               _dev(np.arange(7, 7 + T), torch.int32), torch.zeros(T, dtype=torch.int32, device="cuda"),
               _dev(np.array([0, T]), torch.int32), _dev(np.array([1]), torch.int32), heads, vdim, state, groups, 1,
               1e-5, False)
    assert torch.equal(st, before) and bool(torch.isfinite(out).all())


@pytest.mark.parametrize("experts,top", [(6, 2), (8, 3), (12, 4), (5, 1), (4, 4), (40, 6)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_router_kernel(experts, top, dtype):
    """Scores by softmax over all experts, the `top` largest chosen and weighted by their scores as they are, and the
    shared expert's gate sigmoid(x . w) in the column behind the experts'."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(experts * 10 + top)
    T, W = 40, 72
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    h = _dev(rng.standard_normal((T, W)), td)
    hp = h.float().cpu().numpy().astype(np.float64)
    wr, wg = rng.standard_normal((experts, W)) * 0.4, rng.standard_normal(W) * 0.3
    dense_w = torch.full((T, experts + 3), 7.0, device="cuda")
    chosen = torch.zeros(T, top, dtype=torch.int32, device="cuda")
    weights = torch.zeros(T, top, device="cuda")
    K.moe_route(h, _dev(wr), None, dense_w, chosen, weights, top, 1, 1, 1.0, softmax=True, renorm=False, w_gate=_dev(wg))
    wr32, wg32 = _dev(wr).cpu().numpy().astype(np.float64), _dev(wg).cpu().numpy().astype(np.float64)
    margins = []
    want_c, want_w = V.route_softmax(hp, wr32, top, margins)
    chosen, weights, dense_w = chosen.cpu().numpy(), weights.cpu().numpy(), dense_w.cpu().numpy()
    for t in range(T):
        np.testing.assert_allclose(dense_w[t, experts], V.sigmoid(hp[t] @ wg32), rtol=2e-5)
        assert (dense_w[t, experts + 1:] == 7.0).all()
        if margins and margins[t] < 1e-4:
            continue                                     # a tie within rounding: either choice is right
        got = dict(zip(chosen[t].tolist(), weights[t].tolist()))
        assert sorted(got) == sorted(want_c[t].tolist()), (t, chosen[t], want_c[t])
        row = np.zeros(experts)
        for e, s in zip(want_c[t], want_w[t]):
            assert got[int(e)] == pytest.approx(s, rel=2e-5)
            row[e] = s
        np.testing.assert_allclose(dense_w[t, :experts], row, rtol=2e-5, atol=1e-9)
        if top < experts:
            assert weights[t].sum() < 1.0                # scores as they are: they do not sum to one


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gates_kernel(dtype):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(4)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    for T, H, dv in ((7, 3, 40), (33, 5, 18), (2, 8, 64)):
        a, g = _dev(rng.standard_normal((T, H * dv + 4)), td), _dev(rng.standard_normal((T, H + 3)) * 2, td)
        a0, g0 = a.float().cpu().numpy().astype(np.float64), g.float().cpu().numpy().astype(np.float64)
        K.gate_heads(a, g, H, dv)
        want = a0.copy()
        want[:, :H * dv] = (a0[:, :H * dv].reshape(T, H, dv) * V.sigmoid(g0[:, :H])[:, :, None]).reshape(T, H * dv)
        tol = 2e-6 if dtype == "float32" else 5e-3
        assert np.max(np.abs(a.float().cpu().numpy() - want)) <= tol * np.max(np.abs(want))


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["latent", "ssm", "moe", "dense", "loop"])
def test_one_mechanism_alone(name, dtype, tmp_path):
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / name), name, dtype, seed=7)
    engine = _engine(path, dtype)
    toks = clear_tokens(np.random.default_rng(1), 90, cfg, w, dtype)
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks, list(range(90)))]).cpu().numpy()
    engine.release(slot)
    assert_close(got, plain_logits(cfg, w, toks), dtype, name)


def test_the_stream_after_every_layer_run(tmp_path):
    """The residual stream behind every run of a layer (looped layers count each time), float32, against the plain
    implementation's: a fault shows at the first run that has it, not only in the logits."""
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / "streams"), "A", "float32", seed=13)
    engine = _engine(path, "float32")
    seen = []
    for la in engine.model.layers:
        arr, inner = la.arrangement, la.arrangement.forward
        if type(arr).__name__ == "StreamOpLayer":
            continue

        def wrapped(layer_, x, step, cache, _inner=inner, **kw):
            out = _inner(layer_, x, step, cache, **kw)
            seen.append(x.detach().clone())
            return out
        arr.forward = wrapped
    toks = clear_tokens(np.random.default_rng(2), 23, cfg, w, "float32")
    want = []
    V.forward(toks, w, cfg, want)
    slot = engine.acquire()
    engine.step([StepEntry(slot, toks, [22])])
    engine.release(slot)
    assert len(seen) == len(want) == 8
    for i, (g, r) in enumerate(zip(seen, want)):
        assert np.max(np.abs(g.cpu().numpy() - r)) <= 2e-5 * np.max(np.abs(r)), f"layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["moe", "A", "TC"])
def test_experts_both_ways(name, dtype, tmp_path, monkeypatch):
    """The experts run on stretches of gathered rows (the way of long prompts, here forced on short ones) and as two
    stacked products (the way of decode steps): both against the plain implementation, and against one another."""
    from stratum_b200.engine import StepEntry
    from stratum_b200.parts import moe as M
    path, cfg, w = make(str(tmp_path / name), name, dtype, seed=5)
    engine = _engine(path, dtype)
    n = 150
    toks = clear_tokens(np.random.default_rng(6), n, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    got = {}
    for way, rows in (("stacked", 1 << 30), ("grouped", 0)):
        monkeypatch.setattr(M, "GROUPED_MIN_ROWS", rows)
        slot = engine.acquire()
        a = engine.step([StepEntry(slot, toks[:97], list(range(97)))]).cpu().numpy()
        b = engine.step([StepEntry(slot, toks[97:], list(range(n - 97)))]).cpu().numpy()
        engine.release(slot)
        got[way] = np.concatenate([a, b])
        assert_close(got[way], ref, dtype, f"{name} experts {way}")
    if dtype == "float32":
        assert np.max(np.abs(got["stacked"] - got["grouped"])) <= 2e-5 * np.max(np.abs(ref))


def test_every_expert_is_reached_and_weighted_by_its_score(tmp_path):
    """Float32, routers that choose freely: over a few hundred tokens every expert of every routed layer is chosen
    somewhere (shown on the plain router), so that a wrong expert's matrices or a renormalised weight shows."""
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / "reach"), "moe", "float32", seed=3)
    toks = clear_tokens(np.random.default_rng(9), 200, cfg, w, "float32")
    x0 = w["embed"][toks]
    h = V.layer_norm(x0 + cfg["residual_mult"] * V.layer_norm(
        V.state_space_mixer(V.layer_norm(x0, w["l0.norm1"], 1e-5), V.sub(w, "l0.mix."), cfg["layers"][0]["mixer"], 1e-5),
        w["l0.norm1b"], 1e-5), w["l0.norm2"], 1e-5)
    chosen, score = V.route_softmax(h, w["l0.mlp.router"], 4)
    assert set(chosen.reshape(-1).tolist()) == set(range(12))
    assert score.sum(axis=-1).max() < 1.0 - 1e-3
    engine = _engine(path, "float32")
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks, list(range(200)))]).cpu().numpy()
    engine.release(slot)
    assert_close(got, plain_logits(cfg, w, toks), "float32", "every expert")


@pytest.mark.parametrize("name", ["TC", "latent"])
def test_latent_attention_both_forms(name, tmp_path, monkeypatch):
    """bfloat16 prompts from position 0 form the heads' keys and values (from 256 tokens on; here from 32 on), everything
    else carries the queries into the latent space and attends over the cached rows: both against the plain
    implementation, and decoded tokens read the cache that either form wrote."""
    from stratum_b200.engine import StepEntry
    from stratum_b200.parts import latent_attention as L
    path, cfg, w = make(str(tmp_path / name), name, "bfloat16", seed=8)
    engine = _engine(path, "bfloat16")
    rng = np.random.default_rng(12)
    prompts = [clear_tokens(rng, n, cfg, w, "bfloat16") for n in (130, 70, 41)]
    refs = [plain_logits(cfg, w, p) for p in prompts]
    for minimum in (32, 1 << 30):
        monkeypatch.setattr(L, "PER_HEAD_MIN_TOKENS", minimum)
        slots = [engine.acquire() for _ in prompts]
        cut = [len(p) - 3 for p in prompts]
        out = engine.step([StepEntry(s, p[:c], [0, c // 2, c - 1]) for s, p, c in zip(slots, prompts, cut)]).cpu().numpy()
        for i, c in enumerate(cut):
            assert_close(out[3 * i:3 * i + 3], refs[i][[0, c // 2, c - 1]], "bfloat16", f"{name} form {minimum} prompt {i}")
        for k in range(3):
            out = engine.step([StepEntry(s, [p[c + k]], [0]) for s, p, c in zip(slots, prompts, cut)]).cpu().numpy()
            for i, c in enumerate(cut):
                assert_close(out[i], refs[i][c + k], "bfloat16", f"{name} form {minimum} seq {i} +{k}")
        for s in slots:
            engine.release(s)


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
    back: every run's logits are the same bits (the small kernels begin while the kernel before them still runs; a
    value read too early, or a sum whose order depends on timing, would show here)."""
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
    """A prompt cut into portions of a few sizes, down to two tokens (fewer than the convolutions' taps); portions
    start inside pages and on their borders."""
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
    state-space layer) that another one has just given back; a state row that was not cleared would show at once."""
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
    """Positions 0, 1, 2 one by one (the convolutions still see zeros before the start), then on across several pages."""
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


# ------------------------------------------------------------------------------------------ one key far back decides
def _marked_key_model(path, dtype):
    """One latent layer in which token 7 is the only one with anything in the embedding's first dimension, and token 8
    the only one with anything in the second.  The shared rotated key part reads the first dimension into its slowest
    pair (it is not normed, so the marked token's is large); the queries' latent reads the second dimension, and every
    head's slowest rotated pair reads that latent.  When token 8 asks, the marked key's score stands far above the
    hundreds of others wherever it lies, and the heads' outputs are its value."""
    H, d, r, rank, q_rank = 3, 16, 8, 40, 24
    cfg_raw = config([layer("latent_attention", latent(heads=H, dim=d, rot=r, vdim=24, rank=rank, q_rank=q_rank,
                                                       base=1e6, scale=0.25))], vocab=120, width=64, mult=3.0)

    def edit(t):
        e = t["embed"].float()
        e[:, :2] = 0.0
        e[7, 0] = e[8, 1] = 8.0
        t["embed"] = e.to(t["embed"].dtype)
        m = t["l0.mix.dkv"].float()
        m[:, :2] = 0.0
        m[rank + r - 2, 0] = 4.0
        t["l0.mix.dkv"] = m.to(t["l0.mix.dkv"].dtype)
        m = t["l0.mix.dq"].float()
        m[:, :2] = 0.0
        m[0, 1] = 8.0
        t["l0.mix.dq"] = m.to(t["l0.mix.dq"].dtype)
        m = t["l0.mix.uq"].float()
        for h in range(H):
            m[h * (d + r) + d + r - 2, 0] = 0.5 + 0.25 * h
        t["l0.mix.uq"] = m.to(t["l0.mix.uq"].dtype)
        t["l0.norm1"] = torch.ones_like(t["l0.norm1"])
        t["l0.mix.dq.norm"] = torch.ones_like(t["l0.mix.dq.norm"])
    return make(path, None, dtype, seed=9, edit=edit, cfg=cfg_raw)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_decides(dtype, tmp_path):
    """The marked key 1, 63, 64, 65, 128, 300 places back and at position 0, among 520 keys: the asking token's logits
    are the marked key's (moving it away changes them wholesale, shown on the plain implementation), as a whole
    prompt, as the last token of the second portion of a prompt, and decoded alone after a few decoded tokens."""
    from stratum_b200.engine import StepEntry
    path, cfg, w = _marked_key_model(str(tmp_path / "far"), dtype)
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
        assert np.max(np.abs(plain_logits(cfg, w, moved)[-1] - ref)) > 0.5 * np.max(np.abs(ref))
        slot = engine.acquire()
        whole = engine.step([StepEntry(slot, toks, [n - 1])]).cpu().numpy()[0]
        engine.release(slot)
        slot = engine.acquire()
        engine.step([StepEntry(slot, toks[:201], [])])
        cut = engine.step([StepEntry(slot, toks[201:], [n - 202])]).cpu().numpy()[0]
        engine.release(slot)
        slot = engine.acquire()
        engine.step([StepEntry(slot, toks[:n - 4], [])])
        for t in toks[n - 4:n - 1]:
            engine.step([StepEntry(slot, [t], [])])
        decoded = engine.step([StepEntry(slot, toks[n - 1:], [0])]).cpu().numpy()[0]
        engine.release(slot)
        assert_close(whole, ref, dtype, f"marked key {back} back, whole")
        assert_close(cut, ref, dtype, f"marked key {back} back, second portion")
        assert_close(decoded, ref, dtype, f"marked key {back} back, decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_marked_key_in_a_batch_of_unequal_requests(dtype, tmp_path):
    """Three requests in one batch, each with its marked key elsewhere (one on a page's last place, one with none):
    every request's logits are its own key's, in the prompt step and in the decoded steps that follow."""
    from stratum_b200.engine import StepEntry
    path, cfg, w = _marked_key_model(str(tmp_path / "batch"), dtype)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(5)
    lens, marks = (200, 70, 131), (63, None, 2)
    seqs = []
    for n, at in zip(lens, marks):
        toks = [int(x) for x in rng.integers(9, cfg["vocab"], n + 3)]
        toks[n - 1:] = [8, 8, 8, 8]
        if at is not None:
            toks[at] = 7
        seqs.append(toks)
    refs = [plain_logits(cfg, w, s) for s in seqs]
    assert np.max(np.abs(refs[0][-1] - refs[1][-1])) > 0.3 * np.max(np.abs(refs[0][-1]))
    slots = [engine.acquire() for _ in seqs]
    out = engine.step([StepEntry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy()
    for i, n in enumerate(lens):
        assert_close(out[i], refs[i][n - 1], dtype, f"batch prompt {i}")
    for k in range(3):
        out = engine.step([StepEntry(s, [q[n + k]], [0]) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy()
        for i, n in enumerate(lens):
            assert_close(out[i], refs[i][n + k], dtype, f"batch seq {i} +{k}")
    for s in slots:
        engine.release(s)
    engine.cache.check()


# ------------------------------------------------------------------------------------------ the convolution's edge
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [2, 4, 5])
def test_a_token_at_the_convolutions_edge(taps, dtype, tmp_path):
    """One state-space layer whose state forgets at once (a large decay rate and step size): a token's output then
    depends on the convolution's taps alone.  A marked token taps - 1 places back changes the logits, one place
    further out it changes nothing (shown on the plain implementation); the framework agrees as a whole prompt, with
    the asking token decoded alone (the taps come from the state row), and with the portion's cut between the two."""
    from stratum_b200.engine import StepEntry
    cfg_raw = config([layer("mamba2", ssm(heads=3, vdim=8, state=12, groups=3, conv=taps, norm_groups=1))],
                     vocab=90, width=48, mult=2.0)

    def edit(t):
        t["l0.mix.A_log"] = torch.full_like(t["l0.mix.A_log"], 5.0)
        t["l0.mix.dt_bias"] = torch.full_like(t["l0.mix.dt_bias"], 2.0)
    path, cfg, w = make(str(tmp_path / "edge"), None, dtype, seed=4, edit=edit, cfg=cfg_raw)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(taps)
    n = 140
    for back in (taps - 1, taps):
        toks = [int(x) for x in rng.integers(9, cfg["vocab"], n)]
        toks[n - 1 - back] = 7
        ref = plain_logits(cfg, w, toks)[-1]
        moved = list(toks)
        moved[n - 1 - back] = 9
        changed = np.max(np.abs(plain_logits(cfg, w, moved)[-1] - ref)) / np.max(np.abs(ref))
        assert changed > 0.05 if back == taps - 1 else changed < 1e-9, f"the marked token {back} back changes the logits by {changed}"
        for first in (n, n - 1, n - 1 - back, n - back):          # whole; decoded alone; cuts on either side of the mark
            slot = engine.acquire()
            if first < n:
                engine.step([StepEntry(slot, toks[:first], [])])
                got = engine.step([StepEntry(slot, toks[first:], [n - first - 1])]).cpu().numpy()[0]
            else:
                got = engine.step([StepEntry(slot, toks, [n - 1])]).cpu().numpy()[0]
            engine.release(slot)
            assert_close(got, ref, dtype, f"taps {taps}, mark {back} back, first portion of {first}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("at", [0, 5, 63, 64])
def test_the_state_carries_a_token_from_far_back(at, dtype, tmp_path):
    """One state-space layer that hardly decays and hardly writes (a step size near zero) except for one marked token,
    whose step size is large: hundreds of tokens later the output is still what that token wrote (shown on the plain
    implementation), through a prompt cut in two, a state row used before, and decoded tokens."""
    from stratum_b200.engine import StepEntry
    heads = 2
    cfg_raw = config([layer("mamba2", ssm(heads=heads, vdim=12, state=16, groups=1, conv=3, norm_groups=2))],
                     vocab=90, width=48, mult=2.0)

    def edit(t):
        t["l0.mix.A_log"] = torch.full_like(t["l0.mix.A_log"], -7.0)
        t["l0.mix.dt_bias"] = torch.full_like(t["l0.mix.dt_bias"], -8.0)
        t["l0.norm1"] = torch.ones_like(t["l0.norm1"])
        e = t["embed"].float()
        e[:, 0] = 0.0
        e[1, 0] = 8.0
        t["embed"] = e.to(t["embed"].dtype)
        m = t["l0.mix.in"].float()
        m[:, 0] = 0.0
        m[-heads:, 0] = 3.0                                  # the step sizes' rows read the marked dimension
        t["l0.mix.in"] = m.to(t["l0.mix.in"].dtype)
    path, cfg, w = make(str(tmp_path / "state"), None, dtype, seed=4, edit=edit, cfg=cfg_raw)
    toks = [int(t) for t in np.random.default_rng(1).integers(2, 90, 400)]
    toks[at] = 1
    ref = plain_logits(cfg, w, toks)
    other = list(toks)
    other[at] = 2
    assert np.max(np.abs(plain_logits(cfg, w, other)[-1] - ref[-1])) > 0.2 * np.max(np.abs(ref[-1]))
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


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, tmp_path):
    """Stratum.generate: the scheduler's batches, replayed decode graphs, slots given back; every picked token is the
    plain implementation's best (or within rounding of it)."""
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
            ref = V.forward(seq, w, cfg, margins=margins)[-1]
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
