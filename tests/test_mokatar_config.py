"""Mokatar on the CPU: the configuration reader, the order in which looped layers run, the tensor list, what each
stop of the schedule keeps in the cache, pages behind a window that keeps first tokens, and the plain implementation's
own properties (mechanisms restated a second way)."""
import copy

import numpy as np
import pytest

from mokatar_helpers import CONFIGS, MOK_A, MOK_B, MOK_TC, biased, config, gla, layer, windowed
from plain import mokatar_plain as M


def _cfg(raw):
    from stratum_b200.config import find_architecture
    return find_architecture(raw).config_class.from_dict(raw)


def test_configuration_round_trip_and_registry():
    from stratum_b200.config import find_architecture
    from stratum_b200.config.mokatar import MokatarConfig
    assert find_architecture({"architecture": "Mokatar"}).config_class is MokatarConfig
    for raw in CONFIGS.values():
        cfg = _cfg(raw)
        assert MokatarConfig.from_dict(cfg.to_dict()) == cfg
        assert [la.kind for la in cfg.layers] == [e["type"] for e in raw["layers"]]
        assert (cfg.loop is None) == ("loop" not in raw)
    a = _cfg(MOK_A)
    assert (a.layers[0].mixer.window, a.layers[0].mixer.keep_first) == (50, 3) and a.layers[0].mixer.rot.ramp
    assert a.layers[2].mixer.window == 0 and not a.layers[2].mixer.rot.ramp and a.layers[2].mixer.rot.factor == 3.0
    assert (a.logit_scale, a.embedding_scale, a.bigram.buckets) == (0.7, 3.0, 53)


def test_what_a_file_does_not_mention_does_not_exist():
    """No pair table, no rotation, no window, no loop, no feed-forward: each is left out by leaving its key out."""
    from stratum_b200.config import find_architecture
    from stratum_b200.engine.model import Model
    raw = copy.deepcopy(MOK_A)
    del raw["embedding"]["bigram"]
    del raw["layers"][0]["mixer"]["rot"]
    del raw["layers"][0]["mixer"]["mask"]
    del raw["layers"][2]["mixer"]["rot"]["scaling"]
    del raw["loop"]
    del raw["logit_scale"]
    cfg = _cfg(raw)
    assert cfg.bigram is None and cfg.loop is None and cfg.logit_scale == 1.0
    assert cfg.layers[0].mixer.rot is None and cfg.layers[0].mixer.window == 0 and cfg.layers[2].mixer.rot.factor is None
    assert type(cfg).from_dict(cfg.to_dict()) == cfg
    model = Model(find_architecture(raw).describe_model(cfg), None)
    assert "bigram" not in model.tensors() and "loop.step" not in model.tensors()
    assert len(model.cache_specs()) == len(model.schedule) == 4          # nothing kept for the embedding
    assert model.layers[0].part("mixer").position is None


def test_configuration_problems_are_listed_together():
    from stratum_b200.config import ConfigError
    raw = copy.deepcopy(MOK_A)
    del raw["vocab"]
    raw["layers"][0]["mixer"]["kv_heads"] = 3                # 4 heads on 3 kv heads
    raw["layers"][0]["mlp"]["router"]["top"] = 7             # of 6 experts
    raw["layers"][1]["type"] = "convolution"
    raw["layers"][2]["mixer"]["rot"]["dims"] = 7
    del raw["layers"][3]["mixer"]["tau"]
    del raw["embedding"]["bigram"]["mul_cur"]
    raw["loop"]["stop"] = 1                                  # not behind its start
    with pytest.raises(ConfigError) as e:
        _cfg(raw)
    text = str(e.value)
    for piece in ("vocab", "multiple of kv_heads", "top=7", "convolution", "rot.dims", "tau", "mul_cur", "loop.start"):
        assert piece in text, (piece, text)


def test_the_order_of_layer_runs():
    runs = _cfg(MOK_A).runs()
    assert [i for i, _, _ in runs] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [t for _, t, _ in runs] == [None, 0, 0, 1, 1, 2, 2, None]
    assert [f for _, _, f in runs] == [False, True, False, True, False, True, False, False]
    assert [i for i, _, _ in _cfg(MOK_B).runs()] == [0, 1, 2]
    assert M.runs(MOK_A) == runs and M.runs(MOK_TC) == _cfg(MOK_TC).runs()


def test_tensor_names_and_shapes():
    from stratum_b200.engine.model import expected_tensors
    t = expected_tensors(_cfg(MOK_A))
    W = MOK_A["width"]
    assert {"embed", "bigram", "final.norm", "head", "loop.step"} <= set(t)
    assert t["bigram"].shape == (MOK_A["embedding"]["bigram"]["buckets"] + 1, W) and t["loop.step"].shape == (3, W)
    assert not any(n.startswith(("l2.mlp", "l2.norm2")) for n in t)          # layer 2 is a mixer alone
    a = MOK_A["layers"][0]["mixer"]
    assert t["l0.mix.q"].shape == (a["heads"] * a["dim"], W) and t["l0.mix.k"].shape == (a["kv_heads"] * a["dim"], W)
    assert t["l0.mix.v"].shape == (a["kv_heads"] * a["vdim"], W) and t["l0.mix.o"].shape == (W, a["heads"] * a["vdim"])
    assert t["l0.mix.q.norm"].shape == t["l0.mix.k.norm"].shape == (a["dim"],) and t["l0.mix.sink"].shape == (a["heads"],)
    assert "l0.mix.q.b" not in t
    b = MOK_A["layers"][2]["mixer"]
    assert t["l2.mix.q.norm"].shape == t["l2.mix.q.b"].shape == (b["heads"] * b["dim"],)
    assert t["l2.mix.k.norm"].shape == t["l2.mix.k.b"].shape == (b["kv_heads"] * b["dim"],)
    assert t["l2.mix.v.b"].shape == (b["kv_heads"] * b["vdim"],) and "l2.mix.sink" not in t
    g = MOK_A["layers"][1]["mixer"]
    assert t["l1.mix.a1"].shape == (g["rank"], W) and t["l1.mix.a2"].shape == (g["heads"] * g["dim"], g["rank"])
    assert t["l1.mix.a2.b"].shape == (g["heads"] * g["dim"],) and t["l1.mix.norm"].shape == (g["vdim"],)
    assert t["l1.mix.g"].shape == (g["heads"] * g["vdim"], W) and t["l1.mix.o"].shape == (W, g["heads"] * g["vdim"])
    assert t["l0.mlp.router"].shape == (6, W) and t["l0.mlp.router.b"].shape == (6,)
    assert t["l0.mlp.e5.down"].shape == (W, 40) and t["l1.mlp.gate"].shape == (96, W)
    assert "loop.step" not in expected_tensors(_cfg(MOK_B))


def test_the_decays_inner_size_comes_from_the_tensor():
    """A file's configuration does not name the inner size of the decay's projections; the shape of a1 does."""
    from stratum_b200.config import find_architecture
    from stratum_b200.engine.model import expected_tensors
    raw = copy.deepcopy(MOK_A)
    for e in raw["layers"]:
        e["mixer"].pop("rank", None)
    arch = find_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    with pytest.raises(ValueError, match="a1"):
        arch.describe_model(cfg)
    sized = arch.sizes_from_tensors(cfg, {"l1.mix.a1": (10, 72), "l3.mix.a1": (4, 72), "l0.mix.q": (96, 72)})
    assert sized == _cfg(MOK_A) and expected_tensors(sized)["l3.mix.a2"].shape == (80, 4)


def test_schedule_and_caches():
    """A looped layer is bound once and has a cache per pass; the head of every pass is a stop of its own; the
    embedding keeps one number per sequence behind the stops."""
    from stratum_b200.cache.store import KVSpec, StateSpec
    from stratum_b200.config import find_architecture
    from stratum_b200.engine.model import Model
    arch = find_architecture(MOK_A)
    model = Model(arch.describe_model(_cfg(MOK_A)), None)
    assert [e.layer for e in model.schedule] == [0, 4, 1, 2, 5, 1, 2, 6, 1, 2, 3]
    specs = model.cache_specs()
    assert len(specs) == len(model.schedule) + 1 and specs[-1] == StateSpec((1,), "int32")
    assert specs[1] is None and specs[4] is None and specs[7] is None
    w = specs[0]
    assert isinstance(w, KVSpec) and (w.n_kv_heads, w.head_dim, w.v_dim, w.window, w.keep_first) == (2, 24, 16, 50, 3)
    assert specs[2] == specs[5] == specs[8] == StateSpec((3 * 12 * 20,), "float32")
    assert specs[3] == specs[6] == specs[9] and specs[3].window == 0 and specs[3].key_order != w.key_order
    ops = [model.layers[e.layer].part("op") for e in model.schedule if model.layers[e.layer].spec.arrangement == "stream_op"]
    assert [(o.row, o.readd) for o in ops] == [(0, False), (1, True), (2, True)]
    assert model.spec.keep_embedded
    assert not Model(arch.describe_model(_cfg(MOK_B)), None).spec.keep_embedded


def test_pages_behind_a_window_that_keeps_first_tokens():
    from stratum_b200.cache.pages import PagePool, SequencePages
    pool = PagePool(12)
    for keep, kept_pages in ((0, 0), (3, 1), (64, 1), (70, 2)):
        sp = SequencePages(pool, window=130, keep_first=keep)
        sp.reserve(600)
        sp.advance(600)
        first_seen = (600 - 130 + 1) // 64
        held = [i for i, p in enumerate(sp.table) if p >= 0]
        assert held == list(range(kept_pages)) + list(range(first_seen, 10)), (keep, held)
        sp.reserve(70)
        sp.advance(70)
        assert [i for i, p in enumerate(sp.table) if p >= 0][:kept_pages] == list(range(kept_pages))
        sp.release()
        pool.check()
        assert pool.free_pages == 12


# ------------------------------------------------------------------------------------------ the oracle against itself
def _weights(raw, seed=0):
    from stratum_b200.engine.model import expected_tensors
    rng = np.random.default_rng(seed)
    w = {}
    for name, spec in expected_tensors(_cfg(raw)).items():
        w[name] = rng.standard_normal(spec.shape) * (0.3 if len(spec.shape) == 2 else 0.5)
    return w


def test_plain_gla_is_a_decayed_sum_over_the_past():
    """o_t = sum_{s <= t} (q_t . (prod_{s < r <= t} alpha_r * k_s)) v_s: the recurrence unrolled."""
    rng = np.random.default_rng(0)
    T, H, d, dv = 9, 2, 5, 3
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    alpha = rng.uniform(0.3, 1.0, (T, H, d))
    o, S = M.gla_recurrence(q, k, v, alpha)
    want = np.zeros_like(o)
    for t in range(T):
        for s in range(t + 1):
            decay = np.prod(alpha[s + 1:t + 1], axis=0)
            want[t] += np.einsum("hd,hd->h", q[t], decay * k[s])[:, None] * v[s]
    assert np.allclose(o, want, atol=1e-12)
    o2, _ = M.gla_recurrence(q[5:], k[5:], v[5:], alpha[5:], state=M.gla_recurrence(q[:5], k[:5], v[:5], alpha[:5])[1])
    assert np.allclose(o2, o[5:], atol=1e-12)


def test_plain_window_and_sink():
    """The mask row by row, and the sink as one more key with a zero value."""
    rng = np.random.default_rng(1)
    T, H, G, d, dv = 30, 4, 2, 6, 5
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, G, d)), rng.standard_normal((T, G, dv))
    sink = rng.uniform(-1, 2, H)
    got = M.masked_softmax_attention(q, k, v, 0.4, sink, 7, 2)
    for t in (0, 1, 6, 7, 8, 9, 29):
        for h in range(H):
            seen = [j for j in range(t + 1) if t - j < 7 or j < 2]
            assert (t < 9) == (seen == list(range(t + 1)))
            s = np.array([q[t, h] @ k[j, h // 2] * 0.4 for j in seen] + [sink[h]])
            a = np.exp(s - s.max())
            a /= a.sum()
            assert np.allclose(got[t, h], a[:-1] @ v[seen, h // 2], atol=1e-12)
    everything = M.masked_softmax_attention(q, k, v, 0.4, np.zeros(H), 0, 0)
    s = np.array([q[29, 0] @ k[j, 0] * 0.4 for j in range(30)])
    assert np.allclose(everything[29, 0], (np.exp(s) / (1.0 + np.exp(s).sum())) @ v[:, 0], atol=1e-12)


def test_plain_rotation_keeps_relative_positions():
    """Rotated q . k depends on the distance alone, in both pair layouts, times the magnitude squared."""
    rng = np.random.default_rng(2)
    for rot, neighbours in ((MOK_A["layers"][0]["mixer"]["rot"], True), (MOK_A["layers"][2]["mixer"]["rot"], False)):
        f, mag = M.frequencies(rot)
        d = rot["dims"] + 4
        q, k = rng.standard_normal((1, 1, d)), rng.standard_normal((1, 1, d))
        dots = [float(M.rotate(q, [p + 5], f, mag, neighbours)[0, 0] @ M.rotate(k, [p], f, mag, neighbours)[0, 0])
                for p in (0, 3, 100)]
        assert np.allclose(dots, dots[0], atol=1e-9)
        plain_part = float(q[0, 0, rot["dims"]:] @ k[0, 0, rot["dims"]:])
        same = float(M.rotate(q, [7], f, mag, neighbours)[0, 0] @ M.rotate(k, [7], f, mag, neighbours)[0, 0])
        assert np.isclose(same - plain_part, mag * mag * float(q[0, 0, :rot["dims"]] @ k[0, 0, :rot["dims"]]))
    f, mag = M.frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0}})
    assert mag == 1.0 and np.allclose(f, [0.25 * 100.0 ** (-i / 4) for i in range(4)])


def test_plain_model_token_by_token_embedding_and_loop():
    """The pair table's row depends on the token in front; the passes of a loop add the pass's vector and, from the
    second on, the embedded tokens."""
    w = _weights(MOK_A, 3)
    toks = [5, 9, 9, 200, 0, 17]
    x0 = M.embed(MOK_A, w, toks)
    big = MOK_A["embedding"]["bigram"]
    assert np.allclose(x0[0], w["embed"][5] * 3.0 + w["bigram"][big["buckets"]])
    assert np.allclose(x0[3], w["embed"][200] * 3.0 + w["bigram"][(9 * 7 + 200 * 13) % 53])
    streams = []
    logits = M.forward(MOK_A, w, toks, streams)
    assert len(streams) == 8 and logits.shape == (6, MOK_A["vocab"])
    x = M.layer(MOK_A, w, 0, x0)
    assert np.allclose(streams[0], x)
    x = M.layer(MOK_A, w, 1, x + w["loop.step"][0])
    assert np.allclose(streams[1], x)
    x = M.layer(MOK_A, w, 1, M.layer(MOK_A, w, 2, x) + x0 + w["loop.step"][1])
    assert np.allclose(streams[3], x)
    # causal: a prefix's logits do not depend on what follows
    assert np.allclose(M.forward(MOK_A, w, toks[:4]), logits[:4], atol=1e-9)


def test_plain_router_weights():
    w = _weights(MOK_A, 4)
    h = np.random.default_rng(0).standard_normal((7, MOK_A["width"]))
    f = MOK_A["layers"][0]["mlp"]
    chosen, weights = M.route(f, w, "l0.mlp.", h)
    z = h @ w["l0.mlp.router"].T + w["l0.mlp.router.b"]
    for t in range(7):
        best = sorted(range(6), key=lambda e: -z[t, e])[:2]
        assert list(chosen[t]) == best
        assert np.allclose(weights[t], np.exp(z[t, best]) / np.exp(z[t, best]).sum())
