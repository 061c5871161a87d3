"""Vitinex on the CPU: the configuration reader, the order in which looped layers run, the tensor list, what each
stop of the schedule keeps in the cache, and the plain implementation's own properties (each mechanism restated a
second way)."""
import copy

import numpy as np
import pytest

from vitinex_helpers import CONFIGS, VIT_A, VIT_B, config, latent, layer, ssm
from plain import vitinex_plain as V


def _cfg(raw):
    from stratum_b200.config import find_architecture
    return find_architecture(raw).config_class.from_dict(raw)


def test_configuration_round_trip_and_registry():
    from stratum_b200.config import find_architecture
    from stratum_b200.config.vitinex import VitinexConfig
    assert find_architecture({"architecture": "Vitinex"}).config_class is VitinexConfig
    for raw in CONFIGS.values():
        cfg = _cfg(raw)
        assert VitinexConfig.from_dict(cfg.to_dict()) == cfg
        assert [la.kind for la in cfg.layers] == [e["type"] for e in raw["layers"]]
        assert (cfg.loop is None) == ("loop" not in raw)
    raw = copy.deepcopy(VIT_B)
    raw["loop"] = None                                       # a file may say "no loop" in so many words
    assert _cfg(raw).loop is None


def test_configuration_problems_are_listed_together():
    from stratum_b200.config import ConfigError
    raw = copy.deepcopy(VIT_A)
    del raw["vocab"]
    raw["layers"][0]["mixer"]["groups"] = 3                  # 4 heads in 3 groups
    raw["layers"][0]["mlp"]["router"]["top"] = 7             # of 6 experts
    raw["layers"][1]["type"] = "convolution"
    raw["layers"][2]["mixer"]["norm_groups"] = 7             # 60 outputs in 7 parts
    raw["layers"][3]["mixer"]["rot"]["dims"] = 7
    del raw["layers"][3]["mixer"]["q_rank"]
    raw["loop"]["stop"] = 1                                  # not behind its start
    with pytest.raises(ConfigError) as e:
        _cfg(raw)
    text = str(e.value)
    for piece in ("vocab", "equal groups", "top=7", "convolution", "equal parts", "rot.dims", "q_rank", "loop.start"):
        assert piece in text, (piece, text)


def test_the_order_of_layer_runs():
    """Layers in front of the loop once, the looped stretch `times` times in a row, the rest once; the first layer of
    every pass is marked (the re-entry stands in front of it)."""
    runs = _cfg(VIT_A).runs()
    assert [i for i, _, _ in runs] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [t for _, t, _ in runs] == [None, 0, 0, 1, 1, 2, 2, None]
    assert [f for _, _, f in runs] == [False, True, False, True, False, True, False, False]
    assert [i for i, _, _ in _cfg(VIT_B).runs()] == [0, 1]
    once = copy.deepcopy(VIT_A)
    once["loop"] = {"start": 3, "stop": 4, "times": 1}       # one pass is still a pass: its re-entry runs
    assert [(i, f) for i, _, f in _cfg(once).runs()] == [(0, False), (1, False), (2, False), (3, True)]
    assert V.layer_runs(VIT_A) == runs and V.layer_runs(once) == _cfg(once).runs()


def test_tensor_names_and_shapes():
    from stratum_b200.engine.model import expected_tensors
    t = expected_tensors(_cfg(VIT_A))
    W = VIT_A["width"]
    assert {"embed", "final.norm", "loop.in", "loop.step"} <= set(t) and "head" not in t
    assert t["loop.in"].shape == (W, 2 * W) and t["loop.step"].shape == (3, W)
    assert not any(n.startswith(("l3.mlp", "l3.norm2")) for n in t)          # layer 3 is a mixer alone
    assert {"l3.norm1", "l3.norm1b", "l0.norm2b"} <= set(t)
    s = VIT_A["layers"][2]["mixer"]
    inner, bc = s["heads"] * s["vdim"], 2 * s["groups"] * s["state"]
    assert t["l2.mix.in"].shape == (2 * inner + bc + s["heads"], W)
    assert t["l2.mix.conv"].shape == (inner + bc, s["conv"]) and t["l2.mix.conv.b"].shape == (inner + bc,)
    assert t["l2.mix.A_log"].shape == t["l2.mix.D"].shape == t["l2.mix.dt_bias"].shape == (s["heads"],)
    assert t["l2.mix.norm"].shape == (inner,) and t["l2.mix.o"].shape == (W, inner)
    a = VIT_A["layers"][1]["mixer"]
    assert t["l1.mix.dq"].shape == (a["q_rank"], W) and t["l1.mix.dq.norm"].shape == (a["q_rank"],)
    assert t["l1.mix.uq"].shape == (a["heads"] * (a["dim"] + a["rot_dim"]), a["q_rank"])
    assert t["l1.mix.dkv"].shape == (a["kv_rank"] + a["rot_dim"], W) and t["l1.mix.dkv.norm"].shape == (a["kv_rank"],)
    assert t["l1.mix.uk"].shape == (a["heads"] * a["dim"], a["kv_rank"])
    assert t["l1.mix.uv"].shape == (a["heads"] * a["vdim"], a["kv_rank"])
    assert t["l1.mix.g"].shape == (a["heads"], W) and t["l1.mix.o"].shape == (W, a["heads"] * a["vdim"])
    assert t["l1.mlp.gate.b"].shape == (96,) and t["l1.mlp.down.b"].shape == (W,)
    m = VIT_A["layers"][0]["mlp"]
    assert t["l0.mlp.router"].shape == (m["router"]["experts"], W)
    assert t["l0.mlp.e5.down"].shape == (W, m["expert"]["ff"]) and "l0.mlp.e6.down" not in t
    assert t["l0.mlp.shared.up"].shape == (m["shared"]["ff"], W) and t["l0.mlp.shared.sg"].shape == (1, W)
    assert not any(n.startswith("l2.mlp.shared") for n in t)                   # layer 2's experts have no shared one
    assert "loop.in" not in expected_tensors(_cfg(VIT_B))


def test_what_each_stop_keeps():
    """Every run of a layer has a cache of its own, also the runs that share weights: latent attention keeps one row
    of rank + rotated numbers per token, a state-space layer a block of fixed size (the matrices of all heads and the
    convolution's tail), the re-entry nothing."""
    from stratum_b200.cache.store import KVSpec, StateSpec
    from stratum_b200.config import find_architecture
    from stratum_b200.engine.model import Model
    arch = find_architecture(VIT_A)
    specs = Model(arch.describe_model(_cfg(VIT_A)), None).cache_specs()
    kinds = ["state", None, "kv", "state", None, "kv", "state", None, "kv", "state", "kv"]
    assert len(specs) == len(kinds)
    for spec, kind in zip(specs, kinds):
        assert (spec is None) if kind is None else isinstance(spec, KVSpec if kind == "kv" else StateSpec)
    a = VIT_A["layers"][1]["mixer"]
    assert specs[2].n_kv_heads == 1 and specs[2].head_dim == a["kv_rank"] + a["rot_dim"] and specs[2].window == 0
    assert specs[2] == specs[5] == specs[8] and specs[10] != specs[2]
    s = VIT_A["layers"][2]["mixer"]
    inner = s["heads"] * s["vdim"]
    channels = inner + 2 * s["groups"] * s["state"]
    assert specs[3].shape == (inner * s["state"] + (s["conv"] - 1) * channels,) and specs[3].dtype == "float32"


def test_plain_layer_norm_has_no_bias_and_the_variance_of_deviations():
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((3, 9)) + 4.0, rng.uniform(0.5, 1.5, 9)
    got = V.layer_norm(x, w, 1e-3)
    for i in range(3):
        mu = sum(x[i]) / 9
        var = sum((v - mu) ** 2 for v in x[i]) / 9
        np.testing.assert_allclose(got[i], [(v - mu) / (var + 1e-3) ** 0.5 * g for v, g in zip(x[i], w)], rtol=1e-12)
    np.testing.assert_allclose(V.layer_norm(x + 100.0, w, 1e-3), got, rtol=1e-9)     # a shift changes nothing


def test_plain_state_space_scan_equals_its_sum_over_the_past():
    """y_t = sum over s <= t of (product of the decays after s) dt_s (C_t . B_s) x_s + D x_t: the attention-like form
    of the same recurrence."""
    rng = np.random.default_rng(1)
    T, H, G, N, P = 9, 4, 2, 5, 3
    x, B, C = rng.standard_normal((T, H, P)), rng.standard_normal((T, G, N)), rng.standard_normal((T, G, N))
    dt, a_log, D = rng.uniform(0.1, 1.5, (T, H)), rng.uniform(-1, 0.5, H), rng.standard_normal(H)
    got = V.ssm_scan(x, B, C, dt, a_log, D, H, G)
    for j in range(H):
        g = j // (H // G)
        for t in range(T):
            want = D[j] * x[t, j]
            for s in range(t + 1):
                decay = np.exp(-np.exp(a_log[j]) * dt[s + 1:t + 1, j].sum())
                want = want + decay * dt[s, j] * (C[t, g] @ B[s, g]) * x[s, j]
            np.testing.assert_allclose(got[t, j], want, rtol=1e-10, atol=1e-12)


def test_plain_convolution_ends_on_the_current_token():
    x = np.arange(1.0, 6.0).reshape(5, 1)
    taps = np.array([[100.0, 10.0, 1.0]])
    np.testing.assert_allclose(V.causal_conv(x, taps, [0.5])[:, 0], [1.5, 12.5, 123.5, 234.5, 345.5])


def test_plain_latent_attention_equals_the_form_that_carries_queries_into_the_latent_space():
    """((Wuk_j^T q_j) . c_t + q_rot_j . kr_t) scale over the cached rows [c | kr], and Wuv_j applied to the mixed
    latent: the same numbers as per-head keys and values."""
    rng = np.random.default_rng(2)
    m = latent(heads=2, dim=6, rot=4, vdim=5, rank=7, q_rank=8, base=50.0, scale=0.4)
    T, W = 8, 10
    h = rng.standard_normal((T, W))
    w = {"dq": rng.standard_normal((8, W)), "dq.norm": rng.uniform(0.5, 1.5, 8), "uq": rng.standard_normal((20, 8)),
         "dkv": rng.standard_normal((11, W)), "dkv.norm": rng.uniform(0.5, 1.5, 7), "uk": rng.standard_normal((12, 7)),
         "uv": rng.standard_normal((10, 7)), "g": rng.standard_normal((2, W)), "o": np.eye(10)}
    got = V.latent_attention(h, w, m, 1e-5).reshape(T, 2, 5)
    pos = np.arange(T)
    q = (V.rms_norm(h @ w["dq"].T, w["dq.norm"], 1e-5) @ w["uq"].T).reshape(T, 2, 10)
    low = h @ w["dkv"].T
    c = V.rms_norm(low[:, :7], w["dkv.norm"], 1e-5)
    kr = V.rotate_pairs(low[:, 7:].reshape(T, 1, 4), pos, 50.0, 4)[:, 0]
    qr = V.rotate_pairs(q[:, :, 6:], pos, 50.0, 4)
    gate = 1.0 / (1.0 + np.exp(-(h @ w["g"].T)))
    for j in range(2):
        uk, uv = w["uk"][6 * j:6 * j + 6], w["uv"][5 * j:5 * j + 5]
        for i in range(T):
            s = np.array([((uk.T @ q[i, j, :6]) @ c[t] + qr[i, j] @ kr[t]) * 0.4 for t in range(i + 1)])
            a = np.exp(s - s.max()); a /= a.sum()
            np.testing.assert_allclose(got[i, j], uv @ (a @ c[:i + 1]) * gate[i, j], rtol=1e-9, atol=1e-12)


def test_plain_router_takes_softmax_scores_as_weights():
    h = np.array([[1.0, 0.0], [0.0, 1.0]])
    router = np.array([[2.0, 0.0], [1.0, 3.0], [0.0, 1.0], [2.0, -1.0]])     # expert 0 and 3 tie on the first token
    margins = []
    chosen, score = V.route_softmax(h, router, 2, margins)
    assert list(chosen[0]) == [0, 3] and list(chosen[1]) == [1, 2]           # the lower index first among equals
    z = router @ h[1]
    s = np.exp(z) / np.exp(z).sum()
    np.testing.assert_allclose(score[1], [s[1], s[2]], rtol=1e-12)           # not divided by their sum
    assert score[1].sum() < 1.0 and margins[1] == pytest.approx(1.0)


def test_whole_model_runs_on_every_configuration():
    from stratum_b200.engine.model import expected_tensors
    for name, raw in CONFIGS.items():
        rng = np.random.default_rng(3)
        w = {n: rng.standard_normal(ts.shape) * 0.1 for n, ts in expected_tensors(_cfg(raw)).items()}
        streams = []
        out = V.forward([1, 2, 3, 4, 5, 6, 7], w, raw, streams)
        assert out.shape == (7, raw["vocab"]) and np.isfinite(out).all(), name
        assert len(streams) == len(V.layer_runs(raw))


def test_a_model_of_other_order_and_sizes_is_described():
    """Layer kinds in any order, a loop anywhere, a layer without feed-forward inside the loop."""
    from stratum_b200.config import find_architecture
    raw = config([layer("latent_attention", latent(heads=5, dim=8, rot=2, vdim=4, rank=12, q_rank=6)),
                  layer("latent_attention", latent()),
                  layer("mamba2", ssm(heads=6, vdim=4, state=3, groups=6, conv=1, norm_groups=24))],
                 vocab=33, width=20, loop=(2, 3, 5), mult=2.0)
    spec = find_architecture(raw).describe_model(_cfg(raw))
    assert len(spec.schedule) == 2 + 5 * 2
    assert spec.keep_embedded
