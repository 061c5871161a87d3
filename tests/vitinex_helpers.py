"""Small Vitinex configurations and model folders for the tests.  None of them is anyone's model: sizes are chosen so
that no two of a layer's sizes are equal by accident, that counts are not 1 where the formulas divide by them, and
that the layers of one model differ from one another (heads, ranks, rotated dimensions, states, taps, experts)."""
import numpy as np
import torch

from helpers import load_plain, make_model_dir
from plain import vitinex_plain as V


def latent(heads=3, dim=24, rot=8, vdim=40, rank=56, q_rank=48, base=10000.0, scale=0.19, rot_dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
            "rot": {"base": base, "dims": rot if rot_dims is None else rot_dims}}


def ssm(heads=4, vdim=12, state=24, groups=2, conv=3, norm_groups=3):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff=96):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40, shared=56):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=211, width=72, eps=1e-5, mult=0.7, loop=None):
    d = {"architecture": "Vitinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
         "layers": layers}
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# a state-space layer in front of the loop, two looped layers run three times (latent attention with a dense
# feed-forward, a state-space layer with experts and no shared one), a latent layer without feed-forward behind it
VIT_A = config([layer("mamba2", ssm(), moe()),
                layer("latent_attention", latent(), dense()),
                layer("mamba2", ssm(heads=3, vdim=20, state=40, groups=3, conv=5, norm_groups=2), moe(experts=8, top=3, ff=24, shared=0)),
                layer("latent_attention", latent(heads=2, dim=16, rot=16, vdim=24, rank=40, q_rank=24, base=500.0, scale=0.3))],
               loop=(1, 3, 3))
# no loop; sizes that no vector load divides (width 70, heads of 20 + 6 and 18, a state of 10): every fallback kernel
VIT_B = config([layer("latent_attention", latent(heads=2, dim=20, rot=6, vdim=18, rank=34, q_rank=26, scale=0.3, rot_dims=4), moe(experts=5, top=1, ff=30, shared=22)),
                layer("mamba2", ssm(heads=2, vdim=9, state=10, groups=1, conv=2, norm_groups=1), dense(50))],
               vocab=97, width=70, eps=1e-6, mult=1.3)
# one mechanism each, alone
VIT_LATENT = config([layer("latent_attention", latent(heads=4, dim=16, rot=8, vdim=16, rank=32, q_rank=40))], width=64, mult=1.0)
VIT_SSM = config([layer("mamba2", ssm(heads=4, vdim=8, state=16, groups=1, conv=4, norm_groups=1))], width=64, mult=1.0)
VIT_MOE = config([layer("mamba2", ssm(heads=1, vdim=8, state=8, groups=1, conv=2, norm_groups=1), moe(experts=12, top=4))], width=64)
VIT_DENSE = config([layer("mamba2", ssm(heads=1, vdim=8, state=8, groups=1, conv=2, norm_groups=1), dense(136))], width=64)
VIT_LOOP = config([layer("mamba2", ssm(heads=2, vdim=8, state=8, groups=2, conv=2, norm_groups=2)),
                   layer("latent_attention", latent(heads=2, dim=8, rot=4, vdim=8, rank=16, q_rank=12))],
                  width=64, loop=(0, 2, 4), mult=0.4)
# sizes of the tensor-core kernels: multiples of 16 everywhere, the whole model looped twice, a state of 128
VIT_TC = config([layer("mamba2", ssm(heads=4, vdim=32, state=64, groups=2, conv=4, norm_groups=2), moe(experts=4, top=2, ff=32, shared=48)),
                 layer("latent_attention", latent(heads=4, dim=32, rot=32, vdim=48, rank=96, q_rank=64), moe(experts=4, top=2, ff=32, shared=48)),
                 layer("mamba2", ssm(heads=8, vdim=16, state=128, groups=1, conv=4, norm_groups=4), dense(160))],
                vocab=331, width=128, loop=(0, 3, 2), mult=0.5)

CONFIGS = {"A": VIT_A, "B": VIT_B, "latent": VIT_LATENT, "ssm": VIT_SSM, "moe": VIT_MOE, "dense": VIT_DENSE,
           "loop": VIT_LOOP, "TC": VIT_TC}

STEADY = 12.0        # the embedded tokens' first dimension under `decisive` weights


def lively(tensors, seed=0, decisive=False):
    """Random weights as the writer makes them are tame: norms of gain one, no biases, decays that are all alike,
    routers that hardly prefer anyone.  Give every constant a value of its own and make scores spread.

    decisive: the routers' choices survive the rounding of the bfloat16 path.  Every token's embedding carries the
    same large number in its first dimension, every re-entry hands it on unchanged, and so the first dimension of
    every normed input is a steady positive number; the routers read it with weights that lie half a unit apart (so the
    chosen experts' scores stay comparable) and everything else faintly.  The choice is then nearly the same for every token (the scores,
    which are the weights, still vary); the float32 tests have routers that choose freely."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda t, lo, hi: (torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype)      # noqa: E731
    for name, t in list(tensors.items()):
        if name.endswith((".dq.norm", ".dkv.norm", ".mix.norm", "norm1", "norm2", "norm1b", "norm2b", "final.norm")):
            tensors[name] = rnd(t, 0.5, 1.5)
        elif name.endswith(".A_log"):
            tensors[name] = rnd(t, -2.0, 0.5)
        elif name.endswith(".dt_bias"):
            tensors[name] = rnd(t, -1.0, 1.0)
        elif name.endswith(".D"):
            tensors[name] = rnd(t, -1.0, 1.5)
        elif name.endswith(".conv"):
            tensors[name] = rnd(t, -0.8, 0.8)
        elif name.endswith(".b"):                          # the convolutions' and the dense feed-forwards' biases
            tensors[name] = rnd(t, -0.3, 0.3)
        elif name == "loop.step":
            tensors[name] = rnd(t, -0.5, 0.5)
        elif name.endswith(".router"):
            m = t.float() * (0.1 if decisive else 6.0)
            if decisive:
                n = t.shape[0]
                m[:, 0] = 0.5 * torch.randperm(n, generator=g).float()
            tensors[name] = m.to(t.dtype)
        elif name == "embed":
            m = t.float() * 30
            if decisive:
                m[:, 0] = STEADY
            tensors[name] = m.to(t.dtype)
        elif name == "loop.in":
            m = t.float() * 2.5
            if decisive:
                m[0] = 0.0
                m[0, t.shape[0]] = 1.0                     # the first dimension of the embedded tokens, as it is
            tensors[name] = m.to(t.dtype)
        elif name.endswith((".dq", ".uq", ".dkv", ".uk", ".uv", ".g", ".o", ".in", ".gate", ".up", ".down", ".sg")):
            tensors[name] = (t.float() * 2.5).to(t.dtype)
    if decisive and "loop.step" in tensors:
        m = tensors["loop.step"].float()
        m[:, 0] = 0.0
        tensors["loop.step"] = m.to(tensors["loop.step"].dtype)


def make(path, name, dtype, seed=0, edit=None, cfg=None):
    decisive = dtype == "bfloat16"

    def both(tensors):
        lively(tensors, seed, decisive)
        if edit is not None:
            edit(tensors)
    path = make_model_dir(path, cfg or CONFIGS[name], seed=seed, dtype=dtype, std=0.05, edit=both)
    cfg, w = load_plain(path)
    return path, cfg, w


def plain_logits(cfg, w, tokens):
    return V.forward(tokens, w, cfg)


def clear_tokens(rng, n, cfg, w, dtype, fixed=None):
    """n random tokens (fixed: position -> token) on which no router is near a tie: a choice that rounding could turn
    is no test of anything.  float32 keeps 1e-4 away (in logits), bfloat16 (with decisive routers) 0.1."""
    need = 1e-4 if dtype == "float32" else 0.1
    for _ in range(200):
        toks = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
        for p, t in (fixed or {}).items():
            toks[p] = t
        margins = []
        V.forward(toks, w, cfg, margins=margins)
        if not margins or min(margins) > need:
            return toks
    raise AssertionError("no token sequence keeps the routers away from ties")


def assert_rows_close(got, ref, dtype, what=""):
    """float32: every logit within the float32 tolerance.  bfloat16: a position here and there sits where rounding
    is amplified (a norm behind an output that nearly cancels), so the tolerance holds for 19 of 20 positions and
    three times the tolerance for all of them.  The rows' means are taken off first (the steady dimension of the
    decisive weights shifts all logits of a row alike, which says nothing)."""
    from helpers import TOL, assert_close
    if dtype == "float32":
        return assert_close(got, ref, dtype, what)
    got, ref = np.atleast_2d(np.asarray(got, np.float64)), np.atleast_2d(np.asarray(ref, np.float64))
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    got, ref = got - got.mean(axis=-1, keepdims=True), ref - ref.mean(axis=-1, keepdims=True)
    err = np.max(np.abs(got - ref), axis=-1) / np.max(np.abs(ref))
    assert err.max() <= 3 * TOL[dtype], f"{what}: worst position off by {err.max():.3e} of the largest logit"
    over = int(np.sum(err > TOL[dtype]))
    assert over <= max(1, len(err) // 20), f"{what}: {over} of {len(err)} positions beyond {TOL[dtype]:.0e}"
