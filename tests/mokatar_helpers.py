"""Small Mokatar configurations and model folders for the tests.  None of them is anyone's model: sizes are chosen so
that no two of a layer's sizes are equal by accident, that counts are not 1 where the formulas divide by them, and
that the layers of one model differ from one another (heads, key and value sizes, rotated dimensions, windows, kept
first tokens, decay sizes, experts)."""
import numpy as np
import torch

from helpers import load_plain, make_model_dir
from plain import mokatar_plain as M


def windowed(heads=4, kv=2, dim=24, vdim=16, rot=12, base=10000.0, scale=0.2, factor=4.0, original=64, fast=8.0,
             slow=0.5, size=50, keep=3):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"base": base, "dims": rot, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}}
    if size:
        d["mask"] = {"size": size, "keep_first": keep}
    return d


def biased(heads=6, kv=3, dim=16, vdim=24, rot=8, base=1000.0, scale=0.3, factor=3.0):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": rot, "scaling": {"factor": factor}}}


def gla(heads=3, dim=12, vdim=20, tau=8.0, rank=10):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def dense(ff=96):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=211, width=72, eps=1e-5, logit_scale=0.7, emb_scale=3.0, buckets=53, mul_prev=7, mul_cur=13,
           loop=None):
    d = {"architecture": "Mokatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
         "embedding": {"scale": emb_scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
         "layers": layers}
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# a windowed layer with experts in front of the loop; a gla layer and a biased-attention layer without feed-forward
# looped three times; a gla layer with experts behind
MOK_A = config([layer("attention", windowed(), moe()),
                layer("gla", gla(), dense()),
                layer("attention_2", biased()),
                layer("gla", gla(heads=2, dim=40, vdim=8, tau=2.0, rank=4), moe(experts=8, top=3, ff=24))],
               loop=(1, 3, 3))
# no loop; sizes that no vector load divides (width 70, heads of 18 / 10, 20 / 22, 9 / 7): every fallback kernel; a
# scaling factor below one; a window shorter than a page that keeps nothing; as many kv heads as heads, and one
MOK_B = config([layer("attention_2", biased(heads=2, kv=1, dim=18, vdim=10, rot=18, factor=0.5), moe(experts=5, top=1, ff=30)),
                layer("attention", windowed(heads=3, kv=3, dim=20, vdim=22, rot=6, size=5, keep=0, factor=1.5, original=16), dense(50)),
                layer("gla", gla(heads=1, dim=9, vdim=7, tau=1.0, rank=3), dense(34))],
               vocab=97, width=70, eps=1e-6, logit_scale=1.9, emb_scale=0.6, buckets=11, mul_prev=1, mul_cur=0)
# sizes of the tensor-core kernels: multiples of 16 everywhere, the whole model looped twice, a window that spans pages
# and keeps more than a page of first tokens, eight query heads on a kv head
MOK_TC = config([layer("gla", gla(heads=4, dim=64, vdim=32, tau=16.0, rank=16), moe(experts=4, top=2, ff=32)),
                 layer("attention", windowed(heads=8, kv=1, dim=64, vdim=64, rot=32, scale=0.1, size=130, keep=70, original=32),
                       moe(experts=4, top=2, ff=32)),
                 layer("attention_2", biased(heads=4, kv=4, dim=32, vdim=48, rot=32, scale=0.15, factor=8.0), dense(160))],
                vocab=331, width=128, loop=(0, 3, 2), buckets=1000, mul_prev=1009, mul_cur=3)
# one mechanism each, alone
MOK_WINDOWED = config([layer("attention", windowed(heads=4, kv=2, dim=16, vdim=16, rot=8, size=40, keep=5))], width=64)
MOK_BIASED = config([layer("attention_2", biased(heads=4, kv=2, dim=16, vdim=8, rot=16))], width=64)
MOK_GLA = config([layer("gla", gla(heads=4, dim=8, vdim=16, tau=4.0, rank=6))], width=64)
MOK_MOE = config([layer("gla", gla(heads=1, dim=8, vdim=8, tau=4.0, rank=2), moe(experts=12, top=4))], width=64)
MOK_DENSE = config([layer("gla", gla(heads=1, dim=8, vdim=8, tau=4.0, rank=2), dense(120))], width=64)
MOK_LOOP = config([layer("gla", gla(heads=2, dim=8, vdim=8, tau=4.0, rank=2)),
                   layer("attention_2", biased(heads=2, kv=2, dim=8, vdim=8, rot=4))], width=64, loop=(0, 2, 4))

CONFIGS = {"A": MOK_A, "B": MOK_B, "TC": MOK_TC, "windowed": MOK_WINDOWED, "biased": MOK_BIASED, "gla": MOK_GLA,
           "moe": MOK_MOE, "dense": MOK_DENSE, "loop": MOK_LOOP}


def lively(tensors, seed=0, decisive=False):
    """Random weights as the writer makes them are tame: norms of gain one, sinks and biases of zero, decays that are
    all alike, routers that hardly prefer anyone.  Give every constant a value of its own and make scores spread.

    decisive: the routers' choices survive the rounding of the bfloat16 path: the routers' biases lie 0.7 apart and
    their matrices are faint, so the choice is nearly the same for every token while the weights still vary; the
    float32 tests have routers that choose freely."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda t, lo, hi: (torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype)      # noqa: E731
    for name, t in list(tensors.items()):
        if name.endswith(("norm1", "norm2", "final.norm")):
            tensors[name] = rnd(t, -0.5, 0.5)                       # stored around zero, acts as 1 + w
        elif name.endswith((".q.norm", ".k.norm", ".mix.norm")):
            tensors[name] = rnd(t, 0.5, 1.5)
        elif name.endswith(".sink"):
            tensors[name] = rnd(t, -1.0, 3.0)
        elif name.endswith(".a2.b"):
            tensors[name] = rnd(t, 0.0, 5.0)                        # decays from 0.5^(1/tau) to nearly one
        elif name.endswith(".router.b"):
            n = t.shape[0]
            tensors[name] = ((0.7 if decisive else 0.3) * torch.randperm(n, generator=g).float()).to(t.dtype)
        elif name.endswith(".b"):                                   # the biased attention's q, k, v
            tensors[name] = rnd(t, -0.5, 0.5)
        elif name == "loop.step":
            tensors[name] = rnd(t, -0.5, 0.5)
        elif name.endswith(".router"):
            tensors[name] = (t.float() * (0.1 if decisive else 6.0)).to(t.dtype)
        elif name == "embed":
            tensors[name] = (t.float() * 10).to(t.dtype)
        elif name == "bigram":
            tensors[name] = (t.float() * 20).to(t.dtype)
        elif name.endswith((".q", ".k", ".v", ".g", ".o", ".a1", ".a2", ".gate", ".up", ".down")):
            tensors[name] = (t.float() * 2.5).to(t.dtype)


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
    return M.forward(cfg, w, tokens)


def clear_tokens(rng, n, cfg, w, dtype, fixed=None):
    """n random tokens (fixed: position -> token) on which no router is near a tie: a choice that rounding could turn
    is no test of anything.  float32 keeps 1e-4 away (in logits), bfloat16 (with decisive routers) 0.1."""
    need = 1e-4 if dtype == "float32" else 0.1
    for _ in range(200):
        toks = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
        for p, t in (fixed or {}).items():
            toks[p] = t
        margins = []
        M.forward(cfg, w, toks, margins=margins)
        if not margins or min(margins) > need:
            return toks
    raise AssertionError("no token sequence keeps the routers away from ties")


def assert_rows_close(got, ref, dtype, what=""):
    """float32: every logit within the float32 tolerance.  bfloat16: a position here and there sits where rounding
    is amplified, so the tolerance holds for 19 of 20 positions and three times the tolerance for all of them.  The
    rows' means are taken off first."""
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
