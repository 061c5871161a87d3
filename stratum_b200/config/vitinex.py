"""VitinexConfig: the sizes and constants of a Vitinex decoder, read from config.json.

A Vitinex config.json names its architecture under "architecture", gives "vocab", "width", "norm": {"eps"} and
"residual_mult" (the factor on every sublayer's contribution to the residual stream), and lists its layers one by
one: each entry gives the mixer's kind ("type": "latent_attention" or "mamba2"), the mixer's sizes and constants
("mixer") and its feed-forward ("mlp": dense, a mixture of experts, or null for a layer that is a mixer alone).
"loop": {"start", "stop", "times"} makes the layers start .. stop - 1 run `times` times in a row with the same
weights, each pass with a cache of its own; a file without "loop" runs every layer once and has no re-entry tensors.
Nothing about a layer is assumed from another layer: sizes and constants may differ from one entry to the next, and
the kinds may come in any order.

  latent_attention  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}
  mamba2            heads, vdim, state, groups, conv (taps), norm_groups
  mlp dense         kind "dense"; ff
  mlp moe           kind "moe"; router: {experts, top}; expert: {ff}; shared: {ff} (optional)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import KeyReader, ModelConfig

MIXER_KINDS = ("latent_attention", "mamba2")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class QueryLatentMixerConfig:
    heads: int
    dim: int                 # unrotated query/key dimensions per head
    rot_dim: int             # rotated query/key dimensions per head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int            # how many of the rot_dim dimensions are rotated

    @classmethod
    def from_reader(cls, r: KeyReader) -> "QueryLatentMixerConfig":
        rot = r.child("rot")
        if rot is None:
            r.problems.append("missing required key 'rot'")
        out = cls(heads=r.integer("heads", hi=1 << 14), dim=r.integer("dim", hi=1 << 14),
                  rot_dim=r.integer("rot_dim", hi=1 << 14), vdim=r.integer("vdim", hi=1 << 14),
                  kv_rank=r.integer("kv_rank", hi=1 << 16), q_rank=r.integer("q_rank", hi=1 << 16),
                  scale=r.number("scale", lo=0.0),
                  rot_base=rot.number("base", lo=1.0) if rot else None,
                  rot_dims=rot.integer("dims", hi=1 << 14) if rot else None)
        if rot is not None:
            r.adopt(rot)
        if out.rot_dims and out.rot_dim:
            r.require(out.rot_dims % 2 == 0 and out.rot_dims <= out.rot_dim,
                      f"rot.dims={out.rot_dims} must be even and at most rot_dim={out.rot_dim}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class StateSpaceMixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int                # taps of the short convolution, the current token's included
    norm_groups: int

    @classmethod
    def from_reader(cls, r: KeyReader) -> "StateSpaceMixerConfig":
        out = cls(heads=r.integer("heads", hi=1 << 14), vdim=r.integer("vdim", hi=1 << 14),
                  state=r.integer("state", hi=512), groups=r.integer("groups", default=1, hi=1 << 14),
                  conv=r.integer("conv", hi=64), norm_groups=r.integer("norm_groups", default=1, hi=1 << 14))
        if out.heads and out.groups:
            r.require(out.heads % out.groups == 0, f"heads={out.heads} do not form groups={out.groups} equal groups")
        if out.heads and out.vdim and out.norm_groups:
            r.require((out.heads * out.vdim) % out.norm_groups == 0,
                      f"heads * vdim = {out.heads * out.vdim} does not form norm_groups={out.norm_groups} equal parts")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


_MIXER_CONFIGS = {"latent_attention": QueryLatentMixerConfig, "mamba2": StateSpaceMixerConfig}


@dataclass(frozen=True)
class VitinexMlp:
    kind: str                    # one of MLP_KINDS
    ff: int                      # dense: the feed-forward's size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None     # moe: the shared expert's size; None: no shared expert

    @classmethod
    def from_reader(cls, r: KeyReader) -> "VitinexMlp":
        kind = r.string("kind", choices=MLP_KINDS)
        if kind == "dense":
            return cls(kind=kind, ff=r.integer("ff", hi=1 << 24))
        router, expert, shared = r.child("router"), r.child("expert"), r.child("shared")
        if kind == "moe":
            for key, sub in (("router", router), ("expert", expert)):
                if sub is None:
                    r.problems.append(f"missing required key '{key}'")
        out = cls(kind=kind or "moe", ff=expert.integer("ff", hi=1 << 24) if expert else None,
                  experts=router.integer("experts", hi=4096) if router else None,
                  top=router.integer("top", hi=4096) if router else None,
                  shared_ff=shared.integer("ff", hi=1 << 24) if shared else None)
        for sub in (router, expert, shared):
            if sub is not None:
                r.adopt(sub)
        if out.experts and out.top:
            r.require(out.top <= out.experts, f"router.top={out.top} exceeds router.experts={out.experts}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class VitinexLayer:
    kind: str                          # one of MIXER_KINDS
    mixer: Any                         # QueryLatentMixerConfig | StateSpaceMixerConfig
    mlp: Optional[VitinexMlp]          # None: no feed-forward

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int                # one past the last looped layer
    times: int

    def to_dict(self) -> Dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class VitinexConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[VitinexLayer, ...]
    loop: Optional[LoopConfig] = None
    torch_dtype: str = "bfloat16"

    architecture = "Vitinex"

    def runs(self):
        """The order in which the layers run: (layer, pass or None, first of its pass) per run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        lp = self.loop
        out = [(i, None, False) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t, i == lp.start) for i in range(lp.start, lp.stop)]
        return out + [(i, None, False) for i in range(lp.stop, n)]

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VitinexConfig":
        r = KeyReader(raw)
        vocab = r.integer("vocab", hi=1 << 26)
        width = r.integer("width", hi=1 << 20)
        mult = r.number("residual_mult", default=1.0)
        norm = r.child("norm")
        eps = norm.number("eps", lo=0.0, hi=1.0) if norm is not None else None
        if norm is None:
            r.problems.append("missing required key 'norm'")
        else:
            r.adopt(norm)
        entries = raw.get("layers")
        layers = []
        if not isinstance(entries, list) or not entries:
            r.problems.append("'layers' must be a non-empty list")
            entries = []
        for i, e in enumerate(entries):
            lr = KeyReader(e if isinstance(e, dict) else {}, f"config.json:layers[{i}]")
            if not isinstance(e, dict):
                lr.problems.append("must be an object")
            kind = lr.string("type", choices=MIXER_KINDS)
            mr = lr.child("mixer")
            mixer = None
            if mr is None:
                lr.problems.append("missing required key 'mixer'")
            elif kind is not None:
                mixer = _MIXER_CONFIGS[kind].from_reader(mr)
                lr.adopt(mr)
            mlp = None
            if isinstance(e, dict) and e.get("mlp") is not None:
                fr = lr.child("mlp")
                if fr is not None:
                    mlp = VitinexMlp.from_reader(fr)
                    lr.adopt(fr)
            layers.append(VitinexLayer(kind, mixer, mlp))
            r.adopt(lr)
        loop = None
        lp = r.child("loop")
        if lp is not None:
            n = max(len(layers), 1)
            start = lp.integer("start", lo=0, hi=n - 1)
            stop = lp.integer("stop", lo=1, hi=n)
            times = lp.integer("times", lo=1, hi=1 << 10)
            r.adopt(lp)
            if start is not None and stop is not None:
                r.require(start < stop, f"loop.start={start} must lie before loop.stop={stop}")
            if None not in (start, stop, times):
                loop = LoopConfig(start, stop, times)
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=mult, layers=tuple(layers), loop=loop,
                   torch_dtype=raw.get("torch_dtype", "bfloat16"))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
             "layers": [layer.to_dict() for layer in self.layers], "torch_dtype": self.torch_dtype}
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
