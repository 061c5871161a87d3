"""MokatarConfig: the sizes and constants of a Mokatar decoder, read from config.json.

A Mokatar config.json names its architecture under "architecture", gives "vocab", "width", "norm": {"eps"},
"logit_scale", "embedding": {"scale", "bigram": {"buckets", "mul_prev", "mul_cur"}} (a file without "bigram" has no
pair table) and lists its layers one by one:
each entry gives the mixer's kind ("type": "attention", "attention_2" or "gla"), the mixer's sizes and constants
("mixer") and its feed-forward ("mlp": dense, a mixture of experts, or null for a layer that is a mixer alone).
"loop": {"start", "stop", "times"} makes the layers start .. stop - 1 run `times` times in a row with the same
weights, each pass with a cache of its own; a file without "loop" runs every layer once and has no "loop.step"
tensor.  Nothing about a layer is assumed from another layer: sizes and constants may differ from one entry to the
next, and the kinds may come in any order.

  attention     heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling: {factor, original, fast, slow}},
                mask: {size, keep_first}
  attention_2   heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling: {factor}}
  gla           heads, dim, vdim, tau
  mlp dense     kind "dense"; ff
  mlp moe       kind "moe"; router: {experts, top}; expert: {ff}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import KeyReader, ModelConfig
from .vitinex import LoopConfig

MIXER_KINDS = ("attention", "attention_2", "gla")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    factor: Optional[float] = None          # scaling.factor; None: frequencies as they are
    original: Optional[float] = None        # with original / fast / slow the scaling is the ramp between scaled and
    fast: Optional[float] = None            # unscaled frequencies; with the factor alone every frequency is divided
    slow: Optional[float] = None

    @property
    def ramp(self) -> bool:
        return self.original is not None

    @classmethod
    def from_reader(cls, r: KeyReader, head_dim: Optional[int]) -> "RotationConfig":
        base, dims = r.number("base", lo=1.0), r.integer("dims", lo=0, hi=1 << 14)
        factor = original = fast = slow = None
        sc = r.child("scaling")
        if sc is not None:
            factor = sc.number("factor", lo=1e-6)
            if any(k in sc.raw for k in ("original", "fast", "slow")):
                original = sc.number("original", lo=1e-6)
                fast = sc.number("fast", lo=1e-6)
                slow = sc.number("slow", lo=1e-6)
            r.adopt(sc)
        if dims and head_dim:
            r.require(dims % 2 == 0 and dims <= head_dim, f"rot.dims={dims} must be even and at most dim={head_dim}")
        return cls(base, dims, factor, original, fast, slow)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            d["scaling"] = {"factor": self.factor}
            if self.ramp:
                d["scaling"].update({"original": self.original, "fast": self.fast, "slow": self.slow})
        return d


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]
    window: int = 0              # mask.size; 0: every earlier key
    keep_first: int = 0          # mask.keep_first: the sequence's first tokens stay visible beyond the window

    masked = True                # whether this kind reads a "mask" object

    @classmethod
    def from_reader(cls, r: KeyReader) -> "AttentionMixerConfig":
        heads, kv = r.integer("heads", hi=1 << 14), r.integer("kv_heads", hi=1 << 14)
        dim, vdim = r.integer("dim", hi=1 << 14), r.integer("vdim", hi=1 << 14)
        scale = r.number("scale", lo=0.0)
        rr = r.child("rot")
        rot = None                   # a mixer without "rot" rotates nothing
        if rr is not None:
            rot = RotationConfig.from_reader(rr, dim)
            r.adopt(rr)
        window = keep = 0
        mk = r.child("mask") if cls.masked else None
        if mk is not None:
            window = mk.integer("size", lo=1, hi=1 << 30)
            keep = mk.integer("keep_first", default=0, lo=0, hi=1 << 30)
            r.adopt(mk)
        if heads and kv:
            r.require(heads % kv == 0, f"heads={heads} is not a multiple of kv_heads={kv}")
        return cls(heads, kv, dim, vdim, scale, rot, window or 0, keep or 0)

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.window:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return d


@dataclass(frozen=True)
class BiasedAttentionMixerConfig(AttentionMixerConfig):
    masked = False


@dataclass(frozen=True)
class LinearAttentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None   # the decay's inner size: the rows of the tensor 'a1' (None until a file says)

    @classmethod
    def from_reader(cls, r: KeyReader) -> "LinearAttentionMixerConfig":
        return cls(heads=r.integer("heads", hi=1 << 14), dim=r.integer("dim", hi=512), vdim=r.integer("vdim", hi=1 << 14),
                   tau=r.number("tau", lo=1e-6), rank=r.integer("rank", default=None, hi=1 << 14))

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


_MIXER_CONFIGS = {"attention": AttentionMixerConfig, "attention_2": BiasedAttentionMixerConfig,
                  "gla": LinearAttentionMixerConfig}


@dataclass(frozen=True)
class MokatarMlp:
    kind: str                    # one of MLP_KINDS
    ff: int                      # dense: the feed-forward's size; moe: an expert's
    experts: int = 0
    top: int = 0

    @classmethod
    def from_reader(cls, r: KeyReader) -> "MokatarMlp":
        kind = r.string("kind", choices=MLP_KINDS)
        if kind == "dense":
            return cls(kind=kind, ff=r.integer("ff", hi=1 << 24))
        router, expert = r.child("router"), r.child("expert")
        if kind == "moe":
            for key, sub in (("router", router), ("expert", expert)):
                if sub is None:
                    r.problems.append(f"missing required key '{key}'")
        out = cls(kind=kind or "moe", ff=expert.integer("ff", hi=1 << 24) if expert else None,
                  experts=router.integer("experts", hi=4096) if router else None,
                  top=router.integer("top", hi=4096) if router else None)
        for sub in (router, expert):
            if sub is not None:
                r.adopt(sub)
        if out.experts and out.top:
            r.require(out.top <= out.experts, f"router.top={out.top} exceeds router.experts={out.experts}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}


@dataclass(frozen=True)
class MokatarLayer:
    kind: str                          # one of MIXER_KINDS
    mixer: Any
    mlp: Optional[MokatarMlp]          # None: no feed-forward

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int

    def to_dict(self) -> Dict[str, Any]:
        return {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}


@dataclass(frozen=True)
class MokatarConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    logit_scale: float
    embedding_scale: float
    bigram: Optional[BigramConfig]
    layers: Tuple[MokatarLayer, ...]
    loop: Optional[LoopConfig] = None
    torch_dtype: str = "bfloat16"

    architecture = "Mokatar"

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
    def from_dict(cls, raw: Dict[str, Any]) -> "MokatarConfig":
        r = KeyReader(raw)
        vocab = r.integer("vocab", hi=1 << 26)
        width = r.integer("width", hi=1 << 20)
        logit_scale = r.number("logit_scale", default=1.0)
        norm = r.child("norm")
        eps = norm.number("eps", lo=0.0, hi=1.0) if norm is not None else None
        if norm is None:
            r.problems.append("missing required key 'norm'")
        else:
            r.adopt(norm)
        emb = r.child("embedding")
        emb_scale, bigram = 1.0, None        # without "bigram" the embedding is the token table's row times the scale
        if emb is not None:
            emb_scale = emb.number("scale", default=1.0)
            bg = emb.child("bigram")
            if bg is not None:
                buckets = bg.integer("buckets", hi=1 << 30)
                # the products previous * mul_prev + token * mul_cur are formed in 64 bits on the device
                mp, mc = bg.integer("mul_prev", lo=0, hi=1 << 30), bg.integer("mul_cur", lo=0, hi=1 << 30)
                emb.adopt(bg)
                if None not in (buckets, mp, mc):
                    bigram = BigramConfig(buckets, mp, mc)
            r.adopt(emb)
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
                    mlp = MokatarMlp.from_reader(fr)
                    lr.adopt(fr)
            layers.append(MokatarLayer(kind, mixer, mlp))
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
        return cls(vocab=vocab, width=width, eps=eps, logit_scale=logit_scale, embedding_scale=emb_scale,
                   bigram=bigram, layers=tuple(layers), loop=loop, torch_dtype=raw.get("torch_dtype", "bfloat16"))

    def with_decay_ranks(self, shapes) -> "MokatarConfig":
        """The same configuration with every gla layer's inner decay size taken from the shape of its 'a1' tensor
        (`shapes`: tensor name -> shape), which is where a file says it."""
        layers = []
        for i, layer in enumerate(self.layers):
            shape = shapes.get(f"l{i}.mix.a1")
            if layer.kind == "gla" and shape is not None and len(shape) == 2:
                m = layer.mixer
                layer = MokatarLayer(layer.kind, LinearAttentionMixerConfig(m.heads, m.dim, m.vdim, m.tau, int(shape[0])),
                                     layer.mlp)
            layers.append(layer)
        return MokatarConfig(self.vocab, self.width, self.eps, self.logit_scale, self.embedding_scale, self.bigram,
                             tuple(layers), self.loop, self.torch_dtype)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.eps}, "logit_scale": self.logit_scale,
             "embedding": {"scale": self.embedding_scale},
             "layers": [layer.to_dict() for layer in self.layers], "torch_dtype": self.torch_dtype}
        if self.bigram is not None:
            d["embedding"]["bigram"] = self.bigram.to_dict()
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
