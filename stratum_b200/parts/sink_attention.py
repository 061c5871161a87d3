"""Grouped-query attention over a sliding window, with normalised queries and keys and a sink in the softmax.

Per token, with h the mixer's input and p its position:  q = Wq h ([heads][d]), k = Wk h ([kv heads][d]); v = k as
projected (no value matrix), or (`v_dim`) v = Wv h ([kv heads][dv]); the projections may have biases.  q and k are
each divided by a root mean square (eps inside the root) and multiplied by a gain: of their whole row (all heads
together) with a gain per column, or (`qk_norm: per_head`) of every head by itself with one gain of d values for all
heads; then the first dimensions of every head are rotated by the position encoding, in neighbouring pairs
(2i, 2i + 1) or in pairs (i, i + n/2) as the encoding says.  Head j (kv head j / (heads / kv heads)):

    s_t = (q_j . k_t) * scale         for the keys t with 0 <= p - t < window or t < keep_first (window 0: every t <= p)
    a_t = exp(s_t) / (sum_t exp(s_t) + exp(sink_j))            (the sink has no key and no value and is not scaled)
    o_j = sum_t a_t v_t;      result = Wo concat_j(o_j)

The sink is a learned number per head, the constant 0 (`sink: "zero"`: one added to every denominator), or absent.
The projections run as one product whose float32 sums go to one kernel that normalises, rotates, rounds once and
appends to the cache (csrc/qk_norm_rope.cu); the attention itself is the general kernel (kernels.AttentionShape) with
its window, kept first keys and sink parameters.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS
from ..cache.store import KVSpec, LayerCache
from .base import Mixer
from .latent_attention import padded
from .linear import ADD_TO_F32, STORE_F32, Linear
from .registry import find_part, register_part
from .spec import PartSpec, TensorSpec


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, scale, window (0 = all keys), keep_first (with a window: the
    positions below it stay visible), eps (of the two norms), position (PartSpec of a rotating position encoding, or
    None), sink (True: a learned number per head, the default; "zero": the constant 0; False: none), v_dim (None:
    the values are the keys as projected; else a value matrix of n_kv_heads * v_dim rows), qk_norm ("whole", the
    default, or "per_head"), bias (biases on the projections: name + ".b"), prefix, and the tensor names q, k, v, o,
    q_norm, k_norm, sink (defaults: q, k, v, o, q.norm, k.norm, sink)."""
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads, self.n_kv = int(spec["hidden"]), int(spec["n_heads"]), int(spec["n_kv_heads"])
        self.d = int(spec["head_dim"])
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = int(spec.get("window", 0) or 0)
        self.keep_first = int(spec.get("keep_first", 0) or 0) if self.window else 0
        sink = spec.get("sink", True)
        if sink not in (True, False, "zero"):
            raise ValueError(f"sink_attention: sink {sink!r} is not one of True, False, 'zero'")
        self.has_sink, self.zero_sink = sink is True, sink == "zero"
        v_dim = spec.get("v_dim")
        self.own_values = v_dim is not None
        self.dv = int(v_dim) if self.own_values else self.d
        norm = spec.get("qk_norm", "whole")
        if norm not in ("whole", "per_head"):
            raise ValueError(f"sink_attention: qk_norm {norm!r} is neither 'whole' nor 'per_head'")
        self.per_head = norm == "per_head"
        self.bias = bool(spec.get("bias", False))
        pos: Optional[PartSpec] = spec.get("position")
        self.position = find_part("position", pos.kind)(pos, runtime) if pos is not None else None
        self.half = False
        if self.position is not None:
            layout = self.position.pair_layout()
            if layout is None or 2 * layout[0] > self.d:
                raise ValueError("sink_attention rotates pairs among a head's first dimensions")
            self.half = not layout[1]
        defaults = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
        self.names = {k: self.prefix + str(spec.get(k + "_tensor", v)) for k, v in defaults.items()}
        self.q_cols, self.k_cols = self.n_heads * self.d, self.n_kv * self.d
        self.v_cols = self.n_kv * self.dv if self.own_values else 0
        self.o_cols = self.n_heads * self.dv
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None
        self.shape: Optional[K.AttentionShape] = None

    def _stacked(self):
        return ("q", "k", "v") if self.own_values else ("q", "k")

    def tensors(self) -> Dict[str, TensorSpec]:
        n = self.names
        cols = {"q": self.q_cols, "k": self.k_cols, "v": self.v_cols}
        t = {n[key]: TensorSpec((cols[key], self.hidden)) for key in self._stacked()}
        if self.bias:
            t.update({n[key] + ".b": TensorSpec((cols[key],), role="vector") for key in self._stacked()})
        t[n["o"]] = TensorSpec((self.hidden, self.o_cols))
        t[n["q_norm"]] = TensorSpec((self.d if self.per_head else self.q_cols,), role="vector", init="ones")
        t[n["k_norm"]] = TensorSpec((self.d if self.per_head else self.k_cols,), role="vector", init="ones")
        if self.has_sink:
            t[n["sink"]] = TensorSpec((self.n_heads,), role="vector", init="zeros")
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        b = torch.cat([weights[n[key] + ".b"] for key in self._stacked()]).contiguous() if self.bias else None
        self.w_in = Linear(self.runtime, torch.cat([weights[n[key]] for key in self._stacked()], dim=0).contiguous(), b)
        self.w_o = Linear(self.runtime, weights[n["o"]])
        self.q_gain, self.k_gain = weights[n["q_norm"]].contiguous(), weights[n["k_norm"]].contiguous()
        self.sink = None
        if self.has_sink:
            self.sink = weights[n["sink"]].contiguous()
        elif self.zero_sink:
            self.sink = torch.zeros(self.n_heads, dtype=torch.float32, device=self.q_gain.device)
        self.shape = K.AttentionShape(self.n_heads, self.n_heads // self.n_kv, 1, self.d, self.dv, False, self.scale,
                                      window=self.window, sink=self.sink, keep_first=self.keep_first)

    def cache_spec(self) -> KVSpec:
        order = "normed_rotated" + ("_half" if self.half else "") + ("" if self.own_values else "_values_raw")
        if not self.own_values:
            return KVSpec(self.n_kv, self.d, self.window, order, keep_first=self.keep_first)
        return KVSpec(self.n_kv, self.d, self.window, order, value_heads=self.n_kv, value_dim=self.dv,
                      keep_first=self.keep_first)

    def forward(self, xin, residual: torch.Tensor, step, cache: LayerCache, store: bool = False) -> None:
        T = xin.shape[0]
        width = self.q_cols + self.k_cols + self.v_cols
        proj = self.runtime.empty(T, padded(width), dtype=torch.float32)
        self.w_in(xin, out=proj[:, :width], mode=STORE_F32)
        q = self.runtime.empty(T, padded(self.q_cols))
        rot = self.position.rotary() if self.position is not None else None
        K.qk_norm_rope(proj, step.token_pos, step.token_seq, cache.block_table, self.q_gain, self.k_gain,
                       None if rot is None else rot.inv_freq, self.eps, q, cache.k, cache.v, self.n_heads, self.n_kv,
                       self.d, PAGE_TOKENS, cache.writes, v_dim=self.dv if self.own_values else 0,
                       per_head=self.per_head, half=self.half, magnitude=1.0 if rot is None else rot.magnitude)
        out = self.runtime.empty(T, padded(self.o_cols))
        from . import attention_dispatch
        attention_dispatch.run_general(self, self.shape, q, cache, step, out)
        self.w_o(out[:, :self.o_cols], out=residual, mode=STORE_F32 if store else ADD_TO_F32)
