"""A mixture of experts: routed SwiGLU experts, of which every token uses a few, and a shared one.

Router, in float32:  z = Wr h;  s = sigmoid(z);  the choice score of expert e is s_e + correction_e.  The experts
form equal groups of neighbours; a group's score is the sum of its two largest choice scores, and only the experts
of the `keep` best groups can be chosen (the others' choice scores count as -inf).  The `top` experts with the
largest choice scores are chosen; their weights are s_e / (sum of the chosen s + 1e-20) * scale.

    result = sum_chosen weight_e * Wdown_e (silu(Wgate_e h) * Wup_e h)  +  the shared expert's output (weight 1)

Two ways to run the experts, chosen by the step's size:

* few tokens (decode steps, short prompts): all experts' gate and up matrices are stacked into one matrix (the shared
  expert's last) and all down matrices side by side into another, so the feed-forward is two matrix products whatever
  the number of experts: the first leaves every expert's activations side by side in a token's row, a small kernel
  multiplies each expert's stretch by the token's weight for it (zero where the expert was not chosen), and the second
  sums the weighted outputs.  A step of a few tokens reads most experts' weights anyway, and nothing on this way
  depends on a number the host would have to wait for, so it runs inside a captured decode step.
* many tokens (prompts): the (token, choice) pairs are put in the order of their experts on the device, the host reads
  the experts' counts (one small copy per layer), every expert runs its two products on its own stretch of gathered
  rows, and each token adds up its experts' outputs times its weights in the order of its choices; the shared expert
  runs on all rows.  Only the chosen experts' arithmetic is done.

Either way an expert a token did not choose contributes nothing, and a token's sum has a fixed order, so the result
does not depend on the other tokens of the step beyond the rounding of the products.

Variants, each a parameter: scores by softmax over all experts in sigmoid's place (`score`); the chosen scores used as
they are, not divided by their sum (`renorm` false); no correction tensor (`correction` false); experts without a gate
matrix, Wdown act(Wup h), with the activation named (`gated` false, `activation`); and a shared expert whose output is
multiplied by sigmoid(w_sg . h), one number per token (`shared_gate`: the name of that row of weights): the router's
kernel takes that dot product with the experts' and leaves the gate beside the experts' weights; and a bias on the
router's logits (`router_bias`: tensor router.b).  Softmax scores over all experts, renormalised over the chosen ones,
are the softmax over the chosen logits alone: a design that states its weights that way sets `score: softmax`.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from .base import FeedForward
from .linear import ADD_TO_F32, STORE, STORE_F32, SWIGLU, Linear
from .mlp import GATE_ACTS, interleave_rows
from .registry import register_part
from .spec import TensorSpec


# rows an expert gets on average from which a prompt step takes the grouped way (T * top / experts); measured on layer
# sizes of a 1B-like and an 8B-like model (numbers at `grouped` below).  STRATUM_MOE_GROUPED_MIN_ROWS sets it
# (measurements).
GROUPED_MIN_ROWS = int(os.environ.get("STRATUM_MOE_GROUPED_MIN_ROWS", 96))


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden, n_experts, top, scale, n_groups, keep, intermediate (of an expert), shared_intermediate (of
    the shared expert; None: none), prefix; score ("sigmoid" or "softmax"), renorm, correction, gated, activation
    ("silu", "gelu_tanh", "gelu_erf", "relu_sq"), shared_gate (tensor name under the prefix, or None), router_bias.
    Tensors: router, router.b, correction, e<i>.gate / .up / .down, shared.gate / .up / .down (no .gate when not gated)."""
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_experts, self.top = int(spec["hidden"]), int(spec["n_experts"]), int(spec["top"])
        self.scale = float(spec.get("scale", 1.0))
        self.n_groups, self.keep = int(spec.get("n_groups", 1) or 1), int(spec.get("keep", 1) or 1)
        self.ff = int(spec["intermediate"])
        shared = spec.get("shared_intermediate")
        self.shared_ff = int(shared) if shared else 0
        if self.n_experts % self.n_groups or self.keep > self.n_groups \
                or self.top > (self.n_experts // self.n_groups) * self.keep:
            raise ValueError("routed_experts: experts, groups, keep and top do not fit together")
        score = spec.get("score", "sigmoid")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"routed_experts: score {score!r} is neither 'sigmoid' nor 'softmax'")
        self.softmax = score == "softmax"
        self.renorm = bool(spec.get("renorm", True))
        self.has_correction = bool(spec.get("correction", True))
        self.gated = bool(spec.get("gated", True))
        act = spec.get("activation", "silu")
        if act not in GATE_ACTS or (not self.gated and act == "silu"):
            raise ValueError(f"routed_experts: activation {act!r} is not known"
                             + ("" if self.gated else " to experts without a gate"))
        self.act = GATE_ACTS[act]
        self.shared_gate = spec.get("shared_gate") if self.shared_ff else None
        self.has_router_bias = bool(spec.get("router_bias", False))
        self.correction = self.w_gate = self.router_bias = None
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def _experts(self):
        return [f"e{i}." for i in range(self.n_experts)] + (["shared."] if self.shared_ff else [])

    def tensors(self) -> Dict[str, TensorSpec]:
        p, H = self.prefix, self.hidden
        t = {p + "router": TensorSpec((self.n_experts, H), role="vector")}
        if self.has_correction:
            t[p + "correction"] = TensorSpec((self.n_experts,), role="vector", init="zeros")
        if self.has_router_bias:
            t[p + "router.b"] = TensorSpec((self.n_experts,), role="vector", init="zeros")
        if self.shared_gate:
            t[p + self.shared_gate] = TensorSpec((1, H), role="vector")
        for e in self._experts():
            ff = self.shared_ff if e == "shared." else self.ff
            t.update({p + e + "up": TensorSpec((ff, H)), p + e + "down": TensorSpec((H, ff))})
            if self.gated:
                t[p + e + "gate"] = TensorSpec((ff, H))
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.router = weights[p + "router"].contiguous()
        if self.has_correction:
            self.correction = weights[p + "correction"].contiguous()
        if self.shared_gate:
            self.w_gate = weights[p + self.shared_gate].reshape(-1).contiguous()
        if self.has_router_bias:
            self.router_bias = weights[p + "router.b"].contiguous()
        names = self._experts()
        ups = torch.cat([weights[p + e + "up"] for e in names], dim=0)
        # rows of an expert in the stacked first matrix: gate and up alternating, or the up matrix alone
        per = 2 if self.gated else 1
        stacked = interleave_rows(torch.cat([weights[p + e + "gate"] for e in names], dim=0), ups) if self.gated \
            else ups.contiguous()
        self.gate_up = Linear(self.runtime, stacked)
        self.down = Linear(self.runtime, torch.cat([weights[p + e + "down"] for e in names], dim=1).contiguous())
        # the grouped way: every expert's matrices by themselves (gate|up: stretches of the stacked rows; down: the
        # tensors as loaded, since a stretch of the stacked matrix's columns is not a matrix a product can take)
        first = [per * self.ff * i for i in range(self.n_experts)] + [per * self.ff * self.n_experts]
        sizes = [per * self.ff] * self.n_experts + [per * self.shared_ff]
        self.gate_up_of = [Linear(self.runtime, stacked[a:a + n]) for a, n in zip(first, sizes) if n]
        self.down_of = [Linear(self.runtime, weights[p + e + "down"].contiguous()) for e in names]

    def route(self, xin: torch.Tensor):
        """(dense weights [T, experts] with zeros for experts not chosen, chosen [T, top], their weights [T, top])."""
        T = xin.shape[0]
        dense = self.runtime.empty(T, self.n_experts + (1 if self.w_gate is not None else 0), dtype=torch.float32)
        chosen = self.runtime.empty(T, self.top, dtype=torch.int32)
        weights = self.runtime.empty(T, self.top, dtype=torch.float32)
        K.moe_route(xin, self.router, self.correction, dense, chosen, weights, self.top, self.n_groups, self.keep,
                    self.scale, softmax=self.softmax, renorm=self.renorm, w_gate=self.w_gate, bias=self.router_bias)
        return dense, chosen, weights

    def _first(self, lin: Linear, x: torch.Tensor) -> torch.Tensor:
        """An expert's (or all experts') activations: act(gate) * up, or act(up) where the experts have no gate."""
        if self.gated:
            return lin(x, mode=SWIGLU, act=self.act)
        return lin(x, mode=STORE, act=self.act)

    def grouped(self, step, n_tokens: int) -> bool:
        """Whether this step takes the grouped way: a prompt step (never a step that may be captured and replayed: the
        host waits for the experts' counts) whose experts get enough rows each, and whose experts' products are
        large enough to keep the GPU busy one after the other.  The stacked way does experts / top times the
        arithmetic, at the full rate of one large product; an expert's own product covers `tiles` tiles of 256 x 256
        on 74 pairs of SMs, so it runs at about tiles / (waves x 74) of that rate.  The grouped way is taken where
        that fraction beats top / experts by half again (measured: experts of 512 rows at 2,048 x 1,408 lose to the
        stacked way, 2.3 against 1.7 ms over four layers; at 4,096 x 2,816 they win, 3.9 against 4.9 ms)."""
        if step.all_single or self.top >= self.n_experts:
            return False
        rows = n_tokens * self.top / self.n_experts
        if rows < GROUPED_MIN_ROWS:
            return False
        if GROUPED_MIN_ROWS <= 0:
            return True
        tiles = math.ceil(rows / 256) * math.ceil(2 * self.ff / 256)
        rate = tiles / (math.ceil(tiles / 74) * 74)
        return rate > 1.5 * self.top / self.n_experts

    def forward(self, xin, residual: torch.Tensor, step, store: bool = False) -> None:
        dense, chosen, weights = self.route(xin)
        T = xin.shape[0]
        E = self.n_experts
        if not self.grouped(step, T):
            a = self._first(self.gate_up, xin)
            K.scale_column_blocks(a, dense, self.ff, E)
            if self.w_gate is not None:                   # the shared expert's stretch times the token's gate
                K.scale_column_blocks(a[:, E * self.ff:], dense[:, E:], self.shared_ff, 1)
            self.down(a, out=residual, mode=STORE_F32 if store else ADD_TO_F32)
            return
        counts, order, where = K.moe_group(chosen, self.n_experts)
        counts = counts.tolist()                          # the host waits here, once per layer
        rows = self.runtime.empty(T * self.top, self.hidden)
        K.gather_rows(xin, order, self.top, rows)
        outs = self.runtime.empty(T * self.top, self.hidden, dtype=torch.float32)
        at = 0
        for e, n in enumerate(counts):
            if n:
                a = self._first(self.gate_up_of[e], rows[at:at + n])
                self.down_of[e](a, out=outs[at:at + n], mode=STORE_F32)
                at += n
        if self.shared_ff:
            a = self._first(self.gate_up_of[E], xin)
            if self.w_gate is not None:
                K.scale_column_blocks(a, dense[:, E:], self.shared_ff, 1)
            self.down_of[E](a, out=residual, mode=STORE_F32 if store else ADD_TO_F32)
        K.moe_combine(outs, where, weights, residual, accumulate=bool(self.shared_ff) or not store)
