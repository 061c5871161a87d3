"""Gated linear attention: a recurrent mixer that keeps, per sequence and head, one matrix S [d][dv] in float32.

Per token, with h the mixer's input:  q = Wq h / sqrt(d), k = Wk h ([heads][d]), v = Wv h ([heads][dv]), and a decay
per key channel, alpha = sigmoid(Wa2 (Wa1 h) + b)^(1/tau) ([heads][d]; Wa1 maps to a few inner dimensions).  Head j:

    S <- diag(alpha) S + k v^T;   o = S^T q                          (o sees the token's own write)

    o <- o / sqrt(mean(o^2) + eps) * gain * silu(Wg h)_j;      result = Wo concat_j(o)

What a sequence keeps between steps is S: a block of fixed size per sequence (cache.StateSpec), whatever its length.
The five projections that read h run as one product with float32 sums; the decay's inner values go, rounded to the
compute dtype, through its second projection (a matrix product with float32 sums); everything from there to the
output product is float32 (csrc/gla.cu).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.store import LayerCache, StateSpec
from .base import Mixer
from .latent_attention import padded
from .linear import ADD_TO_F32, STORE_F32, Linear
from .registry import register_part
from .spec import TensorSpec


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    """params: hidden, n_heads, head_dim, v_dim, rank (inner size of the decay's projections), tau, eps (of the output
    norm), q_scale (default head_dim^-1/2), prefix, and the tensor names q, k, v, g, o, norm, a1, a2 (defaults: those
    words; the decay's bias is a2's name + ".b")."""
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads = int(spec["hidden"]), int(spec["n_heads"])
        self.d, self.dv, self.rank = int(spec["head_dim"]), int(spec["v_dim"]), int(spec["rank"])
        self.tau, self.eps = float(spec["tau"]), float(spec["eps"])
        if not self.tau > 0:
            raise ValueError("gated linear attention: tau must be positive")
        self.q_scale = float(spec.get("q_scale") or self.d ** -0.5)
        keys = ("q", "k", "v", "g", "o", "norm", "a1", "a2")
        self.names = {k: self.prefix + str(spec.get(k + "_tensor", k)) for k in keys}
        self.qk_cols, self.v_cols = self.n_heads * self.d, self.n_heads * self.dv
        self.width = 2 * self.qk_cols + 2 * self.v_cols + self.rank          # columns of the fused projection
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n, H = self.names, self.hidden
        return {n["q"]: TensorSpec((self.qk_cols, H)), n["k"]: TensorSpec((self.qk_cols, H)),
                n["v"]: TensorSpec((self.v_cols, H)), n["g"]: TensorSpec((self.v_cols, H)),
                n["a1"]: TensorSpec((self.rank, H)), n["a2"]: TensorSpec((self.qk_cols, self.rank)),
                n["a2"] + ".b": TensorSpec((self.qk_cols,), role="vector", init="zeros"),
                n["o"]: TensorSpec((H, self.v_cols)),
                n["norm"]: TensorSpec((self.dv,), role="vector", init="ones")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        stack = [weights[n[k]] for k in ("q", "k", "v", "g", "a1")]
        self.w_in = Linear(self.runtime, torch.cat(stack, dim=0).contiguous())
        self.w_o = Linear(self.runtime, weights[n["o"]])
        self.w_a2 = Linear(self.runtime, weights[n["a2"]].contiguous(), weights[n["a2"] + ".b"].contiguous())
        self.gain = weights[n["norm"]].contiguous()

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.n_heads * self.d * self.dv,), "float32")

    def forward(self, xin, residual: torch.Tensor, step, cache: LayerCache, store: bool = False) -> None:
        T = xin.shape[0]
        f32 = torch.float32
        proj = self.runtime.empty(T, padded(self.width), dtype=f32)
        self.w_in(xin, out=proj[:, :self.width], mode=STORE_F32)
        step_ = K.GlaStep(proj, self.n_heads, self.d, self.dv, self.rank, self.tau, self.q_scale, self.eps)
        inner = self.runtime.empty(T, padded(self.rank))
        step_.cast(inner)
        alpha = self.runtime.empty(T, self.qk_cols, dtype=f32)
        self.w_a2(inner[:, :self.rank], out=alpha, mode=STORE_F32)
        step_.decay(alpha)
        o_raw = self.runtime.empty(T, self.v_cols, dtype=f32)
        step_.recur(o_raw, cache.state, step.token_seq, step.seq_start, step.seq_slot, cache.writes)
        out = self.runtime.empty(T, padded(self.v_cols))
        step_.finish(self.gain, out)
        self.w_o(out[:, :self.v_cols], out=residual, mode=STORE_F32 if store else ADD_TO_F32)
