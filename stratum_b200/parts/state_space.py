"""A selective state-space mixer with a scalar decay per head (the state-space duality form): a recurrent mixer that
keeps, per sequence and head, one matrix S [n_state][v_dim] in float32.

Per token, with h the mixer's input:  W h = [z | x | B | C | dt]  (inner = heads * v_dim, inner, groups * n_state,
groups * n_state, heads).  x, B and C together pass a short causal convolution over time per channel (taps per channel
and a bias, the last tap the current token's, zeros before the sequence's start) and silu.  dt = softplus(dt +
dt_bias), not clamped.  Head j (its B and C are those of group j / (heads / groups)):

    S <- exp(-exp(A_log_j) dt) S + dt B x^T;      y = S^T C + D_j x

    y <- y silu(z);   the row is cut into `norm_groups` equal parts, each divided by its own root mean square (eps
    inside the root);   times the gain;   result = Wo y.      The gate comes before the norm.

What a sequence keeps between steps is S and the last taps - 1 inputs of the convolution: a block of fixed size per
sequence (cache.StateSpec), whatever its length.  The input projection runs with float32 sums; everything between it
and the output product is float32 (csrc/ssm_scan.cu).
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


@register_part("mixer", "selective_state_space")
class SelectiveStateSpace(Mixer):
    """params: hidden, n_heads, v_dim, n_state, n_groups, taps, norm_groups, eps (of the output norm), prefix, and the
    tensor names in, conv, conv_bias, dt_bias, A_log, D, norm, o (defaults: those words, with "conv.b")."""
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads, self.dv = int(spec["hidden"]), int(spec["n_heads"]), int(spec["v_dim"])
        self.n_state, self.n_groups = int(spec["n_state"]), int(spec["n_groups"])
        self.taps, self.norm_groups = int(spec["taps"]), int(spec.get("norm_groups", 1) or 1)
        self.eps = float(spec["eps"])
        if self.n_heads % self.n_groups:
            raise ValueError(f"state-space mixer: {self.n_heads} heads do not form {self.n_groups} equal groups")
        self.inner = self.n_heads * self.dv
        if self.inner % self.norm_groups:
            raise ValueError(f"state-space mixer: {self.inner} outputs do not form {self.norm_groups} equal parts")
        self.channels = self.inner + 2 * self.n_groups * self.n_state
        self.width = self.inner + self.channels + self.n_heads            # columns of the input projection
        keys = ("in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o")
        self.names = {k: self.prefix + str(spec.get(k + "_tensor", "conv.b" if k == "conv_bias" else k)) for k in keys}
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n, H = self.names, self.hidden
        return {n["in"]: TensorSpec((self.width, H)), n["o"]: TensorSpec((H, self.inner)),
                n["conv"]: TensorSpec((self.channels, self.taps), role="vector"),
                n["conv_bias"]: TensorSpec((self.channels,), role="vector", init="zeros"),
                n["dt_bias"]: TensorSpec((self.n_heads,), role="vector", init="zeros"),
                n["A_log"]: TensorSpec((self.n_heads,), role="vector", init="zeros"),
                n["D"]: TensorSpec((self.n_heads,), role="vector", init="ones"),
                n["norm"]: TensorSpec((self.inner,), role="vector", init="ones")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = Linear(self.runtime, weights[n["in"]])
        self.w_o = Linear(self.runtime, weights[n["o"]])
        self.conv_w, self.conv_b = weights[n["conv"]].contiguous(), weights[n["conv_bias"]].contiguous()
        self.a_log, self.dt_bias = weights[n["A_log"]].contiguous(), weights[n["dt_bias"]].contiguous()
        self.d_skip, self.gain = weights[n["D"]].contiguous(), weights[n["norm"]].contiguous()

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.inner * self.n_state + (self.taps - 1) * self.channels,), "float32")

    def forward(self, xin, residual: torch.Tensor, step, cache: LayerCache, store: bool = False) -> None:
        T = xin.shape[0]
        f32 = torch.float32
        proj = self.runtime.empty(T, padded(self.width), dtype=f32)
        self.w_in(xin, out=proj[:, :self.width], mode=STORE_F32)
        act = self.runtime.empty(T, padded(self.channels + 2 * self.n_heads), dtype=f32)
        y_raw = self.runtime.empty(T, self.inner, dtype=f32)
        out = self.runtime.empty(T, padded(self.inner))
        K.ssm_scan(proj, self.conv_w, self.conv_b, self.a_log, self.dt_bias, self.d_skip, self.gain, act, y_raw, out,
                   cache.state, step.token_pos, step.token_seq, step.seq_start, step.seq_slot, self.n_heads, self.dv,
                   self.n_state, self.n_groups, self.norm_groups, self.eps, cache.writes)
        self.w_o(out[:, :self.inner], out=residual, mode=STORE_F32 if store else ADD_TO_F32)
