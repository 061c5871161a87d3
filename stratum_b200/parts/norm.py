"""Norms on the residual stream.
RMSNorm: y = x / sqrt(mean(x^2) + eps) * gain  (stratum/native/stratum_arch_llama.inc.c:45-76).
Dynamic Tanh: y = tanh(alpha x) * w + b, elementwise: it stands where a norm would and takes no row statistic."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from .base import Handover, Norm
from .registry import register_part
from .spec import TensorSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, prefix (e.g. "input_layernorm."; the gain is prefix + "weight") or tensor (the gain's whole
    name), one_plus (the stored weight w is kept around zero and acts as 1 + w), scale (a constant factor on the
    result, folded into the gain in float32 when it is bound: a factor on the logits rides on the last norm)."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.tensor = spec.get("tensor")
        self.one_plus = bool(spec.get("one_plus", False))
        self.scale = float(spec.get("scale", 1.0))
        self.gain: Optional[torch.Tensor] = None

    @property
    def name(self) -> str:
        """The gain's name (a part that owns this norm may move its prefix after it is made)."""
        return self.tensor or self.prefix + "weight"

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), role="vector", init="zeros" if self.one_plus else "ones")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        w = weights[self.name]
        self.gain = (w + 1.0).contiguous() if self.one_plus else w
        if self.scale != 1.0:
            self.gain = (self.gain * self.scale).contiguous()

    def add_normed(self, y: torch.Tensor, residual: torch.Tensor, accumulate: bool = True,
                   copy: Optional[torch.Tensor] = None) -> None:
        K.norm_into_residual(y, self.gain, self.eps, residual, accumulate, copy)

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = self.runtime.empty(n, self.size)
        K.rmsnorm(x, self.gain, self.eps, out, rows)
        return out

    def forward_pair(self, x: torch.Tensor, other: Norm):
        """This norm's and `other`'s output on the same rows from one pass over them, or None where the two are not
        RMS norms of one size and eps (the caller then runs each by itself)."""
        if not isinstance(other, RMSNorm) or other.size != self.size or other.eps != self.eps:
            return None
        out_a, out_b = self.runtime.empty(x.shape[0], self.size), self.runtime.empty(x.shape[0], self.size)
        K.rmsnorm_pair(x, self.gain, other.gain, self.eps, out_a, out_b)
        return out_a, out_b

    def handover(self) -> Optional[Handover]:
        # the matrix products that can honour it are the bfloat16 ones; sums of squares are kept per 128 columns
        if self.runtime is None or self.runtime.dtype != torch.bfloat16 or self.size % 128 != 0:
            return None
        return Handover(self.gain, self.size, self.eps)

    def forward_heads(self, x: torch.Tensor, first_col: int, n_heads: int, head_dim: int) -> None:
        if head_dim != self.size:
            raise ValueError(f"rmsnorm of size {self.size} asked to normalise heads of {head_dim}")
        K.rmsnorm_heads(x, first_col, n_heads, head_dim, self.gain, self.eps)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean x) / sqrt(var x + eps) * w, a weight and no bias (var: the mean of the squared deviations).
    params: size, eps, tensor (the weight's whole name) or prefix (then prefix + "weight"), scale (a constant factor
    on the result, folded into the weight when it is bound: a layer's residual multiplier rides here at no cost)."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.tensor = spec.get("tensor")
        self.scale = float(spec.get("scale", 1.0))
        self.gain: Optional[torch.Tensor] = None

    @property
    def name(self) -> str:
        return self.tensor or self.prefix + "weight"

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), role="vector", init="ones")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        w = weights[self.name]
        self.gain = (w * self.scale).contiguous() if self.scale != 1.0 else w

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = self.runtime.empty(n, self.size)
        K.layernorm(x, self.gain, self.eps, out, rows)
        return out

    def add_normed(self, y: torch.Tensor, residual: torch.Tensor, accumulate: bool = True,
                   copy: Optional[torch.Tensor] = None, then: Optional[Norm] = None) -> Optional[torch.Tensor]:
        """residual (+)= norm(y).  then: the norm that the next sublayer reads the stream through; where that is a
        layer norm of this size, its output (compute dtype) is made by the same kernel, from the row it has just
        written, and returned; otherwise None comes back and that norm runs by itself."""
        if copy is not None:
            raise ValueError("layernorm: the form behind a sublayer leaves no rounded copy of the stream")
        if isinstance(then, LayerNorm) and then.size == self.size:
            out = self.runtime.empty(*residual.shape)
            K.layernorm_into_residual(y, self.gain, self.eps, residual, accumulate, then.gain, then.eps, out)
            return out
        K.layernorm_into_residual(y, self.gain, self.eps, residual, accumulate)
        return None


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """params: size, name (the weight's tensor name; the bias is name + ".b", the scalar name + ".alpha")."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec["size"])
        self.name = str(spec["name"])
        self.w = self.b = self.alpha = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), role="vector", init="ones"),
                self.name + ".b": TensorSpec((self.size,), role="vector", init="zeros"),
                self.name + ".alpha": TensorSpec((), role="vector", init="ones")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.w, self.b = weights[self.name], weights[self.name + ".b"]
        self.alpha = weights[self.name + ".alpha"].reshape(1)

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = self.runtime.empty(n, self.size)
        K.dynamic_tanh(x, self.alpha, self.w, self.b, out, rows)
        return out
