"""Feed-forwards.
Dense with a GELU: residual += Wd gelu(Wu xn), the exact (erf) GELU or its tanh form, applied to the
float32 sums of the first product before they are rounded and stored.
SwiGLU feed-forward: residual += Wd (silu(Wg xn) * (Wu xn))
(stratum/native/stratum_arch_llama.inc.c:550-555, stratum/native/stratum_engine.h:373-391).

Gate and up run as one matrix product over a weight whose rows alternate gate_j, up_j, so that
an output row holds (g_0, u_0, g_1, u_1, ...) and the activation reads neighbours.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .base import FeedForward
from .. import kernels as K
from .linear import ADD_TO_F32, STORE, STORE_F32, SWIGLU, Linear
from .registry import register_part
from .spec import TensorSpec


def interleave_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Rows a_0, b_0, a_1, b_1, ..."""
    return torch.stack([a, b], dim=1).reshape((a.shape[0] * 2,) + tuple(a.shape[1:])).contiguous()


GATE_ACTS = {"silu": K.ACT_NONE, "gelu_erf": K.ACT_GELU_ERF, "gelu_tanh": K.ACT_GELU_TANH, "relu_sq": K.ACT_RELU_SQ}


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """A gated feed-forward: Wd (act(Wg xn) * (Wu xn)), act = silu unless `activation` names another ("gelu_tanh",
    "gelu_erf", "relu_sq").  params: hidden, intermediate, bias, prefix, activation, and the tensors' names gate, up,
    down (defaults "gate_proj.weight" ... with biases "gate_proj.bias" ...; a name given in full has its bias at
    name + ".b")."""
    replays_prompts = True
    takes_normed_rows = True
    hands_on = True
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden"])
        self.intermediate = int(spec["intermediate"])
        self.bias = bool(spec.get("bias", False))
        act = spec.get("activation", "silu")
        if act not in GATE_ACTS:
            raise ValueError(f"gated feed-forward: activation {act!r} is not one of {sorted(GATE_ACTS)}")
        self.act = GATE_ACTS[act]
        self.w_names, self.b_names = {}, {}
        for key in ("gate", "up", "down"):
            given = spec.get(key)
            self.w_names[key] = self.prefix + (given if given else f"{key}_proj.weight")
            self.b_names[key] = self.prefix + (given + ".b" if given else f"{key}_proj.bias")
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        H, F = self.hidden, self.intermediate
        w, b = self.w_names, self.b_names
        t = {w["gate"]: TensorSpec((F, H)), w["up"]: TensorSpec((F, H)), w["down"]: TensorSpec((H, F))}
        if self.bias:
            t.update({b["gate"]: TensorSpec((F,), role="vector"), b["up"]: TensorSpec((F,), role="vector"),
                      b["down"]: TensorSpec((H,), role="vector")})
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        wn, bn = self.w_names, self.b_names
        w = interleave_rows(weights[wn["gate"]], weights[wn["up"]])
        b = interleave_rows(weights[bn["gate"]], weights[bn["up"]]) if self.bias else None
        self.gate_up = Linear(self.runtime, w, b)
        self.down = Linear(self.runtime, weights[wn["down"]], weights.get(bn["down"]) if self.bias else None)

    def forward(self, xn, residual: torch.Tensor, step, emit=None, store: bool = False) -> None:
        a = self.gate_up(xn, mode=SWIGLU, act=self.act)
        self.down(a, out=residual, mode=STORE_F32 if store else ADD_TO_F32, emit=None if store else emit)


@register_part("feed_forward", "dense_gelu")
class DenseGelu(FeedForward):
    """params: hidden, intermediate, activation ("gelu_erf" | "gelu_tanh"), up / down (tensor names), prefix."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden"])
        self.intermediate = int(spec["intermediate"])
        act = spec.get("activation", "gelu_erf")
        if act not in ("gelu_erf", "gelu_tanh"):
            raise ValueError(f"dense_gelu: activation {act!r} is neither gelu_erf nor gelu_tanh")
        self.act = K.ACT_GELU_ERF if act == "gelu_erf" else K.ACT_GELU_TANH
        self.up_name = self.prefix + spec.get("up", "up")
        self.down_name = self.prefix + spec.get("down", "down")
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.up_name: TensorSpec((self.intermediate, self.hidden)),
                self.down_name: TensorSpec((self.hidden, self.intermediate))}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.up = Linear(self.runtime, weights[self.up_name])
        self.down = Linear(self.runtime, weights[self.down_name])

    def forward(self, xn, residual: torch.Tensor, step) -> None:
        a = self.up(xn, mode=STORE, act=self.act)          # the activation rides on the product's epilogue
        self.down(a, out=residual, mode=ADD_TO_F32)
