"""Re-entry of the embedded tokens into the residual stream at the head of a pass over looped layers: through a
matrix (embedding_reentry), or by plain addition (embedding_readd, at the end of this file).

    x <- W [x ; x0] + b_t

x0 are the embedded tokens of the step (StepBatch.embedded), W is [hidden, 2 hidden] with the stream's columns first,
b_t is row t of a table [passes, hidden], t the number of the pass.  A model that runs some of its layers several
times in a row names this part once per pass, each with its `row`; all passes read the same two tensors.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from .base import StreamOp
from .linear import STORE_F32, Linear
from .registry import register_part
from .spec import TensorSpec


@register_part("stream_op", "embedding_reentry")
class EmbeddingReentry(StreamOp):
    """params: hidden, rows (of the table), row (this pass's), prefix, and the tensor names weight ("in") and table
    ("step")."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.rows, self.row = int(spec["hidden"]), int(spec["rows"]), int(spec["row"])
        if not (0 <= self.row < self.rows):
            raise ValueError(f"embedding_reentry: row {self.row} outside a table of {self.rows}")
        self.w_name = self.prefix + str(spec.get("weight", "in"))
        self.t_name = self.prefix + str(spec.get("table", "step"))
        self.lin: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.w_name: TensorSpec((self.hidden, 2 * self.hidden)),
                self.t_name: TensorSpec((self.rows, self.hidden), role="vector", init="zeros")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.lin = Linear(self.runtime, weights[self.w_name], weights[self.t_name][self.row].contiguous())

    def forward(self, x: torch.Tensor, step) -> None:
        if step.embedded is None:
            raise ValueError("embedding_reentry needs the step's embedded tokens (ModelSpec.keep_embedded)")
        T, H = x.shape
        both = self.runtime.empty(T, 2 * H)              # [x | x0] in the compute dtype: the product's operand
        K.pack_columns(x, both, 0)
        K.pack_columns(step.embedded, both, H)
        self.lin(both, out=x, mode=STORE_F32)


@register_part("stream_op", "embedding_readd")
class EmbeddingReadd(StreamOp):
    """x <- x + x0 + b_t at the head of a pass over looped layers, or x <- x + b_t where the embedded tokens are not
    taken in again (`readd` false: the first pass).  b_t is row t of a table [passes, hidden].  params: hidden, rows
    (of the table), row (this pass's), readd, prefix, table (the tensor's name, default "step")."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.rows, self.row = int(spec["hidden"]), int(spec["rows"]), int(spec["row"])
        if not (0 <= self.row < self.rows):
            raise ValueError(f"embedding_readd: row {self.row} outside a table of {self.rows}")
        self.readd = bool(spec.get("readd", True))
        self.t_name = self.prefix + str(spec.get("table", "step"))
        self.vector: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.t_name: TensorSpec((self.rows, self.hidden), role="vector", init="zeros")}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.vector = weights[self.t_name][self.row].contiguous()

    def forward(self, x: torch.Tensor, step) -> None:
        if self.readd and step.embedded is None:
            raise ValueError("embedding_readd needs the step's embedded tokens (ModelSpec.keep_embedded)")
        K.add_rows(x, step.embedded if self.readd else None, self.vector)
