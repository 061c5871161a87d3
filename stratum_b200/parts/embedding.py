"""Token embedding (a row gather, stratum/native/stratum_arch_llama.inc.c:564-593) and the output
head (logits = W xn with W the head's own matrix if the file has one, else the embedding table,
stratum/native/stratum_arch_llama.inc.c:722-723)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from .base import Embedding, Head
from .linear import STORE_F32, Linear
from .registry import find_part, register_part
from .spec import TensorSpec


@register_part("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab, hidden, prefix (e.g. "model.embed_tokens."; the table is prefix + "weight"), or tensor (the
    table's whole name); norm (PartSpec of a norm the gathered rows pass, in float32 and in place, or None)."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.name = spec.get("tensor") or self.prefix + "weight"
        self._table: Optional[torch.Tensor] = None
        ns = spec.get("norm")
        self.norm = find_part("norm", ns.kind)(ns, runtime) if ns is not None else None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {self.name: TensorSpec((self.vocab, self.hidden))}
        if self.norm is not None:
            t.update(self.norm.tensors())
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self._table = weights[self.name]
        if self.norm is not None:
            self.norm.bind(weights)

    def table(self) -> torch.Tensor:
        return self._table

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = self.runtime.empty(token_ids.numel(), self.hidden, dtype=torch.float32)
        K.embed_gather(self._table, token_ids, out)
        if self.norm is not None:
            self.norm.add_normed(out, out, accumulate=False)
        return out


@register_part("head", "linear_head")
class LinearHead(Head):
    """params: vocab, hidden, tied (the file may leave the matrix out: the embedding table then serves), prefix (e.g.
    "lm_head."; the matrix is prefix + "weight"), or tensor (the matrix's whole name); own_matrix (default true;
    false: the head has no tensor of its own and is always the embedding table)."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.tied = bool(spec.get("tied", False))
        self.name = spec.get("tensor") or self.prefix + "weight"
        self.own_matrix = bool(spec.get("own_matrix", True))
        self.proj: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        if not self.own_matrix:
            return {}
        return {self.name: TensorSpec((self.vocab, self.hidden), optional=self.tied)}

    def bind_with_embedding(self, weights: Mapping[str, torch.Tensor], table: torch.Tensor) -> None:
        w = weights.get(self.name) if self.own_matrix else None
        self.proj = Linear(self.runtime, w if w is not None else table)

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        return self.proj(xn, mode=STORE_F32)
