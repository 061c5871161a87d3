"""Token embedding (a row gather, stratum/native/stratum_arch_llama.inc.c:564-593) and the output
head (logits = W xn with W the head's own matrix if the file has one, else the embedding table,
stratum/native/stratum_arch_llama.inc.c:722-723); and an embedding that adds a row chosen by the token and the one in
front of it."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.store import LayerCache, StateSpec
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


@register_part("embedding", "pair_embedding")
class PairEmbedding(Embedding):
    """x = table[token] * scale + pairs[(previous * mul_prev + token * mul_cur) mod buckets]; a sequence's first token
    reads the last row of `pairs` ([buckets + 1, hidden]).  The token in front of a step's first token is part of what
    a sequence keeps between steps: one int per sequence in a state block of the cache, read and rewritten by the
    kernel that gathers the rows, so that a decode step whose token ids are fed on the device needs nothing from the
    host.  params: vocab, hidden, tensor (the table's name), pairs (the pair table's name; None: no pair table, the
    rows are the token table's times the scale and nothing is kept), buckets, mul_prev, mul_cur, scale."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.name = spec.get("tensor") or self.prefix + "weight"
        self.pairs_name = spec.get("pairs")
        self.buckets, self.mul_prev, self.mul_cur = int(spec["buckets"]), int(spec["mul_prev"]), int(spec["mul_cur"])
        self.scale = float(spec.get("scale", 1.0))
        self._table: Optional[torch.Tensor] = None
        self._pairs: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {self.name: TensorSpec((self.vocab, self.hidden))}
        if self.pairs_name:
            t[self.pairs_name] = TensorSpec((self.buckets + 1, self.hidden))
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self._table = weights[self.name]
        self._pairs = weights[self.pairs_name] if self.pairs_name else None

    def table(self) -> torch.Tensor:
        return self._table

    def cache_spec(self) -> Optional[StateSpec]:
        return StateSpec((1,), "int32") if self.pairs_name else None

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise ValueError("pair_embedding needs the step and its state: forward_step")

    def forward_step(self, step, cache: LayerCache, keep: bool = False) -> torch.Tensor:
        out = self.runtime.empty(step.n_tokens, self.hidden, dtype=torch.float32)
        if keep:
            step.embedded = self.runtime.empty(step.n_tokens, self.hidden, dtype=torch.float32)
        K.embed_pairs(self._table, self._pairs, step.token_ids, step.token_pos, step.token_seq, step.seq_start,
                      step.seq_slot, cache.state, out, step.embedded if keep else None, self.scale, self.mul_prev,
                      self.mul_cur, cache.writes)
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
