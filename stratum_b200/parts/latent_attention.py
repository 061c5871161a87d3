"""Latent attention: keys and values of all heads are expansions of one small vector per token, and only that
vector (with one rotated key part shared by the heads) is kept in the cache.

Per token, with h the mixer's input:  q = Wq h, per head [d plain | r rotated];  Wdkv h = [c' | kr];
c = c' / sqrt(mean(c'^2) + eps) * g;  kr and the rotated part of every query head are rotated by the position.
Head j's key is Wuk_j c and its value Wuv_j c, so its score against token t is

    (q_plain_j . Wuk_j c_t + q_rot_j . kr_t) * scale  =  ((Wuk_j^T q_plain_j) . c_t + q_rot_j . kr_t) * scale

and its output Wuv_j (sum_t a_t c_t).  The right-hand forms are what runs: the query is carried into the latent
space once per token ([Wuk_j^T q_plain_j | q_rot_j], rank + r numbers), every head attends over the same cached
rows [c_t | kr_t], whose first `rank` numbers are also the values, and the head's mixed latent is expanded by
Wuv_j afterwards.  Neither keys nor values of the heads are ever formed for cached tokens, which is the point of
the design: a step reads rank + r numbers per cached token, whatever the number of heads.

A prompt that begins at position 0 has no cached tokens to spare: all its keys are this step's own.  There the
left-hand form costs a quarter of the arithmetic (heads of d + r and dv numbers against rank + r and rank), and on
the bfloat16 path, where attention over a long prompt is bound by the tensor cores, it is what runs: the heads' keys
[Wuk_j c | kr] come from one product of the step's rows [c | kr] with the matrix that stacks [Wuk_j 0; 0 I] per
head, the values from Wuv c, and the general attention reads them as plain matrices.  The cache is written all
the same, for the steps that follow.

Two optional pieces, each a parameter.  Queries through a latent of their own (`q_rank`): cq = Wdq h / rms * gq,
q = Wuq cq; the down projection joins the fused first product, the norm runs in place on its stretch of the row
(float32 statistic), and the up projection writes the queries where the direct projection would have.  A gate per
head (`gate`): head j's output times sigmoid(Wg h)_j, whose pre-activation is one more column stretch of the first
product; the sigmoid is taken in float32 on the heads' outputs, in front of the output projection.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import os

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS
from ..cache.store import KVSpec, LayerCache
from .base import Mixer
from .linear import ADD_TO_F32, STORE, STORE_F32, HeadLinear, Linear
from .registry import find_part, register_part
from .spec import PartSpec, TensorSpec


# prompts from this many tokens on take the per-head form on the bfloat16 path (below it the absorbed form's
# arithmetic is not what a step waits for; STRATUM_LATENT_PER_HEAD=0 turns the form off: measurements)
PER_HEAD_MIN_TOKENS = int(os.environ.get("STRATUM_LATENT_PER_HEAD_MIN", 256))


def padded(n: int, to: int = 8) -> int:
    return (n + to - 1) // to * to


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """params: hidden, n_heads, head_dim (the unrotated query/key size), rot_dim, v_dim, kv_rank, scale, eps (of
    the latents' norms), position (PartSpec of a rotating position encoding over at most rot_dim dimensions, pairs
    (i, i + n/2) or neighbours (2i, 2i + 1) as the encoding says), window (0 = all keys), q_rank (None or 0: queries
    projected directly from the input; else the size of the queries' latent), gate (a sigmoid gate per head on the
    heads' outputs), prefix, and the tensor names q, dkv, dkv_norm, uk, uv, o, and with q_rank dq, dq_norm, uq, with
    gate g (defaults: those words, with "dkv.norm" and "dq.norm")."""
    stores_output = True

    @property
    def replays_prompts(self) -> bool:
        return bool(getattr(self.position, "replays_prompts", False))

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads = int(spec["hidden"]), int(spec["n_heads"])
        self.d, self.r, self.dv, self.rank = (int(spec["head_dim"]), int(spec["rot_dim"]), int(spec["v_dim"]),
                                              int(spec["kv_rank"]))
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = int(spec.get("window", 0) or 0)
        pos: PartSpec = spec["position"]
        self.position = find_part("position", pos.kind)(pos, runtime)
        layout = self.position.pair_layout()
        if layout is None or 2 * layout[0] > self.r:
            raise ValueError("latent attention rotates pairs of at most rot_dim dimensions")
        self.interleaved = bool(layout[1])
        self.q_rank = int(spec.get("q_rank") or 0)
        self.gate = bool(spec.get("gate", False))
        self.names = {k: self.prefix + str(spec.get(k, k.replace("_norm", ".norm")))
                      for k in ("q", "dkv", "dkv_norm", "uk", "uv", "o", "dq", "dq_norm", "uq", "g")}
        # columns of a token's row of projections: [queries | c' kr | the queries' latent | the gates], every
        # stretch starting at a multiple of 8 (16 bytes in bfloat16: rows a product may read or write by vectors)
        self.q_cols = self.n_heads * (self.d + self.r)
        self.kv_col = padded(self.q_cols) if self.q_rank else self.q_cols
        self.cq_col = self.kv_col + padded(self.rank + self.r)
        self.g_col = self.cq_col + padded(self.q_rank)
        self.width = (self.g_col + self.n_heads if self.gate else
                      self.cq_col + self.q_rank if self.q_rank else self.kv_col + self.rank + self.r)
        self.shape = K.AttentionShape(self.n_heads, self.n_heads, 1, self.rank + self.r, self.rank, True, self.scale,
                                      window=self.window)
        self.w_in: Optional[Linear] = None
        self.w_uq: Optional[Linear] = None
        self.w_o: Optional[Linear] = None
        self.uk: Optional[HeadLinear] = None
        self.uv: Optional[HeadLinear] = None
        self.gain: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n, H = self.names, self.n_heads
        t = {n["dkv"]: TensorSpec((self.rank + self.r, self.hidden)),
             n["dkv_norm"]: TensorSpec((self.rank,), role="vector", init="ones"),
             n["uk"]: TensorSpec((H * self.d, self.rank)),
             n["uv"]: TensorSpec((H * self.dv, self.rank)),
             n["o"]: TensorSpec((self.hidden, H * self.dv))}
        if self.q_rank:
            t.update({n["dq"]: TensorSpec((self.q_rank, self.hidden)),
                      n["dq_norm"]: TensorSpec((self.q_rank,), role="vector", init="ones"),
                      n["uq"]: TensorSpec((self.q_cols, self.q_rank))})
        else:
            t[n["q"]] = TensorSpec((self.q_cols, self.hidden))
        if self.gate:
            t[n["g"]] = TensorSpec((H, self.hidden))
        return t

    def _stack_rows(self, pieces) -> torch.Tensor:
        """The matrices of `pieces` ((first row, matrix) pairs) one above the other, each from its row on, zero rows
        between them: the weight of one product whose output stretches start where the row layout says."""
        first = min(at for at, _ in pieces)
        last = max(at + w.shape[0] for at, w in pieces)
        ref = pieces[0][1]
        out = torch.zeros((last - first, self.hidden), dtype=ref.dtype, device=ref.device)
        for at, w in pieces:
            out[at - first:at - first + w.shape[0]] = w
        return out

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n, H = self.names, self.n_heads
        pieces = [(self.kv_col, weights[n["dkv"]])]
        if self.q_rank:
            pieces.append((self.cq_col, weights[n["dq"]]))
            self.w_uq = Linear(self.runtime, weights[n["uq"]])
            self.gain_q = weights[n["dq_norm"]].contiguous()
        else:
            pieces.append((0, weights[n["q"]]))
        if self.gate:
            pieces.append((self.g_col, weights[n["g"]]))
        self.w_in = Linear(self.runtime, self._stack_rows(pieces))
        self.gain = weights[n["dkv_norm"]]
        # head j carries its plain query into the latent space with Wuk_j^T: a matrix [rank, d] per head
        self.uk = HeadLinear(self.runtime, weights[n["uk"]].view(H, self.d, self.rank).transpose(1, 2).contiguous())
        self.uv = HeadLinear(self.runtime, weights[n["uv"]].view(H, self.dv, self.rank))
        self.w_o = Linear(self.runtime, weights[n["o"]])
        # the per-head form of whole prompts (bfloat16): keys of all heads from the rows [c | kr] in one product
        self.w_keys = self.w_values = None
        if self.runtime.dtype == torch.bfloat16 and (self.d + self.r) % 8 == 0 and self.dv % 8 == 0:
            d, r, rank = self.d, self.r, self.rank
            stack = torch.zeros((H, d + r, rank + r), dtype=torch.bfloat16, device=weights[n["uk"]].device)
            stack[:, :d, :rank] = weights[n["uk"]].view(H, d, rank)
            stack[:, d:, rank:] = torch.eye(r, dtype=torch.bfloat16, device=stack.device)
            self.w_keys = Linear(self.runtime, stack.view(H * (d + r), rank + r))
            self.w_values = Linear(self.runtime, weights[n["uv"]])
            self.head_shape = K.AttentionShape(H, 1, 1, d + r, self.dv, False, self.scale, window=self.window)

    def cache_spec(self) -> KVSpec:
        return KVSpec(1, self.rank + self.r, self.window, f"latent_{self.rank}_then_rotated", value_heads=0)

    def _per_head_form(self, step, cache: LayerCache) -> bool:
        """Whether this step forms the heads' keys and values instead of carrying queries into the latent space:
        bfloat16, a prompt step launched launch by launch (a replayed step's shape says nothing about where its
        sequences begin) in which every sequence begins at position 0 and the longest brings PER_HEAD_MIN_TOKENS."""
        if self.w_keys is None or step.all_single or step.fixed_qblocks is not None or step.sizes_seen is not None:
            return False
        if not cache.writes or self.window or os.environ.get("STRATUM_LATENT_PER_HEAD", "1") == "0":
            return False
        before = (step.host or {}).get("before")
        return bool(before) and all(b == 0 for b in before) and step.max_new >= PER_HEAD_MIN_TOKENS

    def _finish(self, heads: torch.Tensor, proj: torch.Tensor, residual: torch.Tensor, store: bool) -> None:
        """The heads' outputs times their gates (where the mixer has them), then the output projection."""
        H, dv = self.n_heads, self.dv
        if self.gate:
            K.gate_heads(heads, proj[:, self.g_col:self.g_col + H], H, dv)
        self.w_o(heads[:, :H * dv], out=residual, mode=STORE_F32 if store else ADD_TO_F32)

    def _forward_per_head(self, proj, step, cache: LayerCache, residual: torch.Tensor, store: bool) -> None:
        H, d, r, rank, dv = self.n_heads, self.d, self.r, self.rank, self.dv
        T = proj.shape[0]
        rows = self.runtime.empty(T, padded(rank + r))            # [c | kr] of the step's tokens
        K.mixer_prep(proj, step.token_pos, step.token_seq, cache.block_table, cache.k, None, PAGE_TOKENS, True,
                     queries=(H, d + r, 0), q_rot_off=d, keys=(1, rank + r, self.kv_col), k_rot_off=rank,
                     inv_freq=self.position.rotary().inv_freq, k_norm_gain=self.gain, eps=self.eps, k_out=rows,
                     interleaved=self.interleaved)
        # 64 rows beyond the step's: the last tile of the last sequence reads (and ignores) them
        keys = self.runtime.empty(T + PAGE_TOKENS, padded(H * (d + r)))
        values = self.runtime.empty(T + PAGE_TOKENS, padded(H * dv))
        keys[T:].zero_()
        values[T:].zero_()
        self.w_keys(rows[:, :rank + r], out=keys[:T, :H * (d + r)], mode=STORE)
        self.w_values(rows[:, :rank], out=values[:T, :H * dv], mode=STORE)
        heads = self.runtime.empty(T, padded(H * dv))
        from . import attention_dispatch
        attention_dispatch.run_general_dense(self, self.head_shape, proj, keys, values, step, heads)
        self._finish(heads, proj, residual, store)

    def forward(self, xn, residual: torch.Tensor, step, cache: LayerCache, emit=None, store: bool = False) -> None:
        H, d, r, rank, dv = self.n_heads, self.d, self.r, self.rank, self.dv
        T = xn.shape[0]
        proj = self.runtime.empty(T, padded(self.width))
        if self.q_rank:
            # [c' kr | cq' | gates] in one product; the queries' latent is normed in place and expanded into the
            # queries' columns
            self.w_in(xn, out=proj[:, self.kv_col:self.width], mode=STORE)
            K.rmsnorm_heads(proj, self.cq_col, 1, self.q_rank, self.gain_q, self.eps)
            self.w_uq(proj[:, self.cq_col:self.cq_col + self.q_rank], out=proj[:, :self.q_cols], mode=STORE)
        else:
            self.w_in(xn, out=proj[:, :self.width], mode=STORE)
        if self._per_head_form(step, cache) and K.attention_general_mma_ok(self.head_shape, proj, proj, PAGE_TOKENS):
            self._forward_per_head(proj, step, cache, residual, store)
            return
        q_lat = self.runtime.empty(T, padded(H * (rank + r)))
        K.mixer_prep(proj, step.token_pos, step.token_seq, cache.block_table, cache.k, None, PAGE_TOKENS, cache.writes,
                     queries=(H, d + r, 0), q_rot_off=d, keys=(1, rank + r, self.kv_col), k_rot_off=rank,
                     inv_freq=self.position.rotary().inv_freq, k_norm_gain=self.gain, eps=self.eps,
                     q_out=q_lat, q_out_step=rank + r, q_out_off=rank, interleaved=self.interleaved)
        self.uk(proj, d + r, q_lat, rank + r)
        mixed = self.runtime.empty(T, padded(H * rank))
        from . import attention_dispatch
        attention_dispatch.run_general(self, self.shape, q_lat, cache, step, mixed)
        heads = self.runtime.empty(T, padded(H * dv))
        self.uv(mixed, rank, heads, dv)
        self._finish(heads, proj, residual, store)
