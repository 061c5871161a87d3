"""Arrangements: how a layer's parts are wired around the residual stream."""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache.store import LayerCache
from .base import Arrangement
from .registry import register_part


@register_part("arrangement", "prenorm_residual")
class PreNormResidual(Arrangement):
    """x += mixer(norm_a(x)); x += feed_forward(norm_b(x)): each norm stands before its part, on the
    residual stream (stratum/native/stratum_arch_llama.inc.c:392-396, :524-532, :555)."""
    replays_prompts = True

    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    optional = ("feed_forward_norm", "feed_forward")       # a layer may be a mixer alone
    carries = True

    def accepts_carry(self, layer):
        return layer.part("mixer_norm") if layer.part("mixer").takes_normed_rows else None

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache, carry=None, hand_to=None):
        """carry: NormedRows of x made for this layer's first norm by the layer before (or None).  hand_to: the
        norm the next layer begins with, if it can begin from NormedRows; they are returned (or None).
        A norm whose rows were handed over runs no kernel: the product in front of it left what it needs."""
        norm_a, mixer = layer.part("mixer_norm"), layer.part("mixer")
        norm_b, ff = layer.part("feed_forward_norm"), layer.part("feed_forward")
        xn = carry if carry is not None else norm_a.forward(x)
        if ff is None or norm_b is None:
            mixer.forward(xn, x, step, cache)
            return None
        ask = norm_b.handover() if mixer.hands_on and ff.takes_normed_rows else None
        if ask is not None:
            mixer.forward(xn, x, step, cache, emit=ask)
        else:
            mixer.forward(xn, x, step, cache)
        xn = ask.result if ask is not None and ask.result is not None else norm_b.forward(x)
        ask = hand_to.handover() if hand_to is not None and ff.hands_on else None
        if ask is not None:
            ff.forward(xn, x, step, emit=ask)
            return ask.result
        ff.forward(xn, x, step)
        return None


@register_part("arrangement", "parallel_residual")
class ParallelResidual(Arrangement):
    """x += mixer(norm_a(x)) + feed_forward(norm_b(x)): both sublayers read the same x, each through a norm of its own,
    and both add into the stream.  Both norms run before either sublayer writes; where they are RMS norms of one size
    and eps (which is what the library's models give) one kernel reads the row once, takes one sum of squares and
    writes both outputs.  A layer may have no feed-forward."""
    replays_prompts = True
    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    optional = ("feed_forward_norm", "feed_forward")

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache) -> None:
        norm_a, mixer = layer.part("mixer_norm"), layer.part("mixer")
        norm_b, ff = layer.part("feed_forward_norm"), layer.part("feed_forward")
        if ff is None or norm_b is None:
            mixer.forward(norm_a.forward(x), x, step, cache)
            return
        pair = getattr(norm_a, "forward_pair", None)
        both = pair(x, norm_b) if pair is not None else None
        xa, xb = both if both is not None else (norm_a.forward(x), norm_b.forward(x))
        mixer.forward(xa, x, step, cache)
        ff.forward(xb, x, step)


class RoundedRows:
    """What an `output_norm_residual` layer asks of the layer in front of it: the rows of the residual stream
    rounded to the compute dtype, which its sublayers read.  (It stands where a layer's first norm stands in the
    carry protocol; it cannot be handed over as a norm can, so a layer of another arrangement in front simply
    makes nothing, and this layer rounds the rows itself.)"""

    def handover(self):
        return None


@register_part("arrangement", "output_norm_residual")
class OutputNormResidual(Arrangement):
    """x += norm_a(mixer(x)); x += norm_b(feed_forward(x)): the sublayers read the residual stream itself (rounded to
    the compute dtype for their matrix products) and each norm stands behind its part, on the part's output, before
    that is added.  The norm's kernel adds into the stream and, on the bfloat16 path, also leaves the rounded rows
    the next sublayer reads, so nothing else passes over the stream between two sublayers."""
    slots = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}
    optional = ("feed_forward", "feed_forward_norm")
    carries = True
    _asks = RoundedRows()

    def accepts_carry(self, layer):
        rt = layer.part("mixer").runtime
        return self._asks if rt is not None and rt.dtype != torch.float32 else None

    @staticmethod
    def _run(part, xin, y, step, cache=None) -> None:
        args = (xin, y, step) if cache is None else (xin, y, step, cache)
        if part.stores_output:
            part.forward(*args, store=True)
        else:
            y.zero_()
            part.forward(*args)

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache, carry=None, hand_to=None):
        mixer, norm_a = layer.part("mixer"), layer.part("mixer_norm")
        ff, norm_b = layer.part("feed_forward"), layer.part("feed_forward_norm")
        rt = mixer.runtime
        rounded = rt.dtype != torch.float32
        if not rounded:
            xin = x
        elif isinstance(carry, torch.Tensor):
            xin = carry
        else:
            xin = rt.empty(*x.shape)
            K.cast_rows(x, xin)
        y = rt.empty(*x.shape, dtype=torch.float32)
        self._run(mixer, xin, y, step, cache)
        last = ff is None or norm_b is None
        want = rounded and (not last or isinstance(hand_to, RoundedRows))
        copy = rt.empty(*x.shape) if want else None
        norm_a.add_normed(y, x, True, copy)
        if last:
            return copy
        self._run(ff, copy if rounded else x, y, step)
        copy = rt.empty(*x.shape) if rounded and isinstance(hand_to, RoundedRows) else None
        norm_b.add_normed(y, x, True, copy)
        return copy


@register_part("arrangement", "sandwich_norm_residual")
class SandwichNormResidual(Arrangement):
    """x += post_a(mixer(pre_a(x))); x += post_b(feed_forward(pre_b(x))): a norm on either side of every sublayer.  A
    constant factor on a sublayer's contribution (a residual multiplier) belongs to the norm behind it (its `scale`).
    The norm behind a sublayer adds into the stream and, where the next thing to read the stream is a norm it can
    make from the row it has just written (the one in front of the next sublayer, also across a layer's border), hands
    that norm's output on, so the stream is passed over once between two sublayers."""
    replays_prompts = True
    slots = {"mixer_norm": "norm", "mixer": "mixer", "mixer_out_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_out_norm": "norm"}
    optional = ("feed_forward_norm", "feed_forward", "feed_forward_out_norm")
    carries = True

    def accepts_carry(self, layer):
        return layer.part("mixer_norm")

    @staticmethod
    def _run(part, xn, y, step, cache=None) -> None:
        args = (xn, y, step) if cache is None else (xn, y, step, cache)
        if part.stores_output:
            part.forward(*args, store=True)
        else:
            y.zero_()
            part.forward(*args)

    @staticmethod
    def _behind(norm, y, x, then):
        """x += norm(y); the output of `then` on the new rows if the norm made it, else None."""
        try:
            return norm.add_normed(y, x, True, then=then) if then is not None else norm.add_normed(y, x, True)
        except TypeError:                  # a norm whose form behind a sublayer knows nothing of the norm after it
            norm.add_normed(y, x, True)
            return None

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache, carry=None, hand_to=None):
        pre_a, mixer, post_a = layer.part("mixer_norm"), layer.part("mixer"), layer.part("mixer_out_norm")
        pre_b, ff, post_b = (layer.part("feed_forward_norm"), layer.part("feed_forward"),
                             layer.part("feed_forward_out_norm"))
        rt = mixer.runtime
        xn = carry if isinstance(carry, torch.Tensor) else pre_a.forward(x)
        y = rt.empty(*x.shape, dtype=torch.float32)
        self._run(mixer, xn, y, step, cache)
        if ff is None or pre_b is None or post_b is None:
            return self._behind(post_a, y, x, hand_to)
        xn = self._behind(post_a, y, x, pre_b)
        if xn is None:
            xn = pre_b.forward(x)
        self._run(ff, xn, y, step)
        return self._behind(post_b, y, x, hand_to)


@register_part("arrangement", "stream_op")
class StreamOpLayer(Arrangement):
    """A stop of the schedule that is no decoder layer: one part (`op`, a stream_op) rewrites the residual stream in
    place (a projection at the head of a pass over looped layers, say).  It keeps nothing per sequence."""
    replays_prompts = True
    slots = {"op": "stream_op"}
    cache_owner = None

    def forward(self, layer, x: torch.Tensor, step, cache: LayerCache) -> None:
        layer.part("op").forward(x, step)
