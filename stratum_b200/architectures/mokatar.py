"""The Mokatar decoder as data: MokatarConfig -> ModelSpec.

The embedded tokens are a row of the token table times a constant plus a row of a second table chosen by the token and
the one in front of it.  Every layer adds both of its sublayers, read from the same stream through a norm each:
x += mixer(norm1(x)) + ff(norm2(x)) (a layer may have no feed-forward); the norms are RMS norms whose stored weight w
acts as 1 + w.  The mixer is attention over a sliding window that keeps the sequence's first tokens, with per-head
normalised queries and keys and a learned sink; causal attention with biases, queries and keys normalised over the
whole projection and a sink of score zero; or gated linear attention with state of a fixed size, layer by layer as the
configuration lists them.  The feed-forward is dense and gated (silu) or a mixture of such experts chosen by router
logit and weighted by the softmax over the chosen logits.  A stretch of layers may run several times in a row with the
same weights: every pass is a run of stops of its own in the schedule (shared weights, own caches), headed by a stop
that adds the pass's vector and, from the second pass on, the embedded tokens again.  The logits are the head's
products times a constant, which rides on the last norm's gain.  Tensor names: embed, bigram, loop.step,
l<i>.norm1 / norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.mokatar import MokatarConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _rotation(rot, neighbours: bool) -> PartSpec:
    scaling = None
    if rot.ramp:
        scaling = {"kind": "yarn", "factor": rot.factor, "original_max_position": rot.original,
                   "beta_fast": rot.fast, "beta_slow": rot.slow}
    elif rot.factor is not None:
        scaling = {"kind": "linear", "factor": rot.factor}
    return PartSpec("rope", {"rope_dim": rot.dims, "theta": rot.base, "interleaved": neighbours, "scaling": scaling,
                             "precise": True})


def _mixer(cfg: MokatarConfig, index: int, layer) -> PartSpec:
    m = layer.mixer
    if layer.kind == "gla":
        if m.rank is None:
            raise ValueError(f"layer {index}: the inner size of the decay's projections is the number of rows of "
                             f"l{index}.mix.a1; without the tensors the mixer needs 'rank'")
        return PartSpec("gated_linear_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "v_dim": m.vdim, "rank": m.rank, "tau": m.tau,
            "eps": cfg.eps, "prefix": "mix."})
    first = layer.kind == "attention"
    return PartSpec("sink_attention", {
        "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
        "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "eps": cfg.eps,
        "position": _rotation(m.rot, neighbours=first) if m.rot is not None and m.rot.dims else None,
        "qk_norm": "per_head" if first else "whole", "bias": not first, "sink": True if first else "zero",
        "prefix": "mix."})


def _feed_forward(cfg: MokatarConfig, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("swiglu", {"hidden": cfg.width, "intermediate": f.ff, "gate": "gate", "up": "up",
                                   "down": "down", "prefix": "mlp."})
    return PartSpec("routed_experts", {
        "hidden": cfg.width, "n_experts": f.experts, "top": f.top, "scale": 1.0, "n_groups": 1, "keep": 1,
        "intermediate": f.ff, "shared_intermediate": None, "score": "softmax", "renorm": True, "correction": False,
        "router_bias": True, "prefix": "mlp."})


def describe_mokatar(cfg: MokatarConfig) -> ModelSpec:
    def norm(name, scale=1.0):
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "tensor": name, "one_plus": True,
                                    "scale": scale})

    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer_norm": norm("norm1"), "mixer": _mixer(cfg, i, layer)}
        if layer.mlp is not None:
            parts.update({"feed_forward_norm": norm("norm2"), "feed_forward": _feed_forward(cfg, layer.mlp)})
        layers.append(LayerSpec("parallel_residual", parts, f"l{i}."))
    schedule = []
    for i, t, first in cfg.runs():
        if first:                      # the head of pass t: one more "layer" whose only part acts on the stream
            schedule.append(ScheduleEntry(len(layers)))
            layers.append(LayerSpec("stream_op", {"op": PartSpec("embedding_readd", {
                "hidden": cfg.width, "rows": cfg.loop.times, "row": t, "readd": t > 0, "prefix": "loop."})}, ""))
        schedule.append(ScheduleEntry(i))
    b = cfg.bigram
    embedding = PartSpec("pair_embedding", {
        "vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed", "pairs": "bigram" if b is not None else None,
        "buckets": b.buckets if b else 0, "mul_prev": b.mul_prev if b else 0, "mul_cur": b.mul_cur if b else 0,
        "scale": cfg.embedding_scale})
    return ModelSpec(
        hidden=cfg.width, vocab=cfg.vocab, embedding=embedding, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("final.norm", cfg.logit_scale),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width, "tied": False, "tensor": "head"}),
        keep_embedded=cfg.loop is not None and cfg.loop.times > 1)


MOKATAR = register_architecture(Architecture(
    names=("Mokatar",),
    description="Mokatar decoder: token-pair embedding, parallel sublayers, windowed attention that keeps the first "
                "tokens with a sink, biased attention with a zero sink, gated linear attention, routed experts, "
                "looped layers",
    config_class=MokatarConfig,
    describe_model=describe_mokatar,
    # a layer without a feed-forward has no use for a second norm; a file that carries one all the same is accepted
    ignored_tensor_suffixes=(".norm2",),
    sizes_from_tensors=lambda cfg, shapes: cfg.with_decay_ranks(shapes)), replace=True)
