"""The Vitinex decoder as data: VitinexConfig -> ModelSpec.

Every layer has a norm on either side of each sublayer, x += m LN1b(mixer(LN1(x))); x += m LN2b(ff(LN2(x))) (a layer
may have no feed-forward): layer norms with a weight and no bias, m the configuration's residual factor (it rides on
the weights of the norms behind the sublayers).  The mixer is latent attention with a latent for the queries too and
a sigmoid gate per head, or a selective state-space mixer with state of a fixed size, layer by layer as the
configuration lists them; the feed-forward is dense and gated (tanh GELU, biases) or a mixture of squared-ReLU
experts chosen by softmax scores, with a gated shared expert.  A stretch of layers may run several times in a row
with the same weights: every pass is a run of stops of its own in the schedule (shared weights, own caches), headed
by a stop that re-enters the embedded tokens, x <- W [x ; x0] + step[pass].  The head is the embedding table.
Tensor names: embed, loop.in, loop.step, l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.*, l<i>.mlp.*, final.norm.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.vitinex import VitinexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(cfg: VitinexConfig, layer) -> PartSpec:
    m = layer.mixer
    if layer.kind == "latent_attention":
        rope = PartSpec("rope", {"rope_dim": m.rot_dims, "theta": m.rot_base, "interleaved": True, "scaling": None})
        return PartSpec("latent_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
            "kv_rank": m.kv_rank, "q_rank": m.q_rank, "gate": True, "scale": m.scale, "eps": cfg.eps,
            "position": rope, "window": 0, "prefix": "mix."})
    return PartSpec("selective_state_space", {
        "hidden": cfg.width, "n_heads": m.heads, "v_dim": m.vdim, "n_state": m.state, "n_groups": m.groups,
        "taps": m.conv, "norm_groups": m.norm_groups, "eps": cfg.eps, "prefix": "mix."})


def _feed_forward(cfg: VitinexConfig, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("swiglu", {"hidden": cfg.width, "intermediate": f.ff, "bias": True, "activation": "gelu_tanh",
                                   "gate": "gate", "up": "up", "down": "down", "prefix": "mlp."})
    return PartSpec("routed_experts", {
        "hidden": cfg.width, "n_experts": f.experts, "top": f.top, "scale": 1.0, "n_groups": 1, "keep": 1,
        "intermediate": f.ff, "shared_intermediate": f.shared_ff, "score": "softmax", "renorm": False,
        "correction": False, "gated": False, "activation": "relu_sq",
        "shared_gate": "shared.sg" if f.shared_ff else None, "prefix": "mlp."})


def describe_vitinex(cfg: VitinexConfig) -> ModelSpec:
    def norm(name, scale=1.0):
        return PartSpec("layernorm", {"size": cfg.width, "eps": cfg.eps, "tensor": name, "scale": scale})

    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer_norm": norm("norm1"), "mixer": _mixer(cfg, layer),
                 "mixer_out_norm": norm("norm1b", cfg.residual_mult)}
        if layer.mlp is not None:
            parts.update({"feed_forward_norm": norm("norm2"), "feed_forward": _feed_forward(cfg, layer.mlp),
                          "feed_forward_out_norm": norm("norm2b", cfg.residual_mult)})
        layers.append(LayerSpec("sandwich_norm_residual", parts, f"l{i}."))
    schedule = []
    for i, t, first in cfg.runs():
        if first:                      # the head of pass t: one more "layer" whose only part rewrites the stream
            schedule.append(ScheduleEntry(len(layers)))
            layers.append(LayerSpec("stream_op", {"op": PartSpec("embedding_reentry", {
                "hidden": cfg.width, "rows": cfg.loop.times, "row": t, "prefix": "loop."})}, ""))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        hidden=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width, "own_matrix": False}),
        keep_embedded=cfg.loop is not None)


VITINEX = register_architecture(Architecture(
    names=("Vitinex",),
    description="Vitinex decoder: latent attention with gated heads and state-space layers between norms on both "
                "sides, squared-ReLU experts, looped layers with re-entry of the embedded tokens",
    config_class=VitinexConfig,
    describe_model=describe_vitinex,
    # a layer without a feed-forward has no use for its norms; a file that carries them all the same is accepted
    ignored_tensor_suffixes=(".norm2", ".norm2b")), replace=True)
