"""The Gemosun decoder as a recipe of parts.

Embedding rows as they are; layers of the arrangement ``parallel`` — the mixer and the feed-forward read the same
stream through a layer norm each (a weight, no bias) and are added at once —; the mixer ``window_pool_attention``:
grouped queries, values that are the keys before the rotation, a rotation of neighbouring entries with stretched
frequencies (``rotary_pairs``), a sliding window with one pooled key and value per block of positions that has left
it, a logistic gate per head; a feed-forward per layer — gated dense with the tanh GELU (``swiglu``), routed experts
with logistic scores, groups of experts, the square of relu and a gated shared expert (``routed_experts``), or none;
behind every layer a learned mixture over the embedding output and all layers' results so far (``depth_average``);
a last layer norm and an untied head.  Tensor names: ``embed``, ``head``, ``final.norm`` and per layer i
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``.
"""
from __future__ import annotations

import re

from ..config.gemosun import ARCHITECTURE, GemosunConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24        # the design sets no limit: angles are computed on the fly


def _mixer(c: GemosunConfig, m, prefix: str) -> PartSpec:
    if m.rot_dims:
        scaling = None
        if m.rot_scaling is not None:
            s = m.rot_scaling
            scaling = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
        position = PartSpec("rotary_pairs", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                             "scaling": scaling})
    else:
        position = PartSpec("none")
    return PartSpec("window_pool_attention", {
        "width": c.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
        "window": m.window, "pool": m.pool, "values_from_keys": True, "gate": True, "position": position}, prefix)


def _ffn(c: GemosunConfig, mlp, prefix: str) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("swiglu", {"width": c.width, "inner": mlp.ff, "activation": "gelu_tanh",
                                   "names": ("gate", "up", "down")}, prefix)
    return PartSpec("routed_experts", {
        "width": c.width, "inner": mlp.ff, "experts": mlp.experts, "top": mlp.top, "activation": "relu2", "gated": False,
        "scoring": "logistic_normalised", "groups": (mlp.groups, mlp.keep) if mlp.groups else None,
        "shared": mlp.shared_ff}, prefix)


def gemosun_model_spec(c: GemosunConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("layernorm", {"width": c.width, "eps": c.norm_eps, "tensor": ""}, name)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        layers.append(LayerSpec(
            block="parallel", mixer_norm=norm(p + "norm1"), mixer=_mixer(c, layer.mixer, p + "mix."),
            ffn_norm=norm(p + "norm2") if layer.mlp is not None else None,
            ffn=_ffn(c, layer.mlp, p + "mlp.") if layer.mlp is not None else None))
        schedule.append(ScheduleEntry(i, after=PartSpec("depth_average", {"index": i, "tensor": "dwa"}, p)))
    return ModelSpec(
        architecture=c.architecture, vocab_size=c.vocab, width=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_table", {"vocab": c.vocab, "width": c.width, "tensor": "embed"}, ""),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": c.vocab, "width": c.width, "tied": False, "tensor": "head"}, ""),
        stop_ids=())


# a layer without a feed-forward has no second norm; a file that carries one all the same is not refused for it
_UNUSED_NORM = re.compile(r"^l\d+\.norm2$")

register_architecture(Architecture(ARCHITECTURE, GemosunConfig.from_dict, gemosun_model_spec,
                                   tolerated_extra_tensors=lambda name: bool(_UNUSED_NORM.match(name))))
