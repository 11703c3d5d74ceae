"""The Renitar decoder as a recipe of parts.

Embedding rows as they are; layers of the arrangement ``parallel_scaled`` — the mixer and the feed-forward read ONE RMS
norm's output (its weight stored around zero: ``one_plus``) and their sum joins the stream times a constant —; a mixer
per layer: ``channel_decay_attention`` (linear attention with a decay per key channel from a low-rank path), or
``side_by_side`` of a ``gated_attention`` (biases, a short convolution on q, k, v, whole-row q and k norms, a rotation of
the first entries, capped scores, a mask of blocks of positions, a logistic gate per output entry) and a
``head_decay_attention`` (linear attention with one constant decay per head); a feed-forward per layer or none:
``routed_experts`` with scores from a softmax over all router outputs, a stored correction in the choice, weights that
are not normalised, experts that hand their input on, the exact GELU and a gated shared expert; a last norm and an
untied head.  Tensor names: ``embed``, ``head``, ``final.norm`` and per layer i ``l<i>.norm1``, ``l<i>.mix.*``
(``.left.*`` and ``.right.*`` for the two mixers side by side), ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.renitar import ARCHITECTURE, RenitarConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24        # the design sets no limit: angles are computed on the fly, and a state has no length


def _mixer(c: RenitarConfig, layer, prefix: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "gla":
        return PartSpec("channel_decay_attention", {"width": c.width, "heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                                    "tau": m.tau, "eps": c.norm_eps, "rank": m.rank}, prefix)
    a, r = m.left, m.right
    position = (PartSpec("rotary_half", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base})
                if a.rot_dims else None)
    left = PartSpec("gated_attention", {
        "width": c.width, "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
        "eps": c.norm_eps, "bias": True, "conv": a.taps, "qk_norm": True, "position": position, "softcap": a.softcap,
        "chunk": a.chunk, "gate": True}, "left.")
    right = PartSpec("head_decay_attention", {"width": c.width, "heads": r.heads, "dim": r.dim, "vdim": r.vdim,
                                              "decay": r.decay, "eps": c.norm_eps}, "right.")
    return PartSpec("side_by_side", {"width": c.width, "eps": c.norm_eps, "left": left, "right": right}, prefix)


def _ffn(c: RenitarConfig, mlp, prefix: str) -> PartSpec:
    return PartSpec("routed_experts", {
        "width": c.width, "inner": mlp.ff, "experts": mlp.experts, "identity": mlp.identity, "top": mlp.top,
        "scale": mlp.scale, "activation": "gelu", "gated": False, "scoring": "softmax_all", "shared": mlp.shared_ff}, prefix)


def renitar_model_spec(c: RenitarConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rms", {"width": c.width, "eps": c.norm_eps, "tensor": "", "one_plus": True}, name)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        layers.append(LayerSpec(
            block="parallel_scaled", mixer_norm=norm(p + "norm1"), mixer=_mixer(c, layer, p + "mix."),
            ffn=_ffn(c, layer.mlp, p + "mlp.") if layer.mlp is not None else None,
            block_params={"residual_mult": c.residual_mult}))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        architecture=c.architecture, vocab_size=c.vocab, width=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_table", {"vocab": c.vocab, "width": c.width, "tensor": "embed"}, ""),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": c.vocab, "width": c.width, "tied": False, "tensor": "head"}, ""),
        stop_ids=())


register_architecture(Architecture(ARCHITECTURE, RenitarConfig.from_dict, renitar_model_spec))
