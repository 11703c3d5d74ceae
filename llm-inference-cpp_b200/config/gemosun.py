"""Typed configuration of the Gemosun decoder.

config.json names the design with ``"architecture": "Gemosun"`` and gives every size and every constant that can
differ between models of the design:

* ``vocab``, ``width``; ``norm.eps`` (of every layer norm);
* ``layers``: a list, one entry per layer, with ``type`` (``attention``), ``mixer`` (the mixer's sizes: ``heads``,
  ``kv_heads``, ``dim``, ``vdim``, ``scale``; ``rot`` with ``base``, ``dims`` and an optional ``scaling`` of ``factor``,
  ``original``, ``fast``, ``slow``; ``mask`` with ``size`` and ``pool``) and ``mlp`` (``null`` for a layer without a
  feed-forward; ``kind`` ``dense`` with ``ff``; or ``kind`` ``moe`` with ``expert.ff``, ``router.experts``,
  ``router.top``, an optional ``router.groups`` of ``count`` and ``keep``, and an optional ``shared.ff``).

A mixer without ``rot`` is not rotated, one without ``rot.scaling`` rotates by the plain frequencies; one without
``mask`` sees every earlier position, one without ``mask.pool`` only its window.  No size has a default: a missing or
ill-typed key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .garodra import _number, _obj, _uint
from .llama import MAX_LAYERS, MAX_VOCAB, ConfigError

ARCHITECTURE = "Gemosun"
MAX_EXPERTS = 256


@dataclass(frozen=True)
class RotationScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float = 1.0
    rot_dims: int = 0                       # 0: no rotation
    rot_scaling: Optional[RotationScaling] = None
    window: int = 0                         # 0: every earlier position
    pool: int = 0                           # 0: nothing beyond the window


@dataclass(frozen=True)
class FeedForwardSizes:
    kind: str                               # "dense" | "moe"
    ff: int                                 # dense: the inner size; moe: of one expert
    experts: int = 0
    top: int = 0
    groups: int = 0                         # 0: every expert can be chosen
    keep: int = 0
    shared_ff: int = 0                      # 0: no shared expert


@dataclass(frozen=True)
class GemosunLayer:
    type: str
    mixer: AttentionSizes
    mlp: Optional[FeedForwardSizes]


def _attention(m: Mapping[str, Any], mw: str) -> AttentionSizes:
    heads, kv_heads = _uint(m, "heads", mw), _uint(m, "kv_heads", mw)
    if heads % kv_heads:
        raise ConfigError(f'config: {mw}"heads" is not a multiple of "kv_heads"')
    dim, vdim = _uint(m, "dim", mw), _uint(m, "vdim", mw)
    if vdim != dim:
        raise ConfigError(f'config: {mw}"vdim" must equal "dim": the values are the keys as projected')
    rot_base, rot_dims, scaling = 1.0, 0, None
    if m.get("rot") is not None:
        rot = _obj(m, "rot", mw)
        rot_dims = _uint(rot, "dims", mw + "rot.", least=0)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f'config: {mw}rot."dims" must be even and at most "dim"')
        rot_base = _number(rot, "base", mw + "rot.")
        if rot.get("scaling") is not None:
            s, sw = _obj(rot, "scaling", mw + "rot."), mw + "rot.scaling."
            scaling = RotationScaling(factor=_number(s, "factor", sw), original=_number(s, "original", sw),
                                      fast=_number(s, "fast", sw), slow=_number(s, "slow", sw))
            if rot_base <= 1.0:
                raise ConfigError(f'config: {mw}rot."base" must be larger than 1 where the rotation is scaled')
    window = pool = 0
    if m.get("mask") is not None:
        mask = _obj(m, "mask", mw)
        window = _uint(mask, "size", mw + "mask.", 1 << 30)
        if mask.get("pool") is not None:
            pool = _uint(mask, "pool", mw + "mask.", 1 << 20)
    return AttentionSizes(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_number(m, "scale", mw),
                          rot_base=rot_base, rot_dims=rot_dims, rot_scaling=scaling, window=window, pool=pool)


def _feed_forward(mlp: Mapping[str, Any], where: str) -> FeedForwardSizes:
    kind = mlp.get("kind")
    if kind == "dense":
        return FeedForwardSizes("dense", _uint(mlp, "ff", where + "mlp."))
    if kind != "moe":
        raise ConfigError(f'config: {where}mlp."kind" must be "dense" or "moe", not {kind!r}')
    r, rw = _obj(mlp, "router", where + "mlp."), where + "mlp.router."
    experts = _uint(r, "experts", rw, MAX_EXPERTS)
    top = _uint(r, "top", rw, experts)
    groups = keep = 0
    if r.get("groups") is not None:
        g = _obj(r, "groups", rw)
        groups = _uint(g, "count", rw + "groups.", experts)
        keep = _uint(g, "keep", rw + "groups.", groups)
        if experts % groups:
            raise ConfigError(f'config: {rw}"experts" is not a multiple of groups."count"')
        if keep * (experts // groups) < top:
            raise ConfigError(f'config: {rw}the kept groups hold fewer than "top" experts')
    shared = 0
    if mlp.get("shared") is not None:
        shared = _uint(_obj(mlp, "shared", where + "mlp."), "ff", where + "mlp.shared.")
    return FeedForwardSizes("moe", _uint(_obj(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert."),
                            experts=experts, top=top, groups=groups, keep=keep, shared_ff=shared)


@dataclass(frozen=True)
class GemosunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "GemosunConfig":
        vocab = _uint(root, "vocab", "", MAX_VOCAB)
        width = _uint(root, "width", "")
        eps = _number(_obj(root, "norm", ""), "eps", "norm.")
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw or len(raw) > MAX_LAYERS:
            raise ConfigError(f'config: "layers" must be a list of 1..{MAX_LAYERS} layers')
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config: layers[{i}] must be an object")
            kind = entry.get("type")
            if kind != "attention":
                raise ConfigError(f'config: {where}"type" must be "attention", not {kind!r}')
            mixer = _attention(_obj(entry, "mixer", where), where + "mixer.")
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f'config: {where}"mlp" must be an object or null')
            layers.append(GemosunLayer(kind, mixer, _feed_forward(mlp, where) if mlp is not None else None))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))
