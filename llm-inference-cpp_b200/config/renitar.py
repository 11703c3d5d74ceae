"""Typed configuration of the Renitar decoder.

config.json names the design with ``"architecture": "Renitar"`` and gives every size and every constant that can
differ between models of the design:

* ``vocab``, ``width``; ``norm.eps`` (of every RMS norm); ``residual_mult`` (what both branches of a layer are
  multiplied by before they join the stream);
* ``layers``: a list, one entry per layer, with ``type`` (``gla`` or ``parallel``), ``mixer`` (that mixer's sizes) and
  ``mlp`` (``null`` for a layer without a feed-forward, else ``kind`` ``moe``).

  - a ``gla`` mixer: ``heads``, ``dim``, ``vdim``, ``tau`` (and optionally ``rank``, the size of the decay's low-rank
    path where random weights are drawn; a file's own size is read from its tensors);
  - a ``parallel`` mixer: ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``; optional ``conv``
    — taps of the short convolution on q, k and v —, ``softcap``, ``mask.size``, ``rot`` with ``base`` and ``dims``) and
    ``right`` (``heads``, ``dim``, ``vdim`` and ``decay``, one factor per head);
  - a ``moe`` feed-forward: ``expert.ff``, ``router`` with ``experts``, ``top``, ``scale`` and an optional ``identity``
    (how many further router outputs stand for experts that hand their input on), and an optional ``shared.ff``.

An attention without ``mask`` sees every earlier position, one without ``rot`` (or with ``rot.dims`` 0) is not rotated,
one without ``conv`` (or with 0 taps) has no convolution, one without ``softcap`` (or with 0) does not cap its scores.
No size has a default: a missing or ill-typed key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .garodra import _number, _obj, _uint
from .llama import MAX_LAYERS, MAX_VOCAB, ConfigError

ARCHITECTURE = "Renitar"
MAX_EXPERTS = 256
MAX_TAPS = 16


@dataclass(frozen=True)
class ChannelDecaySizes:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0            # 0: not given (a file's tensors decide; random weights take a default)


@dataclass(frozen=True)
class BlockAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    taps: int = 0            # 0: no short convolution on q, k, v
    softcap: float = 0.0     # 0: scores are not capped
    chunk: int = 0           # positions per block of the mask (0: no mask beyond causality)
    rot_base: float = 1.0
    rot_dims: int = 0        # 0: no rotation


@dataclass(frozen=True)
class HeadDecaySizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple             # one factor per head


@dataclass(frozen=True)
class SideBySideSizes:
    left: BlockAttentionSizes
    right: HeadDecaySizes


@dataclass(frozen=True)
class ExpertsSizes:
    ff: int
    experts: int             # experts with matrices
    identity: int            # further router outputs: experts that hand their input on
    top: int
    scale: float
    shared_ff: int = 0       # 0: no shared expert


@dataclass(frozen=True)
class RenitarLayer:
    type: str                # "gla" | "parallel"
    mixer: Any
    mlp: Optional[ExpertsSizes]


def _cap(m: Mapping[str, Any], where: str) -> float:
    """The cap on the scores: absent, null or 0 means none."""
    if m.get("softcap") is None:
        return 0.0
    cap = _number(m, "softcap", where, positive=False)
    if cap < 0:
        raise ConfigError(f'config: {where}"softcap" must not be negative')
    return cap


def _block_attention(m: Mapping[str, Any], where: str) -> BlockAttentionSizes:
    heads, kv_heads = _uint(m, "heads", where), _uint(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f'config: {where}"heads" is not a multiple of "kv_heads"')
    dim = _uint(m, "dim", where)
    rot_base, rot_dims = 1.0, 0
    if m.get("rot") is not None:
        rot = _obj(m, "rot", where)
        rot_dims = _uint(rot, "dims", where + "rot.", least=0)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f'config: {where}rot."dims" must be even and at most "dim"')
        if rot_dims:
            rot_base = _number(rot, "base", where + "rot.")
    return BlockAttentionSizes(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=_uint(m, "vdim", where), scale=_number(m, "scale", where),
        taps=_uint(m, "conv", where, MAX_TAPS, least=0) if m.get("conv") is not None else 0,
        softcap=_cap(m, where),
        chunk=_uint(_obj(m, "mask", where), "size", where + "mask.", 1 << 30) if m.get("mask") is not None else 0,
        rot_base=rot_base, rot_dims=rot_dims)


def _head_decay(m: Mapping[str, Any], where: str) -> HeadDecaySizes:
    heads = _uint(m, "heads", where)
    decay = m.get("decay")
    if (not isinstance(decay, list) or len(decay) != heads
            or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not (0.0 <= d < float("inf")) for d in decay)):
        raise ConfigError(f'config: {where}"decay" must be a list of {heads} numbers that are not negative, one per head')
    return HeadDecaySizes(heads=heads, dim=_uint(m, "dim", where), vdim=_uint(m, "vdim", where),
                          decay=tuple(float(d) for d in decay))


def _experts(mlp: Mapping[str, Any], where: str) -> ExpertsSizes:
    if mlp.get("kind") != "moe":
        raise ConfigError(f'config: {where}"kind" must be "moe"')
    r = _obj(mlp, "router", where)
    experts = _uint(r, "experts", where + "router.", MAX_EXPERTS)
    identity = _uint(r, "identity", where + "router.", MAX_EXPERTS, least=0) if r.get("identity") is not None else 0
    top = _uint(r, "top", where + "router.", MAX_EXPERTS)
    if experts + identity > MAX_EXPERTS or top > experts + identity:
        raise ConfigError(f'config: {where}router: "top" is at most "experts" + "identity", which is at most {MAX_EXPERTS}')
    shared = mlp.get("shared")
    return ExpertsSizes(ff=_uint(_obj(mlp, "expert", where), "ff", where + "expert."), experts=experts, identity=identity,
                        top=top, scale=_number(r, "scale", where + "router."),
                        shared_ff=_uint(_obj(mlp, "shared", where), "ff", where + "shared.") if shared is not None else 0)


@dataclass(frozen=True)
class RenitarConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "RenitarConfig":
        vocab = _uint(root, "vocab", "", MAX_VOCAB)
        width = _uint(root, "width", "")
        eps = _number(_obj(root, "norm", ""), "eps", "norm.")
        mult = _number(root, "residual_mult", "", positive=False)
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw or len(raw) > MAX_LAYERS:
            raise ConfigError(f'config: "layers" must be a list of 1..{MAX_LAYERS} layers')
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config: layers[{i}] must be an object")
            kind = entry.get("type")
            m = _obj(entry, "mixer", where)
            mw = where + "mixer."
            if kind == "gla":
                mixer = ChannelDecaySizes(heads=_uint(m, "heads", mw), dim=_uint(m, "dim", mw), vdim=_uint(m, "vdim", mw),
                                          tau=_number(m, "tau", mw),
                                          rank=_uint(m, "rank", mw) if m.get("rank") is not None else 0)
            elif kind == "parallel":
                mixer = SideBySideSizes(left=_block_attention(_obj(m, "left", mw), mw + "left."),
                                        right=_head_decay(_obj(m, "right", mw), mw + "right."))
            else:
                raise ConfigError(f'config: {where}"type" must be "gla" or "parallel", not {kind!r}')
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f'config: {where}"mlp" must be an object or null')
            layers.append(RenitarLayer(kind, mixer, _experts(mlp, where + "mlp.") if mlp is not None else None))
        return cls(vocab=vocab, width=width, norm_eps=eps, residual_mult=mult, layers=tuple(layers))
