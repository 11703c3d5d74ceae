"""Position-encoding parts.

``rotary_half``: inv_freq[i] = 1 / theta^(2i/d) in fp32 (src/model/transformer.cpp:59-65);
pairs (i, i + d/2) rotated by angle = float(pos) · inv_freq[i] (src/model/kernels.cpp:122-134);
applied to q and k, never to v; k is stored rotated (src/model/transformer.cpp:251-262).
``none``: keys and values are stored as they are.

A position part that acts elsewhere (say, a table added to the embeddings) overrides
``at_embedding`` and keeps ``rotary_dim = 0``.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels
from .registry import part


class PositionEncoding:
    rotary_dim = 0
    inv_freq = None
    pairing = 0          # which entries turn together: 0 (i, i + rotary_dim/2), 1 neighbours (2i, 2i + 1)
    amplitude = 1.0      # cos and sin are multiplied by this (1: a plain rotation)

    @classmethod
    def declare(cls, spec):
        return {}

    def at_embedding(self, x, ctx) -> None:
        """Hook after the embedding lookup; the default adds nothing."""

    def fused_rotation(self):
        """(inv_freq, rotary_dim) if all this part does to q, k, v is the rotation of pairs and the append that
        :meth:`rotate_and_store` does — a mixer may then let its attention kernel do both; None for a
        subclass with a ``rotate_and_store`` of its own."""
        if type(self).rotate_and_store is not PositionEncoding.rotate_and_store or self.pairing != 0 or self.amplitude != 1.0:
            return None
        return self.inv_freq, self.rotary_dim

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim) -> None:
        """Rotate q (in place) and k by position and append k, v to the call's cache pages."""
        g = binding.group
        kernels.rope_store(qkv, self.inv_freq, self.rotary_dim, ctx.tok_seq, ctx.tok_pos, ctx.pages_of(g),
                           g.page_size, g.k[binding.index], g.v[binding.index], n_heads, n_kv_heads, head_dim,
                           write_kv=binding.writes)


@part("position", "none")
class NoPosition(PositionEncoding):
    takes_padding_rows = True       # (a step padded to a shape has token rows of no sequence: see engine/graphs.py)

    def __init__(self, spec, tensors, rt, **_):
        pass


@part("position", "rotary_half")
class RotaryHalf(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default: the whole head)."""
    takes_padding_rows = True       # the rotation kernel skips rows of no sequence

    def __init__(self, spec, tensors, rt, **_):
        d = int(spec.params.get("rotary_dim", spec.params["head_dim"]))
        if d % 2 or d > int(spec.params["head_dim"]):
            raise ValueError("rotary_half: rotary_dim must be even and at most head_dim")
        theta = np.float32(spec.params["theta"])
        exponent = (np.arange(0, d, 2, dtype=np.float32)) / np.float32(d)
        inv = (np.float32(1.0) / np.power(theta, exponent, dtype=np.float32)).astype(np.float32)
        self.rotary_dim = d
        self.inv_freq = torch.from_numpy(inv).to(rt.device)


@part("position", "rotary_pairs")
class RotaryPairs(PositionEncoding):
    """Neighbouring entries (2i, 2i + 1) of the first ``rotary_dim`` entries of a head turn by pos * f_i, f_i =
    theta^(-2i / rotary_dim).  With ``scaling`` = (factor, original, fast, slow) the frequencies are stretched for
    contexts longer than ``original`` positions: with n(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta) — the
    pair index whose wavelength makes t turns over the original context — pairs up to lo = max(floor(n(fast)), 0) keep
    their frequency, pairs from hi = min(ceil(n(slow)), rotary_dim - 1) on are divided by ``factor``, and between them
    the share of the divided frequency rises linearly, (i - lo) / max(hi - lo, 0.001); cos and sin are both multiplied
    by 0.1 * ln(factor) + 1.  The frequencies are made in float64 and rounded once to fp32; the angle is an fp32 product.

    params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default: the whole head), optional ``scaling`` (a dict
    with ``factor``, ``original``, ``fast``, ``slow``).  A mixer reads ``inv_freq``, ``rotary_dim``, ``pairing`` and
    ``amplitude`` and hands them to the kernel that rotates."""
    takes_padding_rows = True
    pairing = 1

    def __init__(self, spec, tensors, rt, **_):
        import math
        p = spec.params
        d = int(p.get("rotary_dim", p["head_dim"]))
        if d % 2 or d > int(p["head_dim"]):
            raise ValueError("rotary_pairs: rotary_dim must be even and at most head_dim")
        theta = float(p["theta"])
        f = np.array([theta ** (-2.0 * i / d) for i in range(d // 2)], dtype=np.float64) if d else np.zeros(0)
        sc = p.get("scaling")
        if sc is not None and d:
            factor, original = float(sc["factor"]), float(sc["original"])

            def pair_index(turns):
                return d * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
            lo = max(math.floor(pair_index(float(sc["fast"]))), 0)
            hi = min(math.ceil(pair_index(float(sc["slow"]))), d - 1)
            ramp = np.clip((np.arange(d // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            self.amplitude = 0.1 * math.log(factor) + 1.0
        self.rotary_dim = d
        self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(rt.device) if d else None

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim) -> None:
        raise NotImplementedError("rotary_pairs: rotates inside a mixer's own preparation kernel (qkv_prepare)")
