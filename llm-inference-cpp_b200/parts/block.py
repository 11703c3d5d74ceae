"""Arrangements of a layer.  ``prenorm``: x += mixer(norm(x)); x += ffn(norm(x))
(include/llmi/model/transformer.hpp:49-52); the feed-forward may be absent, and a part in the slot ``mixer_conv``
(family ``conv``) acts on the mixer's input: x += mixer(conv(norm(x))).

Norm deferral (optional, see :class:`ops.kernels.DeferredNorm`): a mixer or feed-forward whose class sets
``defers_norm = True`` accepts a filled deferred norm as its input ``h`` and a keyword ``then_norm`` — a
deferred norm to fill with its last, residual-adding product — and returns whether it filled it.  The block
uses this where both neighbours of a norm take part and the norm offers ``deferred``; everything else runs
the norm the plain way, so parts without these extras work unchanged.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import part


def _defers(p) -> bool:
    return bool(getattr(p, "defers_norm", False))


@part("block", "prenorm")
class PreNormBlock:
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone
    def __init__(self, mixer_norm, mixer, ffn_norm=None, ffn=None, mixer_conv=None):
        """``ffn_norm`` and ``ffn`` come together or not at all (a layer without a feed-forward); ``mixer_conv`` (a part
        of the family ``conv``) reshapes what the mixer reads: x += mixer(conv(norm(x)))."""
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("prenorm: a feed-forward comes with its norm, or not at all")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.mixer_conv = mixer_conv

    @property
    def entry_norm(self):
        """The norm this block applies to x first, if whoever updates x before the block may fill its
        deferred form (``forward(..., entry=)``); else None."""
        if self.mixer_conv is not None:       # the convolution reads the norm's rows themselves
            return None
        return self.mixer_norm if _defers(self.mixer) and hasattr(self.mixer_norm, "deferred") else None

    def forward(self, x, ctx, binding, entry=None, next_norm=None):
        """``entry``: the filled deferred form of this block's first norm, or None.  ``next_norm``: the norm
        that reads x after this block, or None.  Returns that norm's deferred form if the block filled it."""
        T = x.shape[0]
        h = None
        if self.mixer_conv is not None:
            fused = getattr(self.mixer_conv, "forward_from_stream", None)
            h = fused(x, self.mixer_norm, ctx, binding.more["mixer_conv"]) if fused is not None else None
            if h is None:
                h = self.mixer_conv.forward(self.mixer_norm.forward(x), ctx, binding.more["mixer_conv"])
        else:
            h = entry if isinstance(entry, kernels.DeferredNorm) else self.mixer_norm.forward(x)
        if self.ffn is None:
            self.mixer.forward(h, x, ctx, binding)
            return None
        then = None
        if _defers(self.mixer) and _defers(self.ffn) and hasattr(self.ffn_norm, "deferred"):
            then = self.ffn_norm.deferred(T, "deferred_inner")
        if then is not None and self.mixer.forward(h, x, ctx, binding, then_norm=then):
            h = then
        else:
            if then is None:
                self.mixer.forward(h, x, ctx, binding)
            h = self.ffn_norm.forward(x)
        then = next_norm.deferred(T, "deferred_outer") if (hasattr(next_norm, "deferred") and _defers(self.ffn)) else None
        if then is not None:
            return then if self.ffn.forward(h, x, ctx, then_norm=then) else None
        self.ffn.forward(h, x, ctx)
        return None


@part("block", "parallel")
class ParallelBlock:
    """Both sublayers read the SAME x, each through a norm of its own, and are added at once:
    x += mixer(norm1(x)) + ffn(norm2(x)).  The feed-forward (with its norm) may be absent.  Both norms are computed
    before either sublayer touches x — in one pass over x where the norms offer ``forward_pair``."""

    def __init__(self, mixer_norm, mixer, ffn_norm=None, ffn=None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("parallel: a feed-forward comes with its norm, or not at all")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    @property
    def takes_padding_rows(self) -> bool:
        return True          # rows are treated alone

    @property
    def entry_norms(self):
        """The norms this block applies to x first: whoever changes x last before the block may hand their outputs in
        (``forward(..., entry=)``) — one tensor for a layer without a feed-forward, else a pair."""
        return (self.mixer_norm,) if self.ffn is None else (self.mixer_norm, self.ffn_norm)

    def forward(self, x, ctx, binding, entry=None):
        if self.ffn is None:
            self.mixer.forward(entry if entry is not None else self.mixer_norm.forward(x), x, ctx, binding)
            return
        pair = entry
        if pair is None and hasattr(self.mixer_norm, "forward_pair"):
            pair = self.mixer_norm.forward_pair(self.ffn_norm, x)
        if pair is None:
            pair = (self.mixer_norm.forward(x, scratch_name="norm_out"), self.ffn_norm.forward(x, scratch_name="norm_out_b"))
        h1, h2 = pair
        self.mixer.forward(h1, x, ctx, binding)
        self.ffn.forward(h2, x, ctx)


@part("block", "parallel_scaled")
class ScaledParallelBlock:
    """Both sublayers read ONE norm's output, and what they add is multiplied by a constant:
    x += m * (mixer(norm(x)) + ffn(norm(x))).  The feed-forward may be absent.  The sublayers write their sum into an
    fp32 buffer of its own (the mixer stores, the feed-forward adds: both must take ``store=``), and one pass joins it
    to the stream; where the norm that reads x next offers ``after_scaled_add`` (the next block's first norm, handed in
    as ``next_norm``), that norm is computed in the same pass and the next block takes its output as ``entry``.

    Slots: ``mixer_norm``, ``mixer``, optional ``ffn``.  Parameter: ``residual_mult`` (m)."""

    def __init__(self, mixer_norm, mixer, ffn=None, residual_mult: float = 1.0):
        for p in (mixer, ffn):
            if p is not None and not getattr(p, "stores_output", False):
                raise ValueError(f"parallel_scaled: the part {getattr(p, 'kind', p)!r} cannot store its output (store=)")
        self.mixer_norm, self.mixer, self.ffn = mixer_norm, mixer, ffn
        self.m = float(residual_mult)
        self.rt = mixer_norm.rt

    @property
    def takes_padding_rows(self) -> bool:
        return True          # rows are treated alone

    @property
    def entry_norm(self):
        return self.mixer_norm

    def forward(self, x, ctx, binding, entry=None, next_norm=None):
        h = entry if isinstance(entry, torch.Tensor) else self.mixer_norm.forward(x)
        y = self.rt.scratch("branch_out", tuple(x.shape), torch.float32)
        self.mixer.forward(h, y, ctx, binding, store=True)
        if self.ffn is not None:
            self.ffn.forward(h, y, ctx)
        if hasattr(next_norm, "after_scaled_add"):
            return next_norm.after_scaled_add(x, y, self.m)       # (this block's own h is read out by now)
        kernels.stream_axpy_norm(x, y, self.m)
        return None


@part("block", "prepost")
class PrePostNormBlock:
    """A norm ahead of AND behind each sublayer:  x += post1(mixer(pre1(x)));  x += post2(ffn(pre2(x))).
    Slots: ``mixer_norm``, ``mixer``, ``mixer_post`` and, for a layer with a feed-forward, ``ffn_norm``, ``ffn``,
    ``ffn_post``.  The sublayer's output goes to an fp32 buffer of its own (a part that sets ``stores_output``
    takes ``store=True`` and overwrites it; any other part adds into the zeroed buffer), and the norm behind it
    joins it to the stream.  Where that norm offers ``add_to(y, x, then=)``, the norm ahead of the NEXT sublayer —
    this block's ``ffn_norm`` or the next block's first norm — is computed in the same pass (the next block gets it
    as ``entry``)."""

    def __init__(self, mixer_norm, mixer, mixer_post, ffn_norm=None, ffn=None, ffn_post=None):
        if (ffn is None) != (ffn_norm is None) or (ffn is None) != (ffn_post is None):
            raise ValueError("prepost: a feed-forward comes with both of its norms, or not at all")
        self.mixer_norm, self.mixer, self.mixer_post = mixer_norm, mixer, mixer_post
        self.ffn_norm, self.ffn, self.ffn_post = ffn_norm, ffn, ffn_post
        self.rt = mixer_norm.rt

    @property
    def takes_padding_rows(self) -> bool:
        return True

    @property
    def entry_norm(self):
        return self.mixer_norm

    def _branch(self, part, h, x, *args):
        y = self.rt.scratch("branch_out", tuple(x.shape), x.dtype)
        if getattr(part, "stores_output", False):
            part.forward(h, y, *args, store=True)
        else:
            y.zero_()
            part.forward(h, y, *args)
        return y

    @staticmethod
    def _join(post, y, x, then, name):
        """x += post(y); returns then(x) if the two norms could share a pass."""
        if hasattr(post, "add_to"):
            return post.add_to(y, x, then if type(then) is type(post) else None, scratch_name=name)
        x += post.forward(y, scratch_name="post_out").float()
        return None

    def forward(self, x, ctx, binding, entry=None, next_norm=None):
        h = entry if isinstance(entry, torch.Tensor) else self.mixer_norm.forward(x)
        y = self._branch(self.mixer, h, x, ctx, binding)
        if self.ffn is None:
            return self._join(self.mixer_post, y, x, next_norm, "norm_out_b")
        h = self._join(self.mixer_post, y, x, self.ffn_norm, "norm_out_b")
        if h is None:
            h = self.ffn_norm.forward(x)
        y = self._branch(self.ffn, h, x, ctx)
        return self._join(self.ffn_post, y, x, next_norm, "norm_out")
