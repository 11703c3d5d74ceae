"""Norm parts.  ``rms``: y = weight · (x · rsqrt(mean(x²) + eps)), as src/model/kernels.cpp:115-120
computes it (scale first, then weight; plain weight, not 1 + weight), the sum of squares in fp32."""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, part


@part("norm", "rms")
class RMSNorm:
    """params: ``width``, ``eps``, optional ``tensor`` (the weight's local name; default ``weight``), optional
    ``one_plus`` (the file stores the weight around zero: y = (1 + w) · x · rsqrt(mean(x²) + eps); the sum 1 + w is made
    once at load, in fp32).  tensors: the weight [width] (kept in fp32)."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone

    @classmethod
    def declare(cls, spec):
        return {spec.params.get("tensor", "weight"): TensorDecl((spec.params["width"],), "norm_scale")}

    def __init__(self, spec, tensors, rt, **_):
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight = rt.to_f32(tensors[spec.params.get("tensor", "weight")])
        if spec.params.get("one_plus", False):
            self.weight = (self.weight + 1.0).contiguous()
        self.rt = rt

    def forward(self, x, rows=None, scratch_name: str = "norm_out"):
        """x fp32 [tokens, width] -> normalised rows in the compute type; ``rows`` picks input rows."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.rt.scratch(scratch_name, (n, self.width))
        kernels.rmsnorm(x, self.weight, out, self.eps, rows)
        return out

    def after_scaled_add(self, x, y, m: float, scratch_name: str = "norm_out"):
        """x += m * y, and this norm of the new x, in one pass over the rows; returns the norm's output."""
        out = self.rt.scratch(scratch_name, (x.shape[0], self.width))
        kernels.stream_axpy_norm(x, y, m, self.weight, self.eps, out)
        return out

    def deferred(self, n_tokens: int, name: str):
        """This norm for ``n_tokens`` rows as a :class:`kernels.DeferredNorm` — to be filled by the product
        that updates x and read by the product after the norm — or None when the step's size or type does
        not allow it (then :meth:`forward` is the way).  ``name`` keeps apart the buffers of norms that are
        in flight at the same time."""
        if not kernels.norm_deferrable(n_tokens, self.width, self.rt.dtype):
            return None
        h = self.rt.scratch(name + "_h", (n_tokens, self.width))
        ss = self.rt.scratch(name + "_ss", ((self.width + 15) // 16, kernels.DeferredNorm.SS_STRIDE), torch.float32)
        return kernels.DeferredNorm(self.weight, self.eps, h, ss)


@part("norm", "layernorm")
class LayerNorm:
    """y = (x - mean) / sqrt(var + eps) * weight: a layer norm with a weight and no bias; var is the mean of the squared
    deviations, all sums in fp32.  params: ``width``, ``eps``, optional ``tensor`` (the weight's local name; default
    ``weight``).  Two norms of this kind that read the same rows can leave in one pass (:meth:`forward_pair`)."""
    takes_padding_rows = True       # rows are treated alone

    @classmethod
    def declare(cls, spec):
        return {spec.params.get("tensor", "weight"): TensorDecl((spec.params["width"],), "norm_scale")}

    def __init__(self, spec, tensors, rt, **_):
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight = rt.to_f32(tensors[spec.params.get("tensor", "weight")])
        self.rt = rt

    def forward(self, x, rows=None, scratch_name: str = "norm_out"):
        """x fp32 [tokens, width] -> normalised rows in the compute type; ``rows`` picks input rows."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.rt.scratch(scratch_name, (n, self.width))
        kernels.layernorm(x, self.weight, out, self.eps, rows)
        return out

    def forward_pair(self, other, x, scratch_names=("norm_out", "norm_out_b")):
        """(self(x), other(x)) from one read of x, or None if ``other`` is no norm of this kind with the same eps."""
        if type(other) is not LayerNorm or other.eps != self.eps or other.width != self.width:
            return None
        a = self.rt.scratch(scratch_names[0], (x.shape[0], self.width))
        b = self.rt.scratch(scratch_names[1], (x.shape[0], self.width))
        kernels.layernorm(x, self.weight, a, self.eps, None, other.weight, b)
        return a, b

    def after_mix(self, other, x, history, n, coeffs, scratch_names=("norm_out", "norm_out_b")):
        """The mixture over the depth (:func:`ops.kernels.depth_mix`) and, of the mixed x, this norm (with ``other``: a
        second norm of this kind with the same eps) in one pass.  Returns the norms' outputs — one tensor, or a pair —,
        or None with nothing done where the fused kernel does not apply."""
        if other is not None and (type(other) is not LayerNorm or other.eps != self.eps or other.width != self.width):
            return None
        a = self.rt.scratch(scratch_names[0], (x.shape[0], self.width))
        b = self.rt.scratch(scratch_names[1], (x.shape[0], self.width)) if other is not None else None
        if not kernels.mix_layernorm(x, history, n, coeffs, self.weight, a, self.eps, other.weight if other is not None else None, b):
            return None
        return a if other is None else (a, b)


@part("norm", "dyt")
class DynamicTanh:
    """Dynamic Tanh: y = tanh(alpha * x) * weight + bias — a norm without statistics.  params: ``width``.
    tensors (the prefix is the norm's full name): ``""`` weight [width], ``".b"`` bias [width], ``".alpha"`` a scalar;
    all kept in fp32.  Used ahead of a sublayer (:meth:`forward`) and behind one (:meth:`add_to`: the normed
    sublayer output joins the residual stream, and the norm ahead of the next sublayer can ride along)."""
    takes_padding_rows = True       # elementwise: rows are treated alone

    @classmethod
    def declare(cls, spec):
        w = spec.params["width"]
        return {"": TensorDecl((w,), "norm_scale"), ".b": TensorDecl((w,), "bias"), ".alpha": TensorDecl((), "norm_scale")}

    def __init__(self, spec, tensors, rt, **_):
        self.width = int(spec.params["width"])
        self.weight = rt.to_f32(tensors[""])
        self.bias = rt.to_f32(tensors[".b"])
        self.alpha = float(tensors[".alpha"].float().item())
        self.rt = rt

    def forward(self, x, rows=None, scratch_name: str = "norm_out"):
        """x fp32 [tokens, width] -> rows in the compute type; ``rows`` picks input rows."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.rt.scratch(scratch_name, (n, self.width))
        kernels.dyt(x, self.weight, self.bias, self.alpha, out, rows)
        return out

    def add_to(self, y, x, then=None, scratch_name: str = "norm_out"):
        """x += self(y), y fp32 [tokens, width].  ``then``: another norm of this kind; its output for the updated x is
        computed in the same pass and returned (None otherwise)."""
        if isinstance(then, DynamicTanh):
            h = self.rt.scratch(scratch_name, (x.shape[0], self.width))
            kernels.dyt_add(y, self.weight, self.bias, self.alpha, x, (then.weight, then.bias, then.alpha), h)
            return h
        kernels.dyt_add(y, self.weight, self.bias, self.alpha, x)
        return None
