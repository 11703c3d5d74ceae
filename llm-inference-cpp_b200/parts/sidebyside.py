"""Mixer ``side_by_side``: two mixers read the same input; each one's output is RMS-normed over the model width with a
plain weight of its own, and the result is the mean of the two.

The two mixers are parts of the mixer family held in the params (``left``, ``right``: PartSpecs whose prefixes are
relative to this part's); each keeps what it needs in the cache under this call: the left one's request is the call's
main one, everything else (the right one's, and what either keeps beside its main request) is handed on by name.
"""
from __future__ import annotations

import torch

from ..cache.storage import CacheBinding
from ..ops import kernels
from .registry import TensorDecl, nested_build, nested_declare, part


@part("mixer", "side_by_side")
class SideBySide:
    """params: ``width``, ``eps``, ``left``, ``right`` (PartSpecs of the mixer family), optional ``names`` (the local names
    of the two norm weights; default ``left.out``, ``right.out``).  tensors: the two mixers' own, and the two weights
    [width]."""
    stores_output = True

    @classmethod
    def declare(cls, spec):
        p = spec.params
        d = {}
        d.update(nested_declare("mixer", p["left"]))
        d.update(nested_declare("mixer", p["right"]))
        for n in p.get("names", ("left.out", "right.out")):
            d[n] = TensorDecl((p["width"],), "norm_scale")
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width, self.eps = int(p["width"]), float(p["eps"])
        self.left = nested_build("mixer", p["left"], tensors, rt)
        self.right = nested_build("mixer", p["right"], tensors, rt)
        for m in (self.left, self.right):
            if not getattr(m, "stores_output", False):
                raise ValueError(f"side_by_side: the mixer {m.kind!r} cannot store its output (store=)")
        ln, rn = p.get("names", ("left.out", "right.out"))
        self.w_left, self.w_right = rt.to_f32(tensors[ln]), rt.to_f32(tensors[rn])

    # -- cache: the left mixer's request is the call's; the rest goes by name ------------------------------------------
    def cache_request(self):
        return self.left.cache_request()

    def more_cache_requests(self):
        more = {}
        if self.right.cache_request() is not None:
            more["right"] = self.right.cache_request()
        for side, m in (("left", self.left), ("right", self.right)):
            for name, req in (m.more_cache_requests() if hasattr(m, "more_cache_requests") else {}).items():
                more[f"{side}.{name}"] = req
        return more

    def _bindings(self, binding):
        def own(side):
            return {name[len(side) + 1:]: b for name, b in binding.more.items() if name.startswith(side + ".")}
        left = CacheBinding(binding.group, binding.index, binding.writes, own("left"))
        r = binding.more.get("right")
        right = CacheBinding(r.group if r else None, r.index if r else 0, binding.writes, own("right"))
        return left, right

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in (self.left, self.right) if hasattr(m, "weight_bytes"))

    @property
    def takes_padding_rows(self) -> bool:
        return bool(getattr(self.left, "takes_padding_rows", False) and getattr(self.right, "takes_padding_rows", False))

    def step_plan(self, ctx, binding):
        lb, rb = self._bindings(binding)
        return tuple(m.step_plan(ctx, b) if hasattr(m, "step_plan") else None for m, b in ((self.left, lb), (self.right, rb)))

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        lb, rb = self._bindings(binding)
        a = self.rt.scratch("side_left", tuple(x.shape), torch.float32)
        b = self.rt.scratch("side_right", tuple(x.shape), torch.float32)
        self.left.forward(h, a, ctx, lb, store=True)
        self.right.forward(h, b, ctx, rb, store=True)
        kernels.normed_pair(a, self.w_left, b, self.w_right, self.eps, 0.5, x, add=not store)
        return False
