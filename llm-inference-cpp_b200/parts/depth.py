"""What acts on the stream right behind a layer and looks back over the depth of the model.

``depth_average``: with X_0 the embedding output and X_(j+1) the result of scheduled call j, the stream that leaves
call i is a learned mixture of all of them,  x <- sum over j = 0 .. i+1 of c[j] * X_j,  with one coefficient per
earlier result (the tensor has i + 2 entries).  The layer's own result X_(i+1) is filed before the mixing, so later
calls mix the unmixed results.  fp32, elementwise, added in the order of j.
"""
from __future__ import annotations

from ..ops import kernels
from .registry import TensorDecl, part


@part("pass_exit", "depth_average")
class DepthAverage:
    """params: ``index`` (the scheduled call it follows: its tensor has ``index + 2`` coefficients), optional ``tensor``
    (local name of the coefficients; default ``dwa``)."""
    takes_padding_rows = True       # elementwise: rows are treated alone

    @classmethod
    def declare(cls, spec):
        return {spec.params.get("tensor", "dwa"): TensorDecl((int(spec.params["index"]) + 2,), "mix")}

    def __init__(self, spec, tensors, rt, **_):
        self.index = int(spec.params["index"])
        self.coeffs = rt.to_f32(tensors[spec.params.get("tensor", "dwa")])

    def forward(self, x, history, index, ctx) -> None:
        if index != self.index:
            raise ValueError(f"depth_average: built for call {self.index}, run behind call {index}")
        kernels.depth_mix(x, history, index + 1, self.coeffs)
