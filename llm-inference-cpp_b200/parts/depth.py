"""What acts on the stream right behind a layer and looks back over the depth of the model.

``depth_average``: with X_0 the embedding output and X_(j+1) the result of scheduled call j, the stream that leaves
call i is a learned mixture of all of them,  x <- sum over j = 0 .. i+1 of c[j] * X_j,  with one coefficient per
earlier result (the tensor has i + 2 entries).  The layer's own result X_(i+1) is filed before the mixing, so later
calls mix the unmixed results.  fp32, elementwise, added in the order of j.  The norms that read the mixed stream next
can leave in the same pass over it (``then``).
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

    def forward(self, x, history, index, ctx, then=None):
        """``then``: the norms that read x next — (norm,) or (norm_a, norm_b) — where their owner takes them ready made.
        Returns their outputs if they left in the same pass as the mixture (a norm that offers ``after_mix``), else None."""
        if index != self.index:
            raise ValueError(f"depth_average: built for call {self.index}, run behind call {index}")
        if then is not None and hasattr(then[0], "after_mix"):
            done = then[0].after_mix(then[1] if len(then) > 1 else None, x, history, index + 1, self.coeffs)
            if done is not None:
                return done
        kernels.depth_mix(x, history, index + 1, self.coeffs)
        return None
