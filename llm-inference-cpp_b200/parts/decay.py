"""Mixers that are linear attention with a decay: a matrix state per head that forgets by a factor per token and takes
one outer product,

    S <- diag(w) S + k vᵀ ;    o = Sᵀ q

with S [dim, vdim] per head in the cache's state slab (fp32, column by column, zero when a slot is handed out).  The two
kinds differ in where the decay comes from and in what surrounds the recurrence; everything behind the projections is
fp32 (csrc/decay_recurrence.cu).

``channel_decay_attention``: q = W_q h · dim^-1/2, k = W_k h, v = W_v h; a decay per head and key channel and token,
w = logistic(z)^(1/tau) with z = W_a2 (W_a1 h) + b (a low-rank path); each head's o is RMS-normed over its vdim entries
with one weight vector shared by the heads, the heads are multiplied by silu(W_g h) and projected by W_o.

``head_decay_attention``: q, k, v = silu(W h); ONE constant decay per head (a parameter, not a tensor) and no scale on
the queries; the heads' outputs are RMS-normed TOGETHER (one row of heads·vdim entries, a weight per entry), multiplied
by logistic(W_g h) and projected by W_o.
"""
from __future__ import annotations

import torch

from ..cache.storage import StateRequest
from ..ops import kernels
from .registry import FreeDim, TensorDecl, part


class _DecayAttention:
    stores_output = True
    defers_norm = False

    def _sizes(self, p):
        self.width, self.H, self.D, self.Dv = int(p["width"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.eps = float(p["eps"])
        self.n_qk, self.n_v = self.H * self.D, self.H * self.Dv

    def cache_request(self):
        return StateRequest((self.H * self.D * self.Dv,), torch.float32)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    @property
    def takes_padding_rows(self) -> bool:
        return True          # every kernel skips token rows and sequences of no slot

    def _project_out(self, heads, x, store):
        kernels.linear(heads, self.w_o, x, None, kernels.OUT_STORE_F32 if store else kernels.OUT_ADD_F32)
        return False


@part("mixer", "channel_decay_attention")
class ChannelDecayAttention(_DecayAttention):
    """params: ``width``, ``heads``, ``dim``, ``vdim``, ``tau``, ``eps`` (of the heads' RMS norm), optional ``rank`` (the
    low-rank path's size where random weights are drawn; a file's own size is read from its tensors).
    tensors: ``q``, ``k`` [heads*dim, width], ``v``, ``g`` [heads*vdim, width], ``a1`` [rank, width], ``a2`` [heads*dim,
    rank], ``a2.b`` [heads*dim], ``norm`` [vdim], ``o`` [width, heads*vdim]."""

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, N, Nv = p["width"], p["heads"] * p["dim"], p["heads"] * p["vdim"]
        R = FreeDim(int(p.get("rank") or max(1, W // 16)))
        return {"q": TensorDecl((N, W)), "k": TensorDecl((N, W)), "v": TensorDecl((Nv, W)), "g": TensorDecl((Nv, W)),
                "o": TensorDecl((W, Nv)), "norm": TensorDecl((p["vdim"],), "norm_scale"), "a1": TensorDecl((R, W)),
                "a2": TensorDecl((N, R)), "a2.b": TensorDecl((N,), "bias")}

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self._sizes(p)
        self.tau = float(p["tau"])
        if not self.tau > 0:
            raise ValueError("channel_decay_attention: tau must be positive")
        self.R = int(tensors["a1"].shape[0])
        if tensors["a2"].shape[1] != self.R:
            raise ValueError(f"channel_decay_attention: a1 has {self.R} rows but a2 has {tensors['a2'].shape[1]} columns")
        # one product for all projections: rows [q | k | v | gate | low-rank path]
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in ("q", "k", "v", "g", "a1")], dim=0))
        self.w2 = rt.to_f32(tensors["a2"])                            # [heads*dim, rank]: a handful of tokens read it row by row
        self.w2t = self.w2.t().contiguous()                           # [rank, heads*dim]: walked by many tokens, eight a block
        self.a_bias = rt.to_f32(tensors["a2.b"])
        self.w_norm = rt.to_f32(tensors["norm"])
        self.w_o = rt.to_compute(tensors["o"])
        self.q_scale = float(self.D) ** -0.5

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        T = h.shape[0]
        rt, H, D, Dv, N, Nv = self.rt, self.H, self.D, self.Dv, self.n_qk, self.n_v
        proj = rt.scratch("decay_proj", (T, 2 * N + 2 * Nv + self.R), torch.float32)
        kernels.linear(h, self.w_in, proj, None, kernels.OUT_STORE_F32)
        dec = rt.scratch("decay_w", (T, N), torch.float32)
        kernels.channel_decay(proj[:, 2 * N + 2 * Nv:], self.w2t, self.a_bias, self.tau, ctx, dec, self.w2)
        o_raw = rt.scratch("decay_o", (T, Nv), torch.float32)
        kernels.decay_recurrence(proj, 0, N, 2 * N, H, D, Dv, binding.group.data[binding.index], ctx, o_raw, dec=dec,
                                 q_scale=self.q_scale, write_state=binding.writes)
        heads = rt.scratch("attn_out", (T, Nv))
        kernels.delta_finish(o_raw, proj[:, 2 * N + Nv:2 * N + 2 * Nv], self.w_norm, self.eps, H, Dv, ctx, heads, kernels.GATE_SILU)
        return self._project_out(heads, x, store)


@part("mixer", "head_decay_attention")
class HeadDecayAttention(_DecayAttention):
    """params: ``width``, ``heads``, ``dim``, ``vdim``, ``decay`` (one factor per head), ``eps`` (of the RMS norm over all
    heads).  tensors: ``q``, ``k`` [heads*dim, width], ``v``, ``g`` [heads*vdim, width], ``norm`` [heads*vdim],
    ``o`` [width, heads*vdim]."""
    SILU_INSIDE_MAX_TOKENS = 64      # up to here a step has no pass of its own for silu on q, k, v

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, N, Nv = p["width"], p["heads"] * p["dim"], p["heads"] * p["vdim"]
        return {"q": TensorDecl((N, W)), "k": TensorDecl((N, W)), "v": TensorDecl((Nv, W)), "g": TensorDecl((Nv, W)),
                "o": TensorDecl((W, Nv)), "norm": TensorDecl((Nv,), "norm_scale")}

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self._sizes(p)
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.H:
            raise ValueError("head_decay_attention: one decay per head")
        self.head_decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0))      # rows [q | k | v | gate]
        self.w_norm = rt.to_f32(tensors["norm"])
        self.w_o = rt.to_compute(tensors["o"])

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        T = h.shape[0]
        rt, H, D, Dv, N, Nv = self.rt, self.H, self.D, self.Dv, self.n_qk, self.n_v
        proj = rt.scratch("decay_proj", (T, 2 * N + 2 * Nv), torch.float32)
        kernels.linear(h, self.w_in, proj, None, kernels.OUT_STORE_F32)
        few = T <= self.SILU_INSIDE_MAX_TOKENS      # a handful of tokens: the recurrence applies silu as it reads q, k, v
        if not few:
            kernels.rows_silu(proj[:, :2 * N + Nv])
        o_raw = rt.scratch("decay_o", (T, Nv), torch.float32)
        kernels.decay_recurrence(proj, 0, N, 2 * N, H, D, Dv, binding.group.data[binding.index], ctx, o_raw,
                                 head_decay=self.head_decay, write_state=binding.writes, silu_in=few)
        heads = rt.scratch("attn_out", (T, Nv))
        # the norm runs over the whole row: one "head" of heads*vdim entries
        kernels.delta_finish(o_raw, proj[:, 2 * N + Nv:], self.w_norm, self.eps, 1, Nv, ctx, heads, kernels.GATE_SIGMOID)
        return self._project_out(heads, x, store)
