"""Mixer parts.  ``gqa``: causal grouped-query attention over the cache.

Formulas: q, k, v projections with optional biases (src/model/transformer.cpp:245-250;
src/model/model.cpp:145-152); query head hh reads kv head hh / (heads / kv_heads)
(src/model/transformer.cpp:264); scores scaled by 1/sqrt(head_dim) after the dot (:235, :271);
causal by position (:270); softmax and weighted sum (:273-280); output projection without
bias added to the residual stream (:283-284).  The three projections are stored as one
matrix [q; k; v] so that one product serves them.
"""
from __future__ import annotations

import math

import torch

from ..cache.storage import KVRequest, StateRequest
from ..ops import kernels
from .registry import TensorDecl, nested_build, nested_declare, part


@part("mixer", "gqa")
class GQAttention:
    """params: ``width``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``bias`` (q/k/v), ``window`` (0: all),
    ``scale`` (default 1/sqrt(head_dim)), ``position`` (a PartSpec of the position family)."""

    @classmethod
    def declare(cls, spec):
        p = spec.params
        q, kv, w = p["n_heads"] * p["head_dim"], p["n_kv_heads"] * p["head_dim"], p["width"]
        d = {"q_proj.weight": TensorDecl((q, w)), "k_proj.weight": TensorDecl((kv, w)),
             "v_proj.weight": TensorDecl((kv, w)), "o_proj.weight": TensorDecl((w, q))}
        if p.get("bias", False):
            d.update({"q_proj.bias": TensorDecl((q,), "bias"), "k_proj.bias": TensorDecl((kv,), "bias"),
                      "v_proj.bias": TensorDecl((kv,), "bias")})
        d.update(nested_declare("position", p["position"]))      # a position part may have tensors of its own
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width = int(p["width"])
        self.n_heads, self.n_kv_heads, self.head_dim = int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError("gqa: n_heads must be a multiple of n_kv_heads")
        self.window = int(p.get("window", 0))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.w_qkv = rt.to_compute(torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                              tensors["v_proj.weight"]], dim=0))
        self.b_qkv = None
        if p.get("bias", False):
            self.b_qkv = rt.to_f32(torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]))
        self.w_o = rt.to_compute(tensors["o_proj.weight"])
        self.position = nested_build("position", p["position"], tensors, rt)

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    defers_norm = True

    @property
    def takes_padding_rows(self) -> bool:
        """Token rows of no sequence (index -1) do no harm: the rotation skips them, attention gives them no job, and
        the products treat rows alone — if the position part agrees."""
        return bool(getattr(self.position, "takes_padding_rows", False))

    def step_plan(self, ctx, binding):
        """What of this step's launches depends on more than the step's padded shape (a recorded step is replayed
        only for a step with the same answer): the decode kernel's split and variant."""
        if not ctx.decode or self.rt.dtype != torch.bfloat16:
            return None
        g = binding.group
        S, P = ctx.pages_of(g).shape
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if g.page_size != 64 or not kernels.attention_decode_supported(hd, nh // nkv):
            return None
        return kernels.decode_plan_token(ctx, S, P, g.page_size, nkv, hd, nh // nkv)

    def forward(self, h, x, ctx, binding, then_norm=None) -> bool:
        T = h.shape[0]
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.rt.scratch("qkv", (T, (nh + 2 * nkv) * hd))
        kernels.linear(h, self.w_qkv, qkv, self.b_qkv)
        attn = self.rt.scratch("attn_out", (T, nh * hd))
        g = binding.group
        pages = ctx.pages_of(g)
        fused = self.position.fused_rotation()
        if fused is not None and kernels.attention_fuses_rotation(qkv, ctx, pages, g.page_size, nh, nkv, hd, fused[1], self.rt):
            rope = (fused[0], fused[1], binding.writes)        # a decode step: the attention kernel rotates and appends
        else:
            rope = None
            self.position.rotate_and_store(qkv, ctx, binding, nh, nkv, hd)
        kernels.attention(qkv, attn, g.k[binding.index], g.v[binding.index], ctx, pages, g.page_size,
                          nh, nkv, hd, self.scale, self.window, rt=self.rt, rope=rope)
        return kernels.linear(attn, self.w_o, x, None, kernels.OUT_ADD_F32, then_norm)


class _MapsAttention:
    """What the attention mixers below share: one product for the projections (fp32 rows), ``qkv_prepare`` (norms,
    rotation, cache append), attention over the call's pages, an optional join of the maps, the output projection.

    Sizes: ``heads`` query heads over ``kv_heads`` key/value heads (query head h reads kv head h // (heads /
    kv_heads)), ``maps`` score maps per head (query row [head][map][dim]; key heads [kv head][map]), one set of values
    of size ``vdim`` per kv head.  ``chunk`` > 0: a query at position p sees the keys of its own block of ``chunk``
    positions only (blocks counted from position 0); ``window`` > 0: the last ``window`` positions only.  A mixer with
    ``shares_kv`` has no key and value projections: its call reads the cache another call fills (``cache_of`` in the
    schedule) with its own queries."""
    maps = 1

    def _sizes(self, p):
        self.width, self.H, self.G = int(p["width"]), int(p["heads"]), int(p["kv_heads"])
        self.D, self.Dv = int(p["dim"]), int(p["vdim"])
        if self.H % self.G:
            raise ValueError(f"{self.kind}: heads must be a multiple of kv_heads")
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.chunk, self.window = int(p.get("chunk", 0)), int(p.get("window", 0))
        self.shares_kv = bool(p.get("shares_kv", False))

    @classmethod
    def _declare_projections(cls, p, maps):
        W, H, G, D, Dv = p["width"], p["heads"], p["kv_heads"], p["dim"], p["vdim"]
        d = {"q": TensorDecl((H * maps * D, W)), "o": TensorDecl((W, H * Dv))}
        if not p.get("shares_kv", False):
            d.update({"k": TensorDecl((G * maps * D, W)), "v": TensorDecl((G * Dv, W))})
        return d

    def _projections(self, tensors, rt):
        names = ("q",) if self.shares_kv else ("q", "k", "v")
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in names], dim=0))
        self.w_o = rt.to_compute(tensors["o"])

    def cache_request(self):
        return KVRequest(self.G * self.maps, self.D, self.window, True, self.G, self.Dv)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    @property
    def takes_padding_rows(self) -> bool:
        return True          # every kernel skips token rows of no sequence

    defers_norm = True       # the output projection can fill the norm behind the mixer (``then_norm``); the input is plain rows

    def _project_out(self, heads, x, store, then_norm) -> bool:
        if store:
            kernels.linear(heads, self.w_o, x, None, kernels.OUT_STORE_F32)
            return False
        return kernels.linear(heads, self.w_o, x, None, kernels.OUT_ADD_F32, then_norm)

    # what a subclass adds
    q_norm_w = k_norm_w = head_scale = None
    inv_freq, rot_dims = None, 0

    def _attend(self, h, ctx, binding):
        """-> attention output per map, [T, H*maps*Dv] (fp32 if there are several maps, else the compute type)."""
        T = h.shape[0]
        rt, H, G, M, D, Dv = self.rt, self.H, self.G, self.maps, self.D, self.Dv
        if binding.writes == self.shares_kv:
            raise ValueError(f"{self.kind}: a layer without key and value projections must read another call's cache, "
                             f"and only such a layer may")
        proj = rt.scratch("attn_proj", (T, self.w_in.shape[0]), torch.float32)
        kernels.linear(h, self.w_in, proj, None, kernels.OUT_STORE_F32)
        g = binding.group
        pages = ctx.pages_of(g)
        k_cache, v_cache = g.k[binding.index], g.v[binding.index]
        q = rt.scratch("attn_q", (T, H * M * D))
        kernels.qkv_prepare(proj, H * M, G * M, D, G, Dv, self.q_norm_w, self.k_norm_w, self.eps, self.inv_freq, self.rot_dims,
                            ctx, pages, g.page_size, k_cache, v_cache, q, has_kv=not self.shares_kv, write_kv=binding.writes)
        out = rt.scratch("attn_maps" if M > 1 else "attn_out", (T, H * M * Dv), torch.float32 if M > 1 else None)
        kernels.attention_maps(q, out, k_cache, v_cache, ctx, pages, g.page_size, H, G, M, D, Dv, self.scale, self.head_scale,
                               self.window, self.chunk, rt=rt)
        return out


@part("mixer", "diff_attention")
class DiffAttention(_MapsAttention):
    """Differential attention: two softmax maps per head over the same values, o = a1 - lam * a2 with one number lam
    for the layer, lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff; then o / rms(o) over the head's values (no weight)
    times (1 - diff), and the output projection.  Queries and keys are rotated by position on the first entries of
    every map (the position part's ``rotary_dim``).

    params: ``width``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``diff``, ``eps``, optional ``chunk``,
    ``window``, ``shares_kv``, ``position`` (a PartSpec of the position family).
    tensors: ``q`` [heads*2*dim, width], ``k`` [kv_heads*2*dim, width], ``v`` [kv_heads*vdim, width] (k, v absent with
    ``shares_kv``), ``lq1``, ``lk1``, ``lq2``, ``lk2`` [dim], ``o`` [width, heads*vdim]."""
    maps = 2

    @classmethod
    def declare(cls, spec):
        p = spec.params
        d = cls._declare_projections(p, 2)
        d.update({n: TensorDecl((p["dim"],), "bias") for n in ("lq1", "lk1", "lq2", "lk2")})
        d.update(nested_declare("position", p["position"]))
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self._sizes(p)
        self._projections(tensors, rt)
        self.diff = float(p["diff"])
        l = {n: tensors[n].double().cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = float(torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum()) + self.diff)
        self.position = nested_build("position", p["position"], tensors, rt)
        fused = self.position.fused_rotation()
        if fused is None:
            raise ValueError("diff_attention: the position part must be a rotation of pairs (or none)")
        self.inv_freq, self.rot_dims = fused
        if self.rot_dims > self.D:
            raise ValueError("diff_attention: the rotated part is larger than a map")

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        a = self._attend(h, ctx, binding)
        heads = self.rt.scratch("attn_out", (h.shape[0], self.H * self.Dv))
        kernels.diff_combine(a, self.lam, self.eps, 1.0 - self.diff, self.H, self.Dv, ctx, heads)
        return self._project_out(heads, x, store, then_norm)

    stores_output = True


@part("mixer", "qk_normed_attention")
class QKNormedAttention(_MapsAttention):
    """Attention without positions in its scores: q and k each pass an RMS norm over the WHOLE projected row (all heads
    at once, a weight per entry) and every head's scores are multiplied by a learned number of its own.

    params: ``width``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``eps``, optional ``chunk``, ``window``.
    tensors: ``q`` [heads*dim, width], ``k`` [kv_heads*dim, width], ``v`` [kv_heads*vdim, width], ``q.norm``
    [heads*dim], ``k.norm`` [kv_heads*dim], ``temp`` [heads], ``o`` [width, heads*vdim]."""

    @classmethod
    def declare(cls, spec):
        p = spec.params
        d = cls._declare_projections(p, 1)
        d.update({"q.norm": TensorDecl((p["heads"] * p["dim"],), "norm_scale"),
                  "k.norm": TensorDecl((p["kv_heads"] * p["dim"],), "norm_scale"),
                  "temp": TensorDecl((p["heads"],), "norm_scale")})
        return d

    def __init__(self, spec, tensors, rt, **_):
        self.rt = rt
        self._sizes(spec.params)
        if self.shares_kv:
            raise ValueError("qk_normed_attention: has key and value projections of its own")
        self._projections(tensors, rt)
        self.q_norm_w, self.k_norm_w = rt.to_f32(tensors["q.norm"]), rt.to_f32(tensors["k.norm"])
        self.head_scale = rt.to_f32(tensors["temp"])

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        return self._project_out(self._attend(h, ctx, binding), x, store, then_norm)

    stores_output = True


@part("mixer", "window_pool_attention")
class WindowPoolAttention(_MapsAttention):
    """Attention over a sliding window and, beside it, over one pooled key and value per block of positions that has
    left the window — optional pieces, each a parameter:

    * ``window`` (0: every earlier position) and ``pool`` (0: nothing beyond the window): the query at position p sees
      the positions j with 0 <= p - j < window and, for every block b of ``pool`` positions with b*pool + pool - 1 <=
      p - window, ONE key and ONE value: the means of the block's keys and values as the cache holds them (keys after
      the rotation).  Positions that have left the window and whose block is not complete before it are not seen.  All
      visible keys share one softmax.  The pooled rows live in cache pages of their own, one row per block
      (``more_cache_requests``), and are made when a block's last position arrives; the token pages are a windowed
      group, so pages that lie wholly before the window (and before the newest block) go back to the pool early.
    * ``values_from_keys``: there is no value projection; the values are the keys as projected, before the rotation.
    * ``gate``: head h's output is multiplied by logistic(W_g h)_h, one number per head from the mixer's input, before
      the output projection.
    * ``position``: a PartSpec of the position family whose ``inv_freq``, ``rotary_dim``, ``pairing`` and ``amplitude``
      the preparation kernel applies to q and k.

    params: ``width``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``window``, ``pool``, ``values_from_keys``,
    ``gate``, ``position``.  tensors: ``q`` [heads*dim, width], ``k`` [kv_heads*dim, width], ``v`` [kv_heads*vdim, width]
    (absent with ``values_from_keys``), ``g`` [heads, width] (with ``gate``), ``o`` [width, heads*vdim]."""

    @classmethod
    def declare(cls, spec):
        p = spec.params
        d = cls._declare_projections(p, 1)
        if p.get("values_from_keys", False):
            del d["v"]
        if p.get("gate", False):
            d["g"] = TensorDecl((p["heads"], p["width"]))
        d.update(nested_declare("position", p["position"]))
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = dict(spec.params)
        p.setdefault("eps", 0.0)
        self.rt = rt
        self._sizes(p)
        self.pool = int(p.get("pool", 0))
        self.values_from_keys = bool(p.get("values_from_keys", False))
        self.gated = bool(p.get("gate", False))
        if self.pool and not self.window:
            raise ValueError("window_pool_attention: pooled blocks lie before a window; without a window there are none")
        if self.values_from_keys and self.Dv != self.D:
            raise ValueError("window_pool_attention: values that are the keys have the keys' size")
        names = ["q", "k"] + ([] if self.values_from_keys else ["v"]) + (["g"] if self.gated else [])
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in names], dim=0))      # one product: [q | k | (v) | (gate)]
        self.w_o = rt.to_compute(tensors["o"])
        self.n_qkv = self.H * self.D + self.G * self.D + (0 if self.values_from_keys else self.G * self.Dv)
        self.position = nested_build("position", p["position"], tensors, rt)
        self.inv_freq, self.rot_dims = self.position.inv_freq, int(self.position.rotary_dim)
        if self.rot_dims > self.D:
            raise ValueError("window_pool_attention: the rotated part is larger than a head")

    def cache_request(self):
        # the newest block's positions must still be there when its last one arrives: the window of the pages is the
        # larger of the two
        window = max(self.window, self.pool) if self.window else 0
        return KVRequest(self.G, self.D, window, True, self.G, self.Dv)

    def more_cache_requests(self):
        if not self.pool:
            return {}
        return {"pooled": KVRequest(self.G, self.D, 0, True, self.G, self.Dv, every=self.pool)}

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        T = h.shape[0]
        rt, H, G, D, Dv = self.rt, self.H, self.G, self.D, self.Dv
        proj = rt.scratch("attn_proj", (T, self.w_in.shape[0]), torch.float32)
        kernels.linear(h, self.w_in, proj, None, kernels.OUT_STORE_F32)
        g = binding.group
        pages = ctx.pages_of(g)
        k_cache, v_cache = g.k[binding.index], g.v[binding.index]
        q = rt.scratch("attn_q", (T, H * D))
        kernels.qkv_prepare(proj, H, G, D, G, Dv, None, None, 0.0, self.inv_freq, self.rot_dims, ctx, pages, g.page_size,
                            k_cache, v_cache, q, has_kv=True, write_kv=binding.writes, pairing=self.position.pairing,
                            amplitude=float(self.position.amplitude), v_from_k=self.values_from_keys)
        pooled = None
        if self.pool:
            pb = binding.more["pooled"]
            pg = pb.group
            k_pool, v_pool, pool_pages = pg.k[pb.index], pg.v[pb.index], ctx.pages_of(pg)
            if binding.writes:
                kernels.pool_rows(k_cache, v_cache, pages, k_pool, v_pool, pool_pages, g.page_size, self.pool, ctx)
            pooled = (self.pool, k_pool, v_pool, pool_pages)
        gate = proj[:, self.n_qkv:] if self.gated else None
        out = rt.scratch("attn_out", (T, H * Dv))
        kernels.attention_maps(q, out, k_cache, v_cache, ctx, pages, g.page_size, H, G, 1, D, Dv, self.scale, None,
                               self.window, 0, rt=rt, pooled=pooled, gate=gate)
        return self._project_out(out, x, store, then_norm)

    stores_output = True


@part("mixer", "gated_attention")
class GatedAttention(_MapsAttention):
    """Softmax attention of grouped queries with optional pieces, each a parameter:

    * ``bias``: the q, k, v and output projections have biases (the tensor's name + ``.b``);
    * ``conv`` (taps; 0: none): a short causal convolution over time on every channel of q, k and v, right behind the
      projection: y[t] = sum_j w[:, j] * u[t - taps + 1 + j], zeros before the sequence's start, no bias, the input itself
      not added.  The last taps - 1 projected rows of a sequence are kept in the cache's state slab (fp32);
    * ``qk_norm``: an RMS norm over the WHOLE q row and the whole k row (all heads at once, a plain weight per entry),
      before the rotation;
    * ``position``: a PartSpec of the position family whose rotation of pairs the preparation kernel applies to the first
      entries of every q and k head;
    * ``softcap`` (0: none): a score s becomes softcap * tanh(s / softcap) before the softmax;
    * ``chunk`` / ``window``: the keys a query sees (see :class:`_MapsAttention`);
    * ``gate``: every output entry is multiplied by logistic(W_g h) of its own, before the output projection.

    params: ``width``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``eps`` (of the q and k norms), and the
    above.  tensors: ``q`` [heads*dim, width], ``k`` [kv_heads*dim, width], ``v`` [kv_heads*vdim, width], ``o`` [width,
    heads*vdim]; with ``bias`` ``q.b``, ``k.b``, ``v.b``, ``o.b``; with ``conv`` ``q.conv``, ``k.conv``, ``v.conv``
    [channels, taps]; with ``qk_norm`` ``q.norm``, ``k.norm``; with ``gate`` ``g`` [heads*vdim, width]."""
    stores_output = True
    defers_norm = False

    @classmethod
    def declare(cls, spec):
        p = spec.params
        d = cls._declare_projections(p, 1)
        H, G, D, Dv, W = p["heads"], p["kv_heads"], p["dim"], p["vdim"], p["width"]
        if p.get("bias", False):
            d.update({"q.b": TensorDecl((H * D,), "bias"), "k.b": TensorDecl((G * D,), "bias"),
                      "v.b": TensorDecl((G * Dv,), "bias"), "o.b": TensorDecl((W,), "bias")})
        if p.get("conv", 0):
            K = p["conv"]
            d.update({"q.conv": TensorDecl((H * D, K)), "k.conv": TensorDecl((G * D, K)), "v.conv": TensorDecl((G * Dv, K))})
        if p.get("qk_norm", False):
            d.update({"q.norm": TensorDecl((H * D,), "norm_scale"), "k.norm": TensorDecl((G * D,), "norm_scale")})
        if p.get("gate", False):
            d["g"] = TensorDecl((H * Dv, W))
        if p.get("position") is not None:
            d.update(nested_declare("position", p["position"]))
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = dict(spec.params)
        p.setdefault("eps", 0.0)
        self.rt = rt
        self._sizes(p)
        if self.shares_kv:
            raise ValueError("gated_attention: has key and value projections of its own")
        H, G, D, Dv = self.H, self.G, self.D, self.Dv
        self.n_qkv = H * D + G * D + G * Dv
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.gated = bool(p.get("gate", False))
        self.taps = int(p.get("conv", 0) or 0)
        names = ["q", "k", "v"] + (["g"] if self.gated else [])
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in names], dim=0))       # one product: [q | k | v | (gate)]
        self.w_o = rt.to_compute(tensors["o"])
        self.b_in = self.b_o = None
        if p.get("bias", False):
            parts = [tensors["q.b"].float(), tensors["k.b"].float(), tensors["v.b"].float()]
            if self.gated:
                parts.append(torch.zeros(H * Dv, dtype=torch.float32, device=parts[0].device))
            self.b_in, self.b_o = rt.to_f32(torch.cat(parts)), rt.to_f32(tensors["o.b"])
        self.conv_w = None
        if self.taps:        # [taps, channels]: neighbouring channels side by side, the oldest tap first
            self.conv_w = rt.to_f32(torch.cat([tensors[n + ".conv"] for n in ("q", "k", "v")], dim=0)).t().contiguous()
        if p.get("qk_norm", False):
            self.q_norm_w, self.k_norm_w = rt.to_f32(tensors["q.norm"]), rt.to_f32(tensors["k.norm"])
        self.pairing, self.amplitude = 0, 1.0
        if p.get("position") is not None:
            self.position = nested_build("position", p["position"], tensors, rt)
            self.inv_freq, self.rot_dims = self.position.inv_freq, int(self.position.rotary_dim)
            self.pairing, self.amplitude = int(self.position.pairing), float(self.position.amplitude)
            if self.rot_dims > D:
                raise ValueError("gated_attention: the rotated part is larger than a head")

    def more_cache_requests(self):
        if self.taps <= 1:
            return {}
        return {"conv": StateRequest(((self.taps - 1) * self.n_qkv,), torch.float32)}

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        T = h.shape[0]
        rt, H, G, D, Dv = self.rt, self.H, self.G, self.D, self.Dv
        proj = rt.scratch("attn_proj", (T, self.w_in.shape[0]), torch.float32)
        kernels.linear(h, self.w_in, proj, self.b_in, kernels.OUT_STORE_F32)
        qkv = proj
        if self.taps:
            qkv = rt.scratch("attn_conv", (T, self.n_qkv), torch.float32)
            if self.taps > 1:
                cb = binding.more["conv"]
                carry = cb.group.data[cb.index]
            else:
                carry = rt.scratch("attn_conv_none", (1, 1), torch.float32)
            if ctx.decode and self.taps > 1:      # single tokens: the convolution and its state's update in one kernel
                kernels.conv_token(proj[:, :self.n_qkv], self.conv_w, carry, ctx, qkv, write_state=binding.writes)
            else:
                kernels.conv_add(proj[:, :self.n_qkv], self.conv_w, carry, ctx, qkv, write_state=binding.writes, add_input=False)
        g = binding.group
        pages = ctx.pages_of(g)
        k_cache, v_cache = g.k[binding.index], g.v[binding.index]
        q = rt.scratch("attn_q", (T, H * D))
        kernels.qkv_prepare(qkv, H, G, D, G, Dv, self.q_norm_w, self.k_norm_w, self.eps, self.inv_freq, self.rot_dims, ctx, pages,
                            g.page_size, k_cache, v_cache, q, has_kv=True, write_kv=binding.writes, pairing=self.pairing,
                            amplitude=self.amplitude)
        out = rt.scratch("attn_out", (T, H * Dv))
        kernels.attention_maps(q, out, k_cache, v_cache, ctx, pages, g.page_size, H, G, 1, D, Dv, self.scale, None,
                               self.window, self.chunk, rt=rt, gate=proj[:, self.n_qkv:] if self.gated else None,
                               softcap=self.softcap)
        kernels.linear(out, self.w_o, x, self.b_o, kernels.OUT_STORE_F32 if store else kernels.OUT_ADD_F32)
        return False
