"""Feed-forward ``routed_experts``: a mixture of small feed-forwards of which every token runs a few.

Router logits z = W_r h in fp32; the ``top`` experts with the largest logits are chosen (ties: the lower index) and
weighted by the softmax over the CHOSEN logits only; the output is the weighted sum of the chosen experts' outputs,
each W_down (act(W_gate h) * (W_up h)) without biases, summed in the order of the choice.

Variations, each a parameter: ``scoring`` ``logistic_normalised`` — scores s = logistic(z), the ``top`` largest scores
are chosen and weighted by s / (sum of the chosen s + 1e-20); ``groups`` = (count, keep) — the experts form ``count``
equal runs of neighbours, a run's score is the sum of its two largest scores, and only experts of the ``keep`` best runs
can be chosen; ``gated`` False — experts without a gate matrix, W_down act(W_up h); ``shared`` — one more expert of the
same form (inner size ``shared``) that every token runs, added times logistic(W_sg h), one number per token;
``scoring`` ``softmax_all`` — scores s = the softmax over ALL router outputs, the choice goes by s + ``correction`` (a
stored number per router output), the weights are the chosen s times ``scale``, not normalised; ``identity`` = n — the
router has n outputs beyond the experts, each standing for an expert without tensors whose output is its input.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, part


@part("ffn", "routed_experts")
class RoutedExperts:
    """params: ``width``, ``inner`` (of one expert), ``experts``, ``top``, optional ``activation`` (``silu``,
    ``gelu_tanh``, ``relu2``; default ``silu``), ``gated`` (default True), ``scoring`` (``softmax_chosen``,
    ``logistic_normalised``, ``softmax_all``), ``groups`` ((count, keep) or None), ``shared`` (inner size of the shared
    expert; 0: none), ``scale`` (of ``softmax_all``; default 1), ``identity`` (router outputs beyond the experts; default 0).
    tensors: ``router`` [experts + identity, width], with ``softmax_all`` ``correction`` [experts + identity], and per expert i ``e<i>.gate`` (if gated), ``e<i>.up`` [inner, width],
    ``e<i>.down`` [width, inner]; with a shared expert ``shared.up`` [shared, width], ``shared.down`` [width, shared]
    and ``shared.sg`` [1, width]."""
    takes_padding_rows = True       # the router marks token rows of no sequence; they get zeros
    stores_output = True

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, F = p["width"], p["inner"]
        d = {}
        for i in range(p["experts"]):
            if p.get("gated", True):
                d[f"e{i}.gate"] = TensorDecl((F, W))
            d.update({f"e{i}.up": TensorDecl((F, W)), f"e{i}.down": TensorDecl((W, F))})
        n_out = p["experts"] + int(p.get("identity", 0) or 0)
        d["router"] = TensorDecl((n_out, W))
        if p.get("scoring") == "softmax_all":
            d["correction"] = TensorDecl((n_out,), "bias")
        if p.get("shared", 0):
            S = p["shared"]
            d.update({"shared.up": TensorDecl((S, W)), "shared.down": TensorDecl((W, S)), "shared.sg": TensorDecl((1, W))})
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width, self.inner, self.E, self.top = int(p["width"]), int(p["inner"]), int(p["experts"]), int(p["top"])
        activation = p.get("activation", "silu")
        if activation not in kernels.EXPERT_ACTIVATIONS:
            raise ValueError(f"routed_experts: unknown activation {activation!r}")
        self.act = kernels.EXPERT_ACTIVATIONS[activation]
        self.gated = bool(p.get("gated", True))
        if self.gated == (activation in ("relu2", "gelu")):
            raise ValueError("routed_experts: gated experts take silu or gelu_tanh, experts without a gate relu2 or gelu")
        self.plain_act = kernels.PLAIN_ACTIVATION_MODES[kernels.PLAIN_ACTIVATIONS[activation]] if not self.gated else None
        scoring = p.get("scoring", "softmax_chosen")
        if scoring not in kernels.ROUTE_MODES:
            raise ValueError(f"routed_experts: unknown scoring {scoring!r} (known: {sorted(kernels.ROUTE_MODES)})")
        self.route_mode = kernels.ROUTE_MODES[scoring]
        self.identity = int(p.get("identity", 0) or 0)
        self.route_scale = float(p.get("scale", 1.0))
        if self.identity and self.route_mode != kernels.ROUTE_SOFTMAX_ALL:
            raise ValueError("routed_experts: experts that hand their input on come with the scoring softmax_all")
        self.n_out = self.E + self.identity            # router outputs
        if not (1 <= self.top <= self.n_out):
            raise ValueError("routed_experts: top must be between 1 and the number of router outputs")
        self.correction = rt.to_f32(tensors["correction"]) if self.route_mode == kernels.ROUTE_SOFTMAX_ALL else None
        self.n_groups, self.keep = (int(v) for v in (p.get("groups") or (0, 0)))
        if self.n_groups and (self.E % self.n_groups or not (1 <= self.keep <= self.n_groups)
                              or self.keep * (self.E // self.n_groups) < self.top):
            raise ValueError("routed_experts: the groups must divide the experts, and the kept ones hold at least `top` experts")
        self.shared = int(p.get("shared", 0))
        if self.shared and self.gated:
            raise ValueError("routed_experts: a shared expert has the form of experts without a gate matrix")
        router = tensors["router"]
        if self.shared:      # the shared expert's gate rides on the router's product: one more row of logits
            router = torch.cat([router, tensors["shared.sg"].reshape(1, self.width)], dim=0)
            self.w_shared_up, self.w_shared_down = rt.to_compute(tensors["shared.up"]), rt.to_compute(tensors["shared.down"])
        self.w_router = rt.to_compute(router)
        self.w_gate = rt.to_compute(torch.stack([tensors[f"e{i}.gate"] for i in range(self.E)])) if self.gated else None
        self.w_up = rt.to_compute(torch.stack([tensors[f"e{i}.up"] for i in range(self.E)]))
        self.w_down = rt.to_compute(torch.stack([tensors[f"e{i}.down"] for i in range(self.E)]))

    def weight_bytes(self) -> int:
        ws = [self.w_router, self.w_up, self.w_down] + ([self.w_gate] if self.gated else [])
        if self.shared:
            ws += [self.w_shared_up, self.w_shared_down]
        return sum(t.numel() * t.element_size() for t in ws)

    def forward(self, h, x, ctx, store: bool = False) -> bool:
        T = h.shape[0]
        rt = self.rt
        logits = rt.scratch("router_logits", (T, self.w_router.shape[0]), torch.float32)
        kernels.linear(h, self.w_router, logits, None, kernels.OUT_STORE_F32)
        idx = rt.scratch("router_choice", (T, self.top), torch.int32)
        wt = rt.scratch("router_weight", (T, self.top), torch.float32)
        id_wt = rt.scratch("router_identity", (T,), torch.float32) if self.identity else None
        kernels.moe_route(logits, self.top, ctx, idx, wt, self.route_mode, self.n_groups, self.keep, experts=self.n_out,
                          correction=self.correction, scale=self.route_scale, identity=self.identity, id_wt=id_wt)
        if kernels.moe_grouped_applies(h, self.width, self.inner, self.E):
            # (what the chosen experts without tensors add — the token's input times their summed weight — joins the sum there)
            kernels.moe_experts_grouped(h, self.w_gate, self.w_up, self.w_down, idx, wt, self.act, rt, x, add=not store, id_wt=id_wt)
        else:
            a = rt.scratch("experts_act", (T, self.top, self.inner), torch.float32)
            kernels.moe_experts_streamed(h, self.w_gate, self.w_up, self.w_down, idx, wt, self.act, a, x, add=not store)
            if self.identity:
                kernels.moe_identity_add(h, id_wt, x)
        if self.shared:      # every token's expert: x += logistic(z_sg) * W_down act(W_up h); the gate scales the activation rows
            sa = rt.scratch("shared_act", (T, self.shared))
            kernels.linear(h, self.w_shared_up, sa, None, self.plain_act)
            kernels.gate_rows(sa, logits[:, self.n_out:])
            kernels.linear(sa, self.w_shared_down, x, None, kernels.OUT_ADD_F32)
        return False
