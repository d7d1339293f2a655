"""Mixture of experts: every token runs ``top`` of ``experts`` small gated feed-forwards, chosen by a router, and
optionally a shared expert that every token runs.

    s = softmax(x Wr^T) over all experts                          (float32)
    experts form ``groups`` equal groups of neighbours; a group's score is its largest s; only experts of the
    ``keep`` best groups can be chosen; of those, the ``top`` largest s are chosen
    weight_e = s_e / (sum of the chosen s + sum_eps)
    expert(x) = Wd (g' * sigmoid(slope * g') * (u' + 1)),  g' = min(x Wg^T, limit),  u' = clamp(x Wu^T, -limit, limit)
    out = sum over the chosen e of weight_e * expert_e(x)  +  shared(x)          (shared: the same form, own size and limit)

All experts' gate and up matrices (and the shared expert's) are one matrix product on the step's rows; the activation
kernel multiplies an expert's hidden values by the token's weight for that expert, which is zero for an expert the
token does not use; one product with the experts' down matrices side by side then sums the chosen experts. Every
expert's matrices are read once per step whatever the routing, which is what a batch of decoding requests or a prompt
portion does anyway; the multiply-adds of experts a token does not use are spent for nothing (experts / top times the
needed ones).

Tensors: ``router`` [experts, hidden]; per expert i ``e<i>.gate``, ``e<i>.up`` [ff, hidden], ``e<i>.down`` [hidden, ff];
``shared.gate`` / ``shared.up`` / ``shared.down`` likewise. No biases.

Other forms, each a key of the spec:

``router_kind``  "softmax_groups" (above) or "sigmoid": s = sigmoid(x Wr^T); the ``top`` experts with the largest
                 s + correction are chosen (``correction`` [experts], a stored tensor that only the choice sees);
                 weight_e = s_e as it is, not renormalised; no groups. "softmax_top": the ``top`` experts with the
                 largest logits are chosen and their weights are the softmax over the chosen logits only (which is
                 what the form above gives without groups and with sum_eps 0); no groups
``expert_kind``  "clipped_swish_glu" (above), "relu_squared": expert(x) = Wd relu(Wu x)^2, no gate matrix, no limit, or
                 "swish_glu": expert(x) = Wd (g sigmoid(g) * u) with g = Wg x, u = Wu x, no limit
``out_scale``    a constant on the result (default 1), multiplied into the experts' weights in float32: a block's
                 residual multiplier costs nothing this way
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import FeedForward, register_feed_forward
from .linear import Linear


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_experts, self.top = int(spec["hidden_size"]), int(spec["experts"]), int(spec["top"])
        self.groups, self.keep = int(spec.get("groups") or 1), int(spec.get("keep") or 1)
        self.ff, self.limit = int(spec["expert_size"]), float(spec.get("limit") or 0.0)
        self.shared_ff = int(spec.get("shared_size") or 0)
        self.shared_limit = float(spec.get("shared_limit") or 0.0)
        self.slope, self.sum_eps = float(spec.get("slope", 1.702)), float(spec.get("sum_eps", 1e-20))
        self.router_kind = str(spec.get("router_kind", "softmax_groups"))
        self.expert_kind = str(spec.get("expert_kind", "clipped_swish_glu"))
        self.out_scale = float(spec.get("out_scale", 1.0))
        if self.router_kind == "softmax_top":
            if self.groups != 1 or self.keep != 1:
                raise ValueError("a softmax_top router has no groups")
            self.sum_eps = 0.0
        if self.router_kind not in ("softmax_groups", "sigmoid", "softmax_top") or \
                self.expert_kind not in ("clipped_swish_glu", "relu_squared", "swish_glu"):
            raise ValueError(f"routed_experts: unknown router_kind {self.router_kind!r} or expert_kind {self.expert_kind!r}")
        if self.router_kind == "sigmoid" and (self.groups != 1 or self.keep != 1):
            raise ValueError("a sigmoid router has no groups")
        if self.out_scale != 1.0 and (self.router_kind != "sigmoid" or self.shared_ff):
            raise ValueError("out_scale goes into the weights of a sigmoid router and does not reach a shared expert")
        self.correction = None
        if min(self.hidden, self.n_experts, self.top, self.groups, self.keep, self.ff) <= 0 or self.shared_ff < 0:
            raise ValueError("routed_experts needs positive sizes")
        if self.n_experts % self.groups or self.keep > self.groups or self.top > self.keep * (self.n_experts // self.groups):
            raise ValueError(f"{self.n_experts} experts in {self.groups} groups, {self.keep} kept: {self.top} cannot be chosen")
        self.router = self.gate_up = self.down = None

    @classmethod
    def param_shapes(cls, spec):
        H, E, F, Fs = int(spec["hidden_size"]), int(spec["experts"]), int(spec["expert_size"]), int(spec.get("shared_size") or 0)
        gated = str(spec.get("expert_kind", "clipped_swish_glu")) != "relu_squared"
        shapes = {"router": (E, H)}
        if str(spec.get("router_kind", "softmax_groups")) == "sigmoid":
            shapes["correction"] = (E,)
        for u, f in [(f"e{i}", F) for i in range(E)] + ([("shared", Fs)] if Fs else []):
            shapes.update({u + ".up": (f, H), u + ".down": (H, f)})
            if gated:
                shapes[u + ".gate"] = (f, H)
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        if name == "router":
            return 0.5 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        if name == "correction":
            return 0.2 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)

    def load(self, params):
        E = self.n_experts
        shared = ["shared"] if self.shared_ff else []
        units = [f"e{i}" for i in range(E)] + shared
        self.router = Linear(self.rt, params["router"])
        if self.router_kind == "sigmoid":
            self.correction = params["correction"].to(device=self.rt.device, dtype=torch.float32).contiguous()
        self.width = E * self.ff + self.shared_ff
        if self.expert_kind == "relu_squared":
            self.gate_up = Linear(self.rt, torch.cat([params[u + ".up"] for u in units], dim=0))
            self.down = Linear(self.rt, torch.cat([params[u + ".down"] for u in units], dim=1))
            return
        # result rows [gate of expert 0 | .. | gate of the shared expert | up of expert 0 | .. | up of the shared expert]
        self.gate_up = Linear(self.rt, torch.cat([params[u + ".gate"] for u in units] + [params[u + ".up"] for u in units], dim=0))
        self.down = Linear(self.rt, torch.cat([params[u + ".down"] for u in units], dim=1))
        self.width = E * self.ff + self.shared_ff

    def forward(self, x, residual):
        logits = self.router(x, out_dtype=torch.float32)
        if self.router_kind == "sigmoid":
            weights, _ = ops.route_sigmoid(logits, self.correction, self.top, self.out_scale)
        else:
            weights, _ = ops.route(logits, self.top, self.groups, self.keep, self.sum_eps)
        rows = self.gate_up(x)
        if self.expert_kind == "relu_squared":
            if self.shared_ff:
                raise NotImplementedError("a shared expert of the relu_squared form")
            act = ops.scaled_relu_sq(rows, weights, self.ff)
        else:
            act = ops.glu_act(rows, 0, self.width, self.width, "swish" if self.expert_kind == "swish_glu" else "clipped_swish",
                              self.limit, self.shared_limit, self.slope, weights, self.ff, self.n_experts)
        if residual is None:
            return self.down(act, out_dtype=torch.float32)
        return self.down(act, residual=residual)
