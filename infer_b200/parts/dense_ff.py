"""Dense feed-forward with one hidden layer: out = residual + act(x Wup^T) Wdown^T, no biases; with ``gated`` the
hidden layer is act(x Wgate^T) * (x Wup^T) (gate and up are one matrix product).

``activation``: "gelu_tanh" is 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); "relu_squared" is max(z, 0)^2.  ``names`` renames the matrices
(roles up, down, gate).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import FeedForward, own_or_projected, register_feed_forward
from .linear import Linear

_ACTIVATIONS = {"gelu_tanh": ops.gelu_tanh, "relu_squared": ops.relu_sq}        # each: (rows, first column, width) -> contiguous [T, width]
_NAMES = {"up": "up_proj.weight", "down": "down_proj.weight", "gate": "gate_proj.weight"}


@register_feed_forward("dense")
class DenseFeedForward(FeedForward):
    accepts_deferred_norm = True

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        if self.hidden <= 0 or self.inter <= 0:
            raise ValueError("a dense feed-forward needs positive sizes")
        act = spec.get("activation", "gelu_tanh")
        if act not in _ACTIVATIONS:
            raise ValueError(f"activation {act!r} is not among {sorted(_ACTIVATIONS)}")
        self.activation, self.act_name = _ACTIVATIONS[act], act
        self.gated = bool(spec.get("gated", False))
        self.up = self.down = None

    @classmethod
    def param_shapes(cls, spec):
        H, I = int(spec["hidden_size"]), int(spec["intermediate_size"])
        n = {**_NAMES, **dict(spec.get("names") or {})}
        shapes = {n["up"]: (I, H), n["down"]: (H, I)}
        if spec.get("gated", False):
            shapes[n["gate"]] = (I, H)
        return shapes

    def load(self, params):
        n = {**_NAMES, **dict(self.spec.get("names") or {})}
        # gated: result rows [gate | up]
        self.up = Linear(self.rt, torch.cat([params[n["gate"]], params[n["up"]]], dim=0) if self.gated else params[n["up"]])
        self.down = Linear(self.rt, params[n["down"]])

    def input_product(self):
        return self.up, "compute"

    def drop_input_product(self):
        self.up = None

    def forward(self, x, residual):
        rows, c0 = own_or_projected(self, x, self.up)
        if self.gated:
            act = ops.glu_act(rows, c0, c0 + self.inter, self.inter, self.act_name)
        else:
            act = self.activation(rows, c0, self.inter)
        if residual is None:
            return self.down(act, out_dtype=torch.float32)
        return self.down(act, residual=residual)
