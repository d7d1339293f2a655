"""Linear attention whose state fades by a constant of the head (lightning attention).

Per head, with x the mixer's input row at a position:

    q = silu(x Wq^T),  k = silu(x Wk^T)          [dim]
    v = silu(x Wv^T)                             [v_dim]
    S <- decay_h S + k v^T                       S [dim, v_dim], zero for a new request
    o = S^T q                                    [v_dim]  (the read-out sees the token's own write; no other scale)

The heads are joined, divided by ONE root mean square over all heads * v_dim channels (eps inside the root) and multiplied
by a weight per channel, then by sigmoid(x Wg^T), and projected by Wo.  S lives in float32 in a state slot of the
request and is carried from step to step.  The four projections are one matrix product with float32 result rows; the
activations, the state, the norm and the gate are float32 whatever the compute dtype.

``decay`` in the spec: one number per head.  ``names`` renames the local tensors by role (q, k, v, gate, o, norm).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, StateNeed, own_or_projected, register_mixer
from .linear import Linear

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight", "o": "o_proj.weight",
          "norm": "norm.weight"}


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


@register_mixer("constant_decay_attention")
class ConstantDecayAttention(Mixer):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.dim = int(spec["num_heads"]), int(spec["head_dim"])
        self.v_dim = int(spec.get("v_head_dim") or self.dim)
        self.eps = float(spec["norm_eps"])
        self.decay = [float(v) for v in spec["decay"]]
        if min(self.hidden, self.n_heads, self.dim, self.v_dim) <= 0 or self.eps <= 0:
            raise ValueError("constant_decay_attention needs positive sizes and eps")
        if len(self.decay) != self.n_heads:
            raise ValueError(f"constant_decay_attention needs one decay per head ({self.n_heads}), got {len(self.decay)}")
        if self.dim > ops.state_scan_max_dim():
            raise ValueError(f"a key size of {self.dim} is beyond what the recurrence kernel keeps in registers ({ops.state_scan_max_dim()})")
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None

    @classmethod
    def param_shapes(cls, spec):
        H, nh, d = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["head_dim"])
        dv = int(spec.get("v_head_dim") or d)
        n = _names(spec)
        return {n["q"]: (nh * d, H), n["k"]: (nh * d, H), n["v"]: (nh * dv, H), n["gate"]: (nh * dv, H), n["o"]: (H, nh * dv),
                n["norm"]: (nh * dv,)}

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        if name == n["norm"]:
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        if name in (n["q"], n["k"], n["v"]):
            return 0.3 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        # result rows [q | k | v | gate], float32
        self.proj = Linear(self.rt, torch.cat([params[n[r]] for r in ("q", "k", "v", "gate")], dim=0))
        f32 = dict(device=self.rt.device, dtype=torch.float32)
        self.decay_w = torch.tensor(self.decay, dtype=torch.float64).to(**f32).contiguous()
        self.norm_w = params[n["norm"]].to(**f32).contiguous()
        self.o = Linear(self.rt, params[n["o"]])

    def cache_need(self):
        return StateNeed({"S": ((self.n_heads, self.dim, self.v_dim), torch.float32)})

    def input_product(self):
        return self.proj, "float32"

    def drop_input_product(self):
        self.proj = None

    def forward(self, x, step, cache, residual, write_cache=True):
        nq, nv = self.n_heads * self.dim, self.n_heads * self.v_dim
        rows, c0 = own_or_projected(self, x, self.proj, torch.float32)
        # prompt portions: the activation in a pass of its own, so that the scan copies its rows as they lie, a chunk
        # ahead; steps of a few tokens per request: inside the scan's staging (one launch less; the same arithmetic)
        in_scan = step.max_q_len < ops.SCAN_SPREAD_FROM
        if not in_scan:
            ops.silu_rows(rows, c0, 2 * nq + nv)
        o = ops.state_scan(ops.SCAN_HEAD_DECAY, rows, c0, c0 + nq, c0 + 2 * nq, self.decay_w, 0, cache["S"], step.seg_start,
                           step.seg_slot, self.n_heads, 1, self.dim, self.v_dim, write_cache, step.max_q_len, silu=in_scan)
        y = ops.group_norm_gate(o, self.norm_w, self.eps, rows, c0 + 2 * nq + nv, "sigmoid", 1, nv, self.rt.dtype)
        if residual is None:
            return self.o(y, out_dtype=torch.float32)
        return self.o(y, residual=residual)
