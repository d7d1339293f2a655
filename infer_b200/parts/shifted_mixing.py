"""Time mixing over mixtures of a token's row with its predecessor's (the RWKV form with a decay per key channel and
token, and a bonus for the current token).

With h the mixer's input row at a position and h' the row of the token before it (zeros before the sequence), each of
the five projections reads its own mixture m_s = h + (h' - h) * mu_s:

    r = m_r Wr^T,  k = m_k Wk^T,  v = m_v Wv^T        per head [dim]
    gate = silu(m_g Wg^T)
    w = exp(-exp(tanh(m_w W1^T) W2^T + w0))           a decay per head and key channel, through a low rank
    o = (S + diag(u) k v^T)^T r                       the current token is read through the bonus u only
    S <- diag(w) S + k v^T                            S [dim, dim], zero for a new request

Every head's o is divided by its root mean square (eps inside the root); the heads are joined, multiplied by a weight
per channel and by the gate, and projected by Wo.  S (float32) and the last row h of the request (float32) are the
request's state.  The mixtures are formed from the float32 residual stream (``reads_stream``); r, k, v and the low
rank's first factor are matrix products with float32 result rows; tanh, the second factor, both exponentials, the
state and the norms are float32 whatever the compute dtype.

The rank of the decay's low-rank product is ``decay_rank`` in the spec, or, with None, what the stored tensors have.
``names`` renames the local tensors by role (mu_r, mu_k, mu_v, mu_g, mu_w, r, k, v, gate, decay_low, decay_up,
decay_bias, bonus, norm, o).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear

_NAMES = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k", "v": "v", "gate": "g",
          "decay_low": "w1", "decay_up": "w2", "decay_bias": "w0", "bonus": "u", "norm": "norm", "o": "o"}
_MIXES = ("r", "k", "v", "g", "w")


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


@register_mixer("shifted_decay_mixing")
class ShiftedDecayMixing(Mixer):
    reads_stream = True

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.dim = int(spec["num_heads"]), int(spec["head_dim"])
        self.eps = float(spec["norm_eps"])
        if min(self.hidden, self.n_heads, self.dim) <= 0 or self.eps <= 0:
            raise ValueError("shifted_decay_mixing needs positive sizes and eps")
        if self.dim > ops.state_scan_max_dim():
            raise ValueError(f"a key size of {self.dim} is beyond what the recurrence kernel keeps in registers ({ops.state_scan_max_dim()})")
        self.rank = 0
        self.o: Optional[Linear] = None

    @classmethod
    def param_shapes(cls, spec):
        H, nh, d = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["head_dim"])
        r = int(spec["decay_rank"]) if spec.get("decay_rank") is not None else -1
        n = _names(spec)
        C = nh * d
        shapes = {n["mu_" + s]: (H,) for s in _MIXES}
        shapes.update({n["r"]: (C, H), n["k"]: (C, H), n["v"]: (C, H), n["gate"]: (C, H), n["decay_low"]: (r, H), n["decay_up"]: (C, r),
                       n["decay_bias"]: (C,), n["bonus"]: (nh, d), n["norm"]: (C,), n["o"]: (H, C)})
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        kw = dict(generator=gen, dtype=torch.float32, device=gen.device)
        if name in [n["mu_" + s] for s in _MIXES]:
            return torch.rand(shape, **kw)
        if name == n["norm"]:
            return 1.0 + 0.1 * torch.randn(shape, **kw)
        if name == n["decay_bias"]:
            return -1.5 + torch.randn(shape, **kw)
        if name == n["bonus"]:
            return 0.5 * torch.randn(shape, **kw)
        if name in (n["decay_low"], n["decay_up"], n["r"], n["k"], n["v"]):
            return 0.3 * torch.randn(shape, **kw)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        f32 = dict(device=self.rt.device, dtype=torch.float32)
        self.mu = torch.stack([params[n["mu_" + s]].float() for s in _MIXES]).to(**f32).contiguous()      # [5, hidden]
        self.lin = {s: Linear(self.rt, params[n[role]]) for s, role in (("r", "r"), ("k", "k"), ("v", "v"), ("g", "gate"), ("w", "decay_low"))}
        low, up = params[n["decay_low"]], params[n["decay_up"]]
        self.rank = int(low.shape[0])
        if up.shape[1] != self.rank:
            raise ValueError(f"the two factors of the decay's low-rank product disagree: {tuple(low.shape)} and {tuple(up.shape)}")
        # the second factor keeps the values the checkpoint has, widened: its product runs in float32
        self.up = up.to(self.rt.dtype).to(**f32).t().contiguous()              # [rank, channels]
        self.up_bias = params[n["decay_bias"]].to(**f32).contiguous()
        self.bonus = params[n["bonus"]].to(**f32).contiguous()
        self.norm_w = params[n["norm"]].to(**f32).contiguous()
        self.o = Linear(self.rt, params[n["o"]])

    def cache_need(self):
        return StateNeed({"S": ((self.n_heads, self.dim, self.dim), torch.float32), "last": ((self.hidden,), torch.float32)})

    def forward(self, x, step, cache, residual, write_cache=True):
        if x.dtype != torch.float32:
            raise TypeError("shifted_decay_mixing reads the float32 rows of the residual stream")
        T, C = x.shape[0], self.n_heads * self.dim
        mixes = ops.shift_mix(x, cache["last"], self.mu, step, self.rt.dtype, write_cache)          # [5, T, hidden]
        rkv = torch.empty((3, T, C), dtype=torch.float32, device=x.device)
        # In a decode step every kernel is a few microseconds of latency: the five products read five different
        # mixtures and write nothing in common, so two of them and the decays go to a side stream beside the other three.
        from .block import PARALLEL_BRANCHES, _side_streams
        side = _side_streams(x.device)[1] if (PARALLEL_BRANCHES and step.decode_only and self.rt.dtype != torch.float32) else None
        if side is not None:
            main = torch.cuda.current_stream(x.device)
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                low = self.lin["w"](mixes[4], out_dtype=torch.float32)
                decay = ops.double_exp_decay(low, 0, self.rank, self.up, self.up_bias)
                gate = self.lin["g"](mixes[3])
                done = torch.cuda.Event()
                done.record(side)
        for i, s in enumerate(("r", "k", "v")):
            self.lin[s](mixes[i], out=rkv[i])
        if side is not None:
            main.wait_event(done)
        else:
            gate = self.lin["g"](mixes[3])
            low = self.lin["w"](mixes[4], out_dtype=torch.float32)
            decay = ops.double_exp_decay(low, 0, self.rank, self.up, self.up_bias)
        o = ops.state_scan(ops.SCAN_BONUS, rkv, (0, 0), (1, 0), (2, 0), decay, 0, cache["S"], step.seg_start, step.seg_slot,
                           self.n_heads, 1, self.dim, self.dim, write_cache, step.max_q_len, bonus=self.bonus)
        y = ops.group_norm_gate(o, self.norm_w, self.eps, gate, 0, "silu", self.n_heads, self.dim, self.rt.dtype)
        if residual is None:
            return self.o(y, out_dtype=torch.float32)
        return self.o(y, residual=residual)
