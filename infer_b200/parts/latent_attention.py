"""Attention through low-rank latents: a position leaves one row behind for all heads.

    cq = rmsnorm(Wdq x) * wq                       query latent [q_rank]
    q  = Wuq cq                                    per head [head_dim unrotated | rot_dim rotated]
    [kv | r] = Wdkv x;  c = rmsnorm(kv) * wkv      kv latent [kv_rank]; r [rot_dim]: ONE rotated key part for all heads
    head h:  k_h = Wuk_h c,  v_h = Wuv_h c
    score_h(i, j) = (q_h[:head_dim] . k_h(j) + rotate(q_h[head_dim:], i) . rotate(r(j), j)) * softmax_scale
    keys j <= i, and i - j < window if the layer has one; softmax in float32
    out = Wo concat_h(sigmoid(Wg x)[h] * sum_j p_h(i, j) v_h(j)) * out_scale            (gate optional)

The pages hold [c | rotate(r)] per position and nothing else (``PagedKVNeed(values_in_keys=True)``: one row serves as
key and as value). Attention runs in the latent space: q_h[:head_dim] is carried through Wuk_h once
(q_lat = [Wuk_h^T q_plain | rotate(q_rot)], ``ops.latent_query``), the score is q_lat . [c | r], the context is the
weighted sum of the c rows, and Wuv_h is applied to that sum (``ops.latent_output``). Cost per (query, key, head):
kv_rank + rot_dim multiply-adds for the score and kv_rank for the value, whatever head_dim and v_head_dim are; no
per-head key or value is ever formed for a cached position.

That is the form for decoded tokens, which meet every cached row once. A prompt portion of n tokens meets every row n
times, and pays for the latent width each time; for portions (bfloat16, sizes that are multiples of 8) the rows that
the step's portions can see are gathered out of the pages, one matrix product with [Wuk; Wuv] forms the per-head keys
and values of those rows, and a tensor-core kernel runs ordinary attention over them (``ops.latent_gather``,
``ops.latent_prefill``): head_dim + rot_dim and v_head_dim multiply-adds per (query, key, head). Single tokens in
the same step keep the latent form; both write the same rows. Which form a token takes depends on the lengths of the
step's segments alone, and the two differ by rounding only.

Spec keys: hidden_size, num_heads, head_dim, rot_dim, v_head_dim, q_rank, kv_rank, softmax_scale, norm_eps,
``position`` (a position part with ``rotary_tables`` / ``layout`` / ``rotary_dims``, or None), ``window`` (None: all
earlier positions), ``head_gate``, ``out_scale`` (a constant on the result, applied to the gated contexts in float32
before the output product: a block's residual multiplier costs nothing this way), ``own_latent`` (False: the layer
has no Wdkv and reads the rows another layer of the same kv_rank, rot_dim and rotation wrote; the run order names
that layer's cache with write_cache False), ``cache_window`` (how long rows must stay: the largest window of the
layers that read this cache; default ``window``), ``names`` (tensor names by role).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, PagedKVNeed, build_part, register_mixer
from .linear import Linear

PORTION_MIN_TOKENS = 4
PORTION_MAX_BYTES = 2 << 30

_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o"}


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        g = lambda k: int(spec[k])
        self.hidden, self.n_heads, self.head_dim, self.rot_dim = g("hidden_size"), g("num_heads"), g("head_dim"), g("rot_dim")
        self.v_dim, self.q_rank, self.kv_rank = g("v_head_dim"), g("q_rank"), g("kv_rank")
        if min(self.hidden, self.n_heads, self.head_dim, self.v_dim, self.q_rank, self.kv_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent_attention needs positive sizes")
        self.scale = float(spec["softmax_scale"])
        self.eps = float(spec["norm_eps"])
        if self.eps <= 0:
            raise ValueError("latent_attention needs a positive norm_eps")
        self.window = int(spec["window"]) if spec.get("window") is not None else None
        if self.window is not None and self.window <= 0:
            raise ValueError("an attention window must be positive (or None for all keys)")
        cw = spec.get("cache_window", self.window)
        self.cache_window = int(cw) if cw is not None else None
        if self.window is None and self.cache_window is not None or \
                (self.window is not None and self.cache_window is not None and self.cache_window < self.window):
            raise ValueError("cache_window must cover the layer's own window")
        self.head_gate = bool(spec.get("head_gate", False))
        self.own_latent = bool(spec.get("own_latent", True))
        self.out_scale = float(spec.get("out_scale", 1.0))
        pos = spec.get("position")
        self.position = build_part("position", pos, runtime) if pos is not None else None
        if self.position is not None:
            if getattr(self.position, "layout", None) not in ops.ROTATION_LAYOUTS:
                raise ValueError("latent_attention needs a rotation that states its layout ('pairs' or 'half') and gives tables")
            if int(self.position.rotary_dims) > self.rot_dim:
                raise ValueError(f"{self.position.rotary_dims} rotated channels do not fit a shared key part of {self.rot_dim}")
        self.dk = self.kv_rank + self.rot_dim
        max_dk, max_dv = ops.latent_attention_max_dims() if runtime is not None and torch.cuda.is_available() else (1024, 512)
        if self.dk > max_dk or self.kv_rank > max_dv:
            raise ValueError(f"latent rows of {self.kv_rank} + {self.rot_dim} are beyond what the attention kernel takes ({max_dv} + rest up to {max_dk})")
        self.down = self.uq = self.o = self.up_kv = None
        self.portion_build = None
        self.w_uk = self.w_uvT = self.wq = self.wkv = None
        self.q_col = self.kv_col = self.gate_col = 0

    @classmethod
    def param_shapes(cls, spec):
        W, H, d, dr, dv = (int(spec[k]) for k in ("hidden_size", "num_heads", "head_dim", "rot_dim", "v_head_dim"))
        rq, rkv = int(spec["q_rank"]), int(spec["kv_rank"])
        n = _names(spec)
        shapes = {n["dq"]: (rq, W), n["dq_norm"]: (rq,), n["uq"]: (H * (d + dr), rq), n["uk"]: (H * d, rkv), n["uv"]: (H * dv, rkv),
                  n["o"]: (W, H * dv)}
        if spec.get("own_latent", True):
            shapes.update({n["dkv"]: (rkv + dr, W), n["dkv_norm"]: (rkv,)})
        if spec.get("head_gate", False):
            shapes[n["gate"]] = (H, W)
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        if name in (n["dq_norm"], n["dkv_norm"]):
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        # the latents are normalised to unit mean square: up-projections of N(0, 1 / rank) keep that scale
        if name in (n["uq"], n["uk"], n["uv"]):
            return torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device) / float(shape[1]) ** 0.5
        if name == n["gate"]:
            return 0.5 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        # The down-projections (and the gate) read the same rows: one product, float32 results, since they feed norms
        # and a sigmoid. Every part's columns start on a multiple of 8.
        mats, col = [], 0

        def add(w):
            nonlocal col
            start = col
            mats.append(w)
            pad = (-w.shape[0]) % 8
            if pad:
                mats.append(torch.zeros(pad, w.shape[1], dtype=w.dtype, device=w.device))
            col += w.shape[0] + pad
            return start
        self.q_col = add(params[n["dq"]])
        if self.own_latent:
            self.kv_col = add(params[n["dkv"]])
        if self.head_gate:
            self.gate_col = add(params[n["gate"]])
        self.down = Linear(self.rt, torch.cat(mats, dim=0))
        self.uq = Linear(self.rt, params[n["uq"]])
        self.o = Linear(self.rt, params[n["o"]])
        dev = dict(device=self.rt.device, dtype=self.rt.dtype)
        self.w_uk = params[n["uk"]].to(**dev).contiguous()                                   # [heads * head_dim, kv_rank]
        self.w_uvT = params[n["uv"]].to(**dev).view(self.n_heads, self.v_dim, self.kv_rank).transpose(1, 2).contiguous()
        if self.rt.dtype == torch.bfloat16 and self.rot_dim > 0:
            self.portion_build = ops.latent_portion_build(self.head_dim, self.rot_dim, self.v_dim, self.kv_rank)
        if self.portion_build is not None:
            self.up_kv = Linear(self.rt, torch.cat([params[n["uk"]], params[n["uv"]]], dim=0))   # [heads * (head_dim + v_dim), kv_rank]
        f32 = dict(device=self.rt.device, dtype=torch.float32)
        self.wq = params[n["dq_norm"]].to(**f32).contiguous()
        self.wkv = params[n["dkv_norm"]].to(**f32).contiguous() if self.own_latent else None

    def cache_need(self):
        return PagedKVNeed(1, self.dk, self.cache_window, self.kv_rank, values_in_keys=True)

    def _portion_span(self, step, table, pages) -> int:
        """Rows per portion for the form with per-head keys and values, or 0 where the step takes the latent form for
        all its tokens: no build for these sizes, fewer than PORTION_MIN_TOKENS tokens in portions (forming the keys
        of a long context costs more than a few queries over its latent rows), or regions beyond PORTION_MAX_BYTES.
        Only what a captured step keeps fixed enters: the segments' lengths and the table's width."""
        if self.portion_build is None or step.max_q_len <= 1:
            return 0
        portions = [n for n in step.seg_lens if n > 1]
        if sum(portions) < PORTION_MIN_TOKENS:
            return 0
        span = table.shape[1] * pages.shape[1]
        if self.window is not None:
            span = min(span, self.window - 1 + max(portions))
        width = self.n_heads * (self.head_dim + self.v_dim) + self.dk
        if len(portions) * span * width * 2 > PORTION_MAX_BYTES:
            return 0
        return span

    def forward(self, x, step, cache, residual, write_cache=True):
        if write_cache and not self.own_latent:
            raise ValueError("a latent_attention layer without its own kv latent cannot write a cache")
        rows = self.down(x, out_dtype=torch.float32)
        table = step.block_tables[cache.group]
        pages = cache.k.view(cache.k.shape[0], cache.k.shape[2], self.dk)               # one kv head: [pages, page_size, dk]
        cos = sin = None
        layout = "pairs"
        if self.position is not None:
            cos, sin = self.position.rotary_tables(self.rt.max_seq_len)
            layout = self.position.layout
        cq = ops.latent_prepare(rows, self.q_col, self.q_rank, self.kv_col, self.kv_rank, self.rot_dim, self.wq, self.wkv, self.eps,
                                cos, sin, layout, step, table, pages, self.rt.dtype, write_cache and self.own_latent)
        q = self.uq(cq)
        gates = rows if self.head_gate else None
        span = self._portion_span(step, table, pages)
        if span:
            # portions: per-head keys and values of the rows they can see, ordinary attention on the tensor cores
            n_portions = sum(1 for n in step.seg_lens if n > 1)
            c_rows, r_rows = ops.latent_gather(pages, table, step, n_portions, span, self.window, self.kv_rank, self.portion_build)
            kv = self.up_kv(c_rows)
            heads = ops.latent_prefill(q, cos, sin, layout, kv, self.n_heads * self.head_dim, r_rows, gates, self.gate_col, self.out_scale,
                                       step, span, self.n_heads, self.head_dim, self.rot_dim, self.v_dim, self.window, self.scale,
                                       self.portion_build)
            if any(n == 1 for n in step.seg_lens):
                q_lat = ops.latent_query(q, self.w_uk, cos, sin, layout, step.positions, self.n_heads, self.head_dim, self.rot_dim, step)
                ctx = ops.latent_attention(q_lat, pages, table, step, self.kv_rank, self.window, self.scale, single_only=True)
                ops.latent_output(ctx, self.w_uvT, gates, self.gate_col, self.out_scale, heads, step)
        else:
            q_lat = ops.latent_query(q, self.w_uk, cos, sin, layout, step.positions, self.n_heads, self.head_dim, self.rot_dim)
            ctx = ops.latent_attention(q_lat, pages, table, step, self.kv_rank, self.window, self.scale)
            heads = ops.latent_output(ctx, self.w_uvT, gates, self.gate_col, self.out_scale)
        if residual is None:
            return self.o(heads, out_dtype=torch.float32)
        return self.o(heads, residual=residual)
