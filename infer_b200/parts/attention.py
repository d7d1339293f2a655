"""Grouped-query causal attention over the paged cache.

q = x Wq^T + bq, k = x Wk^T + bk, v = x Wv^T + bv (one matrix product over the concatenated rows
[Wq; Wk; Wv], as the reference lays them out on the device, kernels/model_gpu.cu:31-34); positions are
encoded into q and k; k and v go to the request's pages; query head h reads kv head h / (heads /
kv_heads); score = (q . k) * scale with scale = 1/sqrt(head_dim) unless given; keys j <= p, and
j > p - window if the layer has a window; softmax in float32; out = residual + ctx Wo^T
(src/forward.cpp:101-136,208-224; kernels/ops/batch.cu:207-316).

Options beyond that, each a key of the part's spec (absent = off):

``v_head_dim``      values of another size than keys (the value pages and the context rows follow it)
``filter_taps``     q, k and v each pass a causal filter over time, per channel, directly after the projection:
                    y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence; the last taps - 1 projected
                    rows of a request are state beside its pages (``CompositeNeed``)
``position``        kind "rotary_pairs": adjacent channel pairs over the first ``rotary_dims`` channels of a head
``value_norm_eps``  every value head is divided by sqrt(mean(v^2) + eps) before it is cached
``head_gate``       head h's context is multiplied by sigmoid(x Wg^T)[h] before the output product; Wg's rows ride
                    in the same matrix product as q, k and v
``qk_row_norm_eps`` ALL of a token's q channels (every head at once) are divided by their root mean square and
                    multiplied by a weight per channel (role q_norm, [heads * head_dim]); k likewise (k_norm); no
                    rotation follows. One kernel normalises and fills the pages
``distance_bias``   {"buckets": B or None, "max_distance": D}: a learned table (role rel, [B, heads]; B is read from
                    the tensor when the spec gives None) whose row bucket(i - j) is added to the scaled score of query i
                    and key j: bucket(n) = n below B // 2, then logarithmic steps that reach the last row at n = D
``sink``            a learned logit per head (role sink, [heads]) that enters the softmax denominator only
``names``           local tensor names by role (q, k, v, o, q_bias, k_bias, v_bias, q_filter, k_filter, v_filter, gate,
                    q_norm, k_norm, rel, sink) for checkpoints that call them otherwise

A third group of options goes through one kernel that normalises per head, rotates, applies the temperature and
fills the pages (``head_prepare``), then through the attention kernels that take a slope and kept first keys:

``qk_head_norm_eps``   EVERY q head and every k head is divided by its own root mean square over head_dim and
                       multiplied by a weight [head_dim] that the heads share (roles q_norm, k_norm), before any
                       rotation; ``position`` may then be "rotary_interpolated" in the pairs layout (or none)
``query_temperature``  {"coef": c, "every": n}: q at position p is multiplied by 1 + c ln(floor((p + 1) / n) + 1)
``distance_slopes``    a number per head: slope_h * (i - j) is taken off the scaled score of query i and key j
``keep_first``         with a window: query i also sees every key j < keep_first (at its true position)
``values_are_keys``    there is no v matrix: a position's value is its key as projected, before norm and rotation
``channel_gate``       the joined heads are multiplied, channel by channel, by sigmoid(x Wg^T) (role gate,
                       [heads * v_head_dim, hidden]) before the output product; Wg rides in the q/k/v product
``sink``               as above
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import CompositeNeed, Mixer, PagedKVNeed, ProjectedInput, StateNeed, build_part, own_or_projected, register_mixer
from .linear import Linear

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
          "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
          "q_filter": "q_proj.filter", "k_filter": "k_proj.filter", "v_filter": "v_proj.filter", "gate": "gate_proj.weight",
          "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "rel": "distance_bias.weight", "sink": "sinks"}


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


def log_bucket(n: int, buckets: int, max_distance: float) -> int:
    """Row of a distance-bias table of ``buckets`` rows for a distance n >= 0: one row per distance below
    buckets // 2, then logarithmic steps up to ``max_distance``, where the last row is reached."""
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(max_distance / half) * (buckets - half))))


def distance_bias_table(rel: torch.Tensor, max_distance: float, window: Optional[int]) -> torch.Tensor:
    """float32 [L, heads]: row n is the bias of distance n, the last row that of every larger distance (a window
    bounds the distances that are ever asked for)."""
    B = rel.shape[0]
    if B < 2 or not max_distance > B // 2:
        raise ValueError(f"a distance bias of {B} rows needs max_distance above {B // 2}, got {max_distance}")
    rows, n = [], 0
    while True:
        b = log_bucket(n, B, max_distance)
        rows.append(b)
        if b == B - 1 or (window is not None and n + 1 >= window):
            break
        n += 1
    return rel.float()[torch.tensor(rows, dtype=torch.long)].contiguous()


@register_mixer("attention")
class Attention(Mixer):
    accepts_deferred_norm = True

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.n_kv, self.head_dim = int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        self.v_dim = int(spec.get("v_head_dim") or self.head_dim)
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.window = spec.get("window")
        if self.window is not None:
            self.window = int(self.window)
            if self.window <= 0:
                raise ValueError("an attention window must be positive (or None for all keys)")
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError(f"heads ({self.n_heads}) must be a multiple of kv heads ({self.n_kv})")
        if self.head_dim <= 0:
            raise ValueError(f"head_dim must be positive, got {self.head_dim}")
        if max(self.head_dim, self.v_dim) > ops.attention_max_head_dim():
            raise ValueError(f"head_dim {self.head_dim} / {self.v_dim} is beyond what the attention kernels take ({ops.attention_max_head_dim()})")
        scale = spec.get("softmax_scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(self.head_dim))
        pos = spec.get("position")
        self.position = build_part("position", pos, runtime) if pos is not None else None
        self.taps = int(spec.get("filter_taps") or 0)
        self.value_norm_eps = spec.get("value_norm_eps")
        self.head_gate = bool(spec.get("head_gate", False))
        # anything beyond rotate-and-store goes through the prepare kernel (filter, pair rotation, value norm)
        if getattr(self.position, "layout", "half") == "half" and self.position is not None and self.head_dim % 2:
            raise ValueError(f"half-split rotation needs an even head_dim, got {self.head_dim}")
        self.prepared = (self.taps > 0 or self.value_norm_eps is not None or self.v_dim != self.head_dim or self.head_gate
                         or getattr(self.position, "layout", "half") == "pairs")
        # (row norms, distance bias and sink have a path of their own, decided below: its kernels ask for no other library)
        self.head_norm_eps = spec.get("qk_head_norm_eps")
        self.q_temp = dict(spec["query_temperature"]) if spec.get("query_temperature") else None
        self.slopes = [float(v) for v in spec["distance_slopes"]] if spec.get("distance_slopes") is not None else None
        self.keep_first = int(spec.get("keep_first") or 0)
        self.values_are_keys = bool(spec.get("values_are_keys", False))
        self.channel_gate = bool(spec.get("channel_gate", False))
        self.per_head = (self.head_norm_eps is not None or self.q_temp is not None or self.slopes is not None or self.keep_first > 0
                         or self.values_are_keys or self.channel_gate)
        if self.per_head:
            self._check_per_head(spec)
        own_path = self.per_head or spec.get("qk_row_norm_eps") is not None or spec.get("distance_bias") is not None or bool(spec.get("sink", False))
        if self.prepared and not own_path:
            if max(self.head_dim, self.v_dim) > ops.qkv_prepare_max_head_dim():
                raise ValueError(f"the prepare kernel takes head sizes up to {ops.qkv_prepare_max_head_dim()}, "
                                 f"got {self.head_dim} / {self.v_dim}")
            if self.position is not None and getattr(self.position, "layout", None) != "pairs":
                raise ValueError("filters, value norm, gates and other value sizes go with position kind 'rotary_pairs' (or none)")
        self.row_norm_eps = spec.get("qk_row_norm_eps")
        self.distance_bias = spec.get("distance_bias")
        self.has_sink = bool(spec.get("sink", False))
        self.row_norm = self.row_norm_eps is not None
        if self.per_head:
            self.prepared = self.biased = False
        elif self.row_norm or self.distance_bias is not None or self.has_sink:
            # these scores are not the ones the fast kernels compute; the projected rows go through the row-norm kernel
            if self.taps > 0 or self.position is not None or self.value_norm_eps is not None or self.head_gate:
                raise ValueError("row norms, distance bias and sinks do not combine with filters, rotation, value norm or head gates")
            if self.row_norm and float(self.row_norm_eps) <= 0:
                raise ValueError("qk_row_norm_eps must be positive")
            self.prepared = False
            self.biased = True
        else:
            self.biased = False
        self.q_norm_w = self.k_norm_w = self.bias_table = self.bias_by_head = self.sink_w = self.slopes_w = None
        self.n_qkv = (self.n_heads + self.n_kv) * self.head_dim + (0 if self.values_are_keys else self.n_kv * self.v_dim)
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.filter_w = None

    def _check_per_head(self, spec):
        if self.taps > 0 or self.value_norm_eps is not None or self.head_gate or self.qkv_bias or spec.get("qk_row_norm_eps") is not None \
                or spec.get("distance_bias") is not None:
            raise ValueError("per-head norms, temperature, slopes, kept first keys, keys as values and channel gates do not combine "
                             "with filters, value norm, head gates, biases, row norms or a distance table")
        if self.head_norm_eps is not None and float(self.head_norm_eps) <= 0:
            raise ValueError("qk_head_norm_eps must be positive")
        if self.position is not None and (getattr(self.position, "layout", None) != "pairs" or self.position.rotary_tables is None):
            raise ValueError("this attention rotates channel pairs from tables (position kind 'rotary_interpolated' or 'rotary_pairs' in the pairs layout)")
        if self.q_temp is not None and (int(self.q_temp.get("every", 0)) <= 0 or "coef" not in self.q_temp):
            raise ValueError("query_temperature needs 'coef' and a positive 'every'")
        if self.slopes is not None and len(self.slopes) != self.n_heads:
            raise ValueError(f"distance_slopes needs one number per head ({self.n_heads}), got {len(self.slopes)}")
        if self.keep_first < 0 or (self.keep_first > 0 and self.window is None):
            raise ValueError("keep_first goes with a window")
        if self.values_are_keys and self.v_dim != self.head_dim:
            raise ValueError("values that are the keys have the keys' size")

    @classmethod
    def param_shapes(cls, spec):
        H, nh, nkv, hd = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        vd = int(spec.get("v_head_dim") or hd)
        n = _names(spec)
        shapes = {n["q"]: (nh * hd, H), n["k"]: (nkv * hd, H), n["v"]: (nkv * vd, H), n["o"]: (H, nh * vd)}
        if spec.get("values_are_keys", False):
            del shapes[n["v"]]
        if spec.get("channel_gate", False):
            shapes[n["gate"]] = (nh * vd, H)
        if spec.get("qk_head_norm_eps") is not None:
            shapes.update({n["q_norm"]: (hd,), n["k_norm"]: (hd,)})
        if spec.get("qkv_bias", False):
            shapes.update({n["q_bias"]: (nh * hd,), n["k_bias"]: (nkv * hd,), n["v_bias"]: (nkv * vd,)})
        taps = int(spec.get("filter_taps") or 0)
        if taps > 0:
            shapes.update({n["q_filter"]: (nh * hd, taps), n["k_filter"]: (nkv * hd, taps), n["v_filter"]: (nkv * vd, taps)})
        if spec.get("head_gate", False):
            shapes[n["gate"]] = (nh, H)
        if spec.get("qk_row_norm_eps") is not None:
            shapes.update({n["q_norm"]: (nh * hd,), n["k_norm"]: (nkv * hd,)})
        db = spec.get("distance_bias")
        if db is not None:
            shapes[n["rel"]] = (int(db["buckets"]) if db.get("buckets") is not None else -1, nh)
        if spec.get("sink", False):
            shapes[n["sink"]] = (nh,)
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        if name in (n["q_filter"], n["k_filter"], n["v_filter"]):
            # taps that keep a channel's scale: about one on the newest tap, small ones before
            w = 0.3 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
            w[:, -1] += 1.0
            return w
        if name in (n["q_norm"], n["k_norm"]):
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        if name in (n["rel"], n["sink"]):
            return torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        mats = [params[n["q"]], params[n["k"]]] + ([] if self.values_are_keys else [params[n["v"]]])
        if self.head_gate or self.channel_gate:
            mats.append(params[n["gate"]])
        w = torch.cat(mats, dim=0)
        if self.head_gate and w.shape[0] % 8:
            # rows of the product's result stay 16-byte aligned for the kernels that read them
            w = torch.cat([w, torch.zeros(8 - w.shape[0] % 8, w.shape[1], dtype=w.dtype, device=w.device)], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([params[n["q_bias"]].float(), params[n["k_bias"]].float(), params[n["v_bias"]].float()])
            if w.shape[0] > b.numel():
                b = torch.cat([b, torch.zeros(w.shape[0] - b.numel(), device=b.device)])
        self.qkv = Linear(self.rt, w, b)
        self.o = Linear(self.rt, params[n["o"]])
        f32 = dict(device=self.rt.device, dtype=torch.float32)
        if self.head_norm_eps is not None:
            self.q_norm_w, self.k_norm_w = params[n["q_norm"]].to(**f32).contiguous(), params[n["k_norm"]].to(**f32).contiguous()
        if self.slopes is not None:
            self.slopes_w = torch.tensor(self.slopes, **f32)
        if self.row_norm:
            self.q_norm_w, self.k_norm_w = params[n["q_norm"]].to(**f32).contiguous(), params[n["k_norm"]].to(**f32).contiguous()
        if self.distance_bias is not None:
            self.bias_table = distance_bias_table(params[n["rel"]], float(self.distance_bias["max_distance"]), self.window).to(**f32).contiguous()
            # for the tensor-core kernel: a head's biases side by side, divided by the scale (added to the raw score)
            self.bias_by_head = (self.bias_table / self.scale).t().contiguous() if self.scale > 0 else None
        if self.has_sink:
            self.sink_w = params[n["sink"]].to(**f32).contiguous()
        if self.taps > 0:
            # tap-major [taps, channels]: the prepare kernel reads neighbouring channels' taps side by side
            self.filter_w = torch.cat([params[n["q_filter"]], params[n["k_filter"]], params[n["v_filter"]]], dim=0) \
                .to(device=self.rt.device, dtype=torch.float32).t().contiguous()

    def cache_need(self):
        pages = PagedKVNeed(self.n_kv, self.head_dim, self.window, None if self.v_dim == self.head_dim else self.v_dim,
                            keep_first=self.keep_first if self.window is not None else 0)
        if self.taps > 1:
            # the last taps - 1 projected rows of the request, in the compute dtype (copies, not sums)
            return CompositeNeed({"pages": pages, "tails": StateNeed({"qkv": ((self.taps - 1, self.n_qkv), None)})})
        return pages

    def _context(self, q, cache, table, step):
        ctx = None
        if self.rt.fast("attention") and self.v_dim == self.head_dim:
            from .. import fast_ops
            ctx = fast_ops.attention(q, cache, table, step, self.n_heads, self.n_kv, self.head_dim, self.window, self.scale)
        if ctx is None:
            ctx = ops.attention_plain(q, cache.k, cache.v, table, step.token_seg, step.positions, self.n_heads, self.n_kv,
                                      self.head_dim, self.window, self.scale, step.status, self.v_dim)
        return ctx

    def _project_out(self, ctx, residual):
        if residual is None:
            return self.o(ctx, out_dtype=torch.float32)
        return self.o(ctx, residual=residual)

    def input_product(self):
        """The q/k/v(/gate) product, for a block that joins the products of parts reading the same rows. Only the
        prepared path reads its rows by (leading dimension, first column)."""
        return (self.qkv, "compute") if (self.prepared or self.biased or self.per_head) else None

    def drop_input_product(self):
        self.qkv = None

    def _forward_biased(self, qkv, col0, step, cache, residual, write_cache):
        """Row norms of q and k with the cache write in one kernel; then attention whose scores take the distance
        bias and whose denominator takes the sink."""
        table = step.block_tables[cache.group]
        q = ops.rownorm_store(qkv, col0, self.q_norm_w, self.k_norm_w, float(self.row_norm_eps or 0.0), step, table,
                              cache.k, cache.v, self.n_heads, self.n_kv, self.head_dim, self.v_dim, write_cache)
        ctx = None
        if self.rt.fast("attention"):
            ctx = ops.attention_window(q, cache.k, cache.v, table, step, self.n_heads, self.n_kv, self.head_dim, self.v_dim,
                                       self.window, self.scale, self.bias_table, self.sink_w, self.bias_by_head)
        if ctx is None:
            ctx = ops.attention_plain(q, cache.k, cache.v, table, step.token_seg, step.positions, self.n_heads, self.n_kv,
                                      self.head_dim, self.window, self.scale, step.status, self.v_dim, self.bias_table, self.sink_w)
        return self._project_out(ctx, residual)

    def _forward_per_head(self, qkv, col0, step, cache, residual, write_cache):
        """Per-head norms, pair rotation, the queries' temperature and the cache write in one kernel; attention whose
        scores lose a slope times the distance, whose window keeps the first keys and whose denominator takes the sink;
        the gate per channel. The part's columns [q | k | (v) | gate] start at ``col0`` of the rows ``qkv``."""
        table = step.block_tables[cache.group]
        cos = sin = None
        n_rot = 0
        if self.position is not None:
            cos, sin = self.position.rotary_tables(self.rt.max_seq_len)
            n_rot = self.position.rotary_dims
        coef, every = (float(self.q_temp["coef"]), int(self.q_temp["every"])) if self.q_temp is not None else (0.0, 0)
        q = ops.head_prepare(qkv, col0, self.q_norm_w, self.k_norm_w, float(self.head_norm_eps or 0.0), cos, sin, n_rot, coef, every,
                             self.values_are_keys, step, table, cache.k, cache.v, self.n_heads, self.n_kv, self.head_dim, self.v_dim,
                             write_cache)
        ctx = None
        if self.rt.fast("attention") and step.max_q_len <= 1 and self.n_heads // self.n_kv <= ops.ATTENTION_SPLIT_GROUP_MAX:
            # single tokens only: the kernel that merges a token's key chunks also applies the gate
            ctx = ops.attention_split(q, cache.k, cache.v, table, step, self.n_heads, self.n_kv, self.head_dim, self.v_dim, self.window,
                                      self.scale, None, self.sink_w, keep_first=self.keep_first, slopes=self.slopes_w,
                                      gate=qkv if self.channel_gate else None, gate_col=col0 + self.n_qkv)
            return self._project_out(ctx, residual)
        if self.rt.fast("attention"):
            ctx = ops.attention_window(q, cache.k, cache.v, table, step, self.n_heads, self.n_kv, self.head_dim, self.v_dim,
                                       self.window, self.scale, None, self.sink_w, None, self.keep_first, self.slopes_w)
        if ctx is None:
            ctx = ops.attention_plain(q, cache.k, cache.v, table, step.token_seg, step.positions, self.n_heads, self.n_kv,
                                      self.head_dim, self.window, self.scale, step.status, self.v_dim, None, self.sink_w,
                                      keep_first=self.keep_first, slopes=self.slopes_w)
        if self.channel_gate:
            ops.gate_mul(ctx, qkv, col0 + self.n_qkv)
        return self._project_out(ctx, residual)

    def forward(self, x, step, cache, residual, write_cache=True):
        if self.per_head:
            qkv, col0 = own_or_projected(self, x, self.qkv)
            return self._forward_per_head(qkv, col0, step, cache, residual, write_cache)
        if self.biased:
            qkv, col0 = own_or_projected(self, x, self.qkv)
            return self._forward_biased(qkv, col0, step, cache, residual, write_cache)
        if self.prepared:
            qkv, col0 = own_or_projected(self, x, self.qkv)
            return self._forward_prepared(qkv, col0, step, cache, residual, write_cache)
        if isinstance(x, ProjectedInput):
            x = x.rows_in
        qkv = self.qkv(x)                                              # [T, (heads + 2 kv) * head_dim]
        table = step.block_tables[cache.group]
        tables = self.position.rotary_tables(self.rt.max_seq_len) if self.position is not None else None
        if self.position is not None and tables is None:
            T = qkv.shape[0]
            q_view = qkv[:, : self.n_heads * self.head_dim].view(T, self.n_heads, self.head_dim)
            k_view = qkv[:, self.n_heads * self.head_dim: (self.n_heads + self.n_kv) * self.head_dim].view(T, self.n_kv, self.head_dim)
            self.position.apply(q_view, k_view, step.positions)
        cos, sin = tables if tables is not None else (None, None)
        if step.decode_only and cos is not None and self.rt.fast("rope") and self.rt.fast("attention"):
            # one token per request: rotation, cache write and attention in one kernel
            from .. import fast_ops
            ctx = fast_ops.attention_decode_fused(qkv, cos, sin, cache.k, cache.v, table, step.seg_start, step.seg_pos0,
                                                  self.n_heads, self.n_kv, self.head_dim, self.window, self.scale,
                                                  step.max_ctx_len, write_cache)
            if ctx is not None:
                return self._project_out(ctx, residual)
        q = ops.rope_kv_write(qkv, cos, sin, step.positions, step.token_seg, table, cache.k, cache.v,
                              self.n_heads, self.n_kv, self.head_dim, write_cache, step.status)
        return self._project_out(self._context(q, cache, table, step), residual)

    def _forward_prepared(self, qkv, col0, step, cache, residual, write_cache):
        """Filter, pair rotation and value norm in one kernel that also fills the pages; then the filter's tails take
        the step's last projected rows, attention runs over the pages, and the heads are gated. The part's columns
        [q | k | v | gates] start at ``col0`` of the rows ``qkv``."""
        pages = cache["pages"] if isinstance(cache, dict) else cache
        tails = cache["tails"]["qkv"] if isinstance(cache, dict) else None
        table = step.block_tables[pages.group]
        cos = sin = None
        n_rot = 0
        if self.position is not None:
            cos, sin = self.position.rotary_tables(self.rt.max_seq_len)
            n_rot = self.position.rotary_dims
        # with one token per request, the thread that filters a channel is the only reader of its tail and moves it too
        inline_tail = tails is not None and write_cache and step.max_q_len == 1
        q = ops.qkv_prepare(qkv, self.filter_w, tails, cos, sin, n_rot, self.value_norm_eps is not None,
                            float(self.value_norm_eps or 0.0), step, table, pages.k, pages.v, self.n_heads, self.n_kv,
                            self.head_dim, self.v_dim, write_cache, col0, inline_tail)
        if tails is not None and write_cache and not inline_tail:
            ops.filter_tail_update(qkv, col0, tails, step.seg_start, step.seg_slot)
        ctx = self._context(q, pages, table, step)
        if self.head_gate:
            ops.head_gate(ctx, qkv, col0 + self.n_qkv, self.n_heads, self.v_dim)
        return self._project_out(ctx, residual)
