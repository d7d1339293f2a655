"""Arrangements of parts into a layer. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(src/forward.cpp:200-244), over the slots mixer_norm, mixer, feed_forward_norm, feed_forward (the last two may be
absent together: a layer without feed-forward). The residual stream h is float32; the sums happen in the parts'
last matrix product, in float32.

"parallel_gated": ONE norm, whose rows n = norm(h) every sublayer reads, and one sum:
h += sigmoid(G1 n + g1) * mixer(n) + sigmoid(G2 n + g2) * feed_forward(n); the feed-forward (and its gate) may be
absent. Slots: norm, mixer, gate (family "gate": the logits of both gates in one product), feed_forward. A mixer
that is two mixers side by side hands over both results and their constants, so that the weighing, the gating and
the residual sum are one float32 kernel.

"sublayer_norm": the sublayers read the residual stream h itself and the norm sits on what they RETURN:
h += norm_a(mixer(h)); h += norm_b(feed_forward(h)); the feed-forward and its norm may be absent. Slots: mixer,
mixer_out_norm, feed_forward, feed_forward_out_norm. Norm and sum are one float32 kernel, which also leaves h in the
compute dtype for the next sublayer's first matrix product.

"postnorm": the norm comes AFTER the sum and its result IS the stream: h <- norm_a(alpha h + mixer(h));
h <- norm_b(alpha h + feed_forward(h)), with the constant ``residual_scale`` = alpha (an option of the layer's spec);
the feed-forward and its norm may be absent. Slots: mixer, mixer_norm, feed_forward, feed_forward_norm. The sublayers
read h itself. Scaling, sum and norm are one float32 kernel (two mixers side by side hand over both results and their
constants), which also leaves h in the compute dtype for the next sublayer's first matrix product."""
from __future__ import annotations

import os

import torch

from .base import Block, DeferredNorm, ProjectedInput, register_block
from .linear import Linear


# INFER_B200_BRANCHES=0: the sublayers of a parallel block one after the other on one stream (for comparisons).
PARALLEL_BRANCHES = os.environ.get("INFER_B200_BRANCHES", "1") == "1"
_SIDE_STREAMS = {}


def _side_streams(device):
    """Two side streams per device, shared by all layers (a layer's branches join before the next layer forks)."""
    key = str(device)
    if key not in _SIDE_STREAMS:
        from .. import fast_ops
        _SIDE_STREAMS[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        for st in _SIDE_STREAMS[key]:
            fast_ops.register_side_stream(st)
    return _SIDE_STREAMS[key]


def normed_input(norm, consumer, h):
    """norm(h), or, for as few rows as the streaming product takes and a consumer that can normalise inside its
    first kernel, the norm deferred. How many rows that is, is the kernel library's answer, not a constant here."""
    if consumer.accepts_deferred_norm and getattr(norm, "fusable", False) and norm.rt.fast("norm"):
        from .. import fast_ops
        if h.shape[0] <= fast_ops.skinny_limits()[0]:
            return DeferredNorm(norm, h)
    return norm.forward(h)


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer_norm, mixer, feed_forward_norm=None, feed_forward=None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a prenorm block has a feed-forward and its norm, or neither")
        parts = {"mixer_norm": mixer_norm, "mixer": mixer}
        if feed_forward is not None:
            parts.update(feed_forward_norm=feed_forward_norm, feed_forward=feed_forward)
        super().__init__(**parts)
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, h, step, cache, write_cache=True):
        h = self.mixer.forward(normed_input(self.mixer_norm, self.mixer, h), step, cache, h, write_cache)
        if self.feed_forward is None:
            return h
        return self.feed_forward.forward(normed_input(self.feed_forward_norm, self.feed_forward, h), h)


@register_block("parallel_gated")
class ParallelGatedBlock(Block):
    accepts_deferred_norm = True          # (of the joined products: the streaming product normalises inside)

    def __init__(self, norm, mixer, gate=None, feed_forward=None):
        parts = {"norm": norm, "mixer": mixer}
        if gate is not None:
            parts["gate"] = gate
        if feed_forward is not None:
            parts["feed_forward"] = feed_forward
        super().__init__(**parts)
        self.gate, self.feed_forward = gate, feed_forward
        # Every sublayer starts with a matrix product on the same rows. Products whose results have the same dtype
        # are joined into one (two launches per layer instead of four or five, and one read of the rows each).
        self.joined = []                   # (Linear, out dtype or None for the compute dtype, [(part, first column)])
        members = []
        for p in (mixer, gate, feed_forward):
            members += p.members() if hasattr(p, "members") else ([p] if p is not None else [])
        offers = [(p, p.input_product()) for p in members if hasattr(p, "input_product")]
        for kind in ("compute", "float32"):
            group = [(p, o[0]) for p, o in offers if o is not None and o[1] == kind]
            if len(group) >= 2:
                linear, starts = Linear.join(norm.rt, [l for _, l in group])
                self.joined.append((linear, torch.float32 if kind == "float32" else None, [(p, c) for (p, _), c in zip(group, starts)]))
                for p, _ in group:
                    p.drop_input_product()

    def forward(self, h, step, cache, write_cache=True):
        from .. import ops
        n = normed_input(self.norm, self, h)
        x = ProjectedInput(n)
        for linear, out_dtype, places in self.joined:
            rows = linear(n, out_dtype=out_dtype)
            for part, col0 in places:
                x.place(part, rows, col0)

        def arg(part):
            """The joined products' rows for a part that knows them; the normalised rows themselves for any other."""
            if hasattr(part, "input_product") or hasattr(part, "members"):
                return x
            return n.materialize() if isinstance(n, DeferredNorm) else n
        gates, g0 = self.gate.forward(x) if self.gate is not None else (None, 0)
        # The sublayers are independent between the joined products and the sum. In a decode step every kernel is a few
        # microseconds of latency, so the second mixer and the feed-forward run on two side streams beside the first
        # mixer (in a captured graph: three branches), and three chains of two to four kernels take the time of the
        # longest. Not in steps with prompt portions: measured on a 2,048-token prompt, the recurrence's scan beside
        # the persistent products (which count on an SM each) made the step 33 ms instead of 18. The fast kernels'
        # scratch is per side stream (fast_ops.register_side_stream).
        side = _side_streams(h.device) if (PARALLEL_BRANCHES and step.decode_only and hasattr(self.mixer, "forward_sides")) else None
        if side is not None:
            main = torch.cuda.current_stream(h.device)
            fork = torch.cuda.Event()
            fork.record(main)
            for st in side:
                st.wait_event(fork)
            r = None
            if self.feed_forward is not None:
                with torch.cuda.stream(side[1]):
                    r = self.feed_forward.forward(arg(self.feed_forward), None)
            p, q, a, b = self.mixer.forward_sides(arg(self.mixer), step, cache, write_cache, side[0])
            for st in side:
                done = torch.cuda.Event()
                done.record(st)
                main.wait_event(done)
            return ops.gated_sum(h, gates, p, a, q, b, r, g0)
        if hasattr(self.mixer, "forward_sides"):
            p, q, a, b = self.mixer.forward_sides(arg(self.mixer), step, cache, write_cache)
        else:
            p, q, a, b = self.mixer.forward(arg(self.mixer), step, cache, None, write_cache), None, 1.0, 1.0
        r = self.feed_forward.forward(arg(self.feed_forward), None) if self.feed_forward is not None else None
        return ops.gated_sum(h, gates, p, a, q, b, r, g0)


@register_block("sublayer_norm")
class SublayerNormBlock(Block):
    def __init__(self, mixer, mixer_out_norm, feed_forward=None, feed_forward_out_norm=None):
        parts = {"mixer": mixer, "mixer_out_norm": mixer_out_norm}
        if feed_forward is not None:
            if feed_forward_out_norm is None:
                raise ValueError("a feed-forward in a sublayer_norm block needs its norm")
            parts.update(feed_forward=feed_forward, feed_forward_out_norm=feed_forward_out_norm)
        super().__init__(**parts)
        self.feed_forward, self.feed_forward_out_norm = feed_forward, feed_forward_out_norm
        for n in (mixer_out_norm, feed_forward_out_norm):
            if n is not None and not getattr(n, "fusable", False):
                raise ValueError("a sublayer_norm block needs norms of the (weight, eps) root-mean-square kind")

    def forward(self, h, step, cache, write_cache=True):
        from .. import ops
        rt = self.mixer.rt
        x = h if rt.dtype == torch.float32 else self._copy_of(h, step, rt.dtype)
        fused = getattr(self.mixer, "forward_normed", None)
        # In a decode step every kernel is a few microseconds of latency: two mixers side by side run on two streams
        # (two branches in a captured graph) and the chains of five or six kernels take the time of the longer one.
        side = _side_streams(h.device)[0] if (PARALLEL_BRANCHES and step.decode_only and fused is not None and rt.dtype != torch.float32) else None
        got = fused(x, step, cache, write_cache, h, self.mixer_out_norm, rt.dtype, side) if fused is not None else None
        if got is None:
            y = self.mixer.forward(x, step, cache, None, write_cache)
            got = ops.norm_add(h, y, self.mixer_out_norm.weight, self.mixer_out_norm.eps, rt.dtype)
        h, copy = got
        if self.feed_forward is not None:
            y = self.feed_forward.forward(copy if copy is not None else h, None)
            h, copy = ops.norm_add(h, y, self.feed_forward_out_norm.weight, self.feed_forward_out_norm.eps, rt.dtype)
        step.extras["rows_copy"] = (h, copy)
        return h

    @staticmethod
    def _copy_of(h, step, dtype):
        from .. import ops
        have = step.extras.get("rows_copy")
        if have is not None and have[0] is h and have[1] is not None and have[1].dtype == dtype:
            return have[1]
        return ops.cast_rows(h, dtype)


@register_block("postnorm")
class PostNormBlock(Block):
    def __init__(self, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None, residual_scale: float = 1.0):
        parts = {"mixer": mixer, "mixer_norm": mixer_norm}
        if feed_forward is not None:
            if feed_forward_norm is None:
                raise ValueError("a feed-forward in a postnorm block needs its norm")
            parts.update(feed_forward=feed_forward, feed_forward_norm=feed_forward_norm)
        super().__init__(**parts)
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.alpha = float(residual_scale)
        for n in (mixer_norm, feed_forward_norm):
            if n is not None and not getattr(n, "fusable", False):
                raise ValueError("a postnorm block needs norms of the (weight, eps) root-mean-square kind")

    def forward(self, h, step, cache, write_cache=True):
        from .. import ops
        rt = self.mixer.rt
        x = h if (rt.dtype == torch.float32 or self.mixer.reads_stream) else SublayerNormBlock._copy_of(h, step, rt.dtype)
        norm = self.mixer_norm
        sides = getattr(self.mixer, "forward_sides", None)
        if sides is not None and not getattr(self.mixer, "normed", False):
            # In a decode step every kernel is a few microseconds of latency: two mixers side by side run on two streams
            side = _side_streams(h.device)[0] if (PARALLEL_BRANCHES and step.decode_only and rt.dtype != torch.float32) else None
            if side is not None:
                main = torch.cuda.current_stream(h.device)
                fork = torch.cuda.Event()
                fork.record(main)
                side.wait_event(fork)
            a, b, sa, sb = sides(x, step, cache, write_cache, side)
            if side is not None:
                done = torch.cuda.Event()
                done.record(side)
                main.wait_event(done)
            h, copy = ops.sum_norm(h, self.alpha, a, sa, b, sb, norm.weight, norm.eps, rt.dtype)
        else:
            y = self.mixer.forward(x, step, cache, None, write_cache)
            h, copy = ops.sum_norm(h, self.alpha, y, 1.0, None, 0.0, norm.weight, norm.eps, rt.dtype)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(copy if copy is not None else h, None)
            norm = self.feed_forward_norm
            h, copy = ops.sum_norm(h, self.alpha, y, 1.0, None, 0.0, norm.weight, norm.eps, rt.dtype)
        step.extras["rows_copy"] = (h, copy)
        return h
