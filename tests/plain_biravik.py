"""The Biravik decoder written out slowly: whole sequences, no cache, torch on the CPU in float64.

One function per mechanism. It shares no code with ``infer_b200``: it reads the raw config.json dictionary and a
dictionary of checkpoint tensors by their names in the file. Everything the engine does for this design is compared
with this file.

The residual stream x starts as table[token] * embedding.scale. A layer normalises AFTER the sum, and its sublayers
read x itself:

    x <- norm_1(alpha x + mixer(x));    x <- norm_2(alpha x + feed_forward(x))      (second line absent without one)

with norm(y) = y / sqrt(mean(y^2) + eps) * (1 + w). Mixers: ``softmax_attention`` (per-head norms of q and k, an
optional rotation of channel pairs with interpolated frequencies, an optional query temperature, an optional bias
that grows with the distance, a window that keeps the first tokens, a sink, values that may be the projected keys,
an output gate per channel), ``constant_decay_attention`` (a matrix state per head that fades by a constant of the
head), the two side by side (layer type "parallel"), and ``shifted_decay_mixing`` (layer type "wkv": projections of
mixtures of a token's row with its predecessor's, a decay per key channel and token, a bonus for the current token).
Feed-forwards: ``dense_relu_squared`` and ``routed_experts`` (softmax over the chosen logits only).

``ROUNDING``: None computes exactly. Set to ``torch.bfloat16`` (see ``rounded``), activations are rounded where a
bfloat16 serving path stores them, which gives the size of the rounding noise such a path must have.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

F = torch.float64
MAGNITUDE_SLOPE = 0.1       # cosines and sines are multiplied by MAGNITUDE_SLOPE * ln(factor) + 1
MIN_RAMP_SPAN = 0.001       # least width of the frequency ramp
SLOPE_EXPONENT = 8.0        # head h of H takes the slope 2^(-SLOPE_EXPONENT (h + 1) / H)

ROUNDING = None


class rounded:
    """with rounded(torch.bfloat16): ... computes with activations rounded where a serving path stores them."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global ROUNDING
        self.old, ROUNDING = ROUNDING, self.dtype

    def __exit__(self, *exc):
        global ROUNDING
        ROUNDING = self.old


def _rnd(x: torch.Tensor) -> torch.Tensor:
    return x if ROUNDING is None else x.to(ROUNDING).to(x.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w.to(F))


def linear(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    return x @ W.to(F).T


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------- positions

def interpolated_frequencies(dims: int, base: float, scaling: Optional[Mapping]) -> (torch.Tensor, float):
    """Frequencies of the dims / 2 channel pairs and the factor on cosines and sines."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, MIN_RAMP_SPAN), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), MAGNITUDE_SLOPE * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Mapping) -> torch.Tensor:
    """x [T, heads, dim]: channels (2i, 2i + 1) below rot.dims turn by position * frequency_i; the rest pass."""
    dims = int(rot["dims"])
    freq, mag = interpolated_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    a = positions.to(F)[:, None] * freq[None, :]                  # [T, dims / 2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    return 1.0 + coef * torch.log(torch.div(positions + 1, every, rounding_mode="floor").to(F) + 1.0)


def distance_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-SLOPE_EXPONENT * (h + 1) / heads) for h in range(heads)], dtype=F)


def visible(T: int, window: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j if j <= i and (i - j < window or j < keep_first); no window: every j <= i."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


# ----------------------------------------------------------------------------- softmax attention

def attention_weights(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores [H, T, T] -> softmax weights over the visible keys; with ``sink`` [H] the denominator also holds
    exp(sink_h), once, which has no key and no value."""
    scores = scores.masked_fill(~mask[None], -math.inf)
    top = scores.max(dim=-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.to(F)[:, None, None])
    e = torch.exp(scores - top)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(F)[:, None, None] - top)
    return e / den


def softmax_attention(h: torch.Tensor, W: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    """One softmax-attention mixer whose tensors start with ``p``; m is its part of the configuration."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m.get("kv_heads") or m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    x = _rnd(h)
    q = linear(x, W[p + "q"]).view(T, H, d)
    k_raw = linear(x, W[p + "k"]).view(T, G, d)
    v = linear(x, W[p + "v"]).view(T, G, dv) if p + "v" in W else k_raw      # the values may be the keys as projected
    q = rms(q, eps) * W[p + "q.norm"].to(F)
    k = rms(k_raw, eps) * W[p + "k.norm"].to(F)
    if m.get("rot"):
        q, k = rotate_pairs(q, pos, m["rot"]), rotate_pairs(k, pos, m["rot"])
    if m.get("q_temp"):
        q = q * query_temperature(pos, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))[:, None, None]
    q, k, v = _rnd(q), _rnd(k), _rnd(v)
    per = H // G
    kh, vh = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)        # query head a reads kv head a // per
    scores = torch.einsum("ihd,jhd->hij", q, kh) * float(m["scale"])
    if m.get("distance_bias", False):
        dist = (pos[:, None] - pos[None, :]).to(F)
        scores = scores - distance_slopes(H)[:, None, None] * dist[None]
    mask = m.get("mask")
    ok = visible(T, int(mask["size"]) if mask else None, int(mask.get("keep_first", 0)) if mask else 0)
    w = attention_weights(scores, ok, W.get(p + "sink"))
    ctx = torch.einsum("hij,jhd->ihd", w, vh).reshape(T, H * dv)
    ctx = _rnd(_rnd(ctx) * torch.sigmoid(linear(x, W[p + "g"])))
    return linear(ctx, W[p + "o"])


# ----------------------------------------------------------------------------- recurrences

def constant_decay_scan(q, k, v, decay: float, S0=None):
    """One head. S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (the read-out sees the token's own write)."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F) if S0 is None else S0.clone()
    out = []
    for t in range(q.shape[0]):
        S = decay * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return (torch.stack(out) if out else torch.zeros(0, v.shape[1], dtype=F)), S


def constant_decay_attention(h, W, p: str, m: Mapping, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    x = _rnd(h)
    q, k, v = (silu(linear(x, W[p + n])) for n in "qkv")
    q, k, v = q.view(T, H, d), k.view(T, H, d), v.view(T, H, dv)
    o = torch.stack([constant_decay_scan(q[:, a], k[:, a], v[:, a], float(m["decay"][a]))[0] for a in range(H)], dim=1)
    y = rms(o.reshape(T, H * dv), eps) * W[p + "norm"].to(F)            # ONE norm over all heads
    y = _rnd(y * torch.sigmoid(linear(x, W[p + "g"])))
    return linear(y, W[p + "o"])


def bonus_scan(r, k, v, w, u, S0=None):
    """One head. o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, then S_t = diag(w_t) S_(t-1) + k_t v_t^T: the current
    token is read through the bonus u only. r, k, w [T, d]; v [T, dv]; u [d]."""
    S = torch.zeros(r.shape[1], v.shape[1], dtype=F) if S0 is None else S0.clone()
    out = []
    for t in range(r.shape[0]):
        kv = k[t][:, None] * v[t][None, :]
        out.append((S + u[:, None] * kv).T @ r[t])
        S = w[t][:, None] * S + kv
    return (torch.stack(out) if out else torch.zeros(0, v.shape[1], dtype=F)), S


def shifted_decay_mixing(h, W, p: str, m: Mapping, eps: float, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, width = h.shape
    H, d = int(m["heads"]), int(m["dim"])
    prev = torch.cat([torch.zeros(1, width, dtype=F) if before is None else before[None], h[:-1]])
    mix = {s: _rnd(h + (prev - h) * W[p + "mu." + s].to(F)) for s in "rkvgw"}
    r, k, v = (linear(mix[s], W[p + s]).view(T, H, d) for s in "rkv")
    gate = silu(linear(mix["g"], W[p + "g"]))
    low = torch.tanh(linear(mix["w"], W[p + "w1"]))
    w = torch.exp(-torch.exp(linear(low, W[p + "w2"]) + W[p + "w0"].to(F))).view(T, H, d)
    u = W[p + "u"].to(F)
    o = torch.stack([bonus_scan(r[:, a], k[:, a], v[:, a], w[:, a], u[a])[0] for a in range(H)], dim=1)
    y = rms(o, eps).reshape(T, H * d) * W[p + "norm"].to(F)              # every head by its own root mean square
    return linear(_rnd(y * gate), W[p + "o"])


# ----------------------------------------------------------------------------- feed-forwards

def dense_relu_squared(h, W, p: str) -> torch.Tensor:
    x = _rnd(h)
    return linear(_rnd(torch.relu(linear(x, W[p + "up"])) ** 2), W[p + "down"])


def route_top(logits: torch.Tensor, top: int):
    """logits [T, E] -> (chosen [T, top], weights [T, top]): the largest logits (ties: the lower index), softmax over
    the chosen ones only; also the gap between the last chosen and the first refused logit."""
    order = torch.sort(logits, dim=-1, descending=True, stable=True)
    chosen, z = order.indices[:, :top], order.values[:, :top]
    gap = (order.values[:, top - 1] - order.values[:, top]) if logits.shape[1] > top else torch.full((logits.shape[0],), math.inf, dtype=F)
    return chosen, torch.softmax(z, dim=-1), gap


def routed_experts(h, W, p: str, f: Mapping, gaps: Optional[List] = None) -> torch.Tensor:
    x = _rnd(h)
    chosen, weights, gap = route_top(linear(x, W[p + "router"]), int(f["router"]["top"]))
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            u = p + f"e{e}."
            hid = _rnd(silu(linear(x[t], W[u + "gate"])) * linear(x[t], W[u + "up"]) * wt)
            out[t] += linear(hid, W[u + "down"])
    return out


# ----------------------------------------------------------------------------- the model

def mixer(kind: str, h, W, p: str, m: Mapping, eps: float) -> torch.Tensor:
    if kind == "attention":
        return softmax_attention(h, W, p, m, eps)
    if kind == "wkv":
        return shifted_decay_mixing(h, W, p, m, eps)
    if kind == "parallel":
        left = dict(m["left"], distance_bias=True)                       # the left side has no mask and no rotation
        return float(m["left_scale"]) * softmax_attention(h, W, p + "left.", left, eps) + \
            float(m["right_scale"]) * constant_decay_attention(h, W, p + "right.", m["right"], eps)
    raise ValueError(f"unknown layer type {kind!r}")


def forward(cfg: Mapping, W: Mapping[str, torch.Tensor], ids: Sequence[int], layer_outputs: Optional[List] = None,
            gaps: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence; ``layer_outputs`` collects the stream after every layer,
    ``gaps`` every router's distance between the last chosen and the first refused logit, per position."""
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    x = W["embed"].to(F)[torch.tensor(list(ids), dtype=torch.long)] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = norm_one_plus(alpha * x + mixer(layer["type"], x, W, p + "mix.", layer["mixer"], eps), W[p + "norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            y = dense_relu_squared(x, W, p + "mlp.") if f["kind"] == "dense" else routed_experts(x, W, p + "mlp.", f, gaps)
            x = norm_one_plus(alpha * x + y, W[p + "norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return linear(_rnd(norm_one_plus(x, W["final.norm"], eps)), W["head"])


def greedy(cfg: Mapping, W: Mapping[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]
