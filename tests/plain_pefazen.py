"""The Pefazen decoder written out slowly: whole sequences, no cache, torch on the CPU in float64.

One function per mechanism. It shares no code with ``infer_b200``: it reads the raw config.json dictionary and a
dictionary of checkpoint tensors by their names in the file. Everything the engine does for this design is compared
with this file.

    x = table[token]
    per layer:  x <- x + m * mixer(layer_norm(x, w1));   x <- x + m * experts(layer_norm(x, w2))   (second line absent
                without a feed-forward); m is one constant of the model
    logits = cap * tanh(head(layer_norm(x, w_final)) * logit_scale / cap)

The mixer is attention through low-rank latents (``latent_attention``): the query of every head is the up-projection
of a normalised low-rank row; keys and values of every head are up-projections of ONE normalised low-rank row c per
position, and one small rotated key part is shared by all heads, so that (c, rotated part) is all that a position
leaves behind. Two variants: rotation of adjacent pairs, a sliding window and a sigmoid gate per head; or rotation of
the two halves with interpolated frequencies, all earlier positions visible and no gate. A layer may read another
layer's (c, rotated part) instead of making its own.

``ROUNDING``: None computes exactly. Set to ``torch.bfloat16`` (see ``rounded``), activations are rounded where a
bfloat16 serving path stores them, which gives the size of the rounding noise such a path must have.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

F = torch.float64
YARN_MAGNITUDE_SLOPE = 0.1     # cos and sin are multiplied by YARN_MAGNITUDE_SLOPE * ln(factor) + 1
YARN_MIN_SPAN = 0.001          # least width of the ramp between the two ends

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


# ----------------------------------------------------------------------------- norms and small functions

def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w over the last dimension; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(F)


def rms_weighted(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.to(F)


def linear(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    return x @ W.to(F).T


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# ----------------------------------------------------------------------------- rotations

def plain_frequencies(dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2."""
    i = torch.arange(dims // 2, dtype=F)
    return torch.pow(torch.tensor(float(base), dtype=F), -2.0 * i / dims)


def interpolated_frequencies(dims: int, base: float, scaling: Optional[Mapping[str, float]]):
    """(frequencies, magnitude). Without ``scaling``: the plain ones and 1. With it, pair i keeps f_i where it turns
    fast, takes f_i / factor where it turns slowly, and a linear mix between: the ramp runs from the pair index at
    which a full turn takes original / fast positions to the one at which it takes original / slow positions."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=F)
    ramp = torch.clamp((i - lo) / max(hi - lo, YARN_MIN_SPAN), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), YARN_MAGNITUDE_SLOPE * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, layout: str, magnitude: float = 1.0) -> torch.Tensor:
    """x [T, ..., n] with n >= 2 * len(freq): the first 2 * len(freq) channels turn by positions * freq, the rest
    pass. layout "pairs": channel 2i turns with 2i + 1; "halves": channel i with i + len(freq).
    (u, v) -> (u cos - v sin, v cos + u sin), cos and sin times ``magnitude``."""
    n = freq.numel()
    a = positions.to(F)[:, None] * freq[None, :]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    cos, sin = torch.cos(a) * magnitude, torch.sin(a) * magnitude
    out = x.clone()
    if layout == "pairs":
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * cos - v * sin
        out[..., 1:2 * n:2] = v * cos + u * sin
    else:
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n] = u * cos - v * sin
        out[..., n:2 * n] = v * cos + u * sin
    return out


# ----------------------------------------------------------------------------- the mixer

def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """bool [T, T]: query i sees key j if j <= i and, with a window, i - j < window."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    return ok


def latent_pair(W: Mapping[str, torch.Tensor], p: str, m: Mapping, h: torch.Tensor, positions, eps: float, layout: str):
    """What a position leaves behind: (c [T, kv_rank], rotated shared key part [T, rot_dim])."""
    r = int(m["kv_rank"])
    rot = m["rot"]
    freq, mag = interpolated_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    low = linear(h, W[p + "dkv"])
    c = rms_weighted(low[:, :r], W[p + "dkv.norm"], eps)
    shared = rotate(low[:, r:], positions, freq, layout, mag)
    return _rnd(c), _rnd(shared)


def latent_attention(W: Mapping[str, torch.Tensor], p: str, m: Mapping, h: torch.Tensor, eps: float, layout: str, gated: bool,
                     pair, positions=None) -> torch.Tensor:
    """h [T, width] (normalised rows) -> [T, width]. ``pair``: (c, rotated shared key part) of this layer or of the
    layer it reads."""
    T = h.shape[0]
    H, d, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    positions = torch.arange(T) if positions is None else positions
    rot = m["rot"]
    freq, mag = interpolated_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    cq = _rnd(rms_weighted(linear(h, W[p + "dq"]), W[p + "dq.norm"], eps))
    q = _rnd(linear(cq, W[p + "uq"])).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, freq, layout, mag)
    c, shared = pair
    k_plain = linear(c, W[p + "uk"]).view(T, H, d)
    v = linear(c, W[p + "uv"]).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, shared)) * float(m["scale"])
    window = int(m["mask"]["size"]) if m.get("mask") else None
    s = s.masked_fill(~visible(T, window)[None], float("-inf"))
    a = torch.softmax(s, dim=-1)
    ctx = torch.einsum("hij,jhd->ihd", a, v)
    if gated:
        ctx = ctx * torch.sigmoid(linear(h, W[p + "g"]))[:, :, None]
    return linear(_rnd(ctx.reshape(T, H * dv)), W[p + "o"])


# ----------------------------------------------------------------------------- the feed-forward

def choose_experts(h: torch.Tensor, Wr: torch.Tensor, correction: torch.Tensor, top: int):
    """(chosen [T, top] indices, their weights [T, top], gap [T]). Scores are sigmoids of the router's logits; the
    choice is by score + correction, the weights are the scores themselves, as they are. gap: how far the last chosen
    choice score lies above the best one left out (inf if all are chosen)."""
    s = torch.sigmoid(linear(h, Wr))
    choice = s + correction.to(F)
    order = torch.argsort(choice, dim=-1, descending=True, stable=True)
    chosen = order[:, :top]
    ranked = torch.gather(choice, 1, order)
    gap = ranked[:, top - 1] - ranked[:, top] if top < s.shape[1] else torch.full((h.shape[0],), float("inf"), dtype=F)
    return chosen, torch.gather(s, 1, chosen), gap


def routed_experts(W: Mapping[str, torch.Tensor], p: str, f: Mapping, h: torch.Tensor, gaps: Optional[List] = None) -> torch.Tensor:
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    chosen, weight, gap = choose_experts(h, W[p + "router"], W[p + "correction"], top)
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F)
    for e in range(E):
        hidden = _rnd(relu_squared(linear(h, W[p + f"e{e}.up"])))
        y = linear(hidden, W[p + f"e{e}.down"])
        w_e = (weight * (chosen == e)).sum(dim=1)
        out = out + y * w_e[:, None]
    return out


# ----------------------------------------------------------------------------- the model

def forward(cfg: Mapping, W: Mapping[str, torch.Tensor], ids: Sequence[int], layers_out: Optional[List] = None,
            gaps: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence from position 0. ``layers_out`` collects x after every layer;
    ``gaps`` the routers' gaps per layer."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    T = len(ids)
    positions = torch.arange(T)
    x = W["embed"].to(F)[torch.tensor(list(ids), dtype=torch.long)]
    pairs: Dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = layer["mixer"]
        layout, gated = ("pairs", True) if layer["type"] == "latent_attention" else ("halves", False)
        h = _rnd(layer_norm(x, W[p + "norm1"], eps))
        src = mix.get("kv_from")
        if src is None:
            pairs[i] = latent_pair(W, p + "mix.", mix, h, positions, eps, layout)
            src = i
        x = x + m * latent_attention(W, p + "mix.", mix, h, eps, layout, gated, pairs[int(src)])
        if layer.get("mlp") is not None:
            h = _rnd(layer_norm(x, W[p + "norm2"], eps))
            x = x + m * routed_experts(W, p + "mlp.", layer["mlp"], h, gaps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = _rnd(layer_norm(x, W["final.norm"], eps))
    logits = linear(h, W["head"]) * float(cfg.get("logit_scale", 1.0))
    return soft_cap(logits, float(cfg["logit_softcap"])) if cfg.get("logit_softcap") else logits


def greedy(cfg: Mapping, W: Mapping[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    """n_new tokens, each the first index of the largest logit after the whole sequence so far."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(cfg, W, ids)[-1]))
        ids.append(tok)
        out.append(tok)
    return out
