"""Rotary position encodings: half-split over the whole head, and adjacent pairs over part of it.

inv_freq[j] = 1 / theta^(2j / head_dim) in float32, angle = float32(pos) * inv_freq[j] (a float32
product), and element j of a head is rotated together with element j + head_dim/2:
x1' = x1*cos - x2*sin, x2' = x2*cos + x1*sin (src/forward.cpp:52-95).  As in the reference
(kernels/batch_gpu.cu:122-127) the tables are built on the host in float32 and uploaded, so the host's
plain implementation and the device rotate by identical angles.
"""
from __future__ import annotations

import torch

from ..config.specs import PartSpec
from .base import PositionEncoding, register_position


def rotary_tables(head_dim: int, theta: float, n_positions: int):
    """(cos, sin), float32 [n_positions, head_dim/2], on the CPU."""
    half = head_dim // 2
    exponent = torch.arange(0, half, dtype=torch.float32) * 2.0 / float(head_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angle = torch.arange(n_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angle), torch.sin(angle)


@register_position("rotary_half")
class RotaryHalf(PositionEncoding):
    layout = "half"

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.head_dim, self.theta = int(spec["head_dim"]), float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.head_dim % 2 or self.head_dim <= 0:
            raise ValueError(f"rotary_half needs an even head_dim, got {self.head_dim}")
        if self.theta <= 0:
            raise ValueError("rotary_half needs a positive theta")
        self._tables = {}

    def rotary_tables(self, n_positions: int = None):
        """Tables for positions [0, n_positions) on the device; cached per length."""
        n = min(self.max_positions, n_positions or self.max_positions)
        cache_key = (self.head_dim, self.theta, n, str(self.rt.device))
        t = _SHARED_TABLES.get(cache_key)
        if t is None:
            cos, sin = rotary_tables(self.head_dim, self.theta, n)
            t = (cos.to(self.rt.device).contiguous(), sin.to(self.rt.device).contiguous())
            _SHARED_TABLES[cache_key] = t
        return t

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary_half is applied by the attention part's rotate-and-store kernel")


# Layers of one model share their tables (same head size, theta and length).
_SHARED_TABLES = {}


def pair_rotation_tables(rotary_dims: int, theta: float, n_positions: int):
    """(cos, sin), float32 [n_positions, rotary_dims/2], on the CPU: pair i turns by float32(pos) * float32(theta^(-2i /
    rotary_dims)), a float32 product; cosine and sine of that float32 angle are taken in float64 and rounded once."""
    i = torch.arange(rotary_dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / float(rotary_dims)).to(torch.float32)
    angle = (torch.arange(n_positions, dtype=torch.float32)[:, None] * freq[None, :]).to(torch.float64)
    return torch.cos(angle).to(torch.float32), torch.sin(angle).to(torch.float32)


@register_position("rotary_pairs")
class RotaryPairs(PositionEncoding):
    """Channels (2i, 2i + 1) of a head, for 2i < rotary_dims, turn together: (u, v) -> (u cos a - v sin a, v cos a +
    u sin a), a = pos * theta^(-2i / rotary_dims); channels from rotary_dims on pass unchanged. The attention part's
    prepare kernel applies it from the tables."""
    layout = "pairs"

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.head_dim, self.theta = int(spec["head_dim"]), float(spec["theta"])
        self.rotary_dims = int(spec.get("rotary_dims") or self.head_dim)
        self.max_positions = int(spec["max_positions"])
        if self.rotary_dims <= 0 or self.rotary_dims % 2 or self.rotary_dims > self.head_dim:
            raise ValueError(f"rotary_pairs needs an even number of rotated channels within the head, got "
                             f"{self.rotary_dims} of {self.head_dim}")
        if self.theta <= 0:
            raise ValueError("rotary_pairs needs a positive theta")

    def rotary_tables(self, n_positions: int = None):
        n = min(self.max_positions, n_positions or self.max_positions)
        cache_key = ("pairs", self.rotary_dims, self.theta, n, str(self.rt.device))
        t = _SHARED_TABLES.get(cache_key)
        if t is None:
            cos, sin = pair_rotation_tables(self.rotary_dims, self.theta, n)
            t = (cos.to(self.rt.device).contiguous(), sin.to(self.rt.device).contiguous())
            _SHARED_TABLES[cache_key] = t
        return t

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary_pairs is applied by the attention part's prepare kernel")


def interpolated_frequencies(rotary_dims: int, theta: float, scaling):
    """(frequencies float64 [rotary_dims / 2], magnitude). f_i = theta^(-2i / rotary_dims). With ``scaling`` {factor,
    original, fast, slow} (YaRN): pairs that turn fast keep f_i, pairs that turn slowly take f_i / factor, a linear
    ramp between, which runs from the pair index at which a full turn takes original / fast positions to the one
    at which it takes original / slow positions (index(t) = rotary_dims * ln(original / (2 pi t)) / (2 ln theta),
    the lower end rounded down and not below 0, the upper rounded up and not above rotary_dims - 1); cosines and
    sines are multiplied by ``magnitude_slope`` * ln(factor) + 1."""
    import math
    i = torch.arange(rotary_dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / float(rotary_dims))
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return rotary_dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), rotary_dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, float(scaling.get("min_span", 0.001))), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), float(scaling.get("magnitude_slope", 0.1)) * math.log(factor) + 1.0


@register_position("rotary_interpolated")
class RotaryInterpolated(PositionEncoding):
    """A rotation over the first ``rotary_dims`` channels of what it is applied to, in either layout ("pairs":
    channel 2i with 2i + 1; "half": channel i with i + rotary_dims / 2), with optionally interpolated frequencies
    (``scaling``, see interpolated_frequencies). Angles, cosines and sines are computed in float64 on the host and
    rounded once; the magnitude is part of the tables, so the kernels that apply them know nothing of the scaling."""

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.theta = float(spec["theta"])
        self.rotary_dims = int(spec["rotary_dims"])
        self.head_dim = int(spec.get("head_dim") or self.rotary_dims)
        self.layout = str(spec.get("layout", "half"))
        self.scaling = dict(spec["scaling"]) if spec.get("scaling") else None
        self.max_positions = int(spec["max_positions"])
        if self.layout not in ("pairs", "half"):
            raise ValueError(f"a rotation's layout is 'pairs' or 'half', not {self.layout!r}")
        if self.rotary_dims <= 0 or self.rotary_dims % 2 or self.rotary_dims > self.head_dim:
            raise ValueError(f"rotary_interpolated needs an even number of rotated channels within the head, got "
                             f"{self.rotary_dims} of {self.head_dim}")
        if self.theta <= 1:
            raise ValueError("rotary_interpolated needs a theta above 1")
        if self.scaling is not None:
            for k in ("factor", "original", "fast", "slow"):
                if k not in self.scaling or float(self.scaling[k]) <= 0:
                    raise ValueError(f"rotary_interpolated: scaling needs a positive {k!r}")

    def rotary_tables(self, n_positions: int = None):
        n = min(self.max_positions, n_positions or self.max_positions)
        sc = tuple(sorted(self.scaling.items())) if self.scaling else None
        cache_key = ("interpolated", self.rotary_dims, self.theta, sc, n, str(self.rt.device))
        t = _SHARED_TABLES.get(cache_key)
        if t is None:
            freq, mag = interpolated_frequencies(self.rotary_dims, self.theta, self.scaling)
            angle = torch.arange(n, dtype=torch.float64)[:, None] * freq[None, :]
            t = ((torch.cos(angle) * mag).to(torch.float32).to(self.rt.device).contiguous(),
                 (torch.sin(angle) * mag).to(torch.float32).to(self.rt.device).contiguous())
            _SHARED_TABLES[cache_key] = t
        return t

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary_interpolated is applied by the kernels of the mixer that names it")
