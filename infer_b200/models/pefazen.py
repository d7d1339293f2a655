"""Pefazen: typed configuration and its translation into a ModelSpec.

A pre-norm decoder whose sublayers are scaled by one constant m of the model:

    x <- x + m * mixer(layernorm_1(x));    x <- x + m * experts(layernorm_2(x))      (second line absent without one)

The norms are layer norms with a weight and no bias (parts/layernorm.py). Every mixer is attention through low-rank
latents (parts/latent_attention.py): a position leaves one normalised low-rank row and one small rotated key part
behind, which all heads share. Two kinds of layer, in any order:

"latent_attention"    rotation of neighbouring channel pairs, a sliding window (``mask.size``), a sigmoid gate per head
"latent_attention_2"  rotation of the two halves with interpolated frequencies (``rot.scaling``), all earlier
                      positions visible, no gate

A layer with ``kv_from: j`` makes no latent of its own: it reads what layer j left in its cache (the run order names
layer j's cache with write_cache False) through its own up-projections, queries and mask.

Feed-forward: a mixture of ungated experts, relu squared, chosen by sigmoid scores plus a stored correction, weights
the scores as they are (parts/routed_ff.py, router_kind "sigmoid", expert_kind "relu_squared"), or none.
A final layer norm, the output matrix, a scale and a soft cap on the logits (parts/vocab.py).

config.json keys (every size and constant comes from there or from the tensors' shapes; tensor names are fixed):

    architecture "Pefazen"; vocab; width; norm.eps; residual_mult; logit_scale; logit_softcap
    layers[i] = {type, mixer: {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims, scaling:
                 {factor, original, fast, slow} | absent}, mask: {size} | absent, kv_from: j | absent},
                 mlp: {kind: "moe", router: {experts, top}, expert: {ff}} | null}

Tensors: embed, final.norm, head, and per layer l<i>.: norm1, norm2, mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o},
mlp.{router, correction, e<k>.up, e<k>.down}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, ConfigError, register_architecture
from ..config.specs import LayerCall, LayerSpec, ModelSpec, PartSpec

NAME = "Pefazen"
DEFAULT_MAX_POSITIONS = 1 << 20       # the design states no limit; an engine's own sequence limit sizes its tables
# what the design fixes per kind of layer: (rotation layout, gate per head)
LAYER_KINDS = {"latent_attention": ("pairs", True), "latent_attention_2": ("half", False)}
# constants of the interpolated rotation that the design fixes
MAGNITUDE_SLOPE = 0.1                 # cos and sin times MAGNITUDE_SLOPE * ln(factor) + 1
MIN_RAMP_SPAN = 0.001                 # least width of the ramp between kept and divided frequencies


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]     # sorted (key, value) pairs of factor, original, fast, slow


@dataclass(frozen=True)
class LatentMixer:
    kind: str
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Rotation
    window: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class ExpertsFF:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class PefazenLayer:
    mixer: LatentMixer
    mlp: Optional[ExpertsFF]


@dataclass(frozen=True)
class PefazenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    logit_softcap: float               # 0: no cap
    layers: Tuple[PefazenLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS


def _get(raw, key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise ConfigError(f"config.json: {where} is missing key {key!r}")
    return raw[key]


def _int(raw, key, where, minimum=1) -> int:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(raw, key, where, positive=False) -> float:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _rotation(raw, where: str, rot_dim: int) -> Rotation:
    dims = _int(raw, "dims", where, 2)
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json: {where}.dims ({dims}) must be even and at most rot_dim ({rot_dim})")
    base = _num(raw, "base", where, positive=True)
    if base <= 1:
        raise ConfigError(f"config.json: {where}.base must be above 1, got {base!r}")
    sc = raw.get("scaling")
    scaling = None
    if sc is not None:
        scaling = tuple(sorted((k, _num(sc, k, where + ".scaling", positive=True)) for k in ("factor", "original", "fast", "slow")))
    return Rotation(base, dims, scaling)


def _mixer(kind: str, raw, where: str, index: int) -> LatentMixer:
    rot_dim = _int(raw, "rot_dim", where, 2)
    mask = raw.get("mask")
    kv_from = raw.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < index):
        raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer, got {kv_from!r}")
    return LatentMixer(kind, _int(raw, "heads", where), _int(raw, "dim", where), rot_dim, _int(raw, "vdim", where),
                       _int(raw, "q_rank", where), _int(raw, "kv_rank", where), _num(raw, "scale", where),
                       _rotation(_get(raw, "rot", where), where + ".rot", rot_dim),
                       _int(mask, "size", where + ".mask") if mask is not None else None, kv_from)


def _mlp(raw, where: str) -> Optional[ExpertsFF]:
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design ('moe')")
    router = _get(raw, "router", where)
    experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: {top} of {experts} experts")
    return ExpertsFF(experts, top, _int(_get(raw, "expert", where), "ff", where + ".expert"))


def parse(raw: Mapping[str, Any]) -> PefazenConfig:
    top = "the configuration"
    layers = _get(raw, "layers", top)
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    out = []
    for i, l in enumerate(layers):
        where = f"layers[{i}]"
        kind = _get(l, "type", where)
        if kind not in LAYER_KINDS:
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design ({', '.join(map(repr, LAYER_KINDS))})")
        out.append(PefazenLayer(_mixer(kind, _get(l, "mixer", where), where + ".mixer", i), _mlp(l.get("mlp"), where + ".mlp")))
    for i, l in enumerate(out):
        j = l.mixer.kv_from
        if j is None:
            continue
        a, b = l.mixer, out[j].mixer
        if b.kv_from is not None:
            raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {j}, which has no latent of its own")
        if (a.kv_rank, a.rot_dim, a.rot, LAYER_KINDS[a.kind][0]) != (b.kv_rank, b.rot_dim, b.rot, LAYER_KINDS[b.kind][0]):
            raise ConfigError(f"config.json: layers[{i}] reads the latent of layer {j}, whose kv_rank, rot_dim or rotation differ")
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"config.json: max_positions must be a positive integer, got {max_positions!r}")
    cap = raw.get("logit_softcap")
    return PefazenConfig(vocab=_int(raw, "vocab", top), width=_int(raw, "width", top),
                         eps=_num(_get(raw, "norm", top), "eps", "norm", positive=True),
                         residual_mult=_num(raw, "residual_mult", top) if raw.get("residual_mult") is not None else 1.0,
                         logit_scale=_num(raw, "logit_scale", top) if raw.get("logit_scale") is not None else 1.0,
                         logit_softcap=_num(raw, "logit_softcap", top, positive=True) if cap is not None else 0.0,
                         layers=tuple(out), max_positions=max_positions)


def to_dict(cfg: PefazenConfig) -> Dict[str, Any]:
    layers = []
    for l in cfg.layers:
        m = l.mixer
        rot: Dict[str, Any] = {"base": m.rot.base, "dims": m.rot.dims}
        if m.rot.scaling is not None:
            rot["scaling"] = dict(m.rot.scaling)
        mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank,
                                 "kv_rank": m.kv_rank, "scale": m.scale, "rot": rot}
        if m.window is not None:
            mixer["mask"] = {"size": m.window}
        if m.kv_from is not None:
            mixer["kv_from"] = m.kv_from
        f = l.mlp
        mlp = None if f is None else {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.ff}}
        layers.append({"type": m.kind, "mixer": mixer, "mlp": mlp})
    d = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "residual_mult": cfg.residual_mult,
         "logit_scale": cfg.logit_scale, "layers": layers}
    if cfg.logit_softcap:
        d["logit_softcap"] = cfg.logit_softcap
    if cfg.max_positions != DEFAULT_MAX_POSITIONS:
        d["max_positions"] = cfg.max_positions
    return d


def _cache_windows(cfg: PefazenConfig) -> Dict[int, Optional[int]]:
    """Layer that owns a cache -> how long its rows must stay: the largest window of the layers that read them, None
    if one of them sees all earlier positions."""
    windows: Dict[int, list] = {}
    for i, l in enumerate(cfg.layers):
        windows.setdefault(i if l.mixer.kv_from is None else l.mixer.kv_from, []).append(l.mixer.window)
    return {j: (None if any(w is None for w in ws) else max(ws)) for j, ws in windows.items()}


def to_spec(cfg: PefazenConfig) -> ModelSpec:
    W = cfg.width
    keep = _cache_windows(cfg)
    layers, schedule = [], []
    cache_of: Dict[int, int] = {}
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        layout, gated = LAYER_KINDS[m.kind]
        owner = i if m.kv_from is None else m.kv_from
        position = PartSpec("rotary_interpolated", {
            "theta": m.rot.base, "rotary_dims": m.rot.dims, "head_dim": m.rot_dim, "layout": layout,
            "scaling": ({**dict(m.rot.scaling), "magnitude_slope": MAGNITUDE_SLOPE, "min_span": MIN_RAMP_SPAN}
                        if m.rot.scaling is not None else None),
            "max_positions": cfg.max_positions})
        mixer = PartSpec("latent_attention", {
            "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
            "q_rank": m.q_rank, "kv_rank": m.kv_rank, "softmax_scale": m.scale, "norm_eps": cfg.eps, "position": position,
            "window": m.window, "cache_window": keep[owner], "head_gate": gated, "own_latent": m.kv_from is None,
            "out_scale": cfg.residual_mult}, p + "mix.")
        parts = {"mixer_norm": ("norm", PartSpec("layernorm", {"size": W, "eps": cfg.eps, "weight_name": "norm1"}, p)),
                 "mixer": ("mixer", mixer)}
        if l.mlp is not None:
            f = l.mlp
            parts["feed_forward_norm"] = ("norm", PartSpec("layernorm", {"size": W, "eps": cfg.eps, "weight_name": "norm2"}, p))
            parts["feed_forward"] = ("feed_forward", PartSpec("routed_experts", {
                "hidden_size": W, "experts": f.experts, "top": f.top, "expert_size": f.ff, "router_kind": "sigmoid",
                "expert_kind": "relu_squared", "out_scale": cfg.residual_mult}, p + "mlp."))
        layers.append(LayerSpec("prenorm", parts))
        if m.kv_from is None:
            cache_of[i] = len(cache_of)
        schedule.append(LayerCall(i, cache_of[owner], m.kv_from is None))
    spec = ModelSpec(
        architecture=NAME, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions, layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("layernorm", {"size": W, "eps": cfg.eps, "weight_name": "final.norm"}, ""),
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "hidden_size": W, "weight_name": "embed"}, ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False, "weight_name": "head",
                                      "logit_scale": cfg.logit_scale, "softcap": cfg.logit_softcap}, ""),
        eos_token_id=None,
        optional_tensors=tuple(f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.mlp is None))
    spec.validate()
    return spec


ARCHITECTURE = register_architecture(Architecture(NAME, parse, to_spec, to_dict))
