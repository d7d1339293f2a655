"""Biravik: typed configuration and its translation into a ModelSpec.

A decoder whose layers normalise AFTER the residual sum, and whose sublayers read the stream x itself:

    x <- norm_1(alpha x + mixer(x));    x <- norm_2(alpha x + feed_forward(x))          (second line absent without one)

with norm(y) = y / sqrt(mean(y^2) + eps) * (1 + w) (the stored weight lies around zero; parts/rmsnorm.py with
``weight_offset``) and the block kind "postnorm" (parts/block.py). The token table's rows are multiplied by a constant;
the same kind of norm precedes the output matrix. Three kinds of layer, in any order:

"attention"  grouped-query softmax attention (parts/attention.py): q and k normalised per head with a weight the heads
             share, channel pairs rotated with interpolated frequencies (parts/rotary.py), a sliding window that keeps
             the first keys, a sink, the projected keys as values, a sigmoid gate per output channel
"parallel"   two mixers on the same rows (parts/side_by_side.py), left_scale * left + right_scale * right. Left: the same
             attention without rotation, window or shared values, with a temperature on the queries that grows with
             the position and a slope_h * distance taken off the scores, slope_h = 2^(-8 (h + 1) / heads). Right: linear
             attention whose state fades by a constant per head (parts/constant_decay.py)
"wkv"        time mixing over mixtures of a token's row with its predecessor's, a decay per key channel and token, a
             bonus for the current token (parts/shifted_mixing.py)

Feed-forwards: dense with relu squared (parts/dense_ff.py), or a mixture of gated experts whose router takes the
softmax over the chosen logits only (parts/routed_ff.py), or none.

config.json keys (all sizes and constants come from there or from the tensors' shapes; tensor names are fixed):

    architecture "Biravik"; vocab; width; norm.eps; postln_alpha; embedding.scale; layers[i] = {type, mixer, mlp}
      type "attention": mixer {heads, kv_heads, dim, vdim (= dim), scale, mask: {size, keep_first} | null,
                               rot: {base, dims, scaling: {factor, original, fast, slow} | null} | null}
      type "parallel":  mixer {left: {heads, kv_heads, dim, vdim, scale, q_temp: {coef, every} | null}, left_scale,
                               right: {heads, dim, vdim, decay: [per head]}, right_scale}
      type "wkv":       mixer {heads, dim}                    (the decay's rank is the stored tensors')
      mlp {kind: "dense", ff} | {kind: "moe", router: {experts, top}, expert: {ff}} | null

A configuration written for a random model also carries ``rank`` (wkv), which a checkpoint's tensors otherwise state.

Tensors: embed, final.norm, head, and per layer l<i>.: norm1, norm2, mix.* and mlp.* as the parts name them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from ..config.registry import Architecture, ConfigError, register_architecture
from ..config.specs import LayerCall, LayerSpec, ModelSpec, PartSpec

NAME = "Biravik"
DEFAULT_MAX_POSITIONS = 1 << 20       # the design states no limit; an engine's own sequence limit sizes its tables
# constants that the design fixes
SLOPE_EXPONENT = 8.0                  # head h of H takes the slope 2^(-SLOPE_EXPONENT (h + 1) / H)
MAGNITUDE_SLOPE = 0.1                 # cosines and sines times MAGNITUDE_SLOPE * ln(factor) + 1
MIN_RAMP_SPAN = 0.001                 # least width of the ramp between kept and divided frequencies
NORM_WEIGHT_OFFSET = 1.0              # the layers' norms multiply by (1 + stored weight)


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]]     # (factor, original, fast, slow)


@dataclass(frozen=True)
class SoftmaxMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    keep_first: int = 0
    rot: Optional[Rotation] = None
    q_temp: Optional[Tuple[float, int]] = None                # (coef, every)


@dataclass(frozen=True)
class FadingSide:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxMixer
    left_scale: float
    right: FadingSide
    right_scale: float


@dataclass(frozen=True)
class ShiftedMixer:
    heads: int
    dim: int
    rank: Optional[int]                # None: the stored tensors state it


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class BiravikLayer:
    mixer: Union[SoftmaxMixer, ParallelMixer, ShiftedMixer]
    mlp: Union[DenseFF, RoutedFF, None]


@dataclass(frozen=True)
class BiravikConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    embedding_scale: float
    layers: Tuple[BiravikLayer, ...]
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


def _opt_int(raw, key, where, minimum=1) -> Optional[int]:
    return _int(raw, key, where, minimum) if isinstance(raw, Mapping) and raw.get(key) is not None else None


def _num(raw, key, where, positive=False) -> float:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _softmax_mixer(raw, where: str, shared_values: bool) -> SoftmaxMixer:
    heads = _int(raw, "heads", where)
    kv = _opt_int(raw, "kv_heads", where) or heads
    if heads % kv:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv})")
    dim = _int(raw, "dim", where)
    vdim = _opt_int(raw, "vdim", where) or dim
    if shared_values and vdim != dim:
        raise ConfigError(f"config.json: {where}.vdim ({vdim}) must equal dim ({dim}): the values are the projected keys")
    mask, rot, temp = raw.get("mask"), raw.get("rot"), raw.get("q_temp")
    window = _int(mask, "size", where + ".mask") if mask is not None else None
    keep = (_opt_int(mask, "keep_first", where + ".mask", 0) or 0) if mask is not None else 0
    rotation = None
    if rot is not None:
        dims = _int(rot, "dims", where + ".rot", 2)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        base = _num(rot, "base", where + ".rot", positive=True)
        if base <= 1:
            raise ConfigError(f"config.json: {where}.rot.base must be above 1, got {base}")
        sc = rot.get("scaling")
        scaling = tuple(_num(sc, k, where + ".rot.scaling", positive=True) for k in ("factor", "original", "fast", "slow")) if sc is not None else None
        rotation = Rotation(base, dims, scaling)
    q_temp = (_num(temp, "coef", where + ".q_temp"), _int(temp, "every", where + ".q_temp")) if temp is not None else None
    return SoftmaxMixer(heads, kv, dim, vdim, _num(raw, "scale", where), window, keep, rotation, q_temp)


def _mixer(kind: str, raw, where: str):
    if kind == "attention":
        return _softmax_mixer(raw, where, shared_values=True)
    if kind == "wkv":
        return ShiftedMixer(_int(raw, "heads", where), _int(raw, "dim", where), _opt_int(raw, "rank", where))
    lraw, rraw = _get(raw, "left", where), _get(raw, "right", where)
    rw = where + ".right"
    heads = _int(rraw, "heads", rw)
    decay = _get(rraw, "decay", rw)
    if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in decay):
        raise ConfigError(f"config.json: {rw}.decay must list one number per head ({heads})")
    dim = _int(rraw, "dim", rw)
    right = FadingSide(heads, dim, _opt_int(rraw, "vdim", rw) or dim, tuple(float(v) for v in decay))
    return ParallelMixer(_softmax_mixer(lraw, where + ".left", shared_values=False), _num(raw, "left_scale", where), right,
                         _num(raw, "right_scale", where))


def _mlp(raw, where: str):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind == "dense":
        return DenseFF(_int(raw, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design ('dense', 'moe')")
    router, expert = _get(raw, "router", where), _get(raw, "expert", where)
    experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: {top} of {experts} experts cannot be chosen")
    return RoutedFF(experts, top, _int(expert, "ff", where + ".expert"))


def parse(raw: Mapping[str, Any]) -> BiravikConfig:
    layers = _get(raw, "layers", "the configuration")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    out = []
    for i, l in enumerate(layers):
        where = f"layers[{i}]"
        kind = _get(l, "type", where)
        if kind not in ("attention", "parallel", "wkv"):
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design ('attention', 'parallel', 'wkv')")
        out.append(BiravikLayer(_mixer(kind, _get(l, "mixer", where), where + ".mixer"), _mlp(l.get("mlp"), where + ".mlp")))
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"config.json: max_positions must be a positive integer, got {max_positions!r}")
    emb = raw.get("embedding")
    return BiravikConfig(vocab=_int(raw, "vocab", "the configuration"), width=_int(raw, "width", "the configuration"),
                         eps=_num(_get(raw, "norm", "the configuration"), "eps", "norm", positive=True),
                         alpha=_num(raw, "postln_alpha", "the configuration"),
                         embedding_scale=_num(emb, "scale", "embedding") if emb is not None else 1.0,
                         layers=tuple(out), max_positions=max_positions)


def _softmax_dict(a: SoftmaxMixer, shared_values: bool) -> Dict[str, Any]:
    d: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
    if shared_values:
        d["mask"] = {"size": a.window, "keep_first": a.keep_first} if a.window is not None else None
        d["rot"] = None
        if a.rot is not None:
            sc = a.rot.scaling
            d["rot"] = {"base": a.rot.base, "dims": a.rot.dims,
                        "scaling": dict(zip(("factor", "original", "fast", "slow"), sc)) if sc is not None else None}
    else:
        d["q_temp"] = {"coef": a.q_temp[0], "every": a.q_temp[1]} if a.q_temp is not None else None
    return d


def to_dict(cfg: BiravikConfig) -> Dict[str, Any]:
    layers = []
    for l in cfg.layers:
        m = l.mixer
        if isinstance(m, SoftmaxMixer):
            kind, mixer = "attention", _softmax_dict(m, True)
        elif isinstance(m, ShiftedMixer):
            kind, mixer = "wkv", {"heads": m.heads, "dim": m.dim}
            if m.rank is not None:
                mixer["rank"] = m.rank
        else:
            b = m.right
            kind = "parallel"
            mixer = {"left": _softmax_dict(m.left, False), "left_scale": m.left_scale,
                     "right": {"heads": b.heads, "dim": b.dim, "vdim": b.vdim, "decay": list(b.decay)}, "right_scale": m.right_scale}
        f = l.mlp
        if f is None:
            mlp = None
        elif isinstance(f, DenseFF):
            mlp = {"kind": "dense", "ff": f.ff}
        else:
            mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.ff}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    d = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "postln_alpha": cfg.alpha,
         "embedding": {"scale": cfg.embedding_scale}, "layers": layers}
    if cfg.max_positions != DEFAULT_MAX_POSITIONS:
        d["max_positions"] = cfg.max_positions
    return d


_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}


def distance_slopes(heads: int):
    return [2.0 ** (-SLOPE_EXPONENT * (h + 1) / heads) for h in range(heads)]


def _softmax_spec(a: SoftmaxMixer, W: int, eps: float, max_positions: int, shared_values: bool, prefix: str = "") -> PartSpec:
    params: Dict[str, Any] = {
        "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
        "window": a.window, "softmax_scale": a.scale, "position": None, "qk_head_norm_eps": eps, "channel_gate": True, "sink": True,
        "names": _ATTENTION_NAMES}
    if shared_values:
        params["values_are_keys"] = True
        params["keep_first"] = a.keep_first if a.window is not None else 0
    else:
        params["distance_slopes"] = distance_slopes(a.heads)
    if a.q_temp is not None:
        params["query_temperature"] = {"coef": a.q_temp[0], "every": a.q_temp[1]}
    if a.rot is not None:
        sc = a.rot.scaling
        scaling = None if sc is None else {"factor": sc[0], "original": sc[1], "fast": sc[2], "slow": sc[3],
                                           "magnitude_slope": MAGNITUDE_SLOPE, "min_span": MIN_RAMP_SPAN}
        params["position"] = PartSpec("rotary_interpolated", {"theta": a.rot.base, "rotary_dims": a.rot.dims, "head_dim": a.dim,
                                                              "layout": "pairs", "scaling": scaling, "max_positions": max_positions})
    return PartSpec("attention", params, prefix)


def _mixer_spec(m, W: int, eps: float, max_positions: int) -> PartSpec:
    if isinstance(m, SoftmaxMixer):
        return _softmax_spec(m, W, eps, max_positions, True)
    if isinstance(m, ShiftedMixer):
        return PartSpec("shifted_decay_mixing", {"hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "norm_eps": eps,
                                                 "decay_rank": m.rank})
    b = m.right
    right = PartSpec("constant_decay_attention", {
        "hidden_size": W, "num_heads": b.heads, "head_dim": b.dim, "v_head_dim": b.vdim, "decay": list(b.decay), "norm_eps": eps,
        "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm"}}, "right.")
    return PartSpec("side_by_side", {"first": _softmax_spec(m.left, W, eps, max_positions, False, "left."), "second": right,
                                     "first_scale": m.left_scale, "second_scale": m.right_scale, "hidden_size": W})


def _mlp_spec(f, W: int) -> PartSpec:
    if isinstance(f, DenseFF):
        return PartSpec("dense", {"hidden_size": W, "intermediate_size": f.ff, "activation": "relu_squared",
                                  "names": {"up": "up", "down": "down"}})
    return PartSpec("routed_experts", {"hidden_size": W, "experts": f.experts, "top": f.top, "expert_size": f.ff,
                                       "router_kind": "softmax_top", "expert_kind": "swish_glu"})


def _with_prefix(spec: PartSpec, prefix: str) -> PartSpec:
    return PartSpec(spec.kind, spec.params, prefix)


def _norm(W: int, eps: float, name: str, prefix: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": W, "eps": eps, "weight_name": name, "weight_offset": NORM_WEIGHT_OFFSET}, prefix)


def to_spec(cfg: BiravikConfig) -> ModelSpec:
    W = cfg.width
    layers, optional = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {
            "mixer": ("mixer", _with_prefix(_mixer_spec(l.mixer, W, cfg.eps, cfg.max_positions), p + "mix.")),
            "mixer_norm": ("norm", _norm(W, cfg.eps, "norm1", p)),
        }
        if l.mlp is not None:
            parts["feed_forward"] = ("feed_forward", _with_prefix(_mlp_spec(l.mlp, W), p + "mlp."))
            parts["feed_forward_norm"] = ("norm", _norm(W, cfg.eps, "norm2", p))
        else:
            optional.append(p + "norm2")                 # a norm with nothing to normalise may be stored all the same
        layers.append(LayerSpec("postnorm", parts, {"residual_scale": cfg.alpha}))
    spec = ModelSpec(
        architecture=NAME, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions, layers=tuple(layers),
        schedule=tuple(LayerCall(i, i) for i in range(len(layers))),
        final_norm=_norm(W, cfg.eps, "final.norm", ""),
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "hidden_size": W, "weight_name": "embed",
                                           "scale": cfg.embedding_scale}, ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False, "weight_name": "head"}, ""),
        eos_token_id=None, optional_tensors=tuple(optional))
    spec.validate()
    return spec


ARCHITECTURE = register_architecture(Architecture(NAME, parse, to_spec, to_dict))
