"""Tiny Pefazen configurations for the tests, random weights for them, and the comparison with the plain
implementation (plain_pefazen.py). The configurations differ from each other in every size and option and make
unequal what a model may happen to make equal (key, rotated and value sizes, ranks of the two latents, heads of
neighbouring layers, the window of a layer and of the layer whose latent it reads, the order of the layer kinds,
experts of which all or one are chosen, layers without feed-forward, constants that are 1)."""
from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import helpers as H
import plain_pefazen as pp
from ruvenex_cases import check_bf16


def _mix(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, window=None, kv_from=None, scaling=None, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": dims or rot_dim}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


W1, W2 = "latent_attention", "latent_attention_2"

CASES: Dict[str, dict] = {
    # a windowed layer, a layer that reads its latent through a SHORTER window and other heads, a causal layer with
    # interpolated frequencies whose ramp lies inside the pairs, a layer without feed-forward
    "a": {"architecture": "Pefazen", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.4, "logit_scale": 0.7,
          "logit_softcap": 12.0,
          "layers": [{"type": W1, "mixer": _mix(2, 16, 8, 24, 20, 32, 0.2, 500.0, window=24), "mlp": _moe(6, 2, 24)},
                     {"type": W1, "mixer": _mix(3, 8, 8, 16, 12, 32, 0.3, 500.0, window=9, kv_from=0), "mlp": None},
                     {"type": W2, "mixer": _mix(4, 8, 16, 8, 24, 40, 0.25, 10000.0, scaling=(4.0, 64, 8.0, 1.0)), "mlp": _moe(5, 1, 16)}]},
    # nothing a multiple of eight; the causal kind first, without scaling; a reader whose window is LONGER than its
    # writer's; a reader of a causal layer; all experts chosen; residual constant, logit scale 1 and no cap
    "b": {"architecture": "Pefazen", "vocab": 97, "width": 36, "norm": {"eps": 3e-6}, "residual_mult": 1.0, "logit_scale": 1.0,
          "layers": [{"type": W2, "mixer": _mix(3, 10, 6, 7, 11, 13, 0.3, 50.0), "mlp": _moe(4, 4, 10)},
                     {"type": W1, "mixer": _mix(1, 12, 4, 9, 5, 18, 0.4, 30.0, window=5), "mlp": None},
                     {"type": W1, "mixer": _mix(5, 6, 4, 3, 9, 18, 0.5, 30.0, window=33, kv_from=1), "mlp": _moe(9, 3, 5)},
                     {"type": W2, "mixer": _mix(2, 4, 6, 14, 7, 13, 0.6, 50.0, kv_from=0), "mlp": _moe(3, 2, 7)},
                     {"type": W1, "mixer": _mix(2, 14, 10, 6, 8, 7, 0.2, 2000.0, window=1), "mlp": None}]},
    # large: twelve heads (more than one group of a CTA), latents of 192 and 264 (two and four channel passes),
    # a window of 80, fewer rotated channels than the shared part has, scaling whose ramp's ends are clamped
    "c": {"architecture": "Pefazen", "vocab": 256, "width": 128, "norm": {"eps": 2e-6}, "residual_mult": 0.5, "logit_scale": 2.0,
          "logit_softcap": 5.0,
          "layers": [{"type": W1, "mixer": _mix(12, 64, 32, 48, 96, 192, 0.1, 20000.0, window=80, dims=24), "mlp": _moe(8, 2, 32)},
                     {"type": W2, "mixer": _mix(4, 32, 16, 80, 64, 264, 0.12, 1000000.0, scaling=(2.0, 2048, 32.0, 1.0)), "mlp": _moe(16, 4, 16)},
                     {"type": W1, "mixer": _mix(2, 128, 32, 128, 72, 192, 0.08, 20000.0, window=130, kv_from=0, dims=24), "mlp": None}]},
    # sizes that are multiples of eight throughout (the tensor-core forms in bfloat16): eighteen heads (two groups of
    # sixteen), a reader of a layer that sees everything, values of 136 (beyond what the portion kernel takes: portions
    # stay in the latent form there, single tokens do not), windows of 70 and of exactly one key tile
    "d": {"architecture": "Pefazen", "vocab": 160, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.7, "logit_scale": 1.5,
          "logit_softcap": 8.0,
          "layers": [{"type": W2, "mixer": _mix(18, 16, 16, 16, 48, 64, 0.2, 5000.0, scaling=(3.0, 128, 4.0, 0.5)), "mlp": _moe(4, 1, 24)},
                     {"type": W2, "mixer": _mix(2, 24, 16, 136, 40, 64, 0.15, 5000.0, kv_from=0, scaling=(3.0, 128, 4.0, 0.5)), "mlp": None},
                     {"type": W1, "mixer": _mix(4, 8, 8, 40, 24, 72, 0.3, 300.0, window=70), "mlp": _moe(3, 3, 16)},
                     {"type": W1, "mixer": _mix(3, 32, 8, 8, 32, 72, 0.25, 300.0, window=64, kv_from=2), "mlp": _moe(8, 2, 8)}]},
}


def spec_of(cfg: dict):
    return H.spec_of(cfg)


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, sharp: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random weights; with ``sharp`` the weights of the query latent's norm are multiplied by it, so that attention
    weights are peaked: a position's result then hangs on single keys anywhere in what it sees, up to the far end of
    its window or the first position, and a wrong key or a window one token off shows."""
    from infer_b200.weights import random_weights
    W = random_weights(spec_of(cfg), seed, dtype)
    for k in W:
        # router logits of unit size: scores spread over (0, 1) instead of crowding at its ends, and the roundings that
        # reach a choice score stay far below the usual gap between two experts
        if k.endswith(".mlp.router"):
            W[k] = (W[k].float() * (2.0 / cfg["width"] ** 0.5)).to(dtype)
    if sharp:
        for k in W:
            if k.endswith(".mix.dq.norm"):
                W[k] = (W[k].float() * sharp).to(dtype)
    return W


def write_model(folder: str, cfg: dict, seed: int) -> None:
    """A model folder (config.json, model.safetensors) with the weights of ``make_weights``."""
    from infer_b200.weights import write_random_model
    from infer_b200.weights.safetensors_io import write_safetensors
    write_random_model(folder, cfg, seed, torch.bfloat16)
    write_safetensors(f"{folder}/model.safetensors", make_weights(cfg, seed), metadata={"format": "pt"})


def random_ids(cfg: dict, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@functools.lru_cache(maxsize=64)
def _oracle(cfg_json: str, seed: int, sharp: float, compute: str, ids: Tuple[int, ...], rounding: str):
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), getattr(torch, compute))
    if rounding == "none":
        return pp.forward(cfg, W, list(ids)).numpy()
    with pp.rounded(getattr(torch, rounding)):
        return pp.forward(cfg, W, list(ids)).numpy()


def oracle(cfg: dict, seed: int, compute: torch.dtype, ids: Sequence[int], rounding=None, sharp: float = 0.0) -> np.ndarray:
    n = lambda d: str(d).replace("torch.", "")
    return _oracle(json.dumps(cfg, sort_keys=True), seed, float(sharp), n(compute), tuple(int(i) for i in ids),
                   "none" if rounding is None else n(rounding))


CLOSE_CALL = 0.01      # a router's gap between choice scores below which bfloat16 roundings may turn the choice: the rows a
                       # router reads carry the roundings of the layers before, times the size of its logits


@functools.lru_cache(maxsize=64)
def _router_gaps(cfg_json: str, seed: int, sharp: float, ids: Tuple[int, ...]) -> np.ndarray:
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), torch.bfloat16)
    gaps: List[torch.Tensor] = []
    pp.forward(cfg, W, list(ids), None, gaps)
    return torch.stack(gaps).min(dim=0).values.numpy() if gaps else np.full(len(ids), np.inf)


def check(cfg: dict, seed: int, dtype: torch.dtype, got: Dict[str, Dict[int, np.ndarray]], reqs: Dict[str, List[int]],
          sharp: float = 0.0, what: str = ""):
    """The engine's rows against the plain implementation. In bfloat16, positions at which a router's choice is a
    close call are left out (the other expert is as right an answer there). Where the engine's row at such a position
    is far from the plain one, it took the other expert, and the later positions of that request read keys and
    values of another function in every later layer: they are held to three times the bound (a wrong key, window or
    rotation moves a row by far more, and the runs with peaked attention show it). A wrong choice where the call is
    not close is not excused. The float32 comparison leaves out nothing and is the sharp one; cuttings are compared
    bit by bit there. The bound is five times the noise of the plain implementation with bfloat16 roundings: the
    engine rounds in two more places per mixer than that has (the query carried into the latent space, and the
    weighted sum of latent rows before the value up-projection)."""
    kept = asked = 0
    for rid, ids in reqs.items():
        ref = oracle(cfg, seed, dtype, ids, None, sharp)
        rows = sorted(got[rid])
        if dtype != torch.float32:
            rounded = oracle(cfg, seed, dtype, ids, torch.bfloat16, sharp)
            gaps = _router_gaps(json.dumps(cfg, sort_keys=True), seed, float(sharp), tuple(int(i) for i in ids))
            rms = lambda a: float(np.sqrt(np.mean(a ** 2)))
            noise = rms(rounded - ref)
            turned = [p for p in rows if gaps[p] < CLOSE_CALL and rms(got[rid][p] - ref[p]) > 5.0 * max(noise, rms(rounded[p] - ref[p]))]
            end = min(turned) if turned else len(ids)
            clear = [p for p in rows if gaps[p] >= CLOSE_CALL]
            asked += len(rows)
            kept += len(clear)
            after = [p for p in clear if p > end]
            if after:
                check_bf16(np.stack([got[rid][p] for p in after]), ref[after], rounded[after], f"{what}/{rid} (after a turned choice)", factor=15.0)
            rows = [p for p in clear if p < end]
            if not rows:
                continue
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            H.check_f32(g, ref[rows], f"{what}/{rid}")
        else:
            check_bf16(g, ref[rows], rounded[rows], f"{what}/{rid}", factor=5.0)
    assert kept >= 0.3 * asked, f"{what}: only {kept} of {asked} positions are clear of close calls"
