"""Tiny Biravik configurations for the tests, random weights for them, and the comparison with the plain
implementation (plain_biravik.py). The configurations differ from each other in every size and option and make
unequal what a model may happen to make equal (key and value sizes, heads of the two sides, kv heads and 1, the
order of the layer types, windows below and above a page or a key chunk, kept first keys within and across pages,
rotations over all or part of a head with and without interpolation, temperatures that change every token or never,
routers that choose one, some or all experts)."""
from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import helpers as H
import plain_biravik as pb
from ruvenex_cases import check_bf16


def _att(heads, kv, dim, scale, mask, rot):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
            "mask": None if mask is None else {"size": mask[0], "keep_first": mask[1]},
            "rot": None if rot is None else {"base": rot[0], "dims": rot[1],
                                             "scaling": None if rot[2] is None else dict(zip(("factor", "original", "fast", "slow"), rot[2]))}}


def _left(heads, kv, dim, vdim, scale, temp):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
            "q_temp": None if temp is None else {"coef": temp[0], "every": temp[1]}}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _par(left, ls, right, rs):
    return {"left": left, "left_scale": ls, "right": right, "right_scale": rs}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _base(vocab, width, eps, alpha, scale, layers):
    return {"architecture": "Biravik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "embedding": {"scale": scale}, "layers": layers}


CASES: Dict[str, dict] = {
    # a shifted-mixing layer first (its first token mixes with zeros), a window of 24 that keeps 5 keys, rotation over
    # half a head with interpolation, a parallel layer whose temperature steps every 7 tokens
    "a": _base(200, 64, 1e-5, 2.0, 4.0, [
        {"type": "wkv", "mixer": {"heads": 2, "dim": 16, "rank": 4}, "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention", "mixer": _att(4, 2, 16, 0.3, (24, 5), (1000.0, 8, (4.0, 64, 8.0, 1.0))), "mlp": _moe(6, 2, 24)},
        {"type": "parallel", "mixer": _par(_left(4, 2, 16, 24, 0.2, (0.5, 7)), 0.7, _right(2, 16, 32, (0.5, 0.97)), 1.2),
         "mlp": {"kind": "dense", "ff": 40}}]),
    # nothing a multiple of eight; the parallel layer first; a window of 33 keeping 18 (across a page border), one of 5
    # keeping none and one of 3 keeping 1; rotation without interpolation; no temperature; a layer without
    # feed-forward; a router that uses every expert and one that chooses a single one; one kv head; decays 1 and 0
    "b": _base(97, 36, 3e-6, 1.0, 1.0, [
        {"type": "parallel", "mixer": _par(_left(3, 3, 10, 7, 0.3, None), 1.0, _right(3, 5, 9, (1.0, 0.0, 0.9)), 0.5), "mlp": None},
        {"type": "attention", "mixer": _att(3, 1, 10, 0.4, (33, 18), (50.0, 10, None)), "mlp": _moe(4, 4, 10)},
        {"type": "wkv", "mixer": {"heads": 3, "dim": 5, "rank": 3}, "mlp": _moe(9, 1, 5)},
        {"type": "attention", "mixer": _att(2, 2, 6, 0.5, (5, 0), None), "mlp": {"kind": "dense", "ff": 20}},
        {"type": "attention", "mixer": _att(1, 1, 12, 0.25, (3, 1), (10000.0, 2, (2.0, 16, 4.0, 0.5))), "mlp": None},
        {"type": "parallel", "mixer": _par(_left(1, 1, 12, 6, 0.5, (1.5, 1)), 0.3, _right(1, 12, 6, (0.8,)), 2.0), "mlp": _moe(5, 3, 7)}]),
    # sizes the tensor-core kernels take: keys and values of 64 and 128, a window of 150 keeping 40 (both across key
    # chunks of 128), no mask at all, eight heads on two kv heads, states of 128 x 64
    "c": _base(256, 128, 2e-6, 3.0, 12.0, [
        {"type": "parallel", "mixer": _par(_left(8, 2, 64, 64, 0.11, (0.3, 50)), 0.8, _right(3, 24, 40, (0.6, 0.9, 0.999)), 0.9),
         "mlp": _moe(8, 2, 32)},
        {"type": "attention", "mixer": _att(4, 1, 64, 0.12, (150, 40), (30000.0, 64, (6.0, 256, 24.0, 1.5))), "mlp": {"kind": "dense", "ff": 256}},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 128, "rank": 16}, "mlp": None},
        {"type": "attention", "mixer": _att(2, 2, 128, 0.09, None, (500.0, 32, None)), "mlp": _moe(3, 2, 64)},
        {"type": "parallel", "mixer": _par(_left(2, 2, 128, 128, 0.08, None), 1.1, _right(2, 128, 64, (0.95, 0.5)), 0.4),
         "mlp": {"kind": "dense", "ff": 64}}]),
}


def spec_of(cfg: dict):
    return H.spec_of(cfg)


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, sharp: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random weights; with ``sharp`` the weights of the query norms are multiplied by it, so that attention weights
    are peaked: a position's result then hangs on single keys (the farthest its window still holds, a kept first
    key, a key hundreds of positions back), and a wrong key, a lost sink or a window one token off shows."""
    from infer_b200.weights import random_weights
    W = random_weights(spec_of(cfg), seed, dtype)
    if sharp:
        for k in W:
            if k.endswith("q.norm"):
                W[k] = (W[k].float() * sharp).to(dtype)
    return W


def random_ids(cfg: dict, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@functools.lru_cache(maxsize=64)
def _oracle(cfg_json: str, seed: int, sharp: float, compute: str, ids: Tuple[int, ...], rounding: str):
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), getattr(torch, compute))
    if rounding == "none":
        return pb.forward(cfg, W, list(ids)).numpy()
    with pb.rounded(getattr(torch, rounding)):
        return pb.forward(cfg, W, list(ids)).numpy()


def oracle(cfg: dict, seed: int, compute: torch.dtype, ids: Sequence[int], rounding=None, sharp: float = 0.0) -> np.ndarray:
    n = lambda d: str(d).replace("torch.", "")
    return _oracle(json.dumps(cfg, sort_keys=True), seed, float(sharp), n(compute), tuple(int(i) for i in ids),
                   "none" if rounding is None else n(rounding))


CLOSE_CALL = 0.05      # a router's gap between its last chosen and first refused logit below which bfloat16 roundings may turn the choice


@functools.lru_cache(maxsize=64)
def _router_gaps(cfg_json: str, seed: int, sharp: float, ids: Tuple[int, ...]) -> np.ndarray:
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), torch.bfloat16)
    gaps: List[torch.Tensor] = []
    pb.forward(cfg, W, list(ids), None, gaps)
    return torch.stack(gaps).min(dim=0).values.numpy() if gaps else np.full(len(ids), np.inf)


def check(cfg: dict, seed: int, dtype: torch.dtype, got: Dict[str, Dict[int, np.ndarray]], reqs: Dict[str, List[int]],
          sharp: float = 0.0, what: str = ""):
    """The engine's rows against the plain implementation. In bfloat16, positions from the first one at which a
    router's choice is a close call are left out (the other expert is as right an answer there, and every later
    position reads what that one left in the caches and states). The float32 comparison leaves out nothing and is
    the sharp one; cuttings are compared bit by bit there."""
    for rid, ids in reqs.items():
        ref = oracle(cfg, seed, dtype, ids, None, sharp)
        rows = sorted(got[rid])
        if dtype != torch.float32:
            gaps = _router_gaps(json.dumps(cfg, sort_keys=True), seed, float(sharp), tuple(int(i) for i in ids))
            close = np.nonzero(gaps < CLOSE_CALL)[0]
            upto = int(close[0]) if len(close) else len(ids)
            rows = [p for p in rows if p < upto]
            if not rows:
                continue
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            H.check_f32(g, ref[rows], f"{what}/{rid}")
        else:
            check_bf16(g, ref[rows], oracle(cfg, seed, dtype, ids, torch.bfloat16, sharp)[rows], f"{what}/{rid}", factor=4.0)
