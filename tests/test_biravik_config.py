"""Biravik without a GPU: configuration, tensor names, sizes that only a checkpoint states, cache needs with kept first
pages, and the plain implementation's own consistency."""
import copy
import math

import pytest
import torch

import biravik_cases as BC
import infer_b200.models  # noqa: F401  (registers the architectures)
import infer_b200.parts  # noqa: F401
import plain_biravik as pb
from infer_b200.cache.manager import CacheManager
from infer_b200.config import parse_config
from infer_b200.config.registry import ConfigError
from infer_b200.models import load_preset
from infer_b200.models.biravik import distance_slopes
from infer_b200.parts.base import CompositeNeed, PagedKVNeed, StateNeed, part_class
from infer_b200.parts.rotary import interpolated_frequencies
from infer_b200.weights.binder import WeightsError, check_weights, expected_tensors

F = torch.float64


@pytest.mark.parametrize("name", sorted(BC.CASES))
def test_config_round_trip_and_tensor_names(name):
    cfg = BC.CASES[name]
    arch, typed = parse_config(cfg)
    assert arch.name == "Biravik"
    assert arch.parse(arch.to_dict(typed)) == typed
    names = expected_tensors(arch.to_spec(typed))
    W = cfg["width"]
    assert {"embed", "final.norm", "head"} <= set(names)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        assert names[p + "norm1"][0] == (W,)
        assert ((p + "norm2") in names) == (l["mlp"] is not None)
        if l["type"] == "attention":
            assert names[p + "mix.q"][0] == (m["heads"] * m["dim"], W) and names[p + "mix.k"][0] == (m["kv_heads"] * m["dim"], W)
            assert (p + "mix.v") not in names                                    # the values are the projected keys
            assert names[p + "mix.q.norm"][0] == names[p + "mix.k.norm"][0] == (m["dim"],)
            assert names[p + "mix.g"][0] == (m["heads"] * m["dim"], W) and names[p + "mix.o"][0] == (W, m["heads"] * m["dim"])
            assert names[p + "mix.sink"][0] == (m["heads"],)
        elif l["type"] == "wkv":
            C = m["heads"] * m["dim"]
            for s in "rkvgw":
                assert names[p + "mix.mu." + s][0] == (W,)
            assert names[p + "mix.r"][0] == names[p + "mix.k"][0] == names[p + "mix.v"][0] == names[p + "mix.g"][0] == (C, W)
            assert names[p + "mix.w1"][0] == (m["rank"], W) and names[p + "mix.w2"][0] == (C, m["rank"]) and names[p + "mix.w0"][0] == (C,)
            assert names[p + "mix.u"][0] == (m["heads"], m["dim"]) and names[p + "mix.norm"][0] == (C,) and names[p + "mix.o"][0] == (W, C)
        else:
            a, b = m["left"], m["right"]
            assert names[p + "mix.left.q"][0] == (a["heads"] * a["dim"], W) and names[p + "mix.left.k"][0] == (a["kv_heads"] * a["dim"], W)
            assert names[p + "mix.left.v"][0] == (a["kv_heads"] * a["vdim"], W)
            assert names[p + "mix.left.g"][0] == (a["heads"] * a["vdim"], W) and names[p + "mix.left.o"][0] == (W, a["heads"] * a["vdim"])
            assert names[p + "mix.left.q.norm"][0] == (a["dim"],) and names[p + "mix.left.sink"][0] == (a["heads"],)
            assert names[p + "mix.right.q"][0] == names[p + "mix.right.k"][0] == (b["heads"] * b["dim"], W)
            assert names[p + "mix.right.v"][0] == names[p + "mix.right.g"][0] == (b["heads"] * b["vdim"], W)
            assert names[p + "mix.right.norm"][0] == (b["heads"] * b["vdim"],)
        if l["mlp"] and l["mlp"]["kind"] == "moe":
            r = l["mlp"]["router"]
            assert names[p + "mlp.router"][0] == (r["experts"], W)
            assert names[p + f"mlp.e{r['experts'] - 1}.gate"][0] == (l["mlp"]["expert"]["ff"], W)
            assert names[p + f"mlp.e{r['experts'] - 1}.down"][0] == (W, l["mlp"]["expert"]["ff"])
        elif l["mlp"]:
            assert names[p + "mlp.up"][0] == (l["mlp"]["ff"], W) and names[p + "mlp.down"][0] == (W, l["mlp"]["ff"])
            assert (p + "mlp.gate") not in names


def test_presets_parse():
    for n in ("tiny-biravik", "biravik-1.5b", "biravik-7b"):
        arch, typed = parse_config(load_preset(n))
        assert arch.name == "Biravik" and arch.to_spec(typed).layers


def _broken(path, value=None, delete=False):
    cfg = copy.deepcopy(BC.CASES["a"])
    node = cfg
    for k in path[:-1]:
        node = node[k]
    if delete:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,delete,word", [
    (("postln_alpha",), None, True, "postln_alpha"),
    (("norm",), None, True, "norm"),
    (("layers", 0, "type"), "gla", False, "not a layer"),
    (("layers", 1, "mixer", "vdim"), 8, False, "vdim"),
    (("layers", 1, "mixer", "kv_heads"), 3, False, "multiple"),
    (("layers", 1, "mixer", "rot", "dims"), 7, False, "even"),
    (("layers", 1, "mixer", "rot", "dims"), 32, False, "at most"),
    (("layers", 1, "mixer", "mask", "size"), 0, False, "size"),
    (("layers", 2, "mixer", "right", "decay"), [0.5], False, "one number per head"),
    (("layers", 2, "mixer", "left_scale"), None, True, "left_scale"),
    (("layers", 2, "mixer", "left", "q_temp", "every"), 0, False, "every"),
    (("layers", 1, "mlp", "router", "top"), 7, False, "cannot be chosen"),
    (("layers", 0, "mlp", "kind"), "glu", False, "not a feed-forward"),
])
def test_refusals_name_the_key(path, value, delete, word):
    with pytest.raises(ConfigError) as e:
        parse_config(_broken(path, value, delete))
    assert word in str(e.value)


def test_options_that_may_be_absent():
    cfg = copy.deepcopy(BC.CASES["a"])
    cfg["layers"][1]["mixer"]["mask"] = None
    cfg["layers"][1]["mixer"]["rot"]["scaling"] = None
    del cfg["layers"][1]["mixer"]["kv_heads"]
    cfg["layers"][2]["mixer"]["left"]["q_temp"] = None
    del cfg["embedding"]
    arch, typed = parse_config(cfg)
    assert typed.layers[1].mixer.window is None and typed.layers[1].mixer.kv_heads == 4 and typed.embedding_scale == 1.0
    spec = arch.to_spec(typed)
    att = spec.layers[1].part("mixer")
    assert att["window"] is None and att["keep_first"] == 0 and att["position"]["scaling"] is None
    assert "query_temperature" not in spec.layers[2].part("mixer")["first"].params


def test_one_error_lists_what_is_missing_and_a_missing_rank_is_read_from_the_tensors():
    cfg = copy.deepcopy(BC.CASES["a"])
    W = BC.make_weights(cfg, 3)
    del cfg["layers"][0]["mixer"]["rank"]
    arch, typed = parse_config(cfg)
    spec = arch.to_spec(typed)
    check_weights(W, spec)                                     # the rank of 4 is the stored tensors'
    broken = dict(W)
    del broken["l1.mix.sink"], broken["l2.mix.right.norm"]
    broken["l0.mix.u"] = torch.zeros(3, 3)
    with pytest.raises(WeightsError) as e:
        check_weights(broken, spec)
    for word in ("l1.mix.sink", "l2.mix.right.norm", "l0.mix.u"):
        assert word in str(e.value)


def test_cache_needs_and_kept_first_pages():
    arch, typed = parse_config(BC.CASES["b"])
    spec = arch.to_spec(typed)
    needs = {}
    for i, ls in enumerate(spec.layers):
        ps = ls.part("mixer")
        needs[i] = part_class("mixer", ps.kind)(ps, _NoDevice()).cache_need()
    assert isinstance(needs[0], CompositeNeed) and isinstance(needs[0].parts["first"], PagedKVNeed)
    assert needs[0].parts["first"].window is None and needs[0].parts["first"].value_dim == 7
    assert needs[0].parts["second"].shapes["S"][0] == (3, 5, 9)
    assert needs[1] == PagedKVNeed(1, 10, 33, None, keep_first=18)
    assert isinstance(needs[2], StateNeed) and needs[2].shapes["S"][0] == (3, 5, 5) and needs[2].shapes["last"][0] == (36,)
    assert needs[3] == PagedKVNeed(2, 6, 5, None) and needs[4] == PagedKVNeed(1, 12, 3, None, keep_first=1)
    mgr = CacheManager(needs, n_pages=12, page_size=16, n_slots=2)
    group = mgr.group_of_cache[1][0]
    mgr.admit("x")
    for _ in range(10):
        assert mgr.reserve("x", 16)
        mgr.advance("x", 16)
    table = mgr.block_table("x", group)
    # 160 positions, a window of 33 keeping 18: pages 0 and 1 hold kept keys, page 7 (positions 112..127) is the first
    # that a later query's window can reach (160 - 33 + 1 = 128 is its first key), so 2..7 went back
    assert [p >= 0 for p in table] == [True, True] + [False] * 6 + [True, True]
    plain_group = mgr.group_of_cache[3][0]
    assert [p >= 0 for p in mgr.block_table("x", plain_group)] == [False] * 9 + [True]
    mgr.check_invariants()
    mgr.release("x")
    assert mgr.pages_in_use() == [0] * len(mgr.groups)
    mgr.admit("y")
    assert mgr.reserve("y", 40)                                # the pages that came back are used again
    mgr.check_invariants()


class _NoDevice:
    """Enough of a runtime to build a part for its cache need (nothing is loaded)."""
    dtype = torch.float32
    device = torch.device("cpu")
    max_seq_len = 64

    def fast(self, op):
        return False


def test_slopes_and_frequencies():
    assert distance_slopes(4) == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8]
    assert torch.allclose(pb.distance_slopes(3), torch.tensor(distance_slopes(3), dtype=F))
    for dims, base, sc in ((8, 1000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}), (64, 20000.0, None),
                           (2, 10000.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5})):
        f, mag = interpolated_frequencies(dims, base, dict(sc, magnitude_slope=0.1, min_span=0.001) if sc else None)
        g, mag2 = pb.interpolated_frequencies(dims, base, sc)
        assert torch.allclose(f, g, rtol=1e-14) and mag == mag2
        if sc:
            assert math.isclose(mag, 0.1 * math.log(sc["factor"]) + 1.0)
            assert bool((g <= base ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims) + 1e-18).all())


# ----------------------------------------------------------------------------- the plain implementation against itself

def test_what_a_window_with_kept_first_keys_sees():
    ok = pb.visible(12, 4, 2)
    assert ok[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert ok[3].tolist() == [True] * 4 + [False] * 8 and ok[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert ok[6].tolist() == [True, True, False, True, True, True, True] + [False] * 5
    assert pb.visible(5, None, 0).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()


def test_a_sink_takes_weight_and_gives_nothing():
    scores = torch.zeros(1, 1, 3, dtype=F)
    mask = torch.ones(1, 3, dtype=torch.bool)
    w = pb.attention_weights(scores, mask, torch.tensor([math.log(3.0)], dtype=F))
    assert torch.allclose(w, torch.full((1, 1, 3), 1.0 / 6.0, dtype=F))
    assert torch.allclose(pb.attention_weights(scores, mask, None).sum(-1), torch.ones(1, 1, dtype=F))


def test_scans_can_be_cut_anywhere_and_the_bonus_reads_the_current_token_only():
    g = torch.Generator().manual_seed(0)
    r, k, w = (torch.rand(9, 5, generator=g, dtype=F) for _ in range(3))
    v, u = torch.randn(9, 7, generator=g, dtype=F), torch.randn(5, generator=g, dtype=F)
    whole, S = pb.bonus_scan(r, k, v, w, u)
    a, Sa = pb.bonus_scan(r[:4], k[:4], v[:4], w[:4], u)
    b, Sb = pb.bonus_scan(r[4:], k[4:], v[4:], w[4:], u, Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(S, Sb)
    assert torch.allclose(whole[0], (u * k[0] * r[0]).sum() * v[0])            # nothing before it: the bonus alone
    whole2, S2 = pb.constant_decay_scan(r, k, v, 0.9)
    c, Sc = pb.constant_decay_scan(r[:1], k[:1], v[:1], 0.9)
    d, Sd = pb.constant_decay_scan(r[1:], k[1:], v[1:], 0.9, Sc)
    assert torch.allclose(torch.cat([c, d]), whole2) and torch.allclose(S2, Sd)
    assert torch.allclose(pb.constant_decay_scan(r, k, v, 0.0)[0], (r * k).sum(-1, keepdim=True) * v)   # no memory at all


def test_the_router_takes_the_softmax_over_the_chosen_logits_only():
    z = torch.tensor([[1.0, 3.0, 2.0, -1.0]], dtype=F)
    chosen, w, gap = pb.route_top(z, 2)
    assert chosen.tolist() == [[1, 2]] and torch.allclose(w, torch.softmax(torch.tensor([[3.0, 2.0]], dtype=F), -1)) and float(gap) == 1.0
    chosen, w, _ = pb.route_top(z, 4)
    assert sorted(chosen[0].tolist()) == [0, 1, 2, 3] and math.isclose(float(w.sum()), 1.0)


def test_a_prefix_does_not_depend_on_what_follows():
    cfg = BC.CASES["b"]
    W = BC.make_weights(cfg, 5)
    import helpers as H
    Wc = H.as_compute(W, torch.float32)
    ids = BC.random_ids(cfg, 50, 9)
    assert torch.allclose(pb.forward(cfg, Wc, ids)[:30], pb.forward(cfg, Wc, ids[:30]), atol=1e-12)
