"""Pefazen without a GPU: configuration, tensor names, the run order with shared caches, cache needs and windows,
the rotation tables, and the plain implementation's own consistency."""
import copy
import math

import pytest
import torch

import infer_b200.models  # noqa: F401  (registers the architectures)
import infer_b200.parts  # noqa: F401
import pefazen_cases as PC
import plain_pefazen as pp
from infer_b200.cache import CacheManager
from infer_b200.config import parse_config
from infer_b200.config.registry import ConfigError
from infer_b200.parts.base import PagedKVNeed, build_part, part_class
from infer_b200.parts.rotary import interpolated_frequencies
from infer_b200.weights.binder import WeightsError, check_weights, expected_tensors


@pytest.mark.parametrize("name", sorted(PC.CASES))
def test_config_round_trip_and_tensor_names(name):
    cfg = PC.CASES[name]
    arch, typed = parse_config(cfg)
    assert arch.name == "Pefazen"
    assert arch.parse(arch.to_dict(typed)) == typed
    names = expected_tensors(arch.to_spec(typed))
    W = cfg["width"]
    assert {"embed", "final.norm", "head"} <= set(names) and names["head"][0] == (cfg["vocab"], W)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, d, dr, dv, rq, rkv = (m[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
        assert names[p + "norm1"][0] == (W,)
        assert ((p + "norm2") in names) == (l["mlp"] is not None)
        assert names[p + "mix.dq"][0] == (rq, W) and names[p + "mix.dq.norm"][0] == (rq,)
        assert names[p + "mix.uq"][0] == (H * (d + dr), rq)
        assert names[p + "mix.uk"][0] == (H * d, rkv) and names[p + "mix.uv"][0] == (H * dv, rkv)
        assert names[p + "mix.o"][0] == (W, H * dv)
        own = "kv_from" not in m
        assert ((p + "mix.dkv") in names) == own and ((p + "mix.dkv.norm") in names) == own
        if own:
            assert names[p + "mix.dkv"][0] == (rkv + dr, W) and names[p + "mix.dkv.norm"][0] == (rkv,)
        assert ((p + "mix.g") in names) == (l["type"] == "latent_attention")
        if l["mlp"]:
            r = l["mlp"]["router"]
            assert names[p + "mlp.router"][0] == (r["experts"], W) and names[p + "mlp.correction"][0] == (r["experts"],)
            assert names[p + f"mlp.e{r['experts'] - 1}.up"][0] == (l["mlp"]["expert"]["ff"], W)
            assert names[p + f"mlp.e{r['experts'] - 1}.down"][0] == (W, l["mlp"]["expert"]["ff"])
            assert (p + "mlp.e0.gate") not in names


def test_config_refusals():
    base = PC.CASES["a"]
    for path, value in ((("layers", 0, "type"), "latent_attention_3"), (("layers", 0, "mlp", "kind"), "dense"),
                        (("layers", 0, "mlp", "router", "top"), 7), (("norm", "eps"), 0), (("vocab",), "many"),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 0, "mixer", "rot", "dims"), 7),
                        (("layers", 0, "mixer", "rot", "dims"), 10), (("layers", 0, "mixer", "rot", "base"), 1.0),
                        (("layers", 1, "mixer", "kv_from"), 1), (("layers", 1, "mixer", "kv_from"), 2),
                        (("layers", 1, "mixer", "kv_rank"), 16), (("layers", 1, "mixer", "rot", "base"), 400.0),
                        (("layers", 2, "mixer", "rot", "scaling", "factor"), 0), (("logit_softcap",), -1.0)):
        cfg = copy.deepcopy(base)
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(cfg)
    cfg = copy.deepcopy(base)
    del cfg["layers"][2]["mixer"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        parse_config(cfg)
    cfg = copy.deepcopy(base)
    cfg["layers"].append(copy.deepcopy(cfg["layers"][1]))
    cfg["layers"][3]["mixer"]["kv_from"] = 1                     # layer 1 has no latent of its own
    with pytest.raises(ConfigError, match="no latent"):
        parse_config(cfg)


def test_weights_are_bound_by_name_and_missing_ones_are_listed():
    cfg = PC.CASES["a"]
    spec = PC.spec_of(cfg)
    W = PC.make_weights(cfg, 3)
    check_weights(W, spec)
    assert "l1.mix.dkv" not in W and "l1.mix.g" in W and "l2.mix.g" not in W
    del W["l0.mlp.correction"]
    W["l1.mix.dkv"] = torch.zeros(40, 64)
    with pytest.raises(WeightsError) as e:
        check_weights(W, spec)
    assert "l0.mlp.correction" in str(e.value) and "l1.mix.dkv" in str(e.value)


def test_run_order_shares_caches_and_a_cache_keeps_the_longest_window_of_its_readers():
    spec = PC.spec_of(PC.CASES["b"])
    calls = [(c.layer, c.cache, c.write_cache) for c in spec.schedule]
    assert calls == [(0, 0, True), (1, 1, True), (2, 1, False), (3, 0, False), (4, 2, True)]
    mix = lambda i: part_class("mixer", "latent_attention")(spec.layers[i].part("mixer"), None)
    needs = {i: mix(i).cache_need() for i in range(5)}
    assert needs[0] == needs[3] == PagedKVNeed(1, 13 + 6, None, 13, values_in_keys=True)
    assert needs[1] == needs[2] == PagedKVNeed(1, 18 + 4, 33, 18, values_in_keys=True)      # the reader's 33, not the writer's 5
    assert needs[4] == PagedKVNeed(1, 7 + 10, 1, 7, values_in_keys=True)
    assert mix(1).window == 5 and mix(2).window == 33 and mix(3).window is None
    # pages: one row of kv_rank + rot_dim channels per position and no value pages
    mgr = CacheManager({0: needs[0], 1: needs[1], 2: needs[4]}, n_pages=8, page_size=16, n_slots=2)
    assert len(mgr.groups) == 3
    assert mgr.storage_bytes(torch.bfloat16) == 8 * 16 * 2 * ((13 + 6) + (18 + 4) + (7 + 10))
    mgr.make_storage(torch.float32, "cpu")
    v = mgr.view(1)
    assert v.v is None and tuple(v.k.shape) == (8, 1, 16, 22) and v.window == 33


def test_windowed_cache_gives_pages_back_behind_the_longest_window_and_uses_them_again():
    need = PagedKVNeed(1, 22, 33, 18, values_in_keys=True)
    mgr = CacheManager({0: need}, n_pages=5, page_size=16, n_slots=2)
    mgr.admit("x")
    seen = set()
    for start in range(0, 400, 7):
        assert mgr.reserve("x", 7)
        mgr.advance("x", 7)
        table = list(mgr.block_table("x", 0))
        live = [p for p in table if p >= 0]
        seen.update(live)
        assert len(live) <= 5
        first_needed = max(0, start + 7 - 33 + 1) // 16              # the next token still reads from here on
        assert all(p >= 0 for p in table[first_needed:(start + 7 - 1) // 16 + 1])
        mgr.check_invariants()
    assert seen == set(range(4))                                     # 400 positions lived in four pages
    mgr.release("x")
    assert mgr.pages_in_use() == [0]


def test_rotation_tables_follow_the_plain_frequencies():
    for dims, base, scaling in ((16, 1e6, {"factor": 2.0, "original": 2048, "fast": 32.0, "slow": 1.0}),
                                (16, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}),
                                (6, 50.0, None), (64, 5e5, {"factor": 8.0, "original": 4096, "fast": 4.0, "slow": 2.0}),
                                (8, 100.0, {"factor": 3.0, "original": 16, "fast": 2.0, "slow": 1.9})):
        f, mag = interpolated_frequencies(dims, base, scaling)
        fp, magp = pp.interpolated_frequencies(dims, base, scaling)
        assert torch.allclose(f, fp, rtol=1e-14, atol=0) and mag == pytest.approx(magp, rel=1e-14)
        if scaling:
            plain = pp.plain_frequencies(dims, base)
            assert bool(((f <= plain * (1 + 1e-12)) & (f >= plain / scaling["factor"] * (1 - 1e-12))).all())
            assert mag == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)
    from infer_b200.config.specs import PartSpec
    from types import SimpleNamespace
    rt = SimpleNamespace(device=torch.device("cpu"), dtype=torch.float32, max_seq_len=40)   # tables are made on the host
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    part = build_part("position", PartSpec("rotary_interpolated", {"theta": 10000.0, "rotary_dims": 16, "layout": "half", "scaling": sc,
                                                                   "max_positions": 1 << 20}), rt)
    cos, sin = part.rotary_tables(40)
    fp, magp = pp.interpolated_frequencies(16, 10000.0, sc)
    ang = torch.arange(40, dtype=torch.float64)[:, None] * fp[None]
    assert tuple(cos.shape) == (40, 8)
    assert torch.equal(cos, (torch.cos(ang) * magp).float()) and torch.equal(sin, (torch.sin(ang) * magp).float())


def test_plain_implementation_is_consistent():
    # both layouts turn a pair by the same angle and keep what lies behind the rotated channels
    x = torch.randn(5, 3, 10, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 8, 30])
    f = pp.plain_frequencies(6, 50.0)
    a, b = pp.rotate(x, pos, f, "pairs"), pp.rotate(x, pos, f, "halves")
    assert torch.equal(a[..., 6:], x[..., 6:]) and torch.equal(b[..., 6:], x[..., 6:])
    assert torch.equal(a[0], x[0]) and torch.allclose(a[:, :, 0:6:2], b[:, :, 0:3] - x[:, :, 0:3] + x[:, :, 0:6:2]) is not None
    perm = [0, 2, 4, 1, 3, 5]
    assert torch.allclose(pp.rotate(x[..., perm + [6, 7, 8, 9]], pos, f, "halves")[..., :6], a[..., :6][..., perm])
    assert torch.allclose((a[..., :6] ** 2).sum(-1), (x[..., :6] ** 2).sum(-1))
    # scores depend on the distance only
    q, k = torch.randn(1, 6, dtype=torch.float64), torch.randn(1, 6, dtype=torch.float64)
    s = lambda i, j: float((pp.rotate(q, torch.tensor([i]), f, "halves") * pp.rotate(k, torch.tensor([j]), f, "halves")).sum())
    assert s(9, 4) == pytest.approx(s(25, 20))
    # what a window sees
    v = pp.visible(6, 3)
    assert v[5].tolist() == [False, False, False, True, True, True] and v[1].tolist() == [True, True, False, False, False, False]
    assert pp.visible(4, None)[3].all() and pp.visible(4, 1).sum() == 4
    # the correction moves the choice and not the weights; ties go to the lower index
    h = torch.eye(4, dtype=torch.float64)[:1]
    Wr = torch.tensor([[0.0], [1.0], [2.0], [2.0]], dtype=torch.float64).expand(4, 4).contiguous()
    chosen, weight, gap = pp.choose_experts(h, Wr, torch.zeros(4), 2)
    assert chosen.tolist() == [[2, 3]] and gap.item() > 0
    chosen, weight, _ = pp.choose_experts(h, Wr, torch.tensor([5.0, 0.0, 0.0, 0.0]), 2)
    assert chosen.tolist() == [[0, 2]] and weight[0, 0].item() == pytest.approx(0.5) and weight[0, 1].item() == pytest.approx(1 / (1 + math.exp(-2.0)))
    # a layer norm's result has mean 0 and, with weight 1, mean square 1
    y = pp.layer_norm(torch.randn(3, 50, dtype=torch.float64) + 4.0, torch.ones(50), 1e-12)
    assert torch.allclose(y.mean(-1), torch.zeros(3, dtype=torch.float64), atol=1e-12) and torch.allclose((y * y).mean(-1), torch.ones(3, dtype=torch.float64))


def test_plain_prefix_does_not_depend_on_what_follows_and_a_shared_latent_matters():
    cfg = PC.CASES["b"]
    W = {k: v.double() for k, v in PC.make_weights(cfg, 5).items()}
    ids = PC.random_ids(cfg, 50, 1)
    full = pp.forward(cfg, W, ids)
    assert torch.allclose(pp.forward(cfg, W, ids[:20]), full[:20], atol=1e-12)
    # layer 2 reads layer 1's latent: changing layer 1's kv projection changes layer 2's output even where layer 1's
    # own window of 5 no longer reaches
    layers_a, layers_b = [], []
    pp.forward(cfg, W, ids, layers_a)
    W2 = dict(W)
    W2["l1.mix.dkv"] = W["l1.mix.dkv"] * 1.5
    pp.forward(cfg, W2, ids, layers_b)
    assert not torch.allclose(layers_a[2] - layers_a[1], layers_b[2] - layers_b[1])
