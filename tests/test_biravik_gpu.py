"""Biravik in the engine against the plain implementation: every way of cutting requests into steps, in float32 and
bfloat16, on configurations that differ in every size and option; generation through the Python entry point and
the scheduler; the trace and generation programs."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import biravik_cases as BC
import helpers as H
import plain_biravik as pb

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
SEED = 11


def _engine(name, dtype, max_tokens=1024, sharp=0.0, **kw):
    from infer_b200.engine import Engine
    cfg = BC.CASES[name]
    return Engine(BC.spec_of(cfg), BC.make_weights(cfg, SEED, sharp=sharp), dtype=dtype, max_tokens=max_tokens,
                  max_requests=4, **kw)


def _requests(name, lengths, seed0=0):
    return {f"r{i}": BC.random_ids(BC.CASES[name], n, seed0 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_whole(name, dtype):
    reqs = _requests(name, [5, 17, 33, 90, 1, 2])
    eng = _engine(name, dtype)
    got = H.run_trace(eng, H.trace_whole(reqs))
    BC.check(BC.CASES[name], SEED, dtype, got, reqs, what=name)
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_tail_one_by_one(name, dtype):
    """The last 40 tokens decoded one by one: windows of 3, 5, 24 and 33 pass over decoded tokens, kept first keys stay."""
    reqs = _requests(name, [110, 47], seed0=10)
    got = H.run_trace(_engine(name, dtype), H.trace_tail(reqs, 40))
    BC.check(BC.CASES[name], SEED, dtype, got, reqs, what=name)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_portions_of_changing_size(name, dtype):
    reqs = _requests(name, [150, 61], seed0=20)
    got = H.run_trace(_engine(name, dtype), H.trace_portions(reqs))
    BC.check(BC.CASES[name], SEED, dtype, got, reqs, what=name)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_mixed_with_pages_and_slots_used_again(name, dtype):
    lengths = [60, 45, 100, 33, 64, 90, 20, 77]
    ids = _requests(name, lengths, seed0=30)
    reqs = {rid: (t, max(2, len(t) - 16 - 3 * i)) for i, (rid, t) in enumerate(ids.items())}
    max_tokens = 320                                        # 20 pages, 4 slots: fewer than the requests need in total
    steps = H.trace_mixed(reqs, max_tokens, seed=7)
    assert max(len(s["entries"]) for s in steps) >= 3
    eng = _engine(name, dtype, max_tokens=max_tokens)
    got = H.run_trace(eng, steps)
    BC.check(BC.CASES[name], SEED, dtype, got, ids, what=name)
    assert sum(-(-n // 16) for n in lengths) > eng.cache.pages_total()[0] and len(lengths) > eng.cache.n_slots
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups)


@pytest.mark.parametrize("name", ["a", "b"])
def test_cuttings_are_bit_equal_in_float32(name):
    """Prefill against token-by-token decoding and against portions down to two tokens: the state that a cut carries
    (pages, the row of the token before, state matrices) is exactly what the uncut run had in its registers."""
    reqs = _requests(name, [97], seed0=40)
    dtype = torch.float32
    a = H.run_trace(_engine(name, dtype), H.trace_whole(reqs))["r0"]
    b = H.run_trace(_engine(name, dtype), H.trace_tail(reqs, 96))["r0"]          # one token, then 96 one by one
    c = H.run_trace(_engine(name, dtype), H.trace_portions(reqs))["r0"]
    ids = reqs["r0"]
    bounds = list(range(0, 96, 2)) + [97]                        # portions of two tokens; the last one has three
    twos = [{"entries": [("r0", ids[a:b], list(range(b - a)))], "end": []} for a, b in zip(bounds[:-1], bounds[1:])]
    d = H.run_trace(_engine(name, dtype), twos)["r0"]
    for p in a:
        for other in (b, c, d):
            assert np.array_equal(a[p], other[p]), f"position {p} differs between cuttings in float32"


def test_bfloat16_cuttings_differ_by_rounding_only():
    name = "c"
    reqs = _requests(name, [200], seed0=41)
    a = H.run_trace(_engine(name, torch.bfloat16), H.trace_whole(reqs))["r0"]
    b = H.run_trace(_engine(name, torch.bfloat16), H.trace_portions(reqs))["r0"]
    ref = BC.oracle(BC.CASES[name], SEED, torch.bfloat16, reqs["r0"])
    noise = float(np.sqrt(np.mean((BC.oracle(BC.CASES[name], SEED, torch.bfloat16, reqs["r0"], torch.bfloat16) - ref) ** 2)))
    for p in a:
        assert float(np.sqrt(np.mean((a[p] - b[p]) ** 2))) <= 4 * noise


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "c"])
def test_sharp_attention_at_window_edges_and_page_borders(name, dtype):
    """Peaked attention weights: a position's result hangs on single keys: the farthest its window still holds, a kept
    first key, a key hundreds of positions back (the layers without a window). Prompts end and decoding starts around
    page borders (multiples of 16) and key chunks (multiples of 128)."""
    cfg = BC.CASES[name]
    ref_flat = BC.oracle(cfg, SEED, torch.float32, BC.random_ids(cfg, 64, 50))
    ref_sharp = BC.oracle(cfg, SEED, torch.float32, BC.random_ids(cfg, 64, 50), sharp=6.0)
    assert np.abs(ref_flat - ref_sharp).max() > 3e-3 * np.abs(ref_flat).max()            # the sharpening changes the function
    for n, head in ((337, 303), (320, 289), (321, 288)):
        ids = BC.random_ids(cfg, n, 51 + n)
        steps = [{"entries": [("x", ids[:head], [head - 1])], "end": []}]
        steps += [{"entries": [("x", [ids[i]], [0])], "end": []} for i in range(head, n)]
        got = H.run_trace(_engine(name, dtype, sharp=6.0), steps)
        BC.check(cfg, SEED, dtype, got, {"x": ids}, sharp=6.0, what=f"{name}/{n}")


def test_tokens_far_back_reach_the_logits():
    """Changing the first token changes logits 300 positions later (through the kept first keys, the layers without a
    window and the recurrences), by the same amount in the engine as in the plain implementation."""
    name = "a"
    cfg = BC.CASES[name]
    ids = BC.random_ids(cfg, 300, 77)
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    want = BC.oracle(cfg, SEED, torch.float32, other)[-1] - BC.oracle(cfg, SEED, torch.float32, ids)[-1]
    assert np.abs(want).max() > 1e-4
    eng = _engine(name, torch.float32)
    got = H.run_trace(eng, H.trace_portions({"p": ids, "q": other}))
    assert np.allclose(got["q"][299] - got["p"][299], want, atol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_long_decode(dtype):
    name = "b"
    ids = BC.random_ids(BC.CASES[name], 300, 60)
    steps = [{"entries": [("x", ids[:7], [6])], "end": []}]
    steps += [{"entries": [("x", [ids[i]], [0])], "end": []} for i in range(7, 300)]
    got = H.run_trace(_engine(name, dtype), steps)
    BC.check(BC.CASES[name], SEED, dtype, got, {"x": ids}, what=name)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_first_tokens_one_by_one(name, dtype):
    """From position 0: the first token mixes with zeros, the state matrices start from zero, the first query's
    softmax holds itself and the sink."""
    ids = BC.random_ids(BC.CASES[name], 7, 70)
    steps = [{"entries": [("x", [t], [0])], "end": []} for t in ids]
    got = H.run_trace(_engine(name, dtype), steps)
    BC.check(BC.CASES[name], SEED, dtype, got, {"x": ids}, what=name)


def test_a_batch_of_unequal_requests_equals_each_alone():
    name = "b"
    reqs = _requests(name, [3, 90, 41, 2], seed0=80)
    eng = _engine(name, torch.float32)
    alone = H.run_trace(eng, H.trace_whole(reqs))
    together = H.run_trace(eng, [{"entries": [(r, t, list(range(len(t)))) for r, t in reqs.items()], "end": list(reqs)}])
    for r in reqs:
        for p in alone[r]:
            assert np.array_equal(alone[r][p], together[r][p])


def test_the_design_runs_on_its_own_kernels():
    from infer_b200 import ops
    eng = _engine("c", torch.bfloat16)
    ids = BC.random_ids(BC.CASES["c"], 140, 90)
    before = dict(ops.LAUNCH_KINDS)
    H.run_trace(eng, [{"entries": [("x", ids[:139], [138])], "end": []}, {"entries": [("x", ids[139:], [0])], "end": ["x"]}])
    ran = {k: v - before.get(k, 0) for k, v in ops.LAUNCH_KINDS.items() if v != before.get(k, 0)}
    for kind in ("ib_state_scan", "ib_head_prepare", "ib_sum_norm", "ib_gate_mul", "ib_shift_mix", "ib_double_exp_decay",
                 "ib_group_norm_gate", "ib_route", "ib_glu_act", "ib_relu_sq", "ib_silu_rows"):
        assert ran.get(kind, 0) >= 2, (kind, ran)
    assert ran.get("ib_gemm_tc", 0) >= 1                     # the tensor-core product serves the prompt's matrices
    # keys and values of 64 and 128: the prompt's attention runs on the tensor-core kernel, with and without kept first
    # keys and slopes, every decoded token's on the kernel that splits its keys over CTAs, none on the plain one
    assert ran.get("ib_attention_prefill_tc_kept", 0) == 3 and ran.get("ib_attention_prefill_tc_biased", 0) == 1, ran
    assert ran.get("ib_attention_split", 0) == 4 and "ib_attention_plain" not in ran, ran


# ----------------------------------------------------------------------------------------------- generation, programs

@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_the_scheduler(name):
    from infer_b200.engine.generation import LLM
    cfg = BC.CASES[name]
    prompts = [BC.random_ids(cfg, n, 100 + n) for n in (5, 17, 33, 1)]
    llm = LLM(None, dtype=torch.float32, spec=BC.spec_of(cfg), weights=BC.make_weights(cfg, SEED), slots=3, max_seq=128,
              max_batch_tokens=24)
    outs = llm.generate(prompts, max_new=12)
    W = H.as_compute(BC.make_weights(cfg, SEED), torch.float32)
    for p, o in zip(prompts, outs):
        assert o == pb.greedy(cfg, W, p, 12)
    assert llm.engine.cache.pages_in_use() == [0] * len(llm.engine.cache.groups)


def test_bfloat16_generation_with_graphs_picks_the_maximum_up_to_rounding():
    from infer_b200.engine.generation import LLM
    name = "a"
    cfg = BC.CASES[name]
    prompts = [BC.random_ids(cfg, n, 200 + n) for n in (9, 40, 70)]
    llm = LLM(None, dtype=torch.bfloat16, spec=BC.spec_of(cfg), weights=BC.make_weights(cfg, SEED), slots=4, max_seq=128)
    outs = llm.generate(prompts, max_new=24)
    for p, o in zip(prompts, outs):
        assert len(o) == 24
        ids = p + o
        ref = BC.oracle(cfg, SEED, torch.bfloat16, ids)
        refr = BC.oracle(cfg, SEED, torch.bfloat16, ids, torch.bfloat16)
        noise = max(float(np.sqrt(np.mean((refr - ref) ** 2))), 1e-3 * float(np.sqrt(np.mean(ref ** 2))))
        for i, tok in enumerate(o):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - 12 * noise, f"token {i}: chose a logit {row.max() - row[tok]:.4f} below the maximum"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_model_folder(tmp_path, dtype):
    """bin/trace_run on a written folder whose configuration leaves the decay's rank to the checkpoint."""
    import json
    from infer_b200.weights import write_random_model
    name = "a"
    cfg = BC.CASES[name]
    model = tmp_path / "model"
    write_random_model(str(model), cfg, SEED, torch.bfloat16)
    stored = json.loads((model / "config.json").read_text())
    del stored["layers"][0]["mixer"]["rank"]
    (model / "config.json").write_text(json.dumps(stored))
    lengths = [70, 40, 100, 33, 64]
    ids = {f"r{i}": BC.random_ids(cfg, n, 600 + i) for i, n in enumerate(lengths)}
    steps = H.trace_mixed({rid: (t, max(2, len(t) - 20)) for rid, t in ids.items()}, 256, seed=3)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "256"], input=H.trace_to_jsonl(steps), capture_output=True,
                          text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got, pos = {}, {}
    for i, st in enumerate(steps):
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        r = 0
        for rid, toks, want in st["entries"]:
            for w in want:
                got.setdefault(rid, {})[pos.get(rid, 0) + w] = arr[r]
                r += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    BC.check(cfg, SEED, torch.float32 if dtype == "float32" else torch.bfloat16, got, ids, what="program")


def test_generate_program_on_a_model_folder_and_on_a_preset(tmp_path):
    from infer_b200.weights import write_random_model
    cfg = BC.CASES["a"]
    model = tmp_path / "model"
    write_random_model(str(model), cfg, SEED, torch.bfloat16)
    prompt = BC.random_ids(cfg, 21, 1)
    want = pb.greedy(cfg, H.as_compute(BC.make_weights(cfg, SEED), torch.float32), prompt, 10)
    gen = os.path.join(ROOT, "bin", "generate")

    def run(args):
        proc = subprocess.run([sys.executable, gen] + args, capture_output=True, text=True, timeout=900, cwd=ROOT)
        assert proc.returncode == 0, (proc.stdout[-1500:], proc.stderr[-1500:])
        line = next(l for l in proc.stdout.splitlines() if l.startswith("ids:"))
        return [int(t) for t in line.split()[1:]]
    ids = ",".join(map(str, prompt))
    assert run(["0", "10", "--model", str(model), "--dtype", "float32", "--prompt-ids", ids, "--max-seq", "64"]) == want
    assert run(["0", "10", "--model", str(model), "--dtype", "float32", "--prompt-ids", ids, "--max-seq", "64", "--chunk", "5",
                "--kv-blocks", "3"]) == want
    assert len(run(["0", "12", "--random", "tiny-biravik", "--max-seq", "64"])) == 12
