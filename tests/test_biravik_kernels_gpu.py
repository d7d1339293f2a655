"""The kernels behind Biravik's parts, each alone against the plain implementation's function for the same
mechanism (float64), in float and bfloat16 storage, over segments of unequal length with state carried between steps."""
import math

import numpy as np
import pytest
import torch

import plain_biravik as pb
from infer_b200 import ops
from test_fozerax_kernels_gpu import _paged
from test_ruvenex_kernels_gpu import _Step

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F = torch.float64


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("width", [36, 192, 1000])
def test_scaled_sum_and_norm_with_its_copy(width):
    g = torch.Generator().manual_seed(width)
    x, a, b = torch.randn(7, width, generator=g), 5.0 * torch.randn(7, width, generator=g), torch.randn(7, width, generator=g)
    w = torch.randn(width, generator=g)
    want = pb.rms(2.5 * x.double() + 0.8 * a.double() + 0.9 * b.double(), 1e-5) * w.double()
    xd = x.to(DEV)
    out, copy = ops.sum_norm(xd, 2.5, a.to(DEV), 0.8, b.to(DEV), 0.9, w.to(DEV), 1e-5, torch.bfloat16)
    assert out.data_ptr() == xd.data_ptr()                                    # the stream is rewritten in place
    assert torch.allclose(out.double().cpu(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(copy.cpu(), out.cpu().to(torch.bfloat16))
    one, none = ops.sum_norm(x.to(DEV), 1.0, a.to(DEV), 1.0, None, 0.0, w.to(DEV), 3e-6, torch.float32)
    assert none is None and torch.allclose(one.double().cpu(), pb.rms(x.double() + a.double(), 3e-6) * w.double(), rtol=1e-5, atol=1e-5)


def _prepared(q, k, wq, wk, eps, pos, rot, temp):
    qn, kn = pb.rms(q, eps) * wq.double(), pb.rms(k, eps) * wk.double()
    if rot is not None:
        qn, kn = pb.rotate_pairs(qn, pos, rot), pb.rotate_pairs(kn, pos, rot)
    if temp is not None:
        qn = qn * pb.query_temperature(pos, *temp)[:, None, None]
    return qn, kn


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes,rot,temp,shared", [
    ((6, 2, 64, 48), None, (0.3, 64), False), ((3, 3, 10, 7), {"base": 50.0, "dims": 10, "scaling": None}, None, False),
    ((2, 1, 12, 12), {"base": 10000.0, "dims": 2, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}}, (1.5, 1), True),
    ((4, 1, 32, 32), {"base": 1000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}, None, True),
    ((1, 1, 9, 5), None, None, False)])
def test_head_norms_rotation_temperature_and_the_cache_write(dtype, sizes, rot, temp, shared):
    from infer_b200.parts.rotary import interpolated_frequencies
    H, G, d, dv = sizes
    g = torch.Generator().manual_seed(d)
    lens, pos0 = [21, 1, 6], [13, 127, 0]
    step = _Step(lens, pos0, [0, 1, 2])
    T = sum(lens)
    C = (H + G) * d + (0 if shared else G * dv)
    rows = torch.randn(T, C + 5, generator=g).to(dtype)
    wq, wk = torch.randn(d, generator=g), torch.randn(d, generator=g)
    table = torch.tensor([[3, 7, 1] + [-1] * 6, [5, 0, 2, 9, 10, 11, 12, 13, 8], [4] + [-1] * 8], dtype=torch.int32, device=DEV)
    kc = torch.full((14, G, 16, d), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((14, G, 16, dv), float("nan"), dtype=dtype, device=DEV)
    cos = sin = None
    n_rot = 0
    if rot is not None:
        sc = dict(rot["scaling"], magnitude_slope=0.1, min_span=0.001) if rot["scaling"] else None
        f, mag = interpolated_frequencies(rot["dims"], rot["base"], sc)
        ang = torch.arange(200, dtype=F)[:, None] * f[None, :]
        cos, sin, n_rot = (torch.cos(ang) * mag).float().to(DEV), (torch.sin(ang) * mag).float().to(DEV), rot["dims"]
    coef, every = temp if temp is not None else (0.0, 0)
    q_out = ops.head_prepare(rows.to(DEV), 3, wq.to(DEV), wk.to(DEV), 1e-5, cos, sin, n_rot, coef, every, shared, step, table, kc, vc,
                             H, G, d, dv, True)
    assert int(step.status.item()) == 0
    pos = step.positions.cpu().long()
    r = rows.double()
    q, k = r[:, 3:3 + H * d].view(T, H, d), r[:, 3 + H * d:3 + (H + G) * d].view(T, G, d)
    v = k if shared else r[:, 3 + (H + G) * d:3 + C].view(T, G, dv)
    qn, kn = _prepared(q, k, wq, wk, 1e-5, pos, rot, temp)
    assert torch.allclose(q_out.double().cpu().view(T, H, d), qn, **_tol(dtype))
    seg = step.token_seg.cpu().tolist()
    for t in range(T):
        page, place = int(table[seg[t], int(pos[t]) // 16]), int(pos[t]) % 16
        assert torch.allclose(kc[page, :, place].double().cpu(), kn[t], **_tol(dtype))
        assert torch.equal(vc[page, :, place].cpu(), v[t].to(dtype))              # values as projected, bit for bit
    assert int(torch.isnan(kc.float()).sum()) == (14 * 16 - T) * G * d            # nothing else was written
    # without the cache write only q comes out
    kc2 = torch.full_like(kc, float("nan"))
    ops.head_prepare(rows.to(DEV), 3, wq.to(DEV), wk.to(DEV), 1e-5, cos, sin, n_rot, coef, every, shared, step, table, kc2, vc, H, G, d, dv, False)
    assert bool(torch.isnan(kc2.float()).all())


def _attention(q, k, v, scale, window, keep, slopes, sink):
    """q [n, H, d], k [n, G, d], v [n, G, dv] of one sequence -> [n, H, dv] (float64)."""
    n, H = q.shape[0], q.shape[1]
    per = H // k.shape[1]
    kh, vh = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * scale
    if slopes is not None:
        pos = torch.arange(n)
        s = s - slopes.double()[:, None, None] * (pos[:, None] - pos[None, :]).double()[None]
    w = pb.attention_weights(s, pb.visible(n, window, keep), sink)
    return torch.einsum("hij,jhd->ihd", w, vh)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("window,keep", [(None, 0), (5, 0), (70, 20), (128, 3), (150, 130), (300, 1), (40, 200)])
@pytest.mark.parametrize("sizes", [(6, 2, 64, 48), (3, 3, 10, 7), (16, 1, 128, 128), (4, 2, 24, 40)])
def test_attention_with_kept_first_keys_and_slopes_plain_and_split(sizes, window, keep, dtype):
    """Tokens at positions around chunk borders (multiples of 128), page borders and the first positions. One key at
    each edge stands out: the farthest the window holds and the one just outside, the last kept key and the first
    that is not kept. The plain kernel serves portions and single tokens, the split kernel single tokens."""
    H, G, d, dv = sizes
    scale = 0.2
    g = torch.Generator().manual_seed(d + (window or 0) + keep)
    n = 420
    q = torch.randn(n, H, d, generator=g).to(dtype).double()
    k = torch.randn(n, G, d, generator=g).to(dtype).double()
    v = torch.randn(n, G, dv, generator=g).to(dtype).double()
    sink = torch.randn(H, generator=g)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if window is None else None
    probes = [0, 1, 15, 16, 127, 128, 129, 255, 256, 300, 383, 384, 419]

    def stand_out(key, query, head):
        if 0 <= key <= query:
            k[key, head // (H // G)] += 2.0 * q[query, head] / q[query, head].norm() * math.sqrt(d)
    for pr_ in probes:
        if window is not None:
            stand_out(pr_ - (window - 1), pr_, 0)
            stand_out(pr_ - window, pr_, H - 1)
            if keep and pr_ - window >= keep:
                stand_out(keep - 1, pr_, 1 % H)
                stand_out(keep, pr_, 2 % H)
        else:
            stand_out(0, pr_, 0)                                        # as far back as it goes, against the slope
    k = k.to(dtype).double()
    want = _attention(q, k, v, scale, window, keep, slopes, sink)
    table_row = list(np.random.default_rng(1).permutation(30))[:27]
    kc, vc = _paged([k], [v], [table_row], 30, G, d, dv, dtype)
    # every probe is a request of its own that shares the pages (one row of the table each), plus one longer segment
    S = len(probes) + 1
    table = torch.tensor([table_row] * S, dtype=torch.int32, device=DEV)
    step = _Step([1] * len(probes) + [37], probes + [200], list(range(S)))
    step.seg_lens, step.max_q_len, step.max_ctx_len = step.lens, 37, n
    rows = torch.cat([q[probes], q[200:237]]).reshape(-1, H * d).to(dtype).to(DEV).contiguous()
    sl = slopes.to(DEV) if slopes is not None else None
    ref = torch.cat([want[probes], want[200:237]])
    plain = ops.attention_plain(rows, kc.to(DEV), vc.to(DEV), table, step.token_seg, step.positions, H, G, d, window, scale, step.status,
                                dv, None, sink.to(DEV), keep_first=keep, slopes=sl)
    assert torch.allclose(plain.double().cpu().view(-1, H, dv), ref, **_tol(dtype))
    out = torch.full((rows.shape[0], H * dv), 7.0, dtype=dtype, device=DEV)
    ops.attention_split(rows, kc.to(DEV), vc.to(DEV), table, step, H, G, d, dv, window, scale, None, sink.to(DEV), out, single_only=True,
                        keep_first=keep, slopes=sl)
    got = out.double().cpu().view(-1, H, dv)
    assert torch.allclose(got[:len(probes)], want[probes], **_tol(dtype))
    assert float((got[len(probes):] - 7.0).abs().sum()) == 0.0               # the longer segment's rows were left alone
    # the merge may apply a gate per output channel: the same bits as the ungated result through the gate's own kernel
    gate = torch.randn(rows.shape[0], 3 + H * dv, generator=g).to(dtype).to(DEV)
    gated = torch.full((rows.shape[0], H * dv), 7.0, dtype=dtype, device=DEV)
    ops.attention_split(rows, kc.to(DEV), vc.to(DEV), table, step, H, G, d, dv, window, scale, None, sink.to(DEV), gated, single_only=True,
                        keep_first=keep, slopes=sl, gate=gate, gate_col=3)
    assert torch.equal(gated[:len(probes)], ops.gate_mul(out[:len(probes)].clone(), gate[:len(probes)].contiguous(), 3))
    assert int(step.status.item()) == 0


@pytest.mark.parametrize("window,keep", [(None, 0), (150, 40), (128, 3), (300, 200), (40, 130), (520, 1)])
@pytest.mark.parametrize("sizes", [(4, 2, 64), (2, 1, 128)])
def test_prompt_portions_on_the_tensor_core_kernel_with_slopes_and_kept_first_keys(sizes, window, keep):
    """A portion of 470 tokens behind 30 cached ones (four query tiles, the last ragged) beside a single token of another
    request; keys at the window's two edges and at the kept keys' end stand out for the portion's last rows."""
    H, G, d = sizes
    scale, dtype = 0.11, torch.bfloat16
    g = torch.Generator().manual_seed(d + (window or 0) + keep)
    n, m, first = 500, 90, 30
    seqs = [[torch.randn(length, hh, d, generator=g).to(dtype).double() for hh in (H, G, G)] for length in (n, m)]
    sink = torch.randn(H, generator=g)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if window is None else None
    q, k, v = seqs[0]

    def stand_out(key, query, head):
        if 0 <= key <= query:
            k[key, head // (H // G)] += 3.0 * q[query, head] / q[query, head].norm() * math.sqrt(d)
    for probe in (n - 1, n - 70, 300):
        if window is not None:
            stand_out(probe - (window - 1), probe, 0)
            stand_out(probe - window, probe, H - 1)
            if probe - window >= keep:
                stand_out(keep - 1, probe, 1 % H)
                stand_out(keep, probe, 0)
        else:
            stand_out(0, probe, 0)
    seqs[0][1] = k = k.to(dtype).double()
    want = [_attention(*sq, scale, window, keep, slopes, sink) for sq in seqs]
    tables = [list(range(3, 35)), [40, 36, 38, 37, 41, 39]]
    kc, vc = _paged([s_[1] for s_ in seqs], [s_[2] for s_ in seqs], tables, 44, G, d, d, dtype)
    table = torch.full((2, 32), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    step = _Step([n - first, 1], [first, m - 1], [0, 1])
    step.seg_lens, step.seg_pos0 = step.lens, torch.tensor(step.pos0, dtype=torch.int32, device=DEV)
    step.max_q_len, step.max_ctx_len = n - first, n
    rows = torch.cat([q[first:].reshape(n - first, H * d), seqs[1][0][m - 1:].reshape(1, H * d)]).to(dtype).to(DEV).contiguous()
    before = dict(ops.LAUNCH_KINDS)
    out = ops.attention_window(rows, kc.to(DEV), vc.to(DEV), table.to(DEV), step, H, G, d, d, window, scale, None, sink.to(DEV), None, keep,
                               slopes.to(DEV) if slopes is not None else None)
    assert out is not None and ops.LAUNCH_KINDS["ib_attention_prefill_tc_kept"] == before.get("ib_attention_prefill_tc_kept", 0) + 1
    assert ops.LAUNCH_KINDS["ib_attention_split"] == before.get("ib_attention_split", 0) + 1        # the single token beside it
    assert int(step.status.item()) == 0
    got = out.double().cpu().view(-1, H, d)
    ref = torch.cat([want[0][first:], want[1][m - 1:]])
    assert torch.allclose(got, ref, rtol=3e-2, atol=3e-2)
    assert float((got - ref).pow(2).mean().sqrt()) < 4e-3


# a key size below, at and above each number of state rows a lane keeps; value sizes that are no multiple of four
SCAN_SIZES = [(2, 16, 32), (1, 40, 20), (3, 5, 9), (2, 128, 64), (4, 8, 4), (2, 160, 128), (1, 33, 3), (2, 64, 130)]


def _scan_case(H, d, dv, seed):
    g = torch.Generator().manual_seed(seed)
    seqs = {}
    for s, n in ((0, 45), (2, 23)):
        seqs[s] = {"q": torch.randn(n, H, d, generator=g), "k": torch.randn(n, H, d, generator=g) * 0.5,
                   "v": torch.randn(n, H, dv, generator=g), "a": torch.rand(n, H, d, generator=g)}
    return seqs


@pytest.mark.parametrize("sizes", SCAN_SIZES)
def test_constant_decay_scan_over_steps(sizes):
    H, d, dv = sizes
    seqs = _scan_case(H, d, dv, d + dv)
    decay = torch.tensor([0.0, 1.0, 0.9, 0.999][:H] if H <= 4 else [0.9] * H)
    ref = {s: torch.stack([pb.constant_decay_scan(x["q"][:, h].double(), x["k"][:, h].double(), x["v"][:, h].double(), float(decay[h]))[0]
                           for h in range(H)], dim=1) for s, x in seqs.items()}
    state = torch.full((3, H, d, dv), float("nan"), device=DEV)
    state[0].zero_(), state[2].zero_()
    at = {0: 0, 2: 0}
    for lens in ([1, 2], [2, 1], [17, 9], [1, 1], [24, 10]):
        step = _Step(lens, [at[0], at[2]], [0, 2])
        parts = [torch.cat([seqs[s][n][at[s]:at[s] + m].reshape(m, -1) for n in ("q", "k", "v")], dim=1) for s, m in zip((0, 2), lens)]
        rows = torch.cat([torch.zeros(sum(lens), 4), torch.cat(parts)], dim=1).to(DEV).contiguous()
        o = ops.state_scan(ops.SCAN_HEAD_DECAY, rows, 4, 4 + H * d, 4 + 2 * H * d, decay.to(DEV), 0, state, step.seg_start, step.seg_slot,
                           H, 1, d, dv, True, max(lens)).double().cpu().view(-1, H, dv)
        want = torch.cat([ref[s][at[s]:at[s] + m] for s, m in zip((0, 2), lens)])
        assert torch.allclose(o, want, rtol=2e-5, atol=2e-5)
        for s, m in zip((0, 2), lens):
            at[s] += m
    assert bool(torch.isnan(state[1]).all())                                   # the slot nobody holds stayed untouched


@pytest.mark.parametrize("sizes", [(2, 16, 16), (3, 5, 5), (2, 128, 128), (1, 40, 40), (4, 64, 64), (1, 33, 33)])
def test_scan_with_a_bonus_over_steps_from_planes(sizes):
    H, d, dv = sizes
    seqs = _scan_case(H, d, dv, 3 * d + dv)
    g = torch.Generator().manual_seed(1)
    u = torch.randn(H, d, generator=g)
    ref = {s: torch.stack([pb.bonus_scan(x["q"][:, h].double(), x["k"][:, h].double(), x["v"][:, h].double(), x["a"][:, h].double(), u[h].double())[0]
                           for h in range(H)], dim=1) for s, x in seqs.items()}
    state = torch.zeros((3, H, d, dv), device=DEV)
    at = {0: 0, 2: 0}
    whole = {}
    for lens in ([1, 2], [2, 1], [17, 9], [1, 1], [24, 10]):
        step = _Step(lens, [at[0], at[2]], [0, 2])
        planes = torch.stack([torch.cat([seqs[s][n][at[s]:at[s] + m].reshape(m, -1) for s, m in zip((0, 2), lens)]) for n in ("q", "k", "v")])
        aux = torch.cat([seqs[s]["a"][at[s]:at[s] + m].reshape(m, -1) for s, m in zip((0, 2), lens)]).to(DEV).contiguous()
        o = ops.state_scan(ops.SCAN_BONUS, planes.to(DEV).contiguous(), (0, 0), (1, 0), (2, 0), aux, 0, state, step.seg_start, step.seg_slot,
                           H, 1, d, dv, True, max(lens), bonus=u.to(DEV)).double().cpu().view(-1, H, dv)
        want = torch.cat([ref[s][at[s]:at[s] + m] for s, m in zip((0, 2), lens)])
        assert torch.allclose(o, want, rtol=2e-5, atol=2e-5)
        for s, m in zip((0, 2), lens):
            at[s] += m


@pytest.mark.parametrize("sizes", [(2, 16, 32), (3, 5, 9), (2, 128, 64)])
def test_the_activation_inside_the_scan_equals_the_activation_before_it(sizes):
    H, d, dv = sizes
    g = torch.Generator().manual_seed(d)
    lens = [5, 1, 3]
    step = _Step(lens, [0, 0, 0], [0, 1, 2])
    rows = torch.randn(sum(lens), 4 + 2 * H * d + H * dv, generator=g).to(DEV)
    decay = torch.rand(H, generator=g).to(DEV)
    one, two = torch.zeros((3, H, d, dv), device=DEV), torch.zeros((3, H, d, dv), device=DEV)
    a = ops.state_scan(ops.SCAN_HEAD_DECAY, rows, 4, 4 + H * d, 4 + 2 * H * d, decay, 0, one, step.seg_start, step.seg_slot, H, 1, d, dv,
                       True, max(lens), silu=True)
    act = ops.silu_rows(rows.clone(), 4, 2 * H * d + H * dv)
    for max_len in (max(lens), 64):                               # the few-token form, and the form of prompt portions
        two.zero_()
        b = ops.state_scan(ops.SCAN_HEAD_DECAY, act, 4, 4 + H * d, 4 + 2 * H * d, decay, 0, two, step.seg_start, step.seg_slot, H, 1, d, dv,
                           True, max_len)
        assert torch.equal(a, b) and torch.equal(one, two)


def test_scans_with_unequal_key_and_value_sizes_and_bit_equal_cuttings():
    H, d, dv = 2, 40, 24
    x = _scan_case(H, d, dv, 9)[0]
    g = torch.Generator().manual_seed(2)
    u = torch.randn(H, d, generator=g)
    n = 45
    rows = torch.cat([x[m].reshape(n, -1) for m in ("q", "k", "v")], dim=1).to(DEV).contiguous()
    aux = x["a"].reshape(n, -1).to(DEV).contiguous()
    ref = torch.stack([pb.bonus_scan(x["q"][:, h].double(), x["k"][:, h].double(), x["v"][:, h].double(), x["a"][:, h].double(), u[h].double())[0]
                       for h in range(H)], dim=1)
    outs = []
    for cuts in ([45], [1] * 45, [2] * 22 + [1], [7, 30, 8]):
        state = torch.zeros((1, H, d, dv), device=DEV)
        got, at = [], 0
        for m in cuts:
            step = _Step([m], [at], [0])
            got.append(ops.state_scan(ops.SCAN_BONUS, rows[at:at + m].contiguous(), 0, H * d, 2 * H * d, aux[at:at + m].contiguous(), 0, state,
                                      step.seg_start, step.seg_slot, H, 1, d, dv, True, m, bonus=u.to(DEV)))
            at += m
        outs.append(torch.cat(got).cpu())
    assert torch.allclose(outs[0].double().view(n, H, dv), ref, rtol=2e-5, atol=2e-5)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_mixtures_with_the_token_before_over_steps(dtype):
    g = torch.Generator().manual_seed(4)
    W, n_mix = 36, 5
    seqs = {0: torch.randn(30, W, generator=g), 2: torch.randn(11, W, generator=g)}
    mu = torch.rand(n_mix, W, generator=g)
    last = torch.full((3, W), float("nan"), device=DEV)
    last[0].zero_(), last[2].zero_()
    at = {0: 0, 2: 0}
    for lens in ([1, 2], [2, 1], [17, 3], [1, 1], [9, 4]):
        step = _Step(lens, [at[0], at[2]], [0, 2])
        x = torch.cat([seqs[s][at[s]:at[s] + m] for s, m in zip((0, 2), lens)])
        out = ops.shift_mix(x.to(DEV), last, mu.to(DEV), step, dtype, True).double().cpu()
        want = []
        for s, m in zip((0, 2), lens):
            h = seqs[s][at[s]:at[s] + m].double()
            before = torch.cat([(seqs[s][at[s] - 1:at[s]] if at[s] else torch.zeros(1, W)).double(), h[:-1]])
            want.append(h[None] + (before - h)[None] * mu.double()[:, None, :])
            at[s] += m
        assert torch.allclose(out, torch.cat(want, dim=1), **_tol(dtype))
    assert torch.equal(last[0].cpu(), seqs[0][29]) and torch.equal(last[2].cpu(), seqs[2][10]) and bool(torch.isnan(last[1]).all())
    # without the state write the kept row stays
    step = _Step([3], [30], [0])
    ops.shift_mix(torch.randn(3, W, device=DEV), last, mu.to(DEV), step, dtype, False)
    assert torch.equal(last[0].cpu(), seqs[0][29])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes", [(2, 16, 4), (1, 40, 3), (3, 128, 16)])
def test_decays_of_two_exponentials_through_a_low_rank(sizes, dtype):
    H, d, r = sizes
    g = torch.Generator().manual_seed(d)
    T, C = 11, H * d
    rows = torch.randn(T, 3 + r, generator=g).to(dtype)
    up, bias = 0.5 * torch.randn(C, r, generator=g), -1.0 + torch.randn(C, generator=g)
    want = torch.exp(-torch.exp(torch.tanh(rows[:, 3:].double()) @ up.double().T + bias.double()))
    decay = ops.double_exp_decay(rows.to(DEV), 3, r, up.t().contiguous().to(DEV), bias.to(DEV))
    assert decay.dtype == torch.float32 and torch.allclose(decay.double().cpu(), want, rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("gate_dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("groups,size,act", [(1, 192, "sigmoid"), (4, 64, "silu"), (3, 5, "silu"), (1, 7, None)])
def test_group_norms_with_gates(groups, size, act, gate_dtype):
    g = torch.Generator().manual_seed(size)
    T = 6
    o = 4.0 * torch.randn(T, groups * size, generator=g)
    w = torch.randn(groups * size, generator=g)
    gate = torch.randn(T, 3 + groups * size, generator=g).to(gate_dtype)
    z = gate[:, 3:].double()
    mult = {"sigmoid": torch.sigmoid(z), "silu": pb.silu(z), None: z}[act]
    want = (pb.rms(o.double().view(T, groups, size), 1e-5).reshape(T, -1) * w.double()) * mult
    got = ops.group_norm_gate(o.to(DEV), w.to(DEV), 1e-5, gate.to(DEV), 3, act, groups, size, torch.float32)
    assert torch.allclose(got.double().cpu(), want, rtol=2e-5, atol=2e-5)
    bare = ops.group_norm_gate(o.to(DEV), None, 1e-5, None, 0, None, groups, size, torch.bfloat16)
    assert torch.allclose(bare.double().cpu(), pb.rms(o.double().view(T, groups, size), 1e-5).reshape(T, -1), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_elementwise_pieces(dtype):
    g = torch.Generator().manual_seed(8)
    rows = (3.0 * torch.randn(9, 50, generator=g)).to(dtype)
    got = ops.relu_sq(rows.to(DEV), 4, 40).double().cpu()
    assert torch.allclose(got, torch.relu(rows[:, 4:44].double()) ** 2, **_tol(dtype))
    ctx = torch.randn(9, 21, generator=g).to(dtype)
    out = ops.gate_mul(ctx.clone().to(DEV), rows.to(DEV), 7).double().cpu()
    assert torch.allclose(out, ctx.double() * torch.sigmoid(rows[:, 7:28].double()), **_tol(dtype))
    f = rows.float().to(DEV)
    ops.silu_rows(f, 5, 30)
    assert torch.allclose(f[:, 5:35].double().cpu(), pb.silu(rows[:, 5:35].double()), rtol=2e-5, atol=2e-5)
    assert torch.equal(f[:, :5].cpu(), rows[:, :5].float()) and torch.equal(f[:, 35:].cpu(), rows[:, 35:].float())
    # a gated hidden layer of experts, each block times its token's weight
    E, ff = 3, 8
    scale = torch.rand(9, E, generator=g)
    scale[:, 1] = 0.0
    r2 = (2.0 * torch.randn(9, 2 * E * ff, generator=g)).to(dtype)
    want = pb.silu(r2[:, :E * ff].double()) * r2[:, E * ff:].double() * scale.double().repeat_interleave(ff, dim=1)
    got = ops.glu_act(r2.to(DEV), 0, E * ff, E * ff, "swish", 0.0, 0.0, 1.0, scale.to(DEV), ff, E).double().cpu()
    assert torch.allclose(got, want, **_tol(dtype)) and float(got[:, ff:2 * ff].abs().sum()) == 0.0


@pytest.mark.parametrize("shape", [(8, 3), (9, 9), (5, 1), (40, 6), (64, 2)])
def test_router_takes_the_softmax_over_the_chosen(shape):
    E, top = shape
    g = torch.Generator().manual_seed(E)
    logits = 3.0 * torch.randn(33, E, generator=g)
    chosen, w, _ = pb.route_top(logits.double(), top)
    want = torch.zeros(33, E, dtype=F).scatter_(1, chosen, w)
    weights, got_chosen = ops.route(logits.to(DEV), top, 1, 1, 0.0, want_chosen=True)
    assert torch.allclose(weights.double().cpu(), want, rtol=1e-5, atol=1e-6)
    assert torch.equal(got_chosen.cpu().long(), chosen)
