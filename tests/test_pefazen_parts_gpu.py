"""Each kernel of the Pefazen design alone against the plain functions of plain_pefazen.py (or float64 torch): layer
norm, the sigmoid router, relu squared with weights, the capped logits, and the attention through latents in its three
forms (a thread per key, single tokens on the tensor cores, prompt portions with per-head keys and values), over
shuffled pages with NaN in the rows that no position owns, with one far key made to stand out."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_pefazen as pp

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def test_layer_norm_against_the_plain_one():
    from infer_b200 import ops
    g = _gen(1)
    for rows, width in ((5, 36), (33, 128), (2, 1000)):
        x = (torch.randn(rows, width, generator=g) * 3 + 1.5)
        w = 1 + 0.2 * torch.randn(width, generator=g)
        want = pp.layer_norm(x.double(), w.double(), 3e-6).float()
        got = ops.layer_norm(x.to(DEV), w.to(DEV), 3e-6, torch.float32).cpu()
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-5)
        got16 = ops.layer_norm(x.to(DEV), w.to(DEV), 3e-6, torch.bfloat16).float().cpu()
        assert torch.allclose(got16, want, atol=0.03, rtol=0.01)


@pytest.mark.parametrize("experts,top", [(8, 2), (5, 1), (4, 4), (16, 4), (9, 3)])
def test_sigmoid_router_against_the_plain_choice(experts, top):
    from infer_b200 import ops
    g = _gen(experts * 10 + top)
    h = torch.randn(40, 24, generator=g)
    Wr = 0.4 * torch.randn(experts, 24, generator=g)
    corr = 0.3 * torch.randn(experts, generator=g)
    chosen, weights = pp.choose_experts(h.double(), Wr, corr, top)[:2]
    logits = pp.linear(h.double(), Wr).float()
    w_got, c_got = ops.route_sigmoid(logits.to(DEV), corr.to(DEV), top, 0.5, want_chosen=True)
    w_got, c_got = w_got.cpu(), c_got.cpu()
    for t in range(h.shape[0]):
        assert sorted(c_got[t].tolist()) == sorted(int(e) for e in chosen[t].tolist())
        dense = torch.zeros(experts)
        for e, w in zip(chosen[t].tolist(), weights[t].tolist()):
            dense[int(e)] = 0.5 * w
        assert torch.allclose(w_got[t], dense, atol=1e-6)


def test_the_correction_decides_the_choice_but_not_the_weight():
    from infer_b200 import ops
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    corr = torch.tensor([-5.0, 0.0, 0.0, 5.0])
    w, c = ops.route_sigmoid(logits.to(DEV), corr.to(DEV), 2, 1.0, want_chosen=True)
    assert sorted(c.cpu()[0].tolist()) == [1, 3]
    assert torch.allclose(w.cpu()[0], torch.tensor([0.0, torch.sigmoid(torch.tensor(1.0)).item(), 0.0, torch.sigmoid(torch.tensor(-1.0)).item()]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_relu_squared_with_weights_and_capped_logits(dtype):
    from infer_b200 import ops
    g = _gen(3)
    x = torch.randn(7, 5 * 24, generator=g).to(dtype)
    scale = torch.rand(7, 5, generator=g)
    want = (pp.relu_squared(x.double()) * scale.double().repeat_interleave(24, dim=1)).float()
    got = ops.scaled_relu_sq(x.to(DEV), scale.to(DEV), 24).float().cpu()
    assert torch.allclose(got, want, atol=1e-6 if dtype == torch.float32 else 0.02, rtol=1e-6 if dtype == torch.float32 else 0.01)
    z = 20 * torch.randn(3, 50, generator=g)
    want = pp.soft_cap(z.double() * 0.7, 12.0).float()
    assert torch.allclose(ops.scale_softcap(z.clone().to(DEV), 0.7, 12.0).cpu(), want, atol=1e-5)
    assert torch.allclose(ops.scale_softcap(z.clone().to(DEV), 0.7, 0.0).cpu(), z * 0.7, atol=1e-6)


# ---------------------------------------------------------------------------------------------------- attention

def _step(seg_lens, pos0):
    """What the kernels read of a step: segments of the given lengths that start at the given positions."""
    T = sum(seg_lens)
    seg_start = np.concatenate([[0], np.cumsum(seg_lens)]).astype(np.int32)
    token_seg = np.repeat(np.arange(len(seg_lens)), seg_lens).astype(np.int32)
    positions = np.concatenate([p + np.arange(n) for p, n in zip(pos0, seg_lens)]).astype(np.int32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return SimpleNamespace(n_tokens=T, n_segments=len(seg_lens), token_seg=t(token_seg), positions=t(positions), seg_start=t(seg_start),
                           seg_pos0=t(np.asarray(pos0, dtype=np.int32)), seg_lens=list(seg_lens), seg_pos0_host=list(pos0),
                           max_q_len=max(seg_lens), max_ctx_len=max(p + n for p, n in zip(pos0, seg_lens)),
                           decode_only=all(n == 1 for n in seg_lens), status=torch.zeros(1, dtype=torch.int32, device=DEV), extras={})


def _pages(rows_per_seq, dk, dtype, seed, page=16):
    """Each sequence's rows [length, dk] scattered over shuffled pages; rows that no position owns are NaN."""
    g = _gen(seed)
    n_pages = sum(-(-r.shape[0] // page) for r in rows_per_seq) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    cache = torch.full((n_pages, page, dk), float("nan"))
    width = max(-(-r.shape[0] // page) for r in rows_per_seq)
    table = torch.full((len(rows_per_seq), width), -1, dtype=torch.int32)
    for s, r in enumerate(rows_per_seq):
        for b in range(-(-r.shape[0] // page)):
            pg = order.pop()
            table[s, b] = pg
            chunk = r[b * page:(b + 1) * page]
            cache[pg, :chunk.shape[0]] = chunk
    return cache.to(dtype).to(DEV), table.to(DEV)


def _plain_contexts(q_lat, rows, positions, token_seg, R, window, scale):
    """softmax(q_lat . row * scale) over the visible rows, times the rows' first R channels; float64."""
    out = torch.zeros(q_lat.shape[0], q_lat.shape[1], R, dtype=torch.float64)
    for t in range(q_lat.shape[0]):
        seq, pos = rows[token_seg[t]].double(), int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        keys = seq[lo:pos + 1]
        p = torch.softmax(q_lat[t].double() @ keys.T * scale, dim=-1)
        out[t] = p @ keys[:, :R]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 37, 1])
@pytest.mark.parametrize("heads,R,dr", [(3, 32, 8), (12, 72, 24), (17, 264, 8)])
def test_latent_attention_of_single_tokens_and_of_portions_in_the_latent_form(dtype, window, heads, R, dr):
    """Decoded tokens at 0, at chunk and page borders and far out (the tensor-core kernel in bfloat16), and, with the
    thread-per-key kernel, portions; a key far back (or at the window's far edge) is made to stand out."""
    from infer_b200 import ops
    g = _gen(heads * 1000 + R + (window or 0))
    dk = R + dr
    lens = [1, 64, 65, 129, 300, 17]
    rows = [(torch.randn(n, dk, generator=g) * 0.5).to(dtype).float() for n in lens]
    cache, table = _pages(rows, dk, dtype, 5)
    for seg_lens, pos0 in (([1] * 6, [n - 1 for n in lens]), ([1, 30, 2, 1, 120, 17], [0, 34, 63, 128, 180, 0])):
        step = _step(seg_lens, pos0)
        q = (torch.randn(step.n_tokens, heads, dk, generator=g) * 0.5)
        positions, token_seg = step.positions.cpu().tolist(), step.token_seg.cpu().tolist()
        for t in range(step.n_tokens):                    # head 0 looks hard at the farthest key it may see
            far = max(0, positions[t] - window + 1) if window else 0
            q[t, 0] = rows[token_seg[t]][far] * 6.0
        q = q.to(dtype)
        scale = 1.0 / math.sqrt(dk)
        want = _plain_contexts(q.float(), rows, positions, token_seg, R, window, scale)
        got = ops.latent_attention(q.to(DEV), cache, table, step, R, window, scale).double().cpu()
        tol = 2e-5 if dtype == torch.float32 else 0.02
        assert torch.isfinite(got).all()
        assert (got - want).abs().max() < tol, (seg_lens, float((got - want).abs().max()))
        assert int(step.status.item()) == 0


@pytest.mark.parametrize("layout", ["pairs", "half"])
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("heads,d,dr,dv,R,n_rot", [(3, 16, 8, 24, 32, 8), (5, 40, 24, 8, 48, 16), (2, 128, 64, 128, 64, 64)])
def test_portions_with_per_head_keys_and_values(layout, window, heads, d, dr, dv, R, n_rot):
    """ops.latent_gather + a product + ops.latent_prefill against float64: portions that start at 0, in the middle of a
    page and behind a long context, of 2 to 200 tokens, beside single tokens whose rows must stay untouched."""
    from infer_b200 import ops
    g = _gen(heads + d + (window or 0))
    dk = R + dr
    defines = ops.latent_portion_build(d, dr, dv, R)
    assert defines is not None
    ctx_lens = [200, 1, 139, 70, 2]
    seg_lens, pos0 = [200, 1, 9, 2, 2], [0, 0, 130, 68, 0]
    rows = [(torch.randn(p + n, dk, generator=g) * 0.5).to(torch.bfloat16).float() for p, n in zip(pos0, seg_lens)]
    assert [r.shape[0] for r in rows] == ctx_lens
    cache, table = _pages(rows, dk, torch.bfloat16, 9)
    step = _step(seg_lens, pos0)
    T = step.n_tokens
    w_kv = (torch.randn(heads * (d + dv), R, generator=g) / math.sqrt(R)).to(torch.bfloat16)
    q = (torch.randn(T, heads * (d + dr), generator=g) * 0.7).to(torch.bfloat16)
    gates = torch.randn(T, heads + 3, generator=g)
    half = n_rot // 2
    freq = pp.plain_frequencies(n_rot, 100.0)
    ang = torch.arange(400, dtype=torch.float64)[:, None] * freq.double()[None, :]
    cos, sin = ang.cos().float(), ang.sin().float()
    portions = [i for i, n in enumerate(seg_lens) if n > 1]
    span = table.shape[1] * 16 if window is None else min(table.shape[1] * 16, window - 1 + max(seg_lens))
    c_rows, r_rows = ops.latent_gather(cache, table, step, len(portions), span, window, R, defines)
    assert torch.isfinite(c_rows.float()).all() and torch.isfinite(r_rows.float()).all()
    kv = (c_rows.float() @ w_kv.float().to(DEV).T).to(torch.bfloat16)
    out = torch.full((T, heads * dv), 7.0, dtype=torch.bfloat16, device=DEV)
    scale = 0.9 / math.sqrt(d + dr)
    ops.latent_prefill(q.to(DEV), cos.to(DEV), sin.to(DEV), layout, kv, heads * d, r_rows, gates.to(DEV), 2, 0.5, step, span, heads, d, dr, dv,
                       window, scale, defines, out)
    got = out.float().cpu().view(T, heads, dv)
    positions, token_seg = step.positions.cpu().tolist(), step.token_seg.cpu().tolist()
    kvs = kv.float().cpu()
    for t in range(T):
        s = token_seg[t]
        if seg_lens[s] == 1:
            assert (got[t] == 7.0).all()                  # a single token's row is another kernel's
            continue
        pos = positions[t]
        lo = max(0, pos - window + 1) if window else 0
        region0 = max(0, pos0[s] - window + 1) if window else 0
        base = portions.index(s) * span - region0
        qt = q[t].float().view(heads, d + dr).double()
        qr = pp.rotate(qt[:, d:d + n_rot], torch.tensor([pos]), freq, layout).double().view(heads, n_rot)
        for h in range(heads):
            keys_c = rows[s][lo:pos + 1].double()
            k_plain = kvs[base + lo:base + pos + 1, h * d:(h + 1) * d].double()
            v = kvs[base + lo:base + pos + 1, heads * d + h * dv:heads * d + (h + 1) * dv].double()
            sc = k_plain @ qt[h, :d] + keys_c[:, R:R + n_rot] @ qr[h] + keys_c[:, R + n_rot:] @ qt[h, d + n_rot:]
            p = torch.softmax(sc * scale, dim=0)
            want = (p @ v) * torch.sigmoid(gates[t, 2 + h].double()) * 0.5
            assert (got[t, h].double() - want).abs().max() < 0.02, (t, h, float((got[t, h].double() - want).abs().max()))
    assert int(step.status.item()) == 0
