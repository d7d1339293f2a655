"""Python face of the CUDA kernels: checks arguments, passes raw pointers, raises on failure.

There is no other implementation behind these functions.  If the library cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises; nothing falls back to the CPU or to
a library's model code.
"""
from __future__ import annotations

import collections
import ctypes
import os
from typing import Optional

import torch

from .csrc.build import load_module

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 storage, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The raw handle of torch's current stream on the current device (asked of torch's C layer directly: the Python
    wrapper costs several microseconds, which counts when a step launches two hundred kernels)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _check(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_SIGS = {}


def _fn(module: str, name: str, argtypes, defines=None, restype=c_int):
    key = (module, name, tuple(sorted(defines.items())) if defines else None)
    f = _SIGS.get(key)
    if f is None:
        lib = load_module(module, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = restype
        f._lib = lib
        _SIGS[key] = f
    return f


_LAUNCHES = [0]
# How often each kind of launch was made from the host (a replayed CUDA graph does not pass here): tests read it to
# assert that the kernel they mean to cover is the one that ran. Launchers add kinds of their own with ``note``.
LAUNCH_KINDS = collections.Counter()


def note(kind: str) -> None:
    LAUNCH_KINDS[kind] += 1


def kernel_launches() -> int:
    """How many launcher calls of this package's own kernels have been made in this process."""
    return _LAUNCHES[0]


def _call(f, *args) -> None:
    _LAUNCHES[0] += 1
    LAUNCH_KINDS[f.__name__] += 1
    rc = f(*args)
    if rc != 0:
        msg = f._lib.ib_last_error()
        raise KernelError(f"{f.__name__} failed ({rc}): {msg.decode() if msg else 'no message'}")


# ----------------------------------------------------------------------------- plain kernels

def embedding(table: torch.Tensor, ids: torch.Tensor, status: Optional[torch.Tensor] = None,
              feedback: Optional[torch.Tensor] = None, token_seg: Optional[torch.Tensor] = None,
              seg_slot: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """float32 rows of ``table`` ([vocab, hidden], float32 or bfloat16) for int32 ``ids``, times ``scale``. An id of
    -1 is replaced by ``feedback[seg_slot[token_seg[t]]]``: the token the sampler left on the device for that request."""
    _check(table, "table")
    _check(ids, "ids", torch.int32)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    if feedback is not None:
        _check(feedback, "feedback", torch.int32)
        _check(token_seg, "token_seg", torch.int32, (T,))
        _check(seg_slot, "seg_slot", torch.int32)
    f = _fn("plain", "ib_embedding", [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64] + [c_void_p] * 5 + [c_float, c_void_p])
    _call(f, table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), T, H, V, out.data_ptr(), _ptr(status),
          _ptr(feedback), _ptr(token_seg), _ptr(seg_slot), float(scale), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows; ``rows`` (int32) selects and orders the input rows."""
    _check(x, "x", torch.float32)
    H = x.shape[-1]
    _check(weight, "weight", torch.float32, (H,))
    if rows is not None:
        _check(rows, "rows", torch.int32)
    n = rows.numel() if rows is not None else x.numel() // H
    out = torch.empty((n, H), dtype=out_dtype, device=x.device)
    f = _fn("plain", "ib_rmsnorm", [c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, x.data_ptr(), weight.data_ptr(), float(eps), n, H, _ptr(rows), out.data_ptr(), dtype_code(out_dtype), _stream())
    return out


def linear_plain(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ w.T (+ bias) (+ residual) with float accumulation in ascending k."""
    _check(x, "x")
    _check(w, "w", x.dtype)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x is [{M},{K}] but w is {tuple(w.shape)}")
    out_dtype = out_dtype or (out.dtype if out is not None else x.dtype)
    if bias is not None:
        _check(bias, "bias", torch.float32, (N,))
    if residual is not None:
        _check(residual, "residual", torch.float32, (M, N))
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, (M, N))
    f = _fn("plain", "ib_linear_plain", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                         c_int, c_int, c_void_p])
    _call(f, x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(), M, N, K,
          dtype_code(x.dtype), dtype_code(out_dtype), _stream())
    return out


def rope_kv_write(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                  positions: torch.Tensor, token_seg: torch.Tensor, block_table: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                  write_cache: bool = True, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotates q and k of packed rows [q|k|v], stores k and v into their pages, returns q [T, heads*head_dim].
    Caches are [pages, kv_heads, page_size, head_dim]."""
    _check(qkv, "qkv")
    T = qkv.shape[0]
    _check(qkv, "qkv", None, (T, (n_heads + 2 * n_kv) * head_dim))
    _check(k_cache, "k_cache", qkv.dtype)
    _check(v_cache, "v_cache", qkv.dtype, k_cache.shape)
    n_pages, ckv, page_size, chd = k_cache.shape
    if ckv != n_kv or chd != head_dim:
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={n_kv}, head_dim={head_dim}")
    _check(positions, "positions", torch.int32, (T,))
    _check(token_seg, "token_seg", torch.int32, (T,))
    _check(block_table, "block_table", torch.int32)
    if cos is not None:
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != head_dim // 2:
            raise KernelError("rotary tables must be [max_positions, head_dim/2]")
    q = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    f = _fn("plain", "ib_rope_kv_write", [c_void_p] * 6 + [c_int64] + [c_void_p] * 3 + [c_int64] + [c_int] * 5 +
            [c_int64, c_int, c_void_p, c_void_p])
    _call(f, qkv.data_ptr(), _ptr(cos), _ptr(sin), positions.data_ptr(), token_seg.data_ptr(), block_table.data_ptr(),
          block_table.shape[1], q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv, head_dim,
          page_size, int(write_cache), n_pages, dtype_code(qkv.dtype), _ptr(status), _stream())
    return q


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                    token_seg: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                    window: Optional[int], scale: float, status: Optional[torch.Tensor] = None,
                    v_head_dim: Optional[int] = None, dist_bias: Optional[torch.Tensor] = None,
                    sink: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                    single_only: Optional[torch.Tensor] = None, keep_first: int = 0,
                    slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token over its request's pages; returns [T, heads*v_head_dim] (values are as long
    as keys unless ``v_head_dim`` says otherwise; the value pages are [pages, kv_heads, page_size, v_head_dim]).
    ``dist_bias`` float32 [L, heads]: row min(distance, L - 1) is added to the scaled scores of a query's keys;
    ``sink`` float32 [heads]: a logit per head that enters the softmax denominator only. ``out``: write there;
    ``single_only`` (the step's seg_start): only tokens that are a segment of their own are computed, the other rows
    of ``out`` stay as they are. ``keep_first``: a windowed query also sees the keys at positions below it.
    ``slopes`` float32 [heads]: slopes[h] * (query position - key position) is taken off the scaled score."""
    _check(q, "q")
    T = q.shape[0]
    vd = int(v_head_dim or head_dim)
    _check(q, "q", None, (T, n_heads * head_dim))
    _check(k_cache, "k_cache", q.dtype)
    n_pages, ckv, page_size, chd = k_cache.shape
    _check(v_cache, "v_cache", q.dtype, (n_pages, ckv, page_size, vd))
    if ckv != n_kv or chd != head_dim:
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={n_kv}, head_dim={head_dim}")
    _check(positions, "positions", torch.int32, (T,))
    _check(token_seg, "token_seg", torch.int32, (T,))
    _check(block_table, "block_table", torch.int32)
    if out is None:
        out = torch.empty((T, n_heads * vd), dtype=q.dtype, device=q.device)
    else:
        _check(out, "out", q.dtype, (T, n_heads * vd))
    if dist_bias is not None:
        _check(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[1] != n_heads:
            raise KernelError(f"dist_bias must be [distances, {n_heads}], got {tuple(dist_bias.shape)}")
    if sink is not None:
        _check(sink, "sink", torch.float32, (n_heads,))
    if slopes is not None:
        _check(slopes, "slopes", torch.float32, (n_heads,))
    f = _fn("plain", "ib_attention_plain", [c_void_p] * 4 + [c_int64] + [c_void_p] * 3 + [c_int64] + [c_int] * 5 +
            [c_float, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          token_seg.data_ptr(), positions.data_ptr(), out.data_ptr(), T, n_heads, n_kv, head_dim, page_size,
          int(window or 0), float(scale), n_pages, dtype_code(q.dtype), _ptr(status), _stream(), vd,
          _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], _ptr(sink), _ptr(single_only), int(keep_first or 0),
          _ptr(slopes))
    return out


def attention_max_head_dim() -> int:
    """The largest head size the attention kernels of this package take."""
    return int(_fn("plain", "ib_attention_plain_max_head_dim", [])())


def swiglu(gate_up: torch.Tensor, interleave8: bool = False) -> torch.Tensor:
    """rows [gate | up] -> silu(gate) * up. With interleave8 the rows are blocks of 8 gate then 8 up features."""
    _check(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("swiglu input rows must hold gate and up halves")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("plain", "ib_swiglu", [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p])
    _call(f, gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, dtype_code(gate_up.dtype), int(interleave8), _stream())
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
           feedback: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token id per row of float32 logits: argmax at temperature 0, else Gumbel-max with a
    hash of (seed, step, index). temperature float32 [B]; seed, step int64 [B]. Returns int32 [B].
    With ``feedback`` (int32 [slots]) and ``slots`` (int64 [B]) each token is also left at feedback[slots[b]]."""
    _check(logits, "logits", torch.float32)
    B, V = logits.shape
    _check(temperature, "temperature", torch.float32, (B,))
    _check(seed, "seed", torch.int64, (B,))
    _check(step, "step", torch.int64, (B,))
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    f = _fn("plain", "ib_sample", [c_void_p, c_int64, c_int64] + [c_void_p] * 7)
    _call(f, logits.data_ptr(), B, V, temperature.data_ptr(), seed.data_ptr(), step.data_ptr(), out.data_ptr(),
          _ptr(feedback), _ptr(slots), _stream())
    return out


def sample_filtered(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
                    top_k: torch.Tensor, top_p: torch.Tensor, feedback: Optional[torch.Tensor] = None,
                    slots: Optional[torch.Tensor] = None) -> torch.Tensor:
    """As ``sample``, after keeping the top_k (int64 [B], 0 = all) largest logits and then the smallest set of
    largest probabilities whose mass reaches top_p (float32 [B], 1 = all)."""
    _check(logits, "logits", torch.float32)
    B, V = logits.shape
    _check(temperature, "temperature", torch.float32, (B,))
    _check(seed, "seed", torch.int64, (B,))
    _check(step, "step", torch.int64, (B,))
    _check(top_k, "top_k", torch.int64, (B,))
    _check(top_p, "top_p", torch.float32, (B,))
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    f = _fn("plain", "ib_sample_filtered", [c_void_p, c_int64, c_int64] + [c_void_p] * 9)
    _call(f, logits.data_ptr(), B, V, temperature.data_ptr(), seed.data_ptr(), step.data_ptr(), top_k.data_ptr(),
          top_p.data_ptr(), out.data_ptr(), _ptr(feedback), _ptr(slots), _stream())
    return out


# ----------------------------------------------------------------------------- kernels of layers with state

def short_filter(rows: torch.Tensor, col0: int, weight: torch.Tensor, tails: Optional[torch.Tensor],
                 token_seg: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor) -> torch.Tensor:
    """Causal filter over time on columns [col0, col0 + C) of ``rows`` [T, ld]: y[t, c] = sum_j weight[c, j] *
    u[t - (taps - 1) + j, c], where u before a segment's first row comes from ``tails`` [slots, taps - 1, C]
    (oldest first). weight float32 [C, taps]. Returns [T, C] in the rows' dtype; the tails are not changed."""
    _check(rows, "rows")
    T, ld = rows.shape
    _check(weight, "weight", torch.float32)
    C, taps = weight.shape
    if tails is not None:
        _check(tails, "tails", rows.dtype)
        if tuple(tails.shape[1:]) != (taps - 1, C):
            raise KernelError(f"tails must be [slots, {taps - 1}, {C}], got {tuple(tails.shape)}")
    _check(token_seg, "token_seg", torch.int32, (T,))
    out = torch.empty((T, C), dtype=rows.dtype, device=rows.device)
    f = _fn("seq", "ib_short_filter", [c_void_p, c_int64, c_int, c_int, c_void_p, c_int] + [c_void_p] * 5 + [c_int64, c_int, c_void_p])
    _call(f, rows.data_ptr(), ld, int(col0), C, weight.data_ptr(), taps, _ptr(tails), token_seg.data_ptr(),
          seg_start.data_ptr(), seg_slot.data_ptr(), out.data_ptr(), T, dtype_code(rows.dtype), _stream())
    return out


def filter_tail_update(rows: torch.Tensor, col0: int, tails: torch.Tensor, seg_start: torch.Tensor,
                       seg_slot: torch.Tensor) -> None:
    """After a step: tails[slot of s] becomes the last taps - 1 values of (old tail, the rows of segment s)."""
    _check(rows, "rows")
    _check(tails, "tails", rows.dtype)
    keep, C = tails.shape[1], tails.shape[2]
    S = seg_slot.numel()
    f = _fn("seq", "ib_filter_tail", [c_void_p, c_int64, c_int, c_int, c_int] + [c_void_p] * 3 + [c_int, c_int, c_void_p])
    _call(f, rows.data_ptr(), rows.shape[1], int(col0), C, keep + 1, tails.data_ptr(), seg_start.data_ptr(),
          seg_slot.data_ptr(), S, dtype_code(rows.dtype), _stream())


def qkv_prepare_max_head_dim() -> int:
    return int(_fn("seq", "ib_qkv_prepare_max_head_dim", [])())


def qkv_prepare(rows: torch.Tensor, filt_w: Optional[torch.Tensor], tails: Optional[torch.Tensor],
                cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], n_rot: int, norm_v: bool, eps: float,
                step, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                n_heads: int, n_kv: int, head_dim: int, v_head_dim: int, write_cache: bool = True, col0: int = 0,
                inline_tail: bool = False) -> torch.Tensor:
    """Projected rows [... | q | k | v | ...] (q at column ``col0``) -> q [T, heads * head_dim] for attention, k and v
    into their pages. ``inline_tail`` (only for steps of one token per request): the kernel also moves the tails.
    Optional on the way: a short causal filter on every q, k and v channel (``filt_w`` float32 [taps, channels] with
    the requests' ``tails`` [slots, taps - 1, channels]); rotation of adjacent channel pairs of q and k over the
    first ``n_rot`` channels of each head (tables float32 [positions, n_rot / 2]); v divided by its root mean square
    per head (``norm_v``). ``step`` gives positions, token_seg, seg_start, seg_slot and the status word."""
    _check(rows, "rows")
    T, ld = rows.shape
    C = (n_heads + n_kv) * head_dim + n_kv * v_head_dim
    if ld < col0 + C:
        raise KernelError(f"rows of {ld} columns cannot hold q, k and v of {C} from column {col0}")
    n_pages, ckv, page_size, chd = k_cache.shape
    _check(k_cache, "k_cache", rows.dtype, (n_pages, n_kv, page_size, head_dim))
    _check(v_cache, "v_cache", rows.dtype, (n_pages, n_kv, page_size, v_head_dim))
    taps = 0
    if filt_w is not None:
        _check(filt_w, "filt_w", torch.float32)
        if filt_w.shape[1] != C:
            raise KernelError(f"the filter has {filt_w.shape[1]} channels, the rows {C}")
        taps = filt_w.shape[0]
        if taps > 1:
            _check(tails, "tails", rows.dtype)
            if tuple(tails.shape[1:]) != (taps - 1, C):
                raise KernelError(f"tails must be [slots, {taps - 1}, {C}], got {tuple(tails.shape)}")
    if cos is not None:
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != n_rot // 2:
            raise KernelError("rotation tables must be [positions, n_rot / 2]")
    else:
        n_rot = 0
    _check(block_table, "block_table", torch.int32)
    q = torch.empty((T, n_heads * head_dim), dtype=rows.dtype, device=rows.device)
    f = _fn("seq", "ib_qkv_prepare", [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float] +
            [c_void_p] * 5 + [c_int64] + [c_void_p] * 3 + [c_int64] + [c_int] * 6 + [c_int64, c_int, c_void_p, c_void_p])
    _call(f, rows.data_ptr(), ld, int(col0), int(bool(inline_tail) and taps > 1), _ptr(filt_w), taps, _ptr(tails) if taps > 1 else None, _ptr(cos), _ptr(sin),
          int(n_rot), int(bool(norm_v)), float(eps), step.positions.data_ptr(), step.token_seg.data_ptr(),
          step.seg_start.data_ptr(), step.seg_slot.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv, head_dim, v_head_dim, page_size,
          int(write_cache), n_pages, dtype_code(rows.dtype), _ptr(step.status), _stream())
    return q


def head_gate(ctx: torch.Tensor, rows: torch.Tensor, gate_col: int, n_heads: int, v_head_dim: int) -> torch.Tensor:
    """In place: ctx[t, h, :] *= sigmoid(rows[t, gate_col + h])."""
    _check(ctx, "ctx")
    T = ctx.shape[0]
    _check(ctx, "ctx", None, (T, n_heads * v_head_dim))
    _check(rows, "rows", ctx.dtype)
    if rows.shape[0] != T or rows.shape[1] < gate_col + n_heads:
        raise KernelError("the gate columns lie outside the rows")
    f = _fn("seq", "ib_head_gate", [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_int, c_void_p])
    _call(f, ctx.data_ptr(), rows.data_ptr(), rows.shape[1], int(gate_col), T, n_heads, v_head_dim, dtype_code(ctx.dtype), _stream())
    return ctx


def gelu_tanh(x: torch.Tensor, col0: int = 0, width: Optional[int] = None) -> torch.Tensor:
    """0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), element by element, of columns [col0, col0 + width) of the rows
    x [T, ld] (default: all of them); the result is contiguous [T, width]."""
    _check(x, "x")
    T, ld = x.shape
    width = ld - col0 if width is None else int(width)
    if col0 < 0 or width < 0 or col0 + width > ld:
        raise KernelError("the activation's columns lie outside the rows")
    out = torch.empty((T, width), dtype=x.dtype, device=x.device)
    f = _fn("seq", "ib_gelu_tanh", [c_void_p, c_int64, c_int, c_int64, c_void_p, c_int64, c_int, c_void_p])
    _call(f, x.data_ptr(), ld, int(col0), width, out.data_ptr(), T, dtype_code(x.dtype), _stream())
    return out


def gated_sum(x: torch.Tensor, gates: Optional[torch.Tensor], p: torch.Tensor, a: float = 1.0,
              q: Optional[torch.Tensor] = None, b: float = 1.0, r: Optional[torch.Tensor] = None, gate_col: int = 0) -> torch.Tensor:
    """x + sigmoid(gates[:, g:g+W]) * (a p + b q) + sigmoid(gates[:, g+W:g+2W]) * r with g = gate_col, float32 [T, W],
    written over x. q and r may be absent; without gates the terms are added as they are."""
    _check(x, "x", torch.float32)
    T, W = x.shape
    for name, t in (("p", p), ("q", q), ("r", r)):
        if t is not None:
            _check(t, name, torch.float32, (T, W))
    ldg = 0
    if gates is not None:
        _check(gates, "gates", torch.float32)
        ldg = gates.shape[1]
        if gates.shape[0] != T or ldg < gate_col + (2 * W if r is not None else W):
            raise KernelError(f"gates of shape {tuple(gates.shape)} do not cover the terms")
    f = _fn("seq", "ib_gated_sum", [c_void_p, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p,
                                    c_int64, c_int64, c_void_p])
    g_ptr = None if gates is None else gates.data_ptr() + 4 * int(gate_col)
    _call(f, x.data_ptr(), g_ptr, ldg, p.data_ptr(), float(a), _ptr(q), float(b), _ptr(r), x.data_ptr(), T, W, _stream())
    return x


def gated_recurrence_fits(dim: int, v_dim: int) -> bool:
    """True if a head's state of dim x v_dim fits the recurrence kernel's registers."""
    return bool(_fn("seq", "ib_gated_recurrence_fits", [c_int, c_int])(int(dim), int(v_dim)))


# Segments of more tokens than this go through the form of the recurrence that spreads a head's columns over CTAs.
RECURRENCE_SPREAD_FROM = 8
RECURRENCE_COLUMN_BLOCK = int(os.environ.get("INFER_B200_RECURRENCE_COLUMNS", "0"))    # 0: the launcher chooses


def gated_recurrence(proj: torch.Tensor, q_col: int, f_col: int, v_col: int, lower: torch.Tensor,
                     norm_weight: torch.Tensor, eps: float, state: torch.Tensor, seg_start: torch.Tensor,
                     seg_slot: torch.Tensor, n_heads: int, dim: int, v_dim: int, out_dtype: torch.dtype,
                     write_state: bool = True, max_len: int = 1) -> torch.Tensor:
    """The gated linear recurrence S <- diag(f) S + (1 - f) v^T, o = S^T q per head, over the tokens of every
    segment in order, from and into ``state`` float32 [slots, heads, dim, v_dim]; f = lower + (1 - lower) *
    sigmoid(proj[:, f_col:]), q = silu(proj[:, q_col:]), v = proj[:, v_col:] (proj float32 [T, ld]). Each head's o is
    divided by its root mean square and multiplied by ``norm_weight`` [v_dim]. Returns [T, heads * v_dim].
    ``max_len`` is the longest segment (known on the host): from RECURRENCE_SPREAD_FROM tokens on, the columns of a
    head are spread over several CTAs and ``proj`` is overwritten with the gates; the results have the same bits."""
    _check(proj, "proj", torch.float32)
    T, ld = proj.shape
    _check(lower, "lower", torch.float32, (n_heads * dim,))
    _check(norm_weight, "norm_weight", torch.float32, (v_dim,))
    _check(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (n_heads, dim, v_dim):
        raise KernelError(f"state must be [slots, {n_heads}, {dim}, {v_dim}], got {tuple(state.shape)}")
    if max(q_col, f_col) + n_heads * dim > ld or v_col + n_heads * v_dim > ld:
        raise KernelError("the q, f or v columns lie outside the rows")
    S = seg_slot.numel()
    _check(seg_start, "seg_start", torch.int32, (S + 1,))
    out = torch.empty((T, n_heads * v_dim), dtype=out_dtype, device=proj.device)
    spread = int(max_len) >= RECURRENCE_SPREAD_FROM
    scratch = torch.empty((T, n_heads * v_dim), dtype=torch.float32, device=proj.device) if spread else None
    sm_count = torch.cuda.get_device_properties(proj.device).multi_processor_count if spread else 0
    f = _fn("seq", "ib_gated_recurrence", [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_float] + [c_void_p] * 4 +
            [c_int] * 6 + [c_void_p, c_int, c_void_p, c_int64, c_int, c_int])
    _call(f, proj.data_ptr(), ld, int(q_col), int(f_col), int(v_col), lower.data_ptr(), norm_weight.data_ptr(), float(eps),
          state.data_ptr(), seg_start.data_ptr(), seg_slot.data_ptr(), out.data_ptr(), S, n_heads, dim, v_dim,
          int(write_state), dtype_code(out_dtype), _stream(), int(spread), _ptr(scratch), T, sm_count, RECURRENCE_COLUMN_BLOCK)
    return out


# ----------------------------------------------------------------------------- norms on sublayer results, routed
# feed-forwards, whole-row q/k norms, recurrences with a decay per key channel and with the delta rule

def norm_add(x: Optional[torch.Tensor], y: torch.Tensor, weight: torch.Tensor, eps: float,
             copy_dtype: Optional[torch.dtype] = None):
    """x + y / sqrt(mean(y^2) + eps) * weight per row, float32 [T, W], written over x (x None: the norm alone, a new
    tensor). With ``copy_dtype`` also the same rows in that dtype (for a matrix product that reads them); returns
    (rows, copy or None)."""
    _check(y, "y", torch.float32)
    T, W = y.shape
    _check(weight, "weight", torch.float32, (W,))
    if x is not None:
        _check(x, "x", torch.float32, (T, W))
    out = x if x is not None else torch.empty_like(y)
    copy = None
    if copy_dtype is not None and copy_dtype != torch.float32:
        copy = torch.empty((T, W), dtype=copy_dtype, device=y.device)
    f = _fn("mix", "ib_norm_add", [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p])
    _call(f, _ptr(x), y.data_ptr(), weight.data_ptr(), float(eps), out.data_ptr(), _ptr(copy),
          dtype_code(copy.dtype) if copy is not None else 0, T, W, _stream())
    return out, copy


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """float32 rows in ``dtype`` (x itself for float32)."""
    _check(x, "x", torch.float32)
    if dtype == torch.float32:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    f = _fn("mix", "ib_cast_rows", [c_void_p, c_void_p, c_int, c_int64, c_void_p])
    _call(f, x.data_ptr(), out.data_ptr(), dtype_code(dtype), x.numel(), _stream())
    return out


def dual_norm_sum(a: torch.Tensor, wa: torch.Tensor, sa: float, b: torch.Tensor, wb: torch.Tensor, sb: float, eps: float,
                  x: Optional[torch.Tensor] = None, wo: Optional[torch.Tensor] = None, eps_o: float = 0.0,
                  copy_dtype: Optional[torch.dtype] = None):
    """m = sa * a / rms(a) * wa + sb * b / rms(b) * wb per row (float32 [T, W]). Without ``wo`` returns (m, None).
    With ``wo``: x + m / rms(m) * wo, written over x (x None: a new tensor), and its copy in ``copy_dtype`` if given:
    returns (rows, copy or None)."""
    _check(a, "a", torch.float32)
    T, W = a.shape
    _check(b, "b", torch.float32, (T, W))
    _check(wa, "wa", torch.float32, (W,))
    _check(wb, "wb", torch.float32, (W,))
    if wo is not None:
        _check(wo, "wo", torch.float32, (W,))
    if x is not None:
        _check(x, "x", torch.float32, (T, W))
    out = x if (x is not None and wo is not None) else torch.empty_like(a)
    copy = None
    if wo is not None and copy_dtype is not None and copy_dtype != torch.float32:
        copy = torch.empty((T, W), dtype=copy_dtype, device=a.device)
    f = _fn("mix", "ib_dual_norm_sum", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
                                        c_float, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p])
    _call(f, a.data_ptr(), wa.data_ptr(), float(sa), b.data_ptr(), wb.data_ptr(), float(sb), float(eps),
          _ptr(x) if wo is not None else None, _ptr(wo), float(eps_o), out.data_ptr(), _ptr(copy),
          dtype_code(copy.dtype) if copy is not None else 0, T, W, _stream())
    return out, copy


GLU_KINDS = {"gelu_tanh": 0, "clipped_swish": 1, "swish": 2}


def glu_act(rows: torch.Tensor, gate_col: int, up_col: int, width: int, kind: str, limit: float = 0.0,
            limit2: float = 0.0, slope: float = 1.0, scale: Optional[torch.Tensor] = None, group: int = 0,
            n_groups: int = 0) -> torch.Tensor:
    """The hidden layer of a gated feed-forward, from rows [T, ld] that hold gate and up columns -> [T, width].
    "gelu_tanh": gelu_tanh(g) * u. "clipped_swish": g' = min(g, limit), u' = clamp(u, -limit, limit),
    g' * sigmoid(slope * g') * (u' + 1). "swish": g * sigmoid(g) * u. With ``scale`` float32 [T, n_groups]: block e of ``group`` columns is
    multiplied by scale[t, e]; columns from n_groups * group on are not scaled and use ``limit2``."""
    _check(rows, "rows")
    T, ld = rows.shape
    if min(gate_col, up_col) < 0 or max(gate_col, up_col) + width > ld:
        raise KernelError("the gate or up columns lie outside the rows")
    if scale is not None:
        _check(scale, "scale", torch.float32, (T, n_groups))
    out = torch.empty((T, width), dtype=rows.dtype, device=rows.device)
    f = _fn("mix", "ib_glu_act", [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_float, c_float, c_float, c_void_p,
                                  c_int64, c_int64, c_void_p, c_int64, c_int, c_void_p])
    _call(f, rows.data_ptr(), ld, int(gate_col), int(up_col), int(width), GLU_KINDS[kind], float(limit), float(limit2),
          float(slope), _ptr(scale), int(group), int(n_groups), out.data_ptr(), T, dtype_code(rows.dtype), _stream())
    return out


def route(logits: torch.Tensor, top: int, n_groups: int = 1, keep: int = 1, sum_eps: float = 0.0, want_chosen: bool = False):
    """Router of a mixture of experts on float32 logits [T, E]: softmax over all experts; the ``keep`` groups (of
    E / n_groups neighbouring experts) with the largest single score stay; of their experts the ``top`` largest are
    chosen; weights are scores / (their sum + sum_eps). Returns (weights float32 [T, E], zero where not chosen;
    chosen int32 [T, top] or None)."""
    _check(logits, "logits", torch.float32)
    T, E = logits.shape
    weights = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device) if want_chosen else None
    f = _fn("mix", "ib_route", [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    _call(f, logits.data_ptr(), T, E, int(top), int(n_groups), int(keep), float(sum_eps), weights.data_ptr(), _ptr(chosen), _stream())
    return weights, chosen


def rownorm_store(rows: torch.Tensor, col0: int, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float, step,
                  block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv: int,
                  head_dim: int, v_head_dim: int, write_cache: bool = True) -> torch.Tensor:
    """Projected rows [.. | q | k | v | ..] (q at column col0) -> q [T, heads * head_dim] with ALL of a token's q
    channels divided by their root mean square and multiplied by wq [heads * head_dim] (k likewise with wk, into the
    token's page; v into its page as it is)."""
    _check(rows, "rows")
    T, ld = rows.shape
    nq, nk, nv = n_heads * head_dim, n_kv * head_dim, n_kv * v_head_dim
    if ld < col0 + nq + nk + nv:
        raise KernelError("q, k and v lie outside the rows")
    n_pages, ckv, page_size, chd = k_cache.shape
    _check(k_cache, "k_cache", rows.dtype, (n_pages, n_kv, page_size, head_dim))
    _check(v_cache, "v_cache", rows.dtype, (n_pages, n_kv, page_size, v_head_dim))
    if wq is not None:
        _check(wq, "wq", torch.float32, (nq,))
    if wk is not None:
        _check(wk, "wk", torch.float32, (nk,))
    _check(block_table, "block_table", torch.int32)
    q = torch.empty((T, nq), dtype=rows.dtype, device=rows.device)
    f = _fn("mix", "ib_rownorm_store", [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int64,
                                        c_void_p, c_void_p, c_void_p, c_int64] + [c_int] * 6 + [c_int64, c_int, c_void_p, c_void_p])
    _call(f, rows.data_ptr(), ld, int(col0), _ptr(wq), _ptr(wk), float(eps), step.positions.data_ptr(), step.token_seg.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv,
          head_dim, v_head_dim, page_size, int(write_cache), n_pages, dtype_code(rows.dtype), _ptr(step.status), _stream())
    return q


def attention_split(q, k_cache, v_cache, block_table, step, n_heads, n_kv, head_dim, v_head_dim, window, scale,
                    dist_bias=None, sink=None, out=None, single_only=False, keep_first=0, slopes=None, gate=None, gate_col=0):
    """Paged attention with keys split over CTAs (chunks of 128 keys aligned to absolute positions, merged in
    ascending order), for tokens that read a few hundred keys each: decoded tokens of a windowed layer. Takes a
    distance bias float32 [L, heads] and a sink float32 [heads]. With ``single_only`` only tokens that are a segment
    of their own are computed (into ``out``, whose other rows stay). ``keep_first``: a windowed query also sees the keys
    at positions below it; ``slopes`` float32 [heads]: slopes[h] * distance is taken off the scaled score. ``gate``
    (rows in q's dtype, logits of a gate per output channel from column ``gate_col``): the result is multiplied by their
    sigmoid in the merge."""
    _check(q, "q")
    T = q.shape[0]
    n_pages, ckv, page_size, chd = k_cache.shape
    _check(q, "q", None, (T, n_heads * head_dim))
    _check(k_cache, "k_cache", q.dtype, (n_pages, n_kv, page_size, head_dim))
    _check(v_cache, "v_cache", q.dtype, (n_pages, n_kv, page_size, v_head_dim))
    if dist_bias is not None:
        _check(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[1] != n_heads:
            raise KernelError(f"dist_bias must be [distances, {n_heads}], got {tuple(dist_bias.shape)}")
    if sink is not None:
        _check(sink, "sink", torch.float32, (n_heads,))
    if out is None:
        out = torch.empty((T, n_heads * v_head_dim), dtype=q.dtype, device=q.device)
    else:
        _check(out, "out", q.dtype, (T, n_heads * v_head_dim))
    visible = min(int(window), int(step.max_ctx_len)) if window else int(step.max_ctx_len)
    visible = max(visible, 1)
    keep_first = int(keep_first or 0) if window else 0
    if slopes is not None:
        _check(slopes, "slopes", torch.float32, (n_heads,))
    if gate is not None:
        _check(gate, "gate", q.dtype)
        if gate.shape[0] != T or gate_col < 0 or gate_col + n_heads * v_head_dim > gate.shape[1]:
            raise KernelError("the gate columns lie outside the rows")
    n_ws = int(_fn("mix", "ib_attention_split_workspace", [c_int64, c_int, c_int, c_int, c_int], restype=c_int64)(T, n_heads, v_head_dim, visible, keep_first))
    ws = torch.empty(n_ws, dtype=torch.float32, device=q.device)
    f = _fn("mix", "ib_attention_split", [c_void_p] * 4 + [c_int64] + [c_void_p] * 5 + [c_int64] + [c_int] * 6 + [c_float, c_int64,
                                          c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64])
    _call(f, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          step.token_seg.data_ptr(), step.positions.data_ptr(), step.seg_start.data_ptr() if single_only else None, out.data_ptr(),
          ws.data_ptr(), T, n_heads, n_kv, head_dim, v_head_dim, page_size, int(window or 0), float(scale), n_pages,
          _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], _ptr(sink), visible, dtype_code(q.dtype),
          _ptr(step.status), _stream(), keep_first, _ptr(slopes), _ptr(gate), 0 if gate is None else gate.shape[1], int(gate_col))
    return out


ATTENTION_SPLIT_GROUP_MAX = 16


def attention_window(q, k_cache, v_cache, block_table, step, n_heads, n_kv, head_dim, v_head_dim, window, scale,
                     dist_bias, sink, dist_bias_by_head=None, keep_first=0, slopes=None):
    """Attention with a distance bias and a sink on the faster kernels, where they take the shape: prompt portions on
    the tensor-core kernel (bfloat16, keys and values of one size that the kernel is built for), one-token segments
    on the kernel that splits a token's keys over CTAs, into the same rows. None where a shape is refused (the caller
    then uses the plain kernel for everything). ``dist_bias_by_head``: float32 [heads, L], the bias divided by the
    scale. ``keep_first`` and ``slopes`` as in attention_split; both kernels take them."""
    from . import fast_ops
    if n_heads // n_kv > ATTENTION_SPLIT_GROUP_MAX:
        return None
    keep_first = int(keep_first or 0) if window else 0
    if step.max_q_len <= 1:
        return attention_split(q, k_cache, v_cache, block_table, step, n_heads, n_kv, head_dim, v_head_dim, window, scale, dist_bias, sink,
                               keep_first=keep_first, slopes=slopes)
    if v_head_dim != head_dim or (dist_bias is not None and dist_bias_by_head is None):
        return None
    out = fast_ops.attention_prefill_biased(q, k_cache, v_cache, block_table, step, n_heads, n_kv, head_dim, window, scale,
                                            dist_bias_by_head, sink, keep_first, slopes)
    if out is None:
        return None
    if any(n == 1 for n in step.seg_lens):
        attention_split(q, k_cache, v_cache, block_table, step, n_heads, n_kv, head_dim, v_head_dim, window, scale, dist_bias, sink,
                        out, single_only=True, keep_first=keep_first, slopes=slopes)
    return out


def decay_gates(rows: torch.Tensor, q_col: int, low_col: int, rank: int, up: torch.Tensor, bias: Optional[torch.Tensor],
                tau: float, q_scale: float) -> torch.Tensor:
    """decay[t, c] = sigmoid(bias[c] + up[:, c] . rows[t, low_col : low_col + rank]) ^ (1 / tau), float32 [T, C] with
    ``up`` float32 [rank, C] (the low rank's second factor, transposed); also multiplies columns [q_col, q_col + C) of
    the float32 rows by q_scale, in place."""
    _check(rows, "rows", torch.float32)
    T, ld = rows.shape
    _check(up, "up", torch.float32)
    C = up.shape[1]
    if up.shape[0] != rank or low_col + rank > ld or q_col + C > ld:
        raise KernelError("decay_gates: the low-rank columns or q lie outside the rows")
    if bias is not None:
        _check(bias, "bias", torch.float32, (C,))
    decay = torch.empty((T, C), dtype=torch.float32, device=rows.device)
    f = _fn("mix", "ib_decay_gates", [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p,
                                      c_int64, c_int, c_void_p])
    _call(f, rows.data_ptr(), ld, int(q_col), int(low_col), int(rank), up.data_ptr(), _ptr(bias), float(tau), float(q_scale),
          decay.data_ptr(), T, C, _stream())
    return decay


def delta_prepare_max_dim() -> int:
    return int(_fn("mix", "ib_delta_prepare_max_dim", [])())


def state_scan_max_dim() -> int:
    return int(_fn("mix", "ib_state_scan_max_dim", [])())


def delta_prepare(rows: torch.Tensor, col0: int, a_col: int, b_col: int, filt_w: Optional[torch.Tensor],
                  tails: Optional[torch.Tensor], a_log: torch.Tensor, dt_bias: torch.Tensor, unit_eps: float, q_scale: float,
                  step, n_heads: int, n_qk: int, dim: int, v_dim: int, inline_tail: bool = False) -> torch.Tensor:
    """What the gated delta rule reads, from float32 projected rows [.. q (n_qk x dim) | k | v (n_heads x v_dim) ..]
    (from column col0; per-head step-size logits at a_col, write-strength logits at b_col): every q, k, v channel
    through its causal filter (``filt_w`` float32 [taps, channels], ``tails`` float32 [slots, taps - 1, channels]) and
    silu; q and k made unit vectors per head, q times q_scale. Returns float32 [T, q | k | v | g | beta | k.q].
    ``inline_tail`` (only for steps of one token per request): the kernel also moves the tails (no ``tail_update``)."""
    _check(rows, "rows", torch.float32)
    T, ld = rows.shape
    C = 2 * n_qk * dim + n_heads * v_dim
    if col0 + C > ld or a_col + n_heads > ld or b_col + n_heads > ld:
        raise KernelError("delta_prepare: columns lie outside the rows")
    taps = 0
    if filt_w is not None:
        _check(filt_w, "filt_w", torch.float32)
        if filt_w.shape[1] != C:
            raise KernelError(f"the filter has {filt_w.shape[1]} channels, the rows {C}")
        taps = filt_w.shape[0]
        if taps > 1:
            _check(tails, "tails", torch.float32)
            if tuple(tails.shape[1:]) != (taps - 1, C):
                raise KernelError(f"tails must be [slots, {taps - 1}, {C}], got {tuple(tails.shape)}")
    _check(a_log, "a_log", torch.float32, (n_heads,))
    _check(dt_bias, "dt_bias", torch.float32, (n_heads,))
    ldp = (C + 2 * n_heads + n_qk + 3) // 4 * 4
    prep = torch.empty((T, ldp), dtype=torch.float32, device=rows.device)
    f = _fn("mix", "ib_delta_prepare", [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float,
                                        c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p])
    _call(f, rows.data_ptr(), ld, int(col0), int(a_col), int(b_col), _ptr(filt_w), taps, _ptr(tails) if taps > 1 else None,
          int(bool(inline_tail)), a_log.data_ptr(), dt_bias.data_ptr(), float(unit_eps), float(q_scale), step.token_seg.data_ptr(), step.seg_start.data_ptr(),
          step.seg_slot.data_ptr(), prep.data_ptr(), ldp, T, n_heads, n_qk, dim, v_dim, _stream())
    return prep


def tail_update(rows: torch.Tensor, col0: int, tails: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor) -> None:
    """After a step: tails[slot of s] (float32 [slots, taps - 1, C]) becomes the last taps - 1 rows of (old tail,
    columns [col0, col0 + C) of segment s's float32 rows)."""
    _check(rows, "rows", torch.float32)
    _check(tails, "tails", torch.float32)
    keep, C = tails.shape[1], tails.shape[2]
    f = _fn("mix", "ib_tail_update", [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, rows.data_ptr(), rows.shape[1], int(col0), C, keep + 1, tails.data_ptr(), seg_start.data_ptr(), seg_slot.data_ptr(),
          seg_slot.numel(), _stream())


SCAN_ROW_DECAY, SCAN_DELTA_RULE, SCAN_HEAD_DECAY, SCAN_BONUS = 0, 1, 2, 3
SCAN_SPREAD_FROM = 8          # segments of more tokens than this spread a head's columns over more CTAs


def state_scan(mode: int, rows: torch.Tensor, q_col: int, k_col: int, v_col: int, aux: torch.Tensor, aux_col: int,
               state: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor, n_heads: int, heads_per_qk: int,
               dim: int, v_dim: int, write_state: bool = True, max_len: int = 1, bonus: Optional[torch.Tensor] = None,
               silu: bool = False) -> torch.Tensor:
    """A linear recurrence with a float32 matrix state [slots, heads, dim, v_dim], over the tokens of every segment
    in order. SCAN_ROW_DECAY: S <- diag(a) S + k v^T, o = S^T q, with a in ``aux`` columns aux_col + h * dim.
    SCAN_DELTA_RULE: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with ``aux`` columns [g (heads) | beta
    (heads) | k.q (heads / heads_per_qk)] from aux_col. q, k at q_col, k_col + (h // heads_per_qk) * dim and v at
    v_col + h * v_dim of the float32 ``rows``. SCAN_HEAD_DECAY: S <- g_h S + k v^T, o = S^T q, with ``aux`` float32
    [heads] (a constant per head) or [T, ...] with g at column aux_col + h. SCAN_BONUS: o = (S + diag(u) k v^T)^T q, then
    S <- diag(a) S + k v^T, with a as for SCAN_ROW_DECAY and u = ``bonus`` float32 [heads, dim].
    ``silu``: q, k and v are z * sigmoid(z) of what the rows hold (applied while the tokens are staged).
    Returns o float32 [T, heads * v_dim]."""
    _check(rows, "rows", torch.float32)
    _check(aux, "aux", torch.float32)
    _check(state, "state", torch.float32)
    T, ld = rows.shape[-2:]
    if rows.dim() == 3:
        # q, k and v lie in planes [n, T, ld] (the results of separate products); a column is then (plane, column)
        cols = []
        for c, width in ((q_col, (n_heads // heads_per_qk) * dim), (k_col, (n_heads // heads_per_qk) * dim), (v_col, n_heads * v_dim)):
            if not (0 <= c[0] < rows.shape[0] and 0 <= c[1] and c[1] + width <= ld):
                raise KernelError("the q, k or v columns lie outside their plane")
            cols.append(c[0] * T * ld + c[1])
        if max(cols) + ld >= 2 ** 31:
            raise KernelError("the planes are too large for 32-bit columns")
        q_col, k_col, v_col = cols
        planes = True
    else:
        planes = False
    if tuple(state.shape[1:]) != (n_heads, dim, v_dim):
        raise KernelError(f"state must be [slots, {n_heads}, {dim}, {v_dim}], got {tuple(state.shape)}")
    n_qk = n_heads // heads_per_qk
    if not planes and (max(q_col, k_col) + n_qk * dim > ld or v_col + n_heads * v_dim > ld):
        raise KernelError("the q, k or v columns lie outside the rows")
    lda = 0
    if mode == SCAN_HEAD_DECAY and aux.dim() == 1:
        if aux_col + n_heads > aux.shape[0]:
            raise KernelError("a decay per head needs one value per head")
    else:
        need = {SCAN_ROW_DECAY: n_heads * dim, SCAN_BONUS: n_heads * dim, SCAN_DELTA_RULE: 2 * n_heads + n_qk, SCAN_HEAD_DECAY: n_heads}[mode]
        if aux.dim() != 2 or aux.shape[0] != T or aux_col + need > aux.shape[1]:
            raise KernelError("the decay columns lie outside their rows")
        lda = aux.shape[1]
    if mode == SCAN_BONUS:
        if bonus is None:
            raise KernelError("SCAN_BONUS needs the bonus [heads, dim]")
        _check(bonus, "bonus", torch.float32, (n_heads, dim))
    S = seg_slot.numel()
    _check(seg_start, "seg_start", torch.int32, (S + 1,))
    out = torch.empty((T, n_heads * v_dim), dtype=torch.float32, device=rows.device)
    spread = int(max_len) >= SCAN_SPREAD_FROM
    sm_count = torch.cuda.get_device_properties(rows.device).multi_processor_count if spread else 0
    f = _fn("mix", "ib_state_scan", [c_int, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                     c_void_p, c_void_p] + [c_int] * 8 + [c_void_p, c_void_p, c_int])
    _call(f, int(mode), rows.data_ptr(), ld, int(q_col), int(k_col), int(v_col), aux.data_ptr(), lda, int(aux_col),
          state.data_ptr(), seg_start.data_ptr(), seg_slot.data_ptr(), out.data_ptr(), S, n_heads, int(heads_per_qk), dim, v_dim,
          int(write_state), int(spread), sm_count, _stream(), _ptr(bonus) if mode == SCAN_BONUS else None, int(bool(silu)))
    return out


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, eps: float, gate: Optional[torch.Tensor], gate_col: int,
                   n_heads: int, v_dim: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Per (token, head): o / sqrt(mean(o^2) + eps) * weight [v_dim], times silu of the gate's logits (columns
    gate_col + h * v_dim of rows ``gate``, float32 or bfloat16) if given. o float32 [T, heads * v_dim]."""
    _check(o, "o", torch.float32)
    T = o.shape[0]
    _check(o, "o", None, (T, n_heads * v_dim))
    _check(weight, "weight", torch.float32, (v_dim,))
    ldg = 0
    if gate is not None:
        _check(gate, "gate")
        ldg = gate.shape[1]
        if gate.shape[0] != T or gate_col + n_heads * v_dim > ldg:
            raise KernelError("the gate columns lie outside the rows")
    out = torch.empty((T, n_heads * v_dim), dtype=out_dtype, device=o.device)
    f = _fn("mix", "ib_head_norm_gate", [c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int64,
                                         c_int, c_int, c_void_p])
    _call(f, o.data_ptr(), weight.data_ptr(), float(eps), _ptr(gate), ldg, int(gate_col),
          dtype_code(gate.dtype) if gate is not None else 0, out.data_ptr(), dtype_code(out_dtype), T, n_heads, v_dim, _stream())
    return out


# ----------------------------------------------------------------------------- attention through low-rank latents

def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
               rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight per float32 row; ``rows`` (int32) selects and
    orders the input rows."""
    _check(x, "x", torch.float32)
    H = x.shape[-1]
    _check(weight, "weight", torch.float32, (H,))
    if rows is not None:
        _check(rows, "rows", torch.int32)
    n = rows.numel() if rows is not None else x.numel() // H
    out = torch.empty((n, H), dtype=out_dtype, device=x.device)
    f = _fn("latent", "ib_layer_norm", [c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, x.data_ptr(), weight.data_ptr(), float(eps), n, H, _ptr(rows), out.data_ptr(), dtype_code(out_dtype), _stream())
    return out


ROTATION_LAYOUTS = {"pairs": 0, "half": 1}


def latent_prepare(rows: torch.Tensor, q_col: int, q_rank: int, kv_col: int, kv_rank: int, rot_dim: int,
                   wq: Optional[torch.Tensor], wkv: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                   sin: Optional[torch.Tensor], layout: str, step, block_table: torch.Tensor, cache: torch.Tensor,
                   out_dtype: torch.dtype, write: bool = True) -> Optional[torch.Tensor]:
    """Float32 rows of the down-projections -> the normalised query latent cq [T, q_rank] (None with q_rank 0) and,
    with ``write``, each token's row [normalised kv latent | rotated shared key part] in its page of ``cache``
    [pages, page_size, kv_rank + rot_dim]. The tables' width says how many channels of the shared part turn."""
    _check(rows, "rows", torch.float32)
    T, ld = rows.shape
    n_pages, page_size, width = cache.shape
    _check(cache, "cache", out_dtype, (n_pages, page_size, kv_rank + rot_dim))
    if q_col < 0 or q_col + q_rank > ld or (write and (kv_col < 0 or kv_col + kv_rank + rot_dim > ld)):
        raise KernelError("the latents lie outside the rows")
    if q_rank:
        _check(wq, "wq", torch.float32, (q_rank,))
    if write:
        _check(wkv, "wkv", torch.float32, (kv_rank,))
    n_rot = 0
    if cos is not None:
        n_rot = 2 * cos.shape[1]
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, tuple(cos.shape))
    _check(block_table, "block_table", torch.int32)
    cq = torch.empty((T, q_rank), dtype=out_dtype, device=rows.device) if q_rank else None
    f = _fn("latent", "ib_latent_prepare", [c_void_p, c_int64] + [c_int] * 5 + [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                            c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int64, c_int, c_int64,
                                            c_int, c_void_p, c_void_p])
    _call(f, rows.data_ptr(), ld, int(q_col), int(q_rank), int(kv_col), int(kv_rank), int(rot_dim), _ptr(wq), _ptr(wkv), float(eps),
          _ptr(cos), _ptr(sin), ROTATION_LAYOUTS[layout], n_rot, step.positions.data_ptr(), step.token_seg.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], _ptr(cq), cache.data_ptr(), page_size, n_pages, int(write), T,
          dtype_code(out_dtype), _ptr(step.status), _stream())
    return cq


def latent_query(q: torch.Tensor, w_uk: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], layout: str,
                 positions: torch.Tensor, n_heads: int, d: int, dr: int, single_step=None) -> torch.Tensor:
    """q [T, heads * (d + dr)] and the key up-projection w_uk [heads * d, R] -> queries in the latent space
    [T, heads, R + dr]: the unrotated channels carried through w_uk, the rotated ones turned by their position.
    With ``single_step`` (the step) only the rows of tokens that are a segment of their own are computed."""
    _check(q, "q")
    T = q.shape[0]
    R = w_uk.shape[1]
    _check(q, "q", None, (T, n_heads * (d + dr)))
    _check(w_uk, "w_uk", q.dtype, (n_heads * d, R))
    n_rot = 0
    if cos is not None:
        n_rot = 2 * cos.shape[1]
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, tuple(cos.shape))
    out = torch.empty((T, n_heads, R + dr), dtype=q.dtype, device=q.device)
    f = _fn("latent", "ib_latent_query", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64,
                                          c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _call(f, q.data_ptr(), w_uk.data_ptr(), _ptr(cos), _ptr(sin), ROTATION_LAYOUTS[layout], n_rot, positions.data_ptr(), out.data_ptr(),
          T, n_heads, d, dr, R, dtype_code(q.dtype), single_step.token_seg.data_ptr() if single_step is not None else None,
          single_step.seg_start.data_ptr() if single_step is not None else None, _stream())
    return out


def latent_attention_max_dims():
    f = _fn("latent", "ib_latent_attention_max_dims", [ctypes.POINTER(c_int), ctypes.POINTER(c_int)])
    a, b = c_int(0), c_int(0)
    f(ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


LATENT_CHUNK = 128                 # keys of one chunk of the latent attention kernel
LATENT_CHUNK_TC = 64               # ... of its tensor-core form for single tokens
LATENT_PARTS_MAX_BYTES = 512 << 20


def latent_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, step, dv: int, window: Optional[int],
                     scale: float, split: Optional[bool] = None, single_only: bool = False) -> torch.Tensor:
    """q [T, heads, dk] over the rows ``cache`` [pages, page_size, dk] -> contexts [T, heads, dv]: a row's first dv
    channels are its value. Two kernels. A thread per key, chunks of 128 keys, float32 or bfloat16: ``split`` spreads
    a token's chunks over CTAs (default: in steps of single tokens that alone would not fill the device); the
    result's bits do not depend on it. In bfloat16, steps of single tokens (and the single tokens of a mixed step,
    with ``single_only``) take chunks of 64 keys on the tensor cores, always spread over CTAs (``split=False`` keeps
    them on the first kernel); the two kernels differ by rounding. With ``single_only`` only tokens that are a
    segment of their own are computed (the other rows of the result are not written)."""
    _check(q, "q")
    T, H, dk = q.shape
    n_pages, page_size, _ = cache.shape
    _check(cache, "cache", q.dtype, (n_pages, page_size, dk))
    _check(block_table, "block_table", torch.int32)
    singles = T if step.decode_only else sum(1 for n in step.seg_lens if n == 1)
    # single tokens in bfloat16: chunks of 64 keys on the tensor cores, always spread over CTAs (while the parts fit)
    chunk = LATENT_CHUNK
    if q.dtype == torch.bfloat16 and dk % 8 == 0 and dv % 2 == 0 and dv <= 512 and (step.decode_only or single_only) and split is not False:
        chunk = LATENT_CHUNK_TC
    span = step.max_ctx_len if not window else min(step.max_ctx_len, int(window) + chunk - 1)
    chunks = max(1, -(-span // chunk) + (1 if window else 0))
    if chunk == LATENT_CHUNK_TC and T * H * chunks * (dv + 2) * 4 > LATENT_PARTS_MAX_BYTES:
        chunk = LATENT_CHUNK
        chunks = max(1, -(-(step.max_ctx_len if not window else min(step.max_ctx_len, int(window) + chunk - 1)) // chunk) + (1 if window else 0))
    if split is None:
        split = (step.decode_only or single_only) and singles * ((H + 7) // 8) < 256
    n_splits = chunks if (chunk == LATENT_CHUNK_TC or (split and chunks > 1)) else 1
    out = torch.empty((T, H, dv), dtype=q.dtype, device=q.device)
    parts = None
    if n_splits > 1 or chunk == LATENT_CHUNK_TC:
        from .fast_ops import device_state
        parts = device_state(q.device).workspace(T * H * n_splits * (dv + 2))
    f = _fn("latent", "ib_latent_attention", [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                              c_int, c_int, c_int, c_int, c_int, c_float, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                                              c_void_p])
    _call(f, q.data_ptr(), cache.data_ptr(), block_table.data_ptr(), block_table.shape[1], step.token_seg.data_ptr(),
          step.positions.data_ptr(), out.data_ptr(), _ptr(parts), T, H, dk, int(dv), page_size, int(window or 0), float(scale),
          n_pages, n_splits, dtype_code(q.dtype), _ptr(step.status), step.seg_start.data_ptr() if single_only else None, chunk,
          _stream())
    return out


def latent_output(ctx: torch.Tensor, w_uvT: torch.Tensor, gates: Optional[torch.Tensor], gate_col: int, mult: float,
                  out: Optional[torch.Tensor] = None, single_step=None) -> torch.Tensor:
    """Latent contexts [T, heads, R] and the value up-projection transposed per head, w_uvT [heads, R, dv] ->
    [T, heads * dv], each head times sigmoid(gates[t, gate_col + head]) (``gates`` float32 rows; None: no gate) and
    times ``mult``. With ``single_step`` (the step) only the rows of tokens that are a segment of their own are
    written, into ``out`` if given."""
    _check(ctx, "ctx")
    T, H, R = ctx.shape
    dv = w_uvT.shape[2]
    _check(w_uvT, "w_uvT", ctx.dtype, (H, R, dv))
    if gates is not None:
        _check(gates, "gates", torch.float32)
        if gates.shape[0] != T or gate_col < 0 or gate_col + H > gates.shape[1]:
            raise KernelError("the gates lie outside their rows")
    if out is None:
        out = torch.empty((T, H * dv), dtype=ctx.dtype, device=ctx.device)
    else:
        _check(out, "out", ctx.dtype, (T, H * dv))
    f = _fn("latent", "ib_latent_output", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p, c_int64, c_int, c_int, c_int,
                                           c_int, c_void_p, c_void_p, c_void_p])
    _call(f, ctx.data_ptr(), w_uvT.data_ptr(), _ptr(gates), gates.shape[1] if gates is not None else 0,
          int(gate_col) if gates is not None else -1, float(mult), out.data_ptr(), T, H, R, dv, dtype_code(ctx.dtype),
          single_step.token_seg.data_ptr() if single_step is not None else None,
          single_step.seg_start.data_ptr() if single_step is not None else None, _stream())
    return out


LATENT_PORTION_TILE = 64           # queries of one CTA of the portion kernel
LATENT_PORTION_MAX_QK, LATENT_PORTION_MAX_V = 512, 128


def latent_portion_build(d: int, dr: int, dv: int, kv_rank: int):
    """The build of the portion kernel that takes heads of d + dr key channels and dv value channels, as the defines
    of its module; None where the sizes are not multiples of 8 or beyond what the kernel holds in registers."""
    if min(d, dr, dv, kv_rank) <= 0 or d % 8 or dr % 8 or dv % 8 or kv_rank % 8:
        return None
    qk, v = -(-(d + dr) // 16) * 16, -(-dv // 16) * 16
    if qk > LATENT_PORTION_MAX_QK or v > LATENT_PORTION_MAX_V:
        return None
    return {"IB_QK_DIM": qk, "IB_V_DIM": v}


def latent_gather(cache: torch.Tensor, block_table: torch.Tensor, step, n_portions: int, span: int, window: Optional[int],
                  kv_rank: int, defines=None):
    """The rows that the step's portions (segments longer than one token, in order) can see, out of the pages
    ``cache`` [pages, page_size, kv_rank + dr] into one region of ``span`` rows per portion: row j of a region is
    position lo + j, lo = max(0, first position of the portion - window + 1) (0 without a window); rows past the
    portion's last token are zero. Returns (c [portions * span, kv_rank], r [portions * span, dr]). ``defines``: the
    build of the module to take the kernel from (the one the portion kernel of these sizes uses)."""
    _check(cache, "cache", torch.bfloat16)
    n_pages, page_size, dk = cache.shape
    dr = dk - kv_rank
    _check(block_table, "block_table", torch.int32)
    n = n_portions * span
    c = torch.empty((n, kv_rank), dtype=cache.dtype, device=cache.device)
    r = torch.empty((n, dr), dtype=cache.dtype, device=cache.device)
    f = _fn("latent_pf", "ib_latent_gather", [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64,
                                              c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p], defines)
    _call(f, cache.data_ptr(), block_table.data_ptr(), block_table.shape[1], step.seg_start.data_ptr(), step.seg_pos0.data_ptr(),
          step.n_segments, int(span), int(window or 0), page_size, n_pages, int(kv_rank), dr, c.data_ptr(), r.data_ptr(), n,
          _ptr(step.status), _stream())
    return c, r


def latent_prefill(q: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], layout: str, kv: torch.Tensor,
                   v_col: int, r: torch.Tensor, gates: Optional[torch.Tensor], gate_col: int, mult: float, step, span: int,
                   n_heads: int, d: int, dr: int, dv: int, window: Optional[int], scale: float, defines,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of the step's portions over per-head keys and values formed from the gathered rows: q [T, heads *
    (d + dr)] (rotated channels not yet turned), kv [portions * span, ld] with head h's keys at column h * d and its
    values at v_col + h * dv, r [portions * span, dr]. Writes the rows of the portions' tokens of ``out`` [T, heads *
    dv]: softmax(q k^T * scale) v, times sigmoid(gates[t, gate_col + head]) (``gates`` None: no gate) and ``mult``.
    ``defines``: what ``latent_portion_build`` returned for these sizes."""
    _check(q, "q", torch.bfloat16)
    T = q.shape[0]
    _check(q, "q", None, (T, n_heads * (d + dr)))
    _check(kv, "kv", torch.bfloat16)
    _check(r, "r", torch.bfloat16, (kv.shape[0], dr))
    n_rot = 0
    if cos is not None:
        n_rot = 2 * cos.shape[1]
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, tuple(cos.shape))
    if gates is not None:
        _check(gates, "gates", torch.float32)
        if gates.shape[0] != T or gate_col < 0 or gate_col + n_heads > gates.shape[1]:
            raise KernelError("the gates lie outside their rows")
    if out is None:
        out = torch.empty((T, n_heads * dv), dtype=q.dtype, device=q.device)
    else:
        _check(out, "out", q.dtype, (T, n_heads * dv))
    portions = [n for n in step.seg_lens if n > 1]
    if kv.shape[0] != len(portions) * span or v_col + n_heads * dv > kv.shape[1]:
        raise KernelError(f"keys and values of {tuple(kv.shape)} for {len(portions)} portions of {span} rows")
    n_tiles = sum(-(-n // LATENT_PORTION_TILE) for n in portions)
    f = _fn("latent_pf", "ib_latent_prefill", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                               c_int64, c_int, c_float, c_void_p, c_void_p, c_void_p] + [c_int] * 8 + [c_float, c_void_p],
            defines)
    _call(f, q.data_ptr(), _ptr(cos), _ptr(sin), ROTATION_LAYOUTS[layout], n_rot, kv.data_ptr(), kv.shape[1], int(v_col), r.data_ptr(),
          _ptr(gates), gates.shape[1] if gates is not None else 0, int(gate_col) if gates is not None else 0, float(mult), out.data_ptr(),
          step.seg_start.data_ptr(), step.seg_pos0.data_ptr(), step.n_segments, int(span), n_tiles, n_heads, d, dr, dv,
          int(window or 0), float(scale), _stream())
    return out


def route_sigmoid(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, mult: float = 1.0, want_chosen: bool = False):
    """Router on float32 logits [T, E] with sigmoid scores: the ``top`` experts with the largest score + correction
    are chosen (of equal ones the lower index); a chosen expert's weight is its score times ``mult``, not renormalised.
    Returns (weights float32 [T, E], zero where not chosen; chosen int32 [T, top] or None)."""
    _check(logits, "logits", torch.float32)
    T, E = logits.shape
    if correction is not None:
        _check(correction, "correction", torch.float32, (E,))
    weights = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device) if want_chosen else None
    f = _fn("latent", "ib_route_sigmoid", [c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    _call(f, logits.data_ptr(), _ptr(correction), T, E, int(top), float(mult), weights.data_ptr(), _ptr(chosen), _stream())
    return weights, chosen


def scaled_relu_sq(x: torch.Tensor, scale: Optional[torch.Tensor] = None, block: int = 0) -> torch.Tensor:
    """relu(x)^2 per element of x [T, width]; with ``scale`` float32 [T, n]: block e of ``block`` columns times scale[t, e]."""
    _check(x, "x")
    T, width = x.shape
    n_blocks = 0
    if scale is not None:
        n_blocks = scale.shape[1]
        _check(scale, "scale", torch.float32, (T, n_blocks))
    out = torch.empty_like(x)
    f = _fn("latent", "ib_scaled_relu_sq", [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p])
    _call(f, x.data_ptr(), _ptr(scale), T, width, int(block), n_blocks, out.data_ptr(), dtype_code(x.dtype), _stream())
    return out


def scale_softcap(logits: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """In place on float32 logits: cap * tanh(logits * scale / cap); cap 0: the scale alone."""
    _check(logits, "logits", torch.float32)
    f = _fn("latent", "ib_scale_softcap", [c_void_p, c_int64, c_float, c_float, c_void_p])
    _call(f, logits.data_ptr(), logits.numel(), float(scale), float(cap), _stream())
    return logits


# ----------------------------------------------------------------------------- norms after the sum, per-head query/key norms, shifted mixtures

def sum_norm(x: torch.Tensor, alpha: float, a: torch.Tensor, sa: float, b: Optional[torch.Tensor], sb: float, weight: torch.Tensor,
             eps: float, copy_dtype: Optional[torch.dtype] = None):
    """y / sqrt(mean(y^2) + eps) * weight per row with y = alpha x + sa a + sb b (b may be absent), float32 [T, W],
    written over x. With ``copy_dtype`` also the same rows in that dtype (for a matrix product that reads them);
    returns (rows, copy or None)."""
    _check(x, "x", torch.float32)
    T, W = x.shape
    _check(a, "a", torch.float32, (T, W))
    if b is not None:
        _check(b, "b", torch.float32, (T, W))
    _check(weight, "weight", torch.float32, (W,))
    copy = None
    if copy_dtype is not None and copy_dtype != torch.float32:
        copy = torch.empty((T, W), dtype=copy_dtype, device=x.device)
    f = _fn("post", "ib_sum_norm", [c_void_p, c_float, c_void_p, c_float, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p,
                                    c_int, c_int64, c_int64, c_void_p])
    _call(f, x.data_ptr(), float(alpha), a.data_ptr(), float(sa), _ptr(b), float(sb), weight.data_ptr(), float(eps), x.data_ptr(),
          _ptr(copy), dtype_code(copy.dtype) if copy is not None else 0, T, W, _stream())
    return x, copy


def head_prepare(rows: torch.Tensor, col0: int, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], n_rot: int, temp_coef: float, temp_every: int,
                 values_are_keys: bool, step, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 n_heads: int, n_kv: int, head_dim: int, v_head_dim: int, write_cache: bool = True) -> torch.Tensor:
    """Projected rows [.. | q | k | v | ..] (q at column col0; no v columns with ``values_are_keys``: a position's
    value is its key as projected) -> q [T, heads * head_dim]; k and v into the token's page. Every q and k head is
    divided by its root mean square (eps inside the root) and multiplied by wq / wk [head_dim] (None: no norm); then
    channel pairs (2i, 2i + 1) below ``n_rot`` turn by the tables cos, sin [positions, n_rot / 2]; then q is multiplied
    by 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1) (temp_every 0: not)."""
    _check(rows, "rows")
    T, ld = rows.shape
    nq, nk = n_heads * head_dim, n_kv * head_dim
    nv = 0 if values_are_keys else n_kv * v_head_dim
    if col0 < 0 or ld < col0 + nq + nk + nv:
        raise KernelError("q, k and v lie outside the rows")
    n_pages, ckv, page_size, chd = k_cache.shape
    _check(k_cache, "k_cache", rows.dtype, (n_pages, n_kv, page_size, head_dim))
    _check(v_cache, "v_cache", rows.dtype, (n_pages, n_kv, page_size, v_head_dim))
    for name, w in (("wq", wq), ("wk", wk)):
        if w is not None:
            _check(w, name, torch.float32, (head_dim,))
    if n_rot:
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != n_rot // 2:
            raise KernelError(f"rotation tables must be [positions, {n_rot // 2}], got {tuple(cos.shape)}")
    _check(block_table, "block_table", torch.int32)
    q = torch.empty((T, nq), dtype=rows.dtype, device=rows.device)
    f = _fn("post", "ib_head_prepare", [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_float, c_int,
                                        c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64] +
            [c_int] * 6 + [c_int64, c_int, c_void_p, c_void_p])
    _call(f, rows.data_ptr(), ld, int(col0), _ptr(wq), _ptr(wk), float(eps), _ptr(cos) if n_rot else None, _ptr(sin) if n_rot else None,
          int(n_rot), float(temp_coef), int(temp_every), int(bool(values_are_keys)), step.positions.data_ptr(), step.token_seg.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv,
          head_dim, v_head_dim, page_size, int(write_cache), n_pages, dtype_code(rows.dtype), _ptr(step.status), _stream())
    return q


def gate_mul(ctx: torch.Tensor, rows: torch.Tensor, gate_col: int) -> torch.Tensor:
    """ctx[t, i] *= sigmoid(rows[t, gate_col + i]), in place; both in one storage dtype."""
    _check(ctx, "ctx")
    _check(rows, "rows", ctx.dtype)
    T, W = ctx.shape
    if rows.shape[0] != T or gate_col < 0 or gate_col + W > rows.shape[1]:
        raise KernelError("the gate columns lie outside the rows")
    f = _fn("post", "ib_gate_mul", [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p])
    _call(f, ctx.data_ptr(), rows.data_ptr(), rows.shape[1], int(gate_col), W, T, dtype_code(ctx.dtype), _stream())
    return ctx


def silu_rows(rows: torch.Tensor, col0: int, width: int) -> torch.Tensor:
    """z * sigmoid(z) of columns [col0, col0 + width) of float32 rows, in place."""
    _check(rows, "rows", torch.float32)
    T, ld = rows.shape
    if col0 < 0 or col0 + width > ld:
        raise KernelError("the columns lie outside the rows")
    f = _fn("post", "ib_silu_rows", [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p])
    _call(f, rows.data_ptr(), ld, int(col0), int(width), T, _stream())
    return rows


def shift_mix(x: torch.Tensor, last: torch.Tensor, mu: torch.Tensor, step, out_dtype: torch.dtype, write_state: bool = True) -> torch.Tensor:
    """Mixtures of every token's row with the row of the token before it: out[m, t] = x[t] + (x[t - 1] - x[t]) * mu[m],
    x float32 [T, W], mu float32 [n, W] -> [n, T, W] in ``out_dtype``. The row before a segment's first token is the
    request's kept row ``last`` [slots, W] (zeros for a new request), which with ``write_state`` becomes the segment's last row."""
    _check(x, "x", torch.float32)
    T, W = x.shape
    _check(mu, "mu", torch.float32)
    n = mu.shape[0]
    _check(mu, "mu", None, (n, W))
    _check(last, "last", torch.float32)
    if last.dim() != 2 or last.shape[1] != W:
        raise KernelError(f"the kept rows must be [slots, {W}], got {tuple(last.shape)}")
    out = torch.empty((n, T, W), dtype=out_dtype, device=x.device)
    f = _fn("post", "ib_shift_mix", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                                     c_int, c_void_p])
    _call(f, x.data_ptr(), last.data_ptr(), mu.data_ptr(), n, step.token_seg.data_ptr(), step.seg_start.data_ptr(), step.seg_slot.data_ptr(),
          out.data_ptr(), dtype_code(out_dtype), T, W, int(write_state), _stream())
    return out


def double_exp_decay(rows: torch.Tensor, low_col: int, rank: int, up: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """decay[t, c] = exp(-exp(bias[c] + up[:, c] . tanh(rows[t, low_col : low_col + rank]))), float32 [T, C], with ``up``
    float32 [rank, C] (a low rank's second factor, transposed)."""
    _check(rows, "rows")
    T, ld = rows.shape
    _check(up, "up", torch.float32)
    C = up.shape[1]
    if up.shape[0] != rank or low_col < 0 or low_col + rank > ld:
        raise KernelError("double_exp_decay: the low-rank columns lie outside the rows")
    if bias is not None:
        _check(bias, "bias", torch.float32, (C,))
    decay = torch.empty((T, C), dtype=torch.float32, device=rows.device)
    f = _fn("post", "ib_double_exp_decay", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    _call(f, rows.data_ptr(), ld, int(low_col), int(rank), up.data_ptr(), _ptr(bias), decay.data_ptr(), T, C, dtype_code(rows.dtype), _stream())
    return decay


GATE_ACTS = {None: 0, "silu": 1, "sigmoid": 2}


def group_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], eps: float, gate: Optional[torch.Tensor], gate_col: int,
                    act: Optional[str], n_groups: int, size: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Per (token, group of ``size`` channels): o / sqrt(mean(o^2) + eps) * weight [groups * size] (None: no weight),
    times act(gate logits) (columns gate_col + g * size of rows ``gate``, float32 or bfloat16; ``act`` "silu", "sigmoid"
    or None for multipliers as they are) if given. o float32 [T, groups * size]."""
    _check(o, "o", torch.float32)
    T = o.shape[0]
    _check(o, "o", None, (T, n_groups * size))
    if weight is not None:
        _check(weight, "weight", torch.float32, (n_groups * size,))
    ldg = 0
    if gate is not None:
        _check(gate, "gate")
        ldg = gate.shape[1]
        if gate.shape[0] != T or gate_col < 0 or gate_col + n_groups * size > ldg:
            raise KernelError("the gate columns lie outside the rows")
    out = torch.empty((T, n_groups * size), dtype=out_dtype, device=o.device)
    f = _fn("post", "ib_group_norm_gate", [c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int, c_int64,
                                           c_int, c_int, c_void_p])
    _call(f, o.data_ptr(), _ptr(weight), float(eps), _ptr(gate), ldg, int(gate_col), dtype_code(gate.dtype) if gate is not None else 0,
          GATE_ACTS[act], out.data_ptr(), dtype_code(out_dtype), T, int(n_groups), int(size), _stream())
    return out


def relu_sq(x: torch.Tensor, col0: int = 0, width: Optional[int] = None) -> torch.Tensor:
    """max(z, 0)^2, element by element, of columns [col0, col0 + width) of the rows x [T, ld] (default: all of them);
    the result is contiguous [T, width]."""
    _check(x, "x")
    T, ld = x.shape
    width = ld - col0 if width is None else int(width)
    if col0 < 0 or width < 0 or col0 + width > ld:
        raise KernelError("the activation's columns lie outside the rows")
    out = torch.empty((T, width), dtype=x.dtype, device=x.device)
    f = _fn("post", "ib_relu_sq", [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_void_p])
    _call(f, x.data_ptr(), ld, int(col0), width, out.data_ptr(), T, dtype_code(x.dtype), _stream())
    return out
