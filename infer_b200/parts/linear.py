"""A weight matrix on the device and the choice of kernel that multiplies by it.

``out = x @ W.T (+ bias) (+ residual)``; W is kept [out, in] as checkpoints store it (row-major,
so the reduction dimension is contiguous: the layout both the plain kernel and the tensor-core
kernels want).  The matrix is held in the runtime's compute dtype, the bias in float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..runtime import Runtime


class Linear:
    def __init__(self, rt: Runtime, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.rt = rt
        self.weight = weight.to(device=rt.device, dtype=rt.dtype).contiguous()
        self.bias = None if bias is None else bias.to(device=rt.device, dtype=torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape

    @classmethod
    def share(cls, rt: Runtime, weight: torch.Tensor) -> "Linear":
        """A product by a matrix that already lies on the device in the compute dtype (no copy is made)."""
        if weight.device != rt.device or weight.dtype != rt.dtype or not weight.is_contiguous():
            raise ValueError("a shared matrix must lie on the device, contiguous, in the compute dtype")
        self = cls.__new__(cls)
        self.rt, self.weight, self.bias = rt, weight, None
        self.out_features, self.in_features = weight.shape
        return self

    @classmethod
    def join(cls, rt: Runtime, linears, align: int = 8):
        """One product for several that read the same rows: the matrices stacked (each padded with zero rows to a
        multiple of ``align``, so that every part's columns start on a 16-byte boundary of the result), biases
        likewise. Returns (Linear, [first column of each])."""
        mats, biases, starts, n = [], [], [], 0
        any_bias = any(l.bias is not None for l in linears)
        for l in linears:
            pad = (-l.out_features) % align
            starts.append(n)
            mats.append(l.weight)
            if pad:
                mats.append(torch.zeros(pad, l.in_features, dtype=l.weight.dtype, device=l.weight.device))
            if any_bias:
                biases.append(l.bias if l.bias is not None else torch.zeros(l.out_features, dtype=torch.float32, device=l.weight.device))
                if pad:
                    biases.append(torch.zeros(pad, dtype=torch.float32, device=l.weight.device))
            n += l.out_features + pad
        return cls(rt, torch.cat(mats, dim=0), torch.cat(biases) if any_bias else None), starts

    def __call__(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [rows, in] in the compute dtype (or a DeferredNorm of float32 rows). With ``residual`` (float32 [rows, out]) the result is
        float32 and is written over ``residual``. Otherwise the result has ``out_dtype`` (default:
        the compute dtype), and is written into ``out`` (contiguous [rows, out] of that dtype) if given."""
        from .base import DeferredNorm
        if residual is not None:
            out, out_dtype = residual, torch.float32
        elif out is not None:
            out_dtype = out.dtype
        if self.rt.fast("linear"):
            from .. import fast_ops
            y = fast_ops.linear(x, self.weight, self.bias, residual, out_dtype or self.rt.dtype, out)
            if y is not None:
                return y
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        return ops.linear_plain(x, self.weight, self.bias, residual, out_dtype or self.rt.dtype, out)
