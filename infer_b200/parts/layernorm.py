"""Layer norm with a weight and no bias: y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w; eps inside the
root. ``weight_name`` in the spec renames the one tensor (default "weight") under the part's prefix."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Norm, register_norm


@register_norm("layernorm")
class LayerNorm(Norm):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.size, self.eps = int(spec["size"]), float(spec["eps"])
        if self.size <= 0 or self.eps <= 0:
            raise ValueError("layernorm needs a positive size and eps")
        self.weight = None

    @classmethod
    def param_shapes(cls, spec):
        return {str(spec.get("weight_name", "weight")): (int(spec["size"]),)}

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)

    def load(self, params):
        self.weight = params[str(self.spec.get("weight_name", "weight"))].to(device=self.rt.device, dtype=torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.eps, out_dtype or self.rt.dtype, rows)
