"""The two ends of a model: the token table (ids -> rows of the residual stream) and the output matrix
(normalised rows -> logits).

h[t, :] = float32(table[ids[t], :]), optionally times a constant ``scale`` (src/forward.cpp:181-187 has none);
logits = x . W^T without bias, W being the head's own matrix or, when tied, the token table itself
(src/forward.cpp:246-257, src/model.h:52). An architecture whose ends do more (a soft cap on the logits, a bias)
registers its own ``Embedding`` / ``Head`` kinds; the model only calls ``forward``. ``weight_name`` in either spec
renames the part's one tensor (default "weight") under its prefix. A head with ``logit_scale`` and / or ``softcap``
returns cap * tanh(logits * scale / cap) (the scale alone without a cap). With ``norm_weight_name`` (and ``norm_eps``) the
looked-up rows are divided by their root mean square and multiplied by that weight before they enter the residual stream.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Embedding, Head, register_embedding, register_head
from .linear import Linear


@register_embedding("token_table")
class TokenTable(Embedding):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        if self.vocab <= 0 or self.hidden <= 0:
            raise ValueError("token_table needs a positive vocab_size and hidden_size")
        scale = spec.get("scale")
        self.scale = 1.0 if scale is None else float(scale)
        self.weight = None
        self.norm_name = spec.get("norm_weight_name")
        self.norm_eps = float(spec.get("norm_eps") or 0.0)
        if self.norm_name is not None and self.norm_eps <= 0:
            raise ValueError("a norm behind the token table needs a positive norm_eps")
        self.norm_weight = None

    @classmethod
    def param_shapes(cls, spec):
        shapes = {str(spec.get("weight_name", "weight")): (int(spec["vocab_size"]), int(spec["hidden_size"]))}
        if spec.get("norm_weight_name") is not None:
            shapes[str(spec["norm_weight_name"])] = (int(spec["hidden_size"]),)
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        if name == spec.get("norm_weight_name"):
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        # The table is read row by row; it keeps the compute dtype of the matrices (a tied head multiplies by it).
        self.weight = params[str(self.spec.get("weight_name", "weight"))].to(device=self.rt.device, dtype=self.rt.dtype).contiguous()
        if self.norm_name is not None:
            self.norm_weight = params[str(self.norm_name)].to(device=self.rt.device, dtype=torch.float32).contiguous()

    def table(self):
        return self.weight

    def forward(self, step):
        rows = ops.embedding(self.weight, step.token_ids, step.status, getattr(step, "feedback", None),
                             step.token_seg, step.seg_slot, self.scale)
        if self.norm_weight is not None:
            # the norm's kernel also leaves the rows in the compute dtype, for a first layer that reads them unnormalised
            rows, copy = ops.norm_add(None, rows, self.norm_weight, self.norm_eps, self.rt.dtype)
            step.extras["rows_copy"] = (rows, copy)
        return rows


@register_head("linear_head")
class LinearHead(Head):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.logit_scale = float(spec.get("logit_scale") or 1.0)
        self.softcap = float(spec.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ValueError("a head's softcap must be positive (or absent)")
        self.linear = None

    @classmethod
    def param_shapes(cls, spec):
        return {} if spec.get("tied", False) else {str(spec.get("weight_name", "weight")): (int(spec["vocab_size"]), int(spec["hidden_size"]))}

    def load(self, params):
        if not self.tied:
            self.linear = Linear(self.rt, params[str(self.spec.get("weight_name", "weight"))])

    def tie(self, embedding):
        if not self.tied:
            return
        table = embedding.table()
        if table is None or tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError("a tied head needs an embedding part with a [vocab, hidden] table")
        self.linear = Linear.share(self.rt, table)

    def forward(self, x):
        logits = self.linear(x, out_dtype=torch.float32)
        if self.logit_scale != 1.0 or self.softcap > 0:
            ops.scale_softcap(logits, self.logit_scale, self.softcap)
        return logits
