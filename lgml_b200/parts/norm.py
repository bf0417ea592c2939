"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, in float32
(``src/lgml.c:1626-1633``; the weight is the separate multiply of
``lua/lgml/transformer.lua:1760``, ``:2044``, ``:2095``)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


class RMSNorm(Part):
    graph_safe = True
    def __init__(self, width: int, eps: float):
        self.width = width
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self, prefix):
        return [TensorSpec(prefix + ".weight", (self.width,), VECTOR, init=(1.0, 1.0))]

    def bind(self, prefix, tensors, rt):
        self.weight = tensors[prefix + ".weight"]

    def forward(self, rt, x, out_dtype, delta=None, rows=None):
        """Norm of x (+ delta).  x is the float32 residual stream; with ``delta`` the sum
        is written back to x.  ``rows`` (int32 on the device) picks the rows to norm."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows)


register_part("norm", "rmsnorm", RMSNorm)
