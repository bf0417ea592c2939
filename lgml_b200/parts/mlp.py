"""The gated feed-forward: down(act(gate(h)) * up(h)) with act = SiLU
(``lua/lgml/transformer.lua:2047-2049``; silu(a) = a * sigmoid(a),
``src/lgml.c:1476-1482``).  Gate and up are one fused product: the two matrices
are concatenated row-wise when they are bound, gate first."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import MATRIX, VECTOR, TensorSpec
from .base import Part, register_part


class GatedMLP(Part):
    def __init__(self, width: int, inner: int, activation: str = "silu", bias: bool = False):
        if activation != "silu":
            raise ValueError(f"activation '{activation}' is not supported (only 'silu')")
        self.width, self.inner, self.bias = width, inner, bool(bias)
        self.wgu = self.bgu = self.wd = self.bd = None

    def tensor_specs(self, prefix):
        E, F = self.width, self.inner
        specs = [TensorSpec(prefix + ".gate_proj.weight", (F, E)), TensorSpec(prefix + ".up_proj.weight", (F, E)),
                 TensorSpec(prefix + ".down_proj.weight", (E, F))]
        if self.bias:
            specs += [TensorSpec(prefix + ".gate_proj.bias", (F,), VECTOR), TensorSpec(prefix + ".up_proj.bias", (F,), VECTOR),
                      TensorSpec(prefix + ".down_proj.bias", (E,), VECTOR)]
        return specs

    def bind(self, prefix, tensors, rt):
        self.wgu = torch.cat([tensors[prefix + ".gate_proj.weight"], tensors[prefix + ".up_proj.weight"]], dim=0).contiguous()
        self.wd = tensors[prefix + ".down_proj.weight"]
        if self.bias:
            self.bgu = torch.cat([tensors[prefix + ".gate_proj.bias"], tensors[prefix + ".up_proj.bias"]], dim=0).contiguous()
            self.bd = tensors[prefix + ".down_proj.bias"]

    def forward(self, rt, h):
        gu = rt.linear(h, self.wgu, bias=self.bgu)
        act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
        ops.silu_mul(gu, act)
        return rt.linear(act, self.wd, bias=self.bd)


register_part("feed_forward", "gated_mlp", GatedMLP)
