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
    graph_safe = True
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
        wg, wu = tensors[prefix + ".gate_proj.weight"], tensors[prefix + ".up_proj.weight"]
        self.wd = tensors[prefix + ".down_proj.weight"]
        bg = bu = None
        if self.bias:
            bg, bu = tensors[prefix + ".gate_proj.bias"], tensors[prefix + ".up_proj.bias"]
            self.bd = tensors[prefix + ".down_proj.bias"]
        # bfloat16: the gate and up rows of a feature lie next to each other, so the product's
        # epilogue has both and applies the activation itself; float32: gate rows, then up rows.
        self.paired = rt.dtype == torch.bfloat16
        if self.paired:
            self.wgu = torch.stack([wg, wu], dim=1).reshape(2 * self.inner, self.width).contiguous()
            self.bgu = torch.stack([bg, bu], dim=1).reshape(2 * self.inner).contiguous() if self.bias else None
        else:
            self.wgu = torch.cat([wg, wu], dim=0).contiguous()
            self.bgu = torch.cat([bg, bu], dim=0).contiguous() if self.bias else None

    def first_weights(self):
        return [self.wgu]

    def forward(self, rt, h):
        if self.paired and rt.fused_swiglu(h, self.wgu):
            act = ops.gemm_bf16_swiglu(h, self.wgu, self.bgu, rt.status)
        else:
            gu = rt.linear(h, self.wgu, bias=self.bgu)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.silu_mul(gu, act, paired=self.paired)
        return rt.linear(act, self.wd, bias=self.bd, partials_ok=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
