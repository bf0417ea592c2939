"""The attention mixer: q/k/v projections, position encoding, cache write, attention over
the cache, output projection.

Formulas in mischief/lgml's order (``lua/lgml/transformer.lua``): q, k, v = W h
(``:1770``, ``:1779-1781``), rotate q and k (``:1775``, ``:1788``), write k and v to
the cache before attention reads it (``:1838-1839``, ``:2405-2406``), softmax of
(q.k) * scale + causal mask over the request's own cells and the weighted sum of v
(``:1805-1816``), scale 1/sqrt(D) unless given (``:1845``), then W_o (``:1864``).  The
reference loads no bias (``:304-319``); with ``bias`` the four projections add one.

q, k and v are one fused product: the three matrices are concatenated row-wise when
they are bound.

What happens to q and k between the projection and the cache write belongs to the
position part (``position.apply``), so a position encoding that is no rotation needs no
change here.  Optional extras that other families of the reference switch on and Llama
leaves off (``L.q_norm`` / ``L.k_norm`` ``lua/lgml/transformer.lua:1772-1786``,
``hp.softcap``): ``q_norm`` / ``k_norm`` (norm parts over the head size, applied per head
before the position part) and ``softcap`` (a cap on the scaled scores).  Absent, they cost
nothing.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache import PagedKV
from ..weights import MATRIX, VECTOR, TensorSpec
from .base import Part, register_part
from .rope import RotaryPosition


class Attention(Part):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, position, bias: bool = False,
                 out_bias: Optional[bool] = None, window: Optional[int] = None, scale: Optional[float] = None,
                 q_norm=None, k_norm=None, softcap: Optional[float] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are no multiple of {n_kv_heads} KV heads")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.position = position
        self.bias = bool(bias)
        self.out_bias = self.bias if out_bias is None else bool(out_bias)
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_norm, self.k_norm = q_norm, k_norm
        self.softcap = float(softcap) if softcap else 0.0
        self.wqkv = self.bqkv = self.wo = self.bo = None

    @property
    def graph_safe(self):
        """Its own launches are fixed by the batch's shape; whether a step through it can be
        captured is up to the parts it is given."""
        return all(getattr(p, "graph_safe", False) for p in (self.position, self.q_norm, self.k_norm) if p is not None)

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def tensor_specs(self, prefix):
        H, G, D, E = self.n_heads, self.n_kv_heads, self.head_dim, self.width
        specs = [TensorSpec(prefix + ".q_proj.weight", (H * D, E)), TensorSpec(prefix + ".k_proj.weight", (G * D, E)),
                 TensorSpec(prefix + ".v_proj.weight", (G * D, E)), TensorSpec(prefix + ".o_proj.weight", (E, H * D))]
        if self.bias:
            specs += [TensorSpec(prefix + ".q_proj.bias", (H * D,), VECTOR), TensorSpec(prefix + ".k_proj.bias", (G * D,), VECTOR),
                      TensorSpec(prefix + ".v_proj.bias", (G * D,), VECTOR)]
        if self.out_bias:
            specs.append(TensorSpec(prefix + ".o_proj.bias", (E,), VECTOR))
        for part, stem in ((self.q_norm, ".q_norm"), (self.k_norm, ".k_norm")):
            if part is not None:
                specs += part.tensor_specs(prefix + stem)
        return specs + self.position.tensor_specs(prefix)

    def bind(self, prefix, tensors, rt):
        self.wqkv = torch.cat([tensors[prefix + f".{n}_proj.weight"] for n in "qkv"], dim=0).contiguous()
        self.wo = tensors[prefix + ".o_proj.weight"]
        if self.bias:
            self.bqkv = torch.cat([tensors[prefix + f".{n}_proj.bias"] for n in "qkv"], dim=0).contiguous()
        if self.out_bias:
            self.bo = tensors[prefix + ".o_proj.bias"]
        for part, stem in ((self.q_norm, ".q_norm"), (self.k_norm, ".k_norm")):
            if part is not None:
                part.bind(prefix + stem, tensors, rt)
        self.position.bind(prefix, tensors, rt)

    def _norm_heads(self, rt, qkv):
        """q and k normed head by head (each head a row of ``head_dim`` for the norm part); v as it is."""
        H, G, D = self.n_heads, self.n_kv_heads, self.head_dim
        full = (qkv.sum() if isinstance(qkv, ops.Partials) else qkv).float()
        n = full.shape[0]
        out = torch.empty((n, (H + 2 * G) * D), dtype=rt.dtype, device=full.device)
        lo = 0
        for part, heads in ((self.q_norm, H), (self.k_norm, G), (None, G)):
            piece = full[:, lo:lo + heads * D]
            if part is not None:
                piece = part.forward(rt, piece.reshape(n * heads, D).contiguous(), rt.dtype).view(n, heads * D)
            out[:, lo:lo + heads * D] = piece
            lo += heads * D
        return out

    def forward(self, rt, h, batch, cache):
        """h [tokens, width] in the compute type -> delta [tokens, width].  ``cache`` has
        ``k``, ``v`` (pages), ``block_table`` and ``writable`` (False when the cache
        belongs to another layer, which has already written this step's cells)."""
        H, D = self.n_heads, self.head_dim
        # the products may come back as partial sums over K (few tokens): the kernel that
        # reads them next adds them up, so no pass is spent on that alone
        qkv = rt.linear(h, self.wqkv, bias=self.bqkv, partials_ok=True)
        if self.q_norm is not None or self.k_norm is not None:
            qkv = self._norm_heads(rt, qkv)
        apply = getattr(self.position, "apply", None)
        if apply is None:       # a part that gives only the three attributes of a rotation
            apply = lambda *a: RotaryPosition.apply(self.position, *a)
        q = apply(rt, qkv, batch, cache, H, self.n_kv_heads, D)
        o = torch.empty((h.shape[0], H * D), dtype=h.dtype, device=h.device)
        rt.attention(q, batch, cache, o, H, self.scale, self.window or 0, softcap=self.softcap)
        return rt.linear(o, self.wo, bias=self.bo, partials_ok=True)


register_part("mixer", "attention", Attention)
