"""Rotary position encoding.

The first ``n_rot`` dimensions of each head are rotated in pairs by
``pos * theta^(-2i/n_rot) / ff_i`` (``lua/lgml/transformer.lua:1756``,
``:1775``, ``:1788``; ``src/lgml.c:2067-2078``).  mischief/lgml reads the
frequency factors ``ff`` ready-made from the optional tensor ``rope_freqs``
(``lua/lgml/transformer.lua:410``); here they come from ``rope_scaling`` (or
from that tensor when a folder has one).  Pairing: ``half`` pairs dimension i
with i + n_rot/2, the order safetensors checkpoints hold; ``adjacent`` pairs 2i
with 2i+1, the reference's "normal" mode for gguf rows (the two differ by the
row permutation of ``lua/lgml/lora.lua:164-184``).

The frequencies are computed in float64 and stored as two float32 numbers each (the
rounded value and what the rounding lost); the kernel forms the angle from both in
float32 arithmetic, so that a position in the thousands turns as exactly as the first.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


def frequency_factors(head_dim: int, theta: float, scaling, n_rot: Optional[int] = None) -> List[float]:
    """ff_i >= 1 per pair.  ``scaling`` is None or an object with ``rope_type``,
    ``factor``, ``low_freq_factor``, ``high_freq_factor``,
    ``original_max_position_embeddings``."""
    n_rot = n_rot or head_dim
    half = n_rot // 2
    if scaling is None or scaling.rope_type == "default":
        return [1.0] * half
    if scaling.rope_type == "linear":
        return [float(scaling.factor)] * half
    if scaling.rope_type != "llama3":
        raise ValueError(f"unknown rope scaling '{scaling.rope_type}'")
    out = []
    orig = float(scaling.original_max_position_embeddings)
    low, high, factor = float(scaling.low_freq_factor), float(scaling.high_freq_factor), float(scaling.factor)
    for i in range(half):
        f = theta ** (-2.0 * i / n_rot)
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out.append(1.0)
        elif wavelen > orig / low:
            out.append(factor)
        else:
            s = (orig / wavelen - low) / (high - low)
            out.append(1.0 / ((1.0 - s) / factor + s))
    return out


def store_kv(rt, qkv, batch, cache, n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Write the k and v of ``qkv`` ([tokens, (H + 2 Hkv) D], or ``ops.Partials`` of it) into
    the cache as they are and return q: what a position part that has already done its own
    work on q and k (or does none) finishes with."""
    none = torch.zeros(1, dtype=torch.float32, device=rt.device)
    return ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, cache.block_table, none, 0, "half", cache.k, cache.v,
                             n_heads, n_kv_heads, head_dim, rt.status, write_kv=cache.writable)


class RotaryPosition(Part):
    """A position part that rotates pairs of q and k by position x frequency.  It owns what
    happens to q and k between the projection and the cache write (``apply``); for a rotation
    that is one fused kernel that adds up the projection's partial sums, rotates q and k by the
    angles pos * ``inv_freq[i]`` (the first ``n_rot`` dimensions, ``pairing``) and stores k and v
    in their cells.  A subclass only sets ``inv_freq`` (float32 on the device), ``n_rot`` and
    ``pairing``.  A position part that is no rotation gives its own ``apply`` with the same
    signature; ``store_kv`` does the cache write for it."""

    graph_safe = True
    n_rot = 0
    pairing = "half"
    inv_freq = None

    def apply(self, rt, qkv, batch, cache, n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
        """qkv: the fused projection's output [tokens, (H + 2 Hkv) D] in the compute type, or
        ``ops.Partials`` of it.  Writes this step's k and v into ``cache`` (unless it belongs
        to another layer call: ``cache.writable``) and returns q [tokens, H D] in the cache's
        type, ready for attention."""
        return ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, cache.block_table, self.inv_freq, self.n_rot,
                                 self.pairing, cache.k, cache.v, n_heads, n_kv_heads, head_dim, rt.status, write_kv=cache.writable)


class Rope(RotaryPosition):
    def __init__(self, head_dim: int, theta: float, scaling=None, n_rot: Optional[int] = None, pairing: str = "half",
                 factors_tensor: Optional[str] = None):
        self.head_dim = head_dim
        self.n_rot = n_rot if n_rot is not None else head_dim
        if self.n_rot % 2 or self.n_rot > head_dim:
            raise ValueError(f"n_rot {self.n_rot} must be even and at most head_dim {head_dim}")
        if pairing not in ("half", "adjacent"):
            raise ValueError(f"unknown pairing '{pairing}'")
        self.theta = float(theta)
        self.scaling = scaling
        self.pairing = pairing
        self.factors_tensor = factors_tensor  # full name of an optional tensor of ready-made factors
        self.inv_freq = None

    def tensor_specs(self, prefix):
        if self.factors_tensor:
            return [TensorSpec(self.factors_tensor, (self.n_rot // 2,), VECTOR, optional=True)]
        return []

    def bind(self, prefix, tensors, rt):
        half = self.n_rot // 2
        ff = frequency_factors(self.head_dim, self.theta, self.scaling, self.n_rot)
        given = tensors.get(self.factors_tensor) if self.factors_tensor else None
        if given is not None:
            ff = [float(v) for v in given.double().cpu().tolist()]
        inv = [self.theta ** (-2.0 * i / self.n_rot) / ff[i] for i in range(half)]
        exact = torch.tensor(inv or [0.0], dtype=torch.float64)
        hi = exact.to(torch.float32)
        self.inv_freq = torch.stack([hi, (exact - hi.double()).to(torch.float32)]).to(rt.device)


class NoPosition(RotaryPosition):
    """No position encoding: q and k stay as they are (a rotation of no dimensions)."""

    def __init__(self, **_):
        self.inv_freq = None

    def bind(self, prefix, tensors, rt):
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=rt.device)


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
