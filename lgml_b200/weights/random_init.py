"""Random-weights mode: a model folder from a configuration and a seed.

Matrices are N(0, std^2), norm weights 1 + N(0, std^2), biases N(0, std^2);
``TensorSpec.init`` of each part says which.  Value i of a tensor comes from a
counter-based stream keyed by (seed, the tensor's name, i): splitmix64 of key and
index, then Box-Muller, the fill mischief/lgml has for its test tensors
(``src/lgml.c:3064-3079``, ``:3133-3137``).  A tensor's values do not depend on which
others are drawn, nor on where they are drawn: the device kernel that fills full-size
models (``fill_normal_kernel`` in ``csrc/elementwise.cu``) and ``seeded_normal`` here
draw the same bits.  For that, nothing comes from a math library: the logarithm and
the cosine are short polynomials of single, correctly rounded float32 operations in a
fixed order, and all range reduction is integer arithmetic on 24-bit uniform numbers.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Dict, Iterable

import numpy as np
import torch

from .loader import INT_TABLE, MATRIX, TensorSpec
from .safetensors import write_safetensors

_F = np.float32
_U = np.uint64


def _hex(s: str) -> np.float32:
    return np.float32(float.fromhex(s))


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream."""
    return ((int(seed) << 32) ^ zlib.crc32(name.encode("utf-8"))) & 0xFFFFFFFFFFFFFFFF


def _splitmix64(z: np.ndarray) -> np.ndarray:
    z = z + _U(0x9E3779B97F4A7C15)
    z = (z ^ (z >> _U(30))) * _U(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> _U(27))) * _U(0x94D049BB133111EB)
    return z ^ (z >> _U(31))


def _log_u24(k: np.ndarray) -> np.ndarray:
    """ln(k / 2^24) for integers 1 <= k <= 2^24, float32 operation by operation as the device does."""
    bits = k.astype(_F).view(np.uint32)
    e = (bits >> np.uint32(23)).astype(np.int32) - np.int32(127)
    m = ((bits & np.uint32(0x7FFFFF)) | np.uint32(0x3F800000)).view(_F)
    big = m > _hex("0x1.6a09e6p+0")
    m = np.where(big, m * _F(0.5), m)
    e = e + big.astype(np.int32)
    s = (m + _F(-1.0)) / (m + _F(1.0))
    s2 = s * s
    p = _hex("0x1.99999ap-3") + s2 * (_hex("0x1.24924ap-3") + s2 * (_hex("0x1.c71c72p-4") + s2 * _hex("0x1.745d18p-4")))
    p = s2 * (_hex("0x1.555556p-2") + s2 * p)
    lnm = _F(2.0) * (s + s * p)
    return (e - np.int32(24)).astype(_F) * _hex("0x1.62e430p-1") + lnm


def _cos_u24(j: np.ndarray) -> np.ndarray:
    """cos(2 pi j / 2^24) for integers 0 <= j < 2^24."""
    q = j >> np.uint32(21)
    f = j & np.uint32(0x1FFFFF)
    g = np.where((q & np.uint32(1)) != 0, np.uint32(0x200000) - f, f)
    x = g.astype(_F) * _hex("0x1.921fb6p-22")
    x2 = x * x
    ps = _hex("-0x1.555556p-3") + x2 * (_hex("0x1.111112p-7") + x2 * (_hex("-0x1.a01a02p-13") + x2 * _hex("0x1.71de3ap-19")))
    sin = x + x * (x2 * ps)
    pc = _F(-0.5) + x2 * (_hex("0x1.555556p-5") + x2 * (_hex("-0x1.6c16c2p-10") + x2 * _hex("0x1.a01a02p-16")))
    cos = _F(1.0) + x2 * pc
    r = np.where(((q + np.uint32(1)) & np.uint32(2)) != 0, sin, cos)
    return np.where((q >= 2) & (q <= 5), -r, r)


def seeded_normal(key: int, n: int, start: int = 0) -> np.ndarray:
    """Values start .. start + n - 1 of the N(0, 1) stream of ``key``, as float32."""
    with np.errstate(over="ignore"):
        i = np.arange(start, start + n, dtype=_U)
        h = _splitmix64(_U(key) ^ _splitmix64(i))
    k = (h >> _U(40)).astype(np.uint32) + np.uint32(1)
    j = ((h >> _U(8)) & _U(0xFFFFFF)).astype(np.uint32)
    radius = np.sqrt(_F(-2.0) * _log_u24(k))
    return radius * _cos_u24(j)


def fill_normal_host(shape, mean: float, sd: float, key: int, chunk: int = 1 << 22) -> torch.Tensor:
    """float32 tensor of ``shape`` with value i = mean + sd * z_i, in pieces of ``chunk``
    values so that a large tensor needs little more memory than itself."""
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    out = np.empty(n, dtype=_F)
    for a in range(0, n, chunk):
        b = min(a + chunk, n)
        out[a:b] = _F(mean) + _F(sd) * seeded_normal(key, b - a, a)
    return torch.from_numpy(out.reshape(tuple(shape)))


def random_tensors(specs: Iterable[TensorSpec], seed: int, std: float = 0.02,
                   matrix_dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Host tensors for every non-optional spec."""
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.optional:
            continue
        if s.kind == INT_TABLE:
            raise ValueError(f"random-weights mode cannot draw the integer table '{s.name}'")
        mean, scale = s.init
        t = fill_normal_host(s.shape, mean, scale * std, tensor_key(seed, s.name))
        out[s.name] = t.to(matrix_dtype) if s.kind == MATRIX else t
    return out


def write_random_model(folder, config, seed: int, std: float = 0.02, dtype: str = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config``.  ``dtype``
    ("float32" or "bfloat16") is the stored type of the matrices; it defaults to
    the configuration's ``torch_dtype``."""
    from ..config import lookup_architecture
    from ..models import tensor_specs_for

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    dtype = dtype or getattr(config, "torch_dtype", "float32")
    matrix_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    d = config.to_dict()
    d["torch_dtype"] = dtype
    lookup_architecture(config.architecture)  # fails early on an unknown name
    tensors = random_tensors(tensor_specs_for(config), seed, std, matrix_dtype)
    (folder / "config.json").write_text(json.dumps(d, indent=1))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return folder
