"""Random-weights mode: a model folder from a configuration and a seed.

Matrices are N(0, std^2), norm weights 1 + N(0, std^2), biases N(0, std^2);
``TensorSpec.init`` of each part says which.  Each tensor has its own stream
keyed by (seed, name), so a tensor's values do not depend on which others are
drawn.  mischief/lgml has seeded fills of the same kind for its tests
(``src/lgml.c:3096-3155``, ``test/tiny.lua:102-119``).
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


def _stream(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, zlib.crc32(name.encode("utf-8"))]))


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
        a = _stream(seed, s.name).standard_normal(size=s.shape, dtype=np.float32)
        t = torch.from_numpy(a).mul_(scale * std).add_(mean)
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
