"""Weights by tensor name.

A model says which tensors it needs (``TensorSpec``); the loader finds them in
the folder's safetensors index and puts them on the device.  As in
mischief/lgml a required tensor that is absent is an error that gives its name
(``lua/lgml/transformer.lua:272-274``, ``:403-405``) and an optional one may be
absent (``:275-277``); here all faults of a folder (missing and unexpected names,
wrong shapes) are gathered into one error.

Types: a matrix goes to the run's compute type (bfloat16, or float32 on the
32-bit path); a vector (norm weight, bias, frequency factors) is widened to
float32, which loses nothing (precedent: the reader's 1-D widening,
``src/safetensors.c:492-495``); an integer table becomes int32.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors import TensorEntry, index_folder, read_tensor

MATRIX, VECTOR, INT_TABLE = "matrix", "vector", "int"


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs.  ``init`` = (mean, scale): random-weights mode
    draws N(mean, (scale * std)^2)."""

    name: str
    shape: Tuple[int, ...]
    kind: str = MATRIX
    optional: bool = False
    init: Tuple[float, float] = (0.0, 1.0)


class WeightError(ValueError):
    """The folder's tensors do not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the names; the message lists them all."""

    def __init__(self, missing, unexpected, wrong_shape):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        parts = []
        if self.missing:
            parts.append("missing: " + ", ".join(self.missing))
        if self.unexpected:
            parts.append("unexpected: " + ", ".join(self.unexpected))
        if self.wrong_shape:
            parts.append("wrong shape: " + ", ".join(
                f"{n} is {tuple(got)}, expected {tuple(want)}" for n, got, want in self.wrong_shape))
        super().__init__("weights do not fit the model; " + "; ".join(parts))


def check_index(index: Dict[str, TensorEntry], specs: Iterable[TensorSpec], ignore: Sequence[str] = ()) -> None:
    """``ignore``: patterns (``fnmatch``) of tensor names that a folder may hold although the
    model does not read them (buffers that some exporters write); the architecture's builder
    names them, everything else the model did not ask for is reported."""
    specs = list(specs)
    known = {s.name for s in specs}
    missing = [s.name for s in specs if not s.optional and s.name not in index]
    unexpected = sorted(n for n in index if n not in known and not any(fnmatch.fnmatchcase(n, pat) for pat in ignore))
    wrong = [(s.name, index[s.name].shape, s.shape) for s in specs
             if s.name in index and tuple(index[s.name].shape) != tuple(s.shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


def target_dtype(kind: str, compute_dtype: torch.dtype) -> torch.dtype:
    if kind == MATRIX:
        return compute_dtype
    if kind == VECTOR:
        return torch.float32
    return torch.int32


def load_tensors(folder, specs: Iterable[TensorSpec], compute_dtype: torch.dtype, device, ignore: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """name -> device tensor for every spec present in the folder."""
    specs = list(specs)
    index = index_folder(folder)
    check_index(index, specs, ignore)
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        ent = index.get(s.name)
        if ent is None:
            continue
        host = read_tensor(ent)
        want = target_dtype(s.kind, compute_dtype)
        if s.kind == INT_TABLE and host.dtype.is_floating_point:
            raise WeightError([], [], [(s.name + " (type " + ent.dtype + ", expected integers)", ent.shape, s.shape)])
        out[s.name] = host.to(device=device, dtype=want, non_blocking=False).contiguous()
    return out
