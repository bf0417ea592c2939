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


STAGE_BYTES = 64 << 20    # the reference uploads in chunks of 64 MiB through a staging buffer (src/lgml.h:20)


class StagedUpload:
    """File -> pinned staging buffer -> device, in chunks, the read of one chunk beside the copy of
    the one before (two buffers).  The host never holds a whole tensor, and the copies run at
    pinned-memory speed (the reference: ``src/safetensors.c:396-447``)."""

    def __init__(self, device, stage_bytes: int = STAGE_BYTES):
        self.device = torch.device(device)
        self.stage_bytes = stage_bytes
        self.stages = [torch.empty(stage_bytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.events = [None, None]
        self.turn = 0
        self.bytes = 0

    def upload(self, ent: TensorEntry) -> torch.Tensor:
        """The tensor on the device in its stored type."""
        from .. import host
        from .safetensors import SafetensorsError, stored_dtype

        dt = stored_dtype(ent)
        out = torch.empty(ent.shape, dtype=dt, device=self.device)
        nbytes = ent.end - ent.begin
        if nbytes != out.numel() * out.element_size():
            raise SafetensorsError(f"{ent.path}: tensor '{ent.name}' holds {nbytes} bytes, its shape wants {out.numel() * out.element_size()}")
        raw = out.view(-1).view(torch.uint8) if out.numel() else out.view(torch.uint8)
        path = str(ent.path).encode()
        for off in range(0, nbytes, self.stage_bytes):
            n = min(self.stage_bytes, nbytes - off)
            i = self.turn % 2
            self.turn += 1
            if self.events[i] is not None:
                self.events[i].synchronize()          # the copy out of this buffer has run
            if host.lib().lgml_st_read(path, ent.begin + off, n, self.stages[i].data_ptr()):
                raise SafetensorsError(f"{host.last_error()} (tensor '{ent.name}')")
            raw[off:off + n].copy_(self.stages[i][:n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev
        self.bytes += nbytes
        return out

    def finish(self) -> None:
        for ev in self.events:
            if ev is not None:
                ev.synchronize()


def load_tensors(folder, specs: Iterable[TensorSpec], compute_dtype: torch.dtype, device, ignore: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """name -> device tensor for every spec present in the folder."""
    specs = list(specs)
    index = index_folder(folder)
    check_index(index, specs, ignore)
    out: Dict[str, torch.Tensor] = {}
    staged = StagedUpload(device) if torch.device(device).type == "cuda" else None
    for s in specs:
        ent = index.get(s.name)
        if ent is None:
            continue
        want = target_dtype(s.kind, compute_dtype)
        if s.kind == INT_TABLE and ent.dtype in ("F64", "F32", "F16", "BF16"):
            raise WeightError([], [], [(s.name + " (type " + ent.dtype + ", expected integers)", ent.shape, s.shape)])
        if staged is not None:
            # to the device in the stored type through pinned chunks, converted there
            t = staged.upload(ent)
            out[s.name] = t if t.dtype == want else t.to(want)
        else:
            out[s.name] = read_tensor(ent).to(device=device, dtype=want, non_blocking=False).contiguous()
    if staged is not None:
        staged.finish()
    return out
