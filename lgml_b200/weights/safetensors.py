"""safetensors files: index, read, write.

The format and every check follow mischief/lgml's reader (``src/safetensors.c``):
an 8-byte little-endian header length, a JSON header, raw little-endian data
(``st_read`` ``:278-332``); the header length is bounded and must lie inside the
file (``:101``); a tensor has at most four dimensions, each at least one
(``:173-188``); ``begin <= end <= data size`` and ``end - begin`` equals the
element count times the element size (``check_entry`` ``:229-244``); names are
1..63 bytes (``:313-315``); a name that two files hold is an error (``:486-487``)
and so is a folder without tensors (``:545``).
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

from .. import host

MAX_HEADER = 100 << 20
MAX_TENSORS = 65536
MAX_NAME = 63

# dtype -> (bytes per element, numpy type used to view the bytes, torch type of the view)
_DTYPES = {
    "F64": (8, "<f8", torch.float64),
    "F32": (4, "<f4", torch.float32),
    "F16": (2, "<f2", torch.float16),
    "BF16": (2, "<u2", torch.bfloat16),
    "I64": (8, "<i8", torch.int64),
    "I32": (4, "<i4", torch.int32),
    "I16": (2, "<i2", torch.int16),
    "I8": (1, "i1", torch.int8),
}
_TORCH_TO_ST = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8"}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file; the message names the file."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    path: Path
    begin: int  # absolute offsets in the file
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


def read_index(path) -> Dict[str, TensorEntry]:
    """The tensors of one file, every size and offset checked; reads no data.  The header is
    read and checked by the host library (``csrc/host/lgml_host.c``)."""
    path = Path(path)
    lib = host.lib()
    ix = lib.lgml_st_open(str(path).encode())
    if not ix:
        raise SafetensorsError(host.last_error())
    try:
        out: Dict[str, TensorEntry] = {}
        for i in range(lib.lgml_st_count(ix)):
            e = lib.lgml_st_get(ix, i).contents
            name = e.name.decode("utf-8")
            out[name] = TensorEntry(name, host.ST_DTYPES[e.dtype], tuple(int(d) for d in e.shape[: e.rank]), path, int(e.begin), int(e.end))
        return out
    finally:
        lib.lgml_st_close(ix)


def index_folder(folder) -> Dict[str, TensorEntry]:
    """All tensors of a model folder.  With ``model.safetensors.index.json`` the
    files it names are read; else every ``*.safetensors`` in the folder."""
    folder = Path(folder)
    idx_file = folder / "model.safetensors.index.json"
    if idx_file.exists():
        try:
            wm = json.loads(idx_file.read_text())["weight_map"]
            files = sorted({folder / v for v in wm.values()})
        except (KeyError, TypeError, AttributeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{idx_file}: no usable weight_map: {e}") from None
    else:
        files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise SafetensorsError(f"{folder}: no safetensors files")
    out: Dict[str, TensorEntry] = {}
    for f in files:
        if not f.exists():
            raise SafetensorsError(f"{f}: named by the index but missing")
        for name, ent in read_index(f).items():
            if name in out:
                raise SafetensorsError(f"tensor '{name}' is in both {out[name].path.name} and {f.name}")
            out[name] = ent
    if not out:
        raise SafetensorsError(f"{folder}: no tensors")
    return out


def stored_dtype(entry: TensorEntry) -> torch.dtype:
    """The torch type a tensor is stored in."""
    return _DTYPES[entry.dtype][2]


def read_tensor(entry: TensorEntry) -> torch.Tensor:
    """The tensor on the host in its stored type, read by the host library into memory of its own."""
    torch_dtype = _DTYPES[entry.dtype][2]
    t = torch.empty(entry.shape, dtype=torch_dtype)
    nbytes = entry.end - entry.begin
    if nbytes != t.numel() * t.element_size():
        raise SafetensorsError(f"{entry.path}: tensor '{entry.name}' holds {nbytes} bytes, its shape wants {t.numel() * t.element_size()}")
    if nbytes and host.lib().lgml_st_read(str(entry.path).encode(), entry.begin, nbytes, t.data_ptr()):
        raise SafetensorsError(f"{host.last_error()} (tensor '{entry.name}')")
    return t


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    """Write host tensors under their names, in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise SafetensorsError(f"tensor '{name}' has a type safetensors cannot hold: {t.dtype}")
        st = _TORCH_TO_ST[t.dtype]
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": st, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
