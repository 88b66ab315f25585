"""Reading and writing the safetensors container.

Layout (the same the reference parses in src/SharpInference.Core/SafetensorsLoader.cs:190-231):
an 8-byte little-endian header length, a JSON header mapping tensor names to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (plus an optional ``__metadata__``), then
the raw little-endian tensor bytes.  A model folder holds ``model.safetensors``, or shards
listed by ``model.safetensors.index.json`` (``weight_map``), or files matching
``model*.safetensors`` (src/SharpInference.Core/SafetensorsLoader.cs:49-101).

Tensors are memory-mapped and handed out as torch views without a copy.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_DTYPE_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype_name: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: "SafetensorsFile"

    @property
    def dtype(self) -> torch.dtype:
        if self.dtype_name not in _DTYPES:
            raise SafetensorsError(
                f"tensor '{self.name}' in {self.file.path} has dtype {self.dtype_name}, which is not supported "
                f"(supported: {', '.join(sorted(_DTYPES))})")
        return _DTYPES[self.dtype_name][0]

    def load(self) -> torch.Tensor:
        """A CPU tensor viewing the mapped file (read-only memory: copy before writing)."""
        dtype, size = self.dtype, _DTYPES[self.dtype_name][1]
        count = 1
        for s in self.shape:
            count *= s
        if count * size != self.end - self.begin:
            raise SafetensorsError(
                f"tensor '{self.name}' in {self.file.path}: shape {list(self.shape)} of {self.dtype_name} needs "
                f"{count * size} bytes but the header gives {self.end - self.begin}")
        if count == 0:
            return torch.empty(self.shape, dtype=dtype)
        flat = torch.frombuffer(self.file.buffer, dtype=dtype, count=count, offset=self.file.data_start + self.begin)
        return flat.view(self.shape)


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as exc:
            raise SafetensorsError(f"cannot open {path}: {exc}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON: {exc}") from None
        self.data_start = 8 + header_len
        self.metadata = header.pop("__metadata__", {}) or {}
        self.buffer = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else b""
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                begin, end = info["data_offsets"]
                entry = TensorEntry(name, str(info["dtype"]), tuple(int(s) for s in info["shape"]),
                                    int(begin), int(end), self)
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for tensor '{name}': {info!r}") from None
            if not (0 <= entry.begin <= entry.end <= size - self.data_start):
                raise SafetensorsError(f"{path}: tensor '{name}' points outside the file: {info['data_offsets']}")
            self.entries[name] = entry


def discover_files(model_dir: str) -> List[str]:
    """The safetensors files of a model folder (or the one file, if a file is given)."""
    if os.path.isfile(model_dir):
        return [model_dir]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as fh:
            try:
                weight_map = json.load(fh)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as exc:
                raise SafetensorsError(f"{index}: not an index with a 'weight_map': {exc}") from None
        return [os.path.join(model_dir, f) for f in sorted(set(weight_map.values()))]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    shards = sorted(glob.glob(os.path.join(model_dir, "model*.safetensors")))
    if shards:
        return shards
    raise SafetensorsError(f"{model_dir}: no model.safetensors, model.safetensors.index.json or model*.safetensors")


def open_model(model_dir: str) -> Dict[str, TensorEntry]:
    """All tensors of a model folder by name."""
    entries: Dict[str, TensorEntry] = {}
    for path in discover_files(model_dir):
        f = SafetensorsFile(path)
        for name, entry in f.entries.items():
            if name in entries:
                raise SafetensorsError(f"tensor '{name}' appears in both {entries[name].file.path} and {path}")
            entries[name] = entry
    return entries


def save_file(tensors: Iterable[Tuple[str, torch.Tensor]], path: str, metadata: Dict[str, str] | None = None) -> None:
    """Write tensors (name, CPU tensor) in the given order.  The header is laid out first from
    shapes alone, then each tensor's bytes are streamed, so the file never sits in memory twice."""
    items = list(tensors)
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, t in items:
        if t.dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            c = t.detach().contiguous().cpu()
            if c.numel():
                fh.write(c.view(torch.uint8).numpy().tobytes() if c.dim() else c.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
