"""Reading and writing safetensors files.

The container is: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": …}``
and the tensors' bytes, offsets counted from the end of the header.  The
reference parses the same container by hand and maps the file
(src/engine/tq_model.c:185-305, shards :750-842); it checks the header's
bounds only (:686-694), while this reader also rejects offsets that leave the
file or disagree with dtype × shape.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
DTYPE_NAMES = {v[0]: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors container."""


def _numel(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One mapped file: ``entries`` maps a tensor's name to (dtype name, shape)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header ({size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen < 2 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} leaves the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
        self._offsets: Dict[str, Tuple[int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (begin, end) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for tensor '{name}'") from None
            if dtype not in DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype '{dtype}'")
            want = _numel(shape) * DTYPES[dtype][1]
            if not (0 <= begin <= end <= data_len) or end - begin != want:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({dtype} {list(shape)}) needs {want} bytes but its offsets "
                    f"[{begin}, {end}) give {end - begin} within {data_len} bytes of data (file truncated?)")
            self.entries[name] = (dtype, shape)
            self._offsets[name] = (begin, end)
        self._map: Optional[mmap.mmap] = None

    def _mapped(self) -> mmap.mmap:
        if self._map is None:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a CPU tensor that owns its memory)."""
        dtype, shape = self.entries[name]
        begin, end = self._offsets[name]
        tdtype = DTYPES[dtype][0]
        if end == begin:
            return torch.empty(shape, dtype=tdtype)
        buf = self._mapped()[self._data_start + begin:self._data_start + end]
        return torch.frombuffer(bytearray(buf), dtype=tdtype).reshape(shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()


def find_shards(folder: str) -> List[str]:
    """Files that hold a folder's tensors: those the index names, else every
    *.safetensors file, in name order."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            try:
                wm = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no readable 'weight_map'") from None
        files = sorted(set(wm.values()))
    else:
        files = sorted(n for n in os.listdir(folder) if n.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in model folder '{folder}'")
    paths = [os.path.join(folder, n) for n in files]
    for p in paths:
        if not os.path.isfile(p):
            raise FileNotFoundError(f"shard '{p}' named by the index does not exist")
    return paths


class SafetensorsWriter:
    """Streams tensors into one file; the header is fixed up front from
    (name, dtype, shape), so a model larger than host memory can be written."""

    def __init__(self, path: str, entries: Iterable[Tuple[str, torch.dtype, Sequence[int]]],
                 metadata: Optional[Dict[str, str]] = None):
        header: Dict[str, object] = {}
        if metadata:
            header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
        off = 0
        self._order: List[Tuple[str, torch.dtype, Tuple[int, ...], int]] = []
        for name, dtype, shape in entries:
            if name in header:
                raise SafetensorsError(f"tensor '{name}' listed twice")
            nbytes = _numel(shape) * DTYPES[DTYPE_NAMES[dtype]][1]
            header[name] = {"dtype": DTYPE_NAMES[dtype], "shape": [int(s) for s in shape],
                            "data_offsets": [off, off + nbytes]}
            self._order.append((name, dtype, tuple(int(s) for s in shape), nbytes))
            off += nbytes
        blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
        blob += b" " * ((8 - len(blob) % 8) % 8)
        self._f = open(path, "wb")
        self._f.write(struct.pack("<Q", len(blob)))
        self._f.write(blob)
        self._next = 0

    def write(self, name: str, tensor: torch.Tensor) -> None:
        want_name, dtype, shape, nbytes = self._order[self._next]
        if name != want_name:
            raise SafetensorsError(f"tensors must be written in header order: expected '{want_name}', got '{name}'")
        if tuple(tensor.shape) != shape or tensor.dtype != dtype:
            raise SafetensorsError(f"tensor '{name}': header says {dtype} {list(shape)}, got "
                                   f"{tensor.dtype} {list(tensor.shape)}")
        t = tensor.detach().contiguous().cpu()
        if nbytes:
            self._f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                          t.reshape(1).view(torch.uint8).numpy().tobytes())
        self._next += 1

    def close(self) -> None:
        if self._next != len(self._order):
            missing = self._order[self._next][0]
            self._f.close()
            raise SafetensorsError(f"writer closed before tensor '{missing}' was written")
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    w = SafetensorsWriter(path, [(n, t.dtype, t.shape) for n, t in tensors.items()], metadata)
    for n, t in tensors.items():
        w.write(n, t)
    w.close()
