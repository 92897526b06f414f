"""Reading and writing the safetensors container, without a library.

Format and checks follow the reference's ``Checkpoint``
(src/model/safetensors.cc:20-28, 126-147, 161-269): an 8-byte little-endian
header length, a JSON header mapping tensor name to ``dtype``/``shape``/
``data_offsets`` (relative to the end of the header), ``__metadata__`` skipped;
the header must lie inside the file and be at most 256 MiB, offsets must satisfy
``begin <= end <= data size`` and ``end - begin == numel * itemsize``.  A model
folder is either ``model.safetensors`` or ``model.safetensors.index.json`` whose
``weight_map`` names the shard files (safetensors.cc:286-342); a tensor name in
two shards is an error.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


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
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 256 << 20


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int  # absolute file offset
    end: int
    shard: int


class _Shard:
    def __init__(self, path: str):
        self.path = path
        self.file = open(path, "rb")
        size = os.fstat(self.file.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a header length")
        self.map = mmap.mmap(self.file.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self.map[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(
                f"{path}: header length {hlen} exceeds the file ({size} bytes) or 256 MiB")
        try:
            self.header = json.loads(self.map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(self.header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.data_start = 8 + hlen
        self.data_bytes = size - self.data_start

    def close(self):
        try:
            self.map.close()
        except (BufferError, ValueError):
            pass  # tensors that borrow the mapping keep it alive
        self.file.close()


class Checkpoint:
    """Tensors of a model folder (or one file), borrowed from memory maps."""

    def __init__(self, path: str):
        self.shards: List[_Shard] = []
        self.entries: Dict[str, TensorEntry] = {}
        if os.path.isdir(path):
            index = os.path.join(path, "model.safetensors.index.json")
            single = os.path.join(path, "model.safetensors")
            if os.path.isfile(index):
                with open(index, "r", encoding="utf-8") as f:
                    try:
                        wm = json.load(f).get("weight_map")
                    except json.JSONDecodeError as e:
                        raise SafetensorsError(f"{index}: not valid JSON ({e})") from None
                if not isinstance(wm, dict) or not wm:
                    raise SafetensorsError(f"{index}: 'weight_map' missing or empty")
                files = sorted(set(wm.values()))
                for fn in files:
                    self._add_shard(os.path.join(path, fn))
                for name, fn in wm.items():
                    if name not in self.entries:
                        raise SafetensorsError(
                            f"{index}: tensor '{name}' is mapped to {fn} but is in no shard")
            elif os.path.isfile(single):
                self._add_shard(single)
            else:
                raise SafetensorsError(
                    f"{path}: neither model.safetensors.index.json nor model.safetensors found")
        elif os.path.isfile(path):
            self._add_shard(path)
        else:
            raise SafetensorsError(f"{path}: no such file or folder")

    def _add_shard(self, path: str):
        if not os.path.isfile(path):
            raise SafetensorsError(f"{path}: shard file not found")
        sh = _Shard(path)
        idx = len(self.shards)
        self.shards.append(sh)
        for name, meta in sh.header.items():
            if name == "__metadata__":
                continue
            if name in self.entries:
                other = self.shards[self.entries[name].shard].path
                raise SafetensorsError(f"tensor '{name}' appears in both {other} and {path}")
            if not isinstance(meta, dict):
                raise SafetensorsError(f"{path}: entry '{name}' is not an object")
            dt = meta.get("dtype")
            shape = meta.get("shape")
            offs = meta.get("data_offsets")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype {dt!r}")
            if (not isinstance(shape, list)
                    or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape)):
                raise SafetensorsError(f"{path}: tensor '{name}' has a bad shape {shape!r}")
            if (not isinstance(offs, list) or len(offs) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) for o in offs)):
                raise SafetensorsError(f"{path}: tensor '{name}' has bad data_offsets {offs!r}")
            begin, end = offs
            tdtype, isz = _DTYPES[dt]
            numel = 1
            for d in shape:
                numel *= d
            if begin < 0 or begin > end or end > sh.data_bytes:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' data_offsets [{begin}, {end}) leave the data "
                    f"section of {sh.data_bytes} bytes")
            if end - begin != numel * isz:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has {end - begin} bytes but shape {shape} of "
                    f"{dt} needs {numel * isz}")
            self.entries[name] = TensorEntry(name, tdtype, tuple(shape), sh.data_start + begin,
                                             sh.data_start + end, idx)

    def names(self) -> List[str]:
        return list(self.entries.keys())

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def __len__(self) -> int:
        return len(self.entries)

    def entry(self, name: str) -> TensorEntry:
        if name not in self.entries:
            raise SafetensorsError(
                f"checkpoint has no tensor '{name}' (it holds {len(self.entries)} tensors)")
        return self.entries[name]

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor that borrows the file mapping (read-only; copy before writing)."""
        e = self.entry(name)
        sh = self.shards[e.shard]
        n = e.end - e.begin
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = np.frombuffer(sh.map, dtype=np.uint8, count=n, offset=e.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # read-only buffer; nothing here writes to it
            t = torch.from_numpy(buf)
        return t.view(e.dtype).reshape(e.shape)

    def close(self):
        for sh in self.shards:
            sh.close()
        self.shards = []


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] = None) -> None:
    """Write tensors (name, CPU tensor) in the given order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    off = 0
    for name, t in tensors:
        if name in header:
            raise SafetensorsError(f"duplicate tensor name '{name}'")
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hbytes) % 8) % 8
    hbytes += b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hbytes)))
        f.write(hbytes)
        for b in blobs:
            f.write(b)
