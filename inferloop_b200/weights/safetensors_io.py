"""Reader and writer for the safetensors container, written against the format itself.

Layout: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`, then
the payload.  The checks are the reference's (crates/model/package/src/storage/
safetensors.rs:220-314): header at most 16 MiB, no duplicate names, every tensor's byte
length equal to shape x dtype size, tensors tiling the payload with no overlap, gap or
trailing bytes.  The file is mapped read-only and tensors are views of the mapping
(safetensors.rs:161-173); nothing is copied until a tensor is moved to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

MAX_HEADER_BYTES = 16 << 20   # safetensors.rs:14
MAX_INDEX_BYTES = 16 << 20    # storage/source.rs:128-183

_DTYPES: Dict[str, Tuple[torch.dtype, int]] = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise SafetensorsError(f"duplicate tensor name {k!r} in header")
        seen[k] = v
    return seen


class SafetensorsFile:
    """One mapped .safetensors file."""

    def __init__(self, path: str) -> None:
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file is shorter than its 8-byte length field")
        self._fh = open(path, "rb")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: header of {n} bytes exceeds {MAX_HEADER_BYTES}")
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} runs past the end of the file")
        try:
            header = json.loads(self._fh.read(n).decode("utf-8"),
                                object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self.data_start = 8 + n
        payload = size - self.data_start
        entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: {name}: unsupported dtype {dtype}")
            if any(s < 0 for s in shape) or begin < 0 or end < begin or end > payload:
                raise SafetensorsError(f"{path}: {name}: offsets [{begin}, {end}) outside payload")
            count = 1
            for s in shape:
                count *= s
            if count * _DTYPES[dtype][1] != end - begin:
                raise SafetensorsError(
                    f"{path}: {name}: shape {list(shape)} of {dtype} needs "
                    f"{count * _DTYPES[dtype][1]} bytes, entry spans {end - begin}")
            entries[name] = TensorEntry(name, dtype, shape, begin, end)
        cursor = 0
        for e in sorted(entries.values(), key=lambda e: (e.begin, e.end)):
            if e.begin < cursor:
                raise SafetensorsError(f"{path}: {e.name} overlaps the tensor before it")
            if e.begin > cursor:
                raise SafetensorsError(f"{path}: gap of {e.begin - cursor} bytes before {e.name}")
            cursor = e.end
        if cursor != payload:
            raise SafetensorsError(f"{path}: {payload - cursor} trailing bytes after the last tensor")
        self.entries = entries
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only view of the mapped bytes (do not write through it)."""
        e = self.entries[name]
        dtype, width = _DTYPES[e.dtype]
        count = (e.end - e.begin) // width
        if count == 0:
            return torch.empty(e.shape, dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only by design
            flat = torch.frombuffer(self._map, dtype=dtype, count=count,
                                    offset=self.data_start + e.begin)
        return flat.view(e.shape)

    def close(self) -> None:
        # Views handed out keep the mapping alive through the buffer protocol; closing
        # with live views raises BufferError, which is left to the garbage collector.
        try:
            if self._map is not None:
                self._map.close()
        except BufferError:
            pass
        self._fh.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor] | Iterable[Tuple[str, torch.Tensor]],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors (CPU, contiguous) in the given order."""
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            c = t.detach().cpu().contiguous()
            fh.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")


class TensorSource:
    """All tensors of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names (crates/model/package/src/storage/source.rs:
    128-183, index.rs:17-40).  Shard names that leave the folder are refused."""

    def __init__(self, folder: str) -> None:
        self.folder = folder
        index_path = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        if os.path.exists(index_path):
            if os.path.getsize(index_path) > MAX_INDEX_BYTES:
                raise SafetensorsError(f"{index_path}: larger than {MAX_INDEX_BYTES} bytes")
            try:
                with open(index_path, "r", encoding="utf-8") as fh:
                    index = json.load(fh)
                weight_map = dict(index["weight_map"])
            except (json.JSONDecodeError, KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{index_path}: malformed index: {e}") from None
            root = os.path.realpath(folder)
            for name, shard in weight_map.items():
                if (not isinstance(shard, str) or os.path.isabs(shard)
                        or os.path.realpath(os.path.join(folder, shard)) != os.path.join(root, shard)
                        or os.sep in shard or shard in ("", ".", "..")):
                    raise SafetensorsError(f"{index_path}: shard path {shard!r} leaves the folder")
                if shard not in self.files:
                    p = os.path.join(folder, shard)
                    if not os.path.exists(p):
                        raise SafetensorsError(f"{index_path}: shard {shard} does not exist")
                    self.files[shard] = SafetensorsFile(p)
                if name not in self.files[shard].entries:
                    raise SafetensorsError(f"{index_path}: {name} is not in {shard}")
                self.where[name] = shard
            for shard, f in self.files.items():
                for name in f.entries:
                    if self.where.get(name) != shard:
                        raise SafetensorsError(
                            f"{shard}: holds {name}, which the index does not map to it")
        elif os.path.exists(single):
            self.files["model.safetensors"] = SafetensorsFile(single)
            for name in self.files["model.safetensors"].entries:
                self.where[name] = "model.safetensors"
        else:
            raise SafetensorsError(
                f"{folder}: neither model.safetensors nor model.safetensors.index.json exists")

    def names(self) -> List[str]:
        return list(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.files[self.where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()
