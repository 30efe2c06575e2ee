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

import ctypes
import json
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
            raise SafetensorsError(f"duplicate name {k!r}")
        seen[k] = v
    return seen


class SafetensorsFile:
    """One mapped .safetensors file.  The mapping, the header's parse and every check of
    it are the C++ host library's (`host/ilb_host.cpp`, `st_*`); tensors are views of the
    mapped bytes."""

    def __init__(self, path: str) -> None:
        from .. import host
        self.path = path
        self._lib = host.lib()
        h = ctypes.c_void_p()
        rc = self._lib.ilb_st_open(os.fsencode(path), ctypes.byref(h))
        if rc:
            msg = host.last_error()
            if rc == host.IO and not os.path.exists(path):
                raise FileNotFoundError(msg)
            raise SafetensorsError(msg)
        self._h = h
        self.data_start = self._lib.ilb_st_data_start(h)
        self._payload = self._lib.ilb_st_payload(h) or 0
        meta = self._lib.ilb_st_metadata(h).decode("utf-8", "replace")
        try:
            self.metadata = (json.loads(meta) if meta else None) or {}
        except json.JSONDecodeError:
            self.metadata = {}
        entries: Dict[str, TensorEntry] = {}
        name, dtype = ctypes.c_char_p(), ctypes.c_char_p()
        ndim = ctypes.c_int()
        shape = ctypes.POINTER(ctypes.c_longlong)()
        begin, end = ctypes.c_longlong(), ctypes.c_longlong()
        for i in range(self._lib.ilb_st_count(h)):
            self._lib.ilb_st_entry(h, i, ctypes.byref(name), ctypes.byref(dtype), ctypes.byref(ndim),
                                   ctypes.byref(shape), ctypes.byref(begin), ctypes.byref(end))
            n = name.value.decode("utf-8")
            d = dtype.value.decode("ascii")
            if d not in _DTYPES:
                self.close()
                raise SafetensorsError(f"{path}: {n}: unsupported dtype {d}")
            entries[n] = TensorEntry(n, d, tuple(int(shape[k]) for k in range(ndim.value)), begin.value, end.value)
        self.entries = entries

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only view of the mapped bytes (do not write through it).  The view keeps
        this object, and with it the mapping, alive."""
        e = self.entries[name]
        dtype, width = _DTYPES[e.dtype]
        nbytes = e.end - e.begin
        if nbytes == 0:
            return torch.empty(e.shape, dtype=dtype)
        buf = (ctypes.c_ubyte * nbytes).from_address(self._payload + e.begin)
        buf._keep = self                      # the mapping must outlive the view
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only by design
            flat = torch.frombuffer(buf, dtype=dtype, count=nbytes // width)
        return flat.view(e.shape)

    def close(self) -> None:
        """Drops this object's own hold on the mapping; it is unmapped when the last tensor
        view is gone too."""
        self.entries = dict(getattr(self, "entries", {}))

    def __del__(self) -> None:
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            self._lib.ilb_st_close(h)
            self._h = None


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
                    index = json.load(fh, object_pairs_hook=_no_duplicates)
                weight_map = dict(index["weight_map"])
            except (json.JSONDecodeError, RecursionError, KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{index_path}: malformed index: {e}") from None
            root = os.path.realpath(folder)
            for name, shard in weight_map.items():
                if (not isinstance(shard, str) or "\x00" in shard or os.path.isabs(shard)
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
            self._check_total_size(index_path, index)
        elif os.path.exists(single):
            self.files["model.safetensors"] = SafetensorsFile(single)
            for name in self.files["model.safetensors"].entries:
                self.where[name] = "model.safetensors"
        else:
            raise SafetensorsError(
                f"{folder}: neither model.safetensors nor model.safetensors.index.json exists")

    def _check_total_size(self, index_path: str, index: Mapping) -> None:
        """`metadata.total_size`, when the index declares one, must equal the shards'
        payload bytes, or the payload plus the shards' headers (some exporters count
        those): crates/model/package/src/storage/source.rs:160-181.  A whole number written
        as a float is taken (index.rs:60-81); absence is not an error."""
        meta = index.get("metadata") if isinstance(index, dict) else None
        if not isinstance(meta, dict) or "total_size" not in meta:
            return
        declared = meta["total_size"]
        if isinstance(declared, bool) or not isinstance(declared, (int, float)):
            raise SafetensorsError(f"{index_path}: invalid total_size {declared!r}")
        if isinstance(declared, float):
            if declared != declared or declared in (float("inf"), float("-inf")) or declared != int(declared):
                raise SafetensorsError(f"{index_path}: invalid total_size {declared!r}")
            declared = int(declared)
        if declared <= 0:
            raise SafetensorsError(f"{index_path}: total_size {declared} declares empty weights")
        payload = sum(e.end - e.begin for f in self.files.values() for e in f.entries.values())
        with_headers = payload + sum(int(f.data_start) for f in self.files.values())
        if declared not in (payload, with_headers):
            raise SafetensorsError(
                f"{index_path}: total_size {declared} disagrees with the shards "
                f"({payload} bytes of tensors, {with_headers} with their headers)")

    def names(self) -> List[str]:
        return list(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.files[self.where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()
