"""Reader and writer of the safetensors container.

The file is an 8-byte little-endian header length, a JSON header that maps a
tensor name to ``{dtype, shape, data_offsets}``, then the raw bytes.  The
checks at open time are those the reference makes (loader/safetensors/
safetensors.go:78-143,167-199): header length within the file, offsets ordered
and inside the data section, byte count equal to numel x sizeof(dtype).  A
folder holds either ``model.safetensors`` or ``model.safetensors.index.json``
with a ``weight_map`` from tensor name to shard file
(loader/weights/weights.go:28-45).

Tensors come back in the dtype they are stored in (bfloat16 stays bfloat16, a
32-bit tensor stays 32-bit); 64-bit integer tables come back as int32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Mapping, Tuple

import torch


class SafetensorsError(ValueError):
    """The container is malformed."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int32: "I32", torch.int64: "I64"}


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One mapped file.  `entries[name] = (dtype name, shape, begin, end)`."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise FileNotFoundError(f"{path} does not exist") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors header")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._base = 8 + hlen
        data_len = size - self._base
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dt = meta["dtype"]
                shape = tuple(int(s) for s in meta["shape"])
                begin, end = (int(o) for o in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: entry {name!r} is malformed: {meta!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r} "
                                       f"(supported: {sorted(_DTYPES)})")
            if any(s < 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has a negative extent {shape}")
            if not (0 <= begin <= end <= data_len):
                raise SafetensorsError(f"{path}: tensor {name!r} offsets [{begin}, {end}) lie "
                                       f"outside the data section of {data_len} bytes")
            want = _numel(shape) * _DTYPES[dt][1]
            if end - begin != want:
                raise SafetensorsError(f"{path}: tensor {name!r} of shape {list(shape)} and dtype "
                                       f"{dt} needs {want} bytes but has {end - begin}")
            self.entries[name] = (dt, shape, begin, end)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        dt = self.entries[name][0]
        return torch.int32 if dt == "I64" else _DTYPES[dt][0]

    def tensor(self, name: str, copy: bool = True) -> torch.Tensor:
        """The tensor in its stored dtype (int64 narrowed to int32): a host copy,
        or with copy=False a read-only view of the mapped file that is valid while
        the file is open -- a loader that sends it straight to the device then
        copies each tensor once, not twice."""
        dt, shape, begin, end = self.entries[name]
        tdt, size = _DTYPES[dt]
        if end == begin:
            out = torch.empty(shape, dtype=tdt)
        elif not copy and (self._base + begin) % size == 0:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", UserWarning)     # the map is read-only; nobody writes to the view
                out = torch.frombuffer(self._mm, dtype=tdt, count=_numel(shape),
                                       offset=self._base + begin).reshape(shape)
        else:
            buf = memoryview(self._mm)[self._base + begin: self._base + end]
            out = torch.frombuffer(bytearray(buf), dtype=tdt).reshape(shape)
        if tdt == torch.int64:
            if out.numel() and (out.max() > 2**31 - 1 or out.min() < -2**31):
                raise SafetensorsError(f"{self.path}: integer table {name!r} does not fit int32")
            out = out.to(torch.int32)
        return out

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass              # a view handed out with copy=False is still alive; the map goes with it
        finally:
            self._f.close()


class TensorSource:
    """All tensors of a model folder by name, across shards."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.exists(index):
            with open(index) as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no usable 'weight_map'") from None
            for name, shard in weight_map.items():
                if shard not in self._files:
                    path = os.path.join(folder, shard)
                    if not os.path.exists(path):
                        raise SafetensorsError(f"{index} names shard {shard!r}, which is missing")
                    self._files[shard] = SafetensorsFile(path)
                if name not in self._files[shard].entries:
                    raise SafetensorsError(f"{index} places {name!r} in {shard!r}, which lacks it")
                self._where[name] = shard
        elif os.path.exists(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].entries:
                self._where[name] = "model.safetensors"
        else:
            raise FileNotFoundError(f"{folder} has neither model.safetensors nor "
                                    f"model.safetensors.index.json")

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._files[self._where[name]].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._files[self._where[name]].dtype(name)

    def tensor(self, name: str, copy: bool = True) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name, copy=copy)

    def close(self) -> None:
        for f in self._files.values():
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] = None) -> None:
    """Write tensors (host or device) to one file, names in sorted order, data
    8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store {name!r} of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * ((8 - len(head) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
