"""Reader and writer of the safetensors container, by tensor name.

File layout (as the reference reads it, io/SafetensorsFile.cajeta:59-139): an unsigned
64-bit little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (the ``__metadata__`` entry is
skipped, io/SafetensorsFile.cajeta:337-347), then the raw little-endian payload.  The
reader checks every byte range against the payload and against shape x element size
(io/SafetensorsFile.cajeta:113-118,298-312).  A folder may hold one
``model.safetensors`` or an index ``model.safetensors.index.json`` whose ``weight_map``
names the shard of each tensor (io/Checkpoint.cajeta:52-65,432-492).

Tensors come back in the dtype the file stores (bfloat16 stays bfloat16, a 32-bit
tensor stays 32-bit); 64-bit integer tables are narrowed to int32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch


class WeightFileError(ValueError):
    """A weight file that cannot be read; names the file and the tensor."""


# name -> (numpy dtype used to view the bytes, element size, torch dtype handed out)
_DTYPES = {
    "F32": (np.dtype("<f4"), 4, torch.float32),
    "F16": (np.dtype("<f2"), 2, torch.float16),
    "BF16": (np.dtype("<u2"), 2, torch.bfloat16),
    "I32": (np.dtype("<i4"), 4, torch.int32),
    "I64": (np.dtype("<i8"), 8, torch.int32),
    "F64": (np.dtype("<f8"), 8, torch.float32),
}

_TORCH_TO_NAME = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                  torch.int32: "I32", torch.int64: "I64"}


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise WeightFileError(f"{path}: cannot open ({e.strerror})") from None
        if size < 8:
            raise WeightFileError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen <= 0 or 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise WeightFileError(f"{path}: header must be a JSON object")
        self._payload = 8 + hlen
        payload_size = size - self._payload
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = info["dtype"]
                shape = tuple(int(d) for d in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise WeightFileError(f"{path}: tensor '{name}' has a malformed header entry") from None
            if dtype not in _DTYPES:
                raise WeightFileError(
                    f"{path}: tensor '{name}' has dtype {dtype}; supported: {', '.join(sorted(_DTYPES))}")
            if begin < 0 or end < begin or end > payload_size:
                raise WeightFileError(
                    f"{path}: tensor '{name}' byte range [{begin}, {end}) lies outside the payload ({payload_size} bytes)")
            count = 1
            for d in shape:
                count *= d
            want = count * _DTYPES[dtype][1]
            if end - begin != want:
                raise WeightFileError(
                    f"{path}: tensor '{name}' of shape {list(shape)} {dtype} needs {want} bytes, its range holds {end - begin}")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape_of(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype_of(self, name: str) -> str:
        return self.entries[name][0]

    def load(self, name: str) -> torch.Tensor:
        """A host tensor that owns its memory (copied out of the map)."""
        if name not in self.entries:
            raise WeightFileError(f"{self.path}: no tensor named '{name}'")
        dtype, shape, begin, end = self.entries[name]
        np_dtype, _, torch_dtype = _DTYPES[dtype]
        raw = np.frombuffer(self._map, dtype=np_dtype, count=(end - begin) // np_dtype.itemsize,
                            offset=self._payload + begin)
        if dtype == "BF16":
            t = torch.from_numpy(raw.astype(np.int16, copy=True)).view(torch.bfloat16)
        elif dtype == "I64":
            if raw.size and (raw.max() > np.iinfo(np.int32).max or raw.min() < np.iinfo(np.int32).min):
                raise WeightFileError(f"{self.path}: integer tensor '{name}' does not fit 32 bits")
            t = torch.from_numpy(raw.astype(np.int32))
        elif dtype == "F64":
            t = torch.from_numpy(raw.astype(np.float32))
        else:
            t = torch.from_numpy(raw.copy())
        return t.reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        finally:
            self._fh.close()


class Checkpoint:
    """All tensors of a model folder under one name -> tensor surface."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.isfile(single):
            f = self._open(single)
            for n in f.names():
                self._where[n] = single
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as fh:
                try:
                    weight_map = json.load(fh)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise WeightFileError(f"{index}: no 'weight_map' object") from None
            for n, shard in weight_map.items():
                path = os.path.join(model_dir, shard)
                f = self._open(path)
                if n not in f.entries:
                    raise WeightFileError(f"{index}: maps '{n}' to {shard}, which does not hold it")
                self._where[n] = path
        else:
            raise WeightFileError(
                f"{model_dir}: holds neither model.safetensors nor model.safetensors.index.json")

    def _open(self, path: str) -> SafetensorsFile:
        if path not in self._files:
            self._files[path] = SafetensorsFile(path)
        return self._files[path]

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape_of(self, name: str) -> Tuple[int, ...]:
        return self._files[self._where[name]].shape_of(name)

    def dtype_of(self, name: str) -> str:
        return self._files[self._where[name]].dtype_of(name)

    def load(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise WeightFileError(f"{self.model_dir}: no tensor named '{name}'")
        return self._files[self._where[name]].load(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()
        self._files.clear()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor] | Iterable[Tuple[str, torch.Tensor]],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write host tensors to one ``.safetensors`` file (names in the given order)."""
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs: List[bytes] = []
    for name, t in items:
        if t.dtype not in _TORCH_TO_NAME:
            raise WeightFileError(f"{path}: tensor '{name}' has unsupported dtype {t.dtype}")
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            data = t.view(torch.int16).numpy().tobytes()
        else:
            data = t.numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(data)]}
        offset += len(data)
        blobs.append(data)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * ((8 - len(head) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
