"""The safetensors container: read by tensor name, and write.

Format (`safetensors/safetensors.go:1-11`): an 8-byte little-endian header
length, a JSON header `name -> {dtype, shape, data_offsets}` (plus an optional
`__metadata__` map of strings), then the raw bytes.  A model folder holds
`model.safetensors`, or `model.safetensors.index.json` whose `weight_map` names
the shard files; the shards' own headers are the authority on what they hold
(`safetensors/safetensors.go:74-107`).  The writer emits sorted names into a
temporary file and renames it into place (`safetensors/write.go:26-77`).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch


class SafetensorsError(ValueError):
    """A safetensors file or model folder that cannot be read."""


_TORCH_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NP_VIEW = {  # how the raw bytes are viewed before torch reinterprets them
    "F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16,
    "I64": np.int64, "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.uint8,
    "U32": np.uint32, "U16": np.uint16,
}
_ITEMSIZE = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1,
             "U8": 1, "BOOL": 1, "U32": 4, "U16": 2}
_NAMES = {v: k for k, v in _TORCH_DTYPES.items()}


@dataclass(frozen=True)
class TensorInfo:
    dtype: str                # the container's dtype string, e.g. "BF16"
    shape: tuple[int, ...]
    begin: int                # byte range inside the data section
    end: int


class SafetensorsFile:
    """One .safetensors file: header parsed at open, tensors read on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"open {path}: {e.strerror or e}") from e
        size = os.fstat(self._f.fileno()).st_size
        head = self._f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: file too short for a header length ({size} bytes)")
        (hlen,) = struct.unpack("<Q", head)
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata: dict[str, str] = {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self._infos: dict[str, TensorInfo] = {}
        for name, info in header.items():
            if name == "__metadata__":
                if isinstance(info, dict):
                    self.metadata = {str(k): str(v) for k, v in info.items()}
                continue
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{path}: malformed header entry for tensor {name!r}") from e
            if dtype not in _ITEMSIZE:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
            n = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor {name!r} has a negative dimension")
                n *= s
            if begin < 0 or end < begin or end > data_len:
                raise SafetensorsError(f"{path}: tensor {name!r} data_offsets [{begin}, {end}) lie outside "
                                       f"the data section ({data_len} bytes)")
            if end - begin != n * _ITEMSIZE[dtype]:
                raise SafetensorsError(f"{path}: tensor {name!r} has {end - begin} bytes, its shape "
                                       f"{list(shape)} and dtype {dtype} need {n * _ITEMSIZE[dtype]}")
            self._infos[name] = TensorInfo(dtype, shape, begin, end)
        self._mm = None

    def names(self) -> list[str]:
        return sorted(self._infos)

    def info(self, name: str) -> TensorInfo:
        try:
            return self._infos[name]
        except KeyError:
            raise SafetensorsError(f"tensor {name!r} not found in {self.path}") from None

    def __contains__(self, name: str) -> bool:
        return name in self._infos

    def read(self, name: str) -> torch.Tensor:
        """The tensor on the host, in the dtype it is stored in (U32/U16 come back as int32)."""
        info = self.info(name)
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        lo = self._data_start + info.begin
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=info.end - info.begin, offset=lo)
        arr = raw.view(_NP_VIEW[info.dtype]).reshape(info.shape).copy()
        if info.dtype == "BF16":
            return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
        if info.dtype == "BOOL":
            return torch.from_numpy(arr).to(torch.bool)
        if info.dtype in ("U32", "U16"):
            return torch.from_numpy(arr.astype(np.int64)).to(torch.int32)
        return torch.from_numpy(arr)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


class ModelFiles:
    """All tensors of a model folder, whichever shard holds them."""

    def __init__(self, files: list[SafetensorsFile]):
        self.files = files
        self._where: dict[str, SafetensorsFile] = {}
        for f in files:
            for n in f.names():
                if n in self._where:   # safetensors/safetensors.go:167-170
                    raise SafetensorsError(f"duplicate tensor {n!r} across shards "
                                           f"({self._where[n].path} and {f.path})")
                self._where[n] = f

    def names(self) -> list[str]:
        return sorted(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str) -> TensorInfo:
        if name not in self._where:
            raise SafetensorsError(f"tensor {name!r} not found")
        return self._where[name].info(name)

    def read(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise SafetensorsError(f"tensor {name!r} not found")
        return self._where[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def open_model(model_dir: str) -> ModelFiles:
    """model.safetensors, or the shards that model.safetensors.index.json names."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(single):
        return ModelFiles([SafetensorsFile(single)])
    if os.path.exists(index):
        try:
            with open(index, "r", encoding="utf-8") as f:
                idx = json.load(f)
        except (OSError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{index}: cannot read the shard index: {e}") from e
        wm = idx.get("weight_map") if isinstance(idx, dict) else None
        if not isinstance(wm, dict) or not wm:        # safetensors/safetensors.go:96-98
            raise SafetensorsError(f"{index}: weight_map is missing or empty")
        shards = sorted(set(str(v) for v in wm.values()))
        return ModelFiles([SafetensorsFile(os.path.join(model_dir, s)) for s in shards])
    raise SafetensorsError(f"{model_dir}: no model.safetensors and no model.safetensors.index.json")


def write_safetensors(path: str, tensors: dict[str, torch.Tensor],
                      metadata: dict[str, str] | None = None) -> None:
    """Write host tensors under sorted names; the file appears whole or not at all."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = f"{path}.tmp.{os.getpid()}"
    try:
        with open(tmp, "wb") as f:
            f.write(struct.pack("<Q", len(blob)))
            f.write(blob)
            for name in order:
                t = tensors[name].detach().cpu().contiguous()
                if t.dtype == torch.bfloat16:
                    f.write(t.view(torch.int16).numpy().tobytes())
                elif t.dtype == torch.bool:
                    f.write(t.to(torch.uint8).numpy().tobytes())
                else:
                    f.write(t.numpy().tobytes())
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)
