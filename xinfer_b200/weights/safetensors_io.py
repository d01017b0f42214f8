"""Reader and writer for the safetensors container: 8 bytes little-endian header length, a JSON
header ``{name: {dtype, shape, data_offsets}}``, then the raw little-endian tensor bytes.

The reference memory-maps the same files through its tensor library
(src/models/layers/mod.rs:129-135) and finds them as ``model.safetensors`` or through
``model.safetensors.index.json`` (src/utils/downloader.rs:170-177, src/utils/mod.rs:106-125).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: str


class SafetensorsFile:
    """One memory-mapped file; ``tensor(name)`` returns a CPU tensor viewing the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype, isz = _DTYPES[info["dtype"]]
            except KeyError:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {info.get('dtype')!r}") from None
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if end - begin != n * isz or begin < 0 or self._data_start + end > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has offsets [{begin}, {end}) that do not match shape {shape} / file size")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, path)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e.end - e.begin,
                            offset=self._data_start + e.begin)
        # the mapping is read-only; torch only reads from it before the copy to the device
        with _quiet_readonly():
            t = torch.from_numpy(buf)
        return t.view(e.dtype).reshape(e.shape)

    def close(self) -> None:
        # views handed out earlier keep the mapping alive through numpy's reference
        self._fh.close()


class _quiet_readonly:
    def __enter__(self):
        import warnings
        self._cm = warnings.catch_warnings()
        self._cm.__enter__()
        warnings.simplefilter("ignore")

    def __exit__(self, *a):
        self._cm.__exit__(*a)


def find_weight_files(model_dir: str) -> List[str]:
    """``model.safetensors``, else the files named by ``model.safetensors.index.json``."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        files = sorted({os.path.join(model_dir, v) for v in weight_map.values()})
        missing = [p for p in files if not os.path.isfile(p)]
        if missing:
            raise SafetensorsError("index names files that do not exist: " + ", ".join(missing))
        if files:
            return files
    raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in '{model_dir}'")


def write_safetensors(path: str, tensors: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      produce, metadata: Optional[Mapping[str, str]] = None) -> None:
    """Stream a file: ``tensors`` lists (name, shape, dtype) in file order and ``produce(name)``
    returns each tensor when its turn comes, so only one tensor is in memory at a time."""
    specs = list(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, shape, dtype in specs:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(s) for s in shape],
                        "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype in specs:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise SafetensorsError(f"producer returned {tuple(t.shape)}/{t.dtype} for '{name}', expected {tuple(shape)}/{dtype}")
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
