"""Reading and writing the safetensors file format.

A file is: 8 bytes little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``, then
the raw little-endian tensor bytes.  Reading maps the file into memory and returns
views, so a tensor is only paged in when it is used.  The reference reads
checkpoints through the ``safetensors`` package (cpmcu/llm.py:139-175).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One file, memory-mapped.  ``entries`` maps a name to (dtype, shape, begin, end)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes); truncated?")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(x) for x in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: bad header entry for '{name}': {info!r}") from None
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * torch.empty((), dtype=dtype).element_size():
                raise SafetensorsError(f"{path}: '{name}' has {end - begin} bytes, its shape {shape} needs "
                                       f"{count * torch.empty((), dtype=dtype).element_size()}")
            if self._base + end > size:
                raise SafetensorsError(f"{path}: '{name}' ends at byte {self._base + end}, the file has {size}; truncated?")
            self.entries[name] = (dtype, shape, begin, end)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._base + begin:self._base + end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the map is read-only; the view is never written
            flat = torch.frombuffer(buf, dtype=dtype)
        return flat.view(shape)

    def close(self) -> None:
        # tensors handed out keep the map alive through their buffer; only the file handle is closed
        self._f.close()


def model_files(model_dir: str) -> List[str]:
    """The safetensors files of a model folder (sharded folders list theirs in an index)."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        return [os.path.join(model_dir, n) for n in sorted(set(weight_map.values()))]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    found = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not found:
        raise SafetensorsError(f"no model.safetensors (or index, or any *.safetensors) in {model_dir}")
    return [os.path.join(model_dir, n) for n in found]


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"'{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
