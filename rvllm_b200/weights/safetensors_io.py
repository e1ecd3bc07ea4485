"""Reading and writing safetensors files without any library for the format.

Format and checks as the reference's parser (v3/crates/rvllm-loader/src/safetensors.rs:34-141):
8 bytes little-endian header length, a JSON header {name: {dtype, shape, data_offsets}},
`__metadata__` skipped, offsets relative to the end of the header, and end - start must equal
dtype bytes x product(shape).  Shards are found through model.safetensors.index.json
(safetensors.rs:156-208).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..errors import LoaderError

# name -> (bytes per element, numpy storage dtype, torch dtype)
_DTYPES = {
    "F32": (4, np.float32, torch.float32),
    "F16": (2, np.float16, torch.float16),
    "BF16": (2, np.uint16, torch.bfloat16),
    "I32": (4, np.int32, torch.int32),
    "I64": (8, np.int64, torch.int64),
}
_TORCH_TO_NAME = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                  torch.int32: "I32", torch.int64: "I64"}
_MAX_HEADER = 100 * 1024 * 1024


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "start", "end", "file")

    def __init__(self, name, dtype, shape, start, end, file):
        self.name, self.dtype, self.shape, self.start, self.end, self.file = name, dtype, shape, start, end, file


class SafetensorsFile:
    """One memory-mapped file; tensors are read by name."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise LoaderError(f"cannot open weight file: {e}", path=path) from None
        if size < 8:
            raise LoaderError(f"file of {size} bytes is too short for a safetensors header", path=path)
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise LoaderError(f"header length {hlen} exceeds the file size {size}", path=path)
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise LoaderError(f"header is not valid JSON: {e}", path=path) from None
        if not isinstance(header, dict):
            raise LoaderError("header must be a JSON object", path=path)
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        self.entries: Dict[str, TensorEntry] = {}
        for name, e in header.items():
            try:
                dtype, shape, (s, t) = e["dtype"], [int(d) for d in e["shape"]], e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise LoaderError(f"malformed header entry for tensor {name!r}", path=path) from None
            if dtype not in _DTYPES:
                raise LoaderError(f"tensor {name!r} has unsupported dtype {dtype} "
                                  f"(known: {', '.join(_DTYPES)})", path=path)
            n = 1
            for d in shape:
                n *= d
            if t - s != n * _DTYPES[dtype][0] or s < 0:
                raise LoaderError(f"tensor {name!r}: offset range {s}..{t} != dtype*shape "
                                  f"{n * _DTYPES[dtype][0]} bytes", path=path)
            if t > data_len:
                raise LoaderError(f"tensor {name!r}: offsets {s}..{t} lie beyond the file's data "
                                  f"({data_len} bytes)", path=path)
            self.entries[name] = TensorEntry(name, dtype, tuple(shape), s, t, self)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (copy it before the file is closed)."""
        e = self.entries[name]
        _, np_dtype, torch_dtype = _DTYPES[e.dtype]
        count = (e.end - e.start) // np.dtype(np_dtype).itemsize
        arr = np.frombuffer(self._mm, dtype=np_dtype, count=count, offset=self.data_start + e.start)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # read-only buffer: nothing writes through the view
            t = torch.from_numpy(arr)
        if e.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor],
                      metadata: Optional[Dict[str, str]] = None) -> None:
    """Write tensors in name order; every data block starts on an 8-byte boundary."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise LoaderError(f"tensor {name!r}: dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())


def open_model_files(model_dir: str) -> Dict[str, TensorEntry]:
    """name -> entry over all shards of a model folder."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(index):
        try:
            with open(index) as f:
                weight_map = json.load(f)["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            raise LoaderError(f"shard index is malformed: {e}", path=index) from None
        files = {name: SafetensorsFile(os.path.join(model_dir, name)) for name in sorted(set(weight_map.values()))}
        out: Dict[str, TensorEntry] = {}
        missing = []
        for tname, fname in weight_map.items():
            if tname not in files[fname].entries:
                missing.append(f"{tname} (index says {fname})")
            else:
                out[tname] = files[fname].entries[tname]
        if missing:
            raise LoaderError("the shard index names tensors that their shard does not hold",
                              path=index, missing=missing)
        return out
    if os.path.exists(single):
        return dict(SafetensorsFile(single).entries)
    raise LoaderError(f"no weights found: neither {single} nor {index} exists", path=model_dir)
