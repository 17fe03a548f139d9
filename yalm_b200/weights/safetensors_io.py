"""Reading and writing the safetensors container: an 8-byte little-endian
header length, a JSON header ``{name: {dtype, shape, data_offsets}}`` and the
raw tensor bytes.  The reference's codec parses the same container
(codec.cpp:39-156: dtype string, offsets inside the file, numel*size == bytes);
the checks here raise exceptions that name the tensor instead of returning -1.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype string -> (bytes per element, numpy carrier dtype, torch dtype)
_DTYPES = {
    "F32": (4, np.uint32, torch.float32),
    "F16": (2, np.uint16, torch.float16),
    "BF16": (2, np.uint16, torch.bfloat16),
    "F64": (8, np.uint64, torch.float64),
    "I64": (8, np.int64, torch.int64),
    "I32": (4, np.int32, torch.int32),
    "I16": (2, np.int16, torch.int16),
    "I8": (1, np.int8, torch.int8),
    "U8": (1, np.uint8, torch.uint8),
    "BOOL": (1, np.uint8, torch.bool),
}
_TORCH_TO_NAME = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                  torch.float64: "F64", torch.int64: "I64", torch.int32: "I32",
                  torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}


def read_header(path: str) -> Tuple[Dict[str, dict], int, int]:
    """Returns (entries, data_start, file_size); validates every entry."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    data_start = 8 + n
    entries = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        dt = ent.get("dtype")
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
        shape = ent.get("shape")
        offs = ent.get("data_offsets")
        if (not isinstance(shape, list) or not isinstance(offs, list) or len(offs) != 2
                or any((not isinstance(s, int)) or s < 0 for s in shape)):
            raise SafetensorsError(f"{path}: tensor {name!r} has a malformed entry")
        b, e = offs
        numel = 1
        for s in shape:
            numel *= s
        if not (0 <= b <= e) or data_start + e > size:
            raise SafetensorsError(
                f"{path}: tensor {name!r} lies outside the file "
                f"(offsets {b}..{e}, data section {size - data_start} bytes): truncated file?")
        if numel * _DTYPES[dt][0] != e - b:
            raise SafetensorsError(
                f"{path}: tensor {name!r} with shape {shape} and dtype {dt} needs "
                f"{numel * _DTYPES[dt][0]} bytes but has {e - b}")
        entries[name] = ent
    return entries, data_start, size


def read_metadata(path: str) -> Dict[str, str]:
    """The string-to-string ``__metadata__`` of a file ({} if it has none)."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > os.path.getsize(path):
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    meta = header.get("__metadata__") or {}
    return {str(k): str(v) for k, v in meta.items()}


def read_file(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one file, in their stored dtype, as CPU tensors that
    share the file's memory map (copy-on-write: nothing is written back)."""
    entries, data_start, _ = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    if not entries:
        return out
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    for name, ent in entries.items():
        nbytes, carrier, tdtype = _DTYPES[ent["dtype"]]
        b, e = ent["data_offsets"]
        count = (e - b) // nbytes
        arr = np.frombuffer(mm, dtype=carrier, count=count, offset=data_start + b)
        t = torch.from_numpy(arr)
        if t.dtype != tdtype:
            t = t.view(tdtype)
        out[name] = t.reshape(ent["shape"])
    return out


def write_file(path: str, tensors: Dict[str, torch.Tensor],
               metadata: Dict[str, str] | None = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            carrier = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
            f.write(t.view(carrier).numpy().tobytes())


def list_files(model_dir: str) -> Iterable[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r") as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_dir, n) for n in names]
    files = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    return [os.path.join(model_dir, n) for n in files]
