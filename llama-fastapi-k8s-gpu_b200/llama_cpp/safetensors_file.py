"""Reader and writer for safetensors files (memory-mapped), the weight container of the config.json model folders.

Layout: an 8-byte little-endian header length, that many bytes of JSON mapping tensor name ->
{"dtype", "shape", "data_offsets": [begin, end)} (offsets relative to the end of the header; the key
"__metadata__" holds free-form strings), then the raw little-endian tensor bytes. BF16 has no numpy dtype: such
tensors are exposed as uint16 bit patterns; `to_float32` widens them exactly.

The GGUF side of the loader is `gguf_file.py`; this is its counterpart for models that ship as a folder.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np

# safetensors dtype -> (numpy dtype that carries the bytes, bytes per element)
DTYPES = {"BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4), "F64": (np.float64, 8),
          "I32": (np.int32, 4), "I64": (np.int64, 8), "U8": (np.uint8, 1), "I8": (np.int8, 1)}


@dataclass
class STensor:
    name: str
    dtype: str                 # safetensors dtype string
    shape: Tuple[int, ...]     # row-major, outermost first
    data: np.ndarray           # view into the mapping (uint16 bit patterns for BF16)

    def to_float32(self) -> np.ndarray:
        if self.dtype == "BF16":
            return (self.data.astype(np.uint32) << 16).view(np.float32).reshape(self.shape)
        return self.data.astype(np.float32).reshape(self.shape)


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", head)
        size = self._f.seek(0, 2)
        if n <= 0 or 8 + n > size:
            raise ValueError(f"{path}: bad safetensors header length {n}")
        self._f.seek(8)
        header = json.loads(self._f.read(n).decode("utf-8"))
        self.metadata: Dict[str, str] = header.pop("__metadata__", None) or {}
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        base = 8 + n
        self.tensors: Dict[str, STensor] = {}
        for name, info in header.items():
            dt = info["dtype"]
            if dt not in DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
            np_dt, width = DTYPES[dt]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            count = int(np.prod(shape)) if shape else 1
            if e - b != count * width or base + e > size or b < 0:
                raise ValueError(f"{path}: tensor {name}: byte range does not match its shape")
            arr = np.frombuffer(self._mm, dtype=np_dt, count=count, offset=base + b).reshape(shape)
            self.tensors[name] = STensor(name, dt, shape, arr)

    def close(self):
        self.tensors = {}
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass            # numpy views still alive: the mapping goes with them
        self._f.close()


def float32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r.reshape(a.shape)


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], bf16: bool = True) -> None:
    """Write float arrays as BF16 (or F32 when bf16 is false) and integer arrays as I32."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.asarray(a)
        if np.issubdtype(a.dtype, np.integer):
            raw, dt = np.ascontiguousarray(a, dtype="<i4").tobytes(), "I32"
        elif bf16:
            raw, dt = float32_to_bf16_bits(a.astype(np.float32)).astype("<u2").tobytes(), "BF16"
        else:
            raw, dt = np.ascontiguousarray(a, dtype="<f4").tobytes(), "F32"
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
