"""Minimal reader / writer of the safetensors container (8-byte little-endian header length, JSON header
name -> {dtype, shape, data_offsets}, raw little-endian data).  numpy only; bfloat16 tensors travel as uint16 bit patterns."""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

_NP = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "I32": np.int32, "I64": np.int64, "U8": np.uint8}


def read(path) -> dict:
    """name -> (dtype string, numpy array); BF16 arrays hold the 16-bit patterns."""
    raw = np.fromfile(str(path), np.uint8)
    n = struct.unpack("<Q", raw[:8].tobytes())[0]
    header = json.loads(raw[8:8 + n].tobytes())
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = info["dtype"]
        if dt not in _NP:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
        out[name] = (dt, raw[8 + n + lo:8 + n + hi].view(_NP[dt]).reshape(info["shape"]))
    return out


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bfloat16 bit patterns of a float32 array."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16).reshape(np.shape(a))


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def write(path, tensors: dict) -> None:
    """tensors: name -> (dtype string, numpy array) as read() returns them."""
    header, off, blobs = {}, 0, []
    for name, (dt, arr) in tensors.items():
        b = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(np.shape(arr)), "data_offsets": [off, off + len(b)]}       # () stays (): a scalar tensor
        off += len(b)
        blobs.append(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(Path(path), "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def read_as_bf16(path, known: dict, family: str) -> dict:
    """name -> bfloat16 bit patterns of a checkpoint whose family stores bfloat16: float16 / float32 tensors are converted, tensors of
    other types are left out unless the description (known: name -> shape) needs them, which is an error."""
    out = {}
    for name, (dt, arr) in read(path).items():
        if dt == "BF16":
            out[name] = arr
        elif dt in ("F32", "F16"):
            out[name] = f32_to_bf16_bits(arr.astype(np.float32))
        elif name in known:
            raise ValueError(f"tensor {name}: dtype {dt} where a {family} checkpoint holds bfloat16")
    return out
