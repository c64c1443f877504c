"""Minimal safetensors reader / writer (numpy only).

File layout: 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets relative
to the end of the header), then the raw little-endian data.  bfloat16 has no numpy dtype: such tensors are returned
as uint16 arrays holding the bit patterns (`is_bf16` tells), which is what the drivers' load_tensor entry points take.
"""
import json
import struct

import numpy as np

_DTYPES = {"BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4), "I32": (np.int32, 4),
           "I64": (np.int64, 8), "U8": (np.uint8, 1), "I8": (np.int8, 1)}


class Bf16Array(np.ndarray):
    """uint16 view whose values are bfloat16 bit patterns."""


def is_bf16(a):
    return isinstance(a, Bf16Array)


def bf16_to_f32(a):
    return (np.asarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(a):
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r.view(Bf16Array)


def load_file(path):
    """-> {name: numpy array}; bfloat16 tensors come back as Bf16Array (uint16 bit patterns)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _DTYPES:
            raise ValueError("unsupported safetensors dtype %s for %s" % (info["dtype"], name))
        dt, size = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        count = 1
        for d in info["shape"]:
            count *= d
        if hi - lo != count * size or hi > len(data):
            raise ValueError("bad data_offsets for %s" % name)
        a = np.frombuffer(data, dtype=dt, count=count, offset=lo).reshape(info["shape"])
        out[name] = a.view(Bf16Array) if info["dtype"] == "BF16" else a
    return out


def save_file(tensors, path):
    """tensors: name -> numpy array (Bf16Array is written as BF16, float32 as F32, int32 as I32)."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        if is_bf16(a):
            code = "BF16"
        else:
            code = {np.dtype(np.float32): "F32", np.dtype(np.int32): "I32", np.dtype(np.float16): "F16"}[np.asarray(a).dtype]
        raw = np.ascontiguousarray(a).tobytes()
        header[name] = {"dtype": code, "shape": list(np.asarray(a).shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode("utf-8")
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
