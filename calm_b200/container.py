"""Reader and writer of the tensor container the models come in: a u64 little-endian header length, that many bytes
of JSON (name -> dtype, shape, data_offsets; "__metadata__" is free-form), then the raw data.  calm's `.calm` files use
the same container with padded headers, so one parser serves both (the calm host's own parser is tensors.c of the
reference, which the drop-in binary keeps using)."""
from __future__ import annotations

import json
import struct
from typing import Dict, Tuple

import torch

DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32, "U8": torch.uint8, "F8_E5M2": torch.uint8}
NAMES = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32", torch.uint8: "U8"}


def read_tensors(path: str) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    """All tensors of the file (sharing one host buffer) and its metadata."""
    with open(path, "rb") as f:
        raw = bytearray(f.read())
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(bytes(raw[8:8 + n]).decode("utf-8"))
    meta = header.pop("__metadata__", {}) or {}
    body = memoryview(raw)[8 + n:]
    out = {}
    for name, info in header.items():
        if info["dtype"] not in DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
        lo, hi = info["data_offsets"]
        dt = DTYPES[info["dtype"]]
        count = 1
        for d in info["shape"]:
            count *= d
        if hi - lo != count * torch.empty((), dtype=dt).element_size():
            raise ValueError(f"{path}: tensor {name} has {hi - lo} bytes for shape {info['shape']}")
        t = torch.frombuffer(body[lo:hi], dtype=dt) if count else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"])
    return out, meta


def write_tensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header, chunks, at = {}, [], 0
    for name, t in tensors.items():
        t = t.contiguous()
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(b)]}
        chunks.append(b)
        at += len(b)
    if metadata:
        header["__metadata__"] = metadata
    h = json.dumps(header).encode("utf-8")
    h += b" " * (-(8 + len(h)) % 16)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in chunks:
            f.write(b)
