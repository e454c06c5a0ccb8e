"""safetensors read / write without external packages: u64 header length, JSON header
(``name -> {dtype, shape, data_offsets}`` + ``__metadata__``), raw little-endian payload.
(Reference: tensorplay/serialization/archive.py:1534-1800.)"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Mapping, Optional

import torch

_DT = {
    torch.bool: "BOOL", torch.uint8: "U8", torch.int8: "I8", torch.int16: "I16", torch.uint16: "U16",
    torch.int32: "I32", torch.uint32: "U32", torch.int64: "I64", torch.uint64: "U64",
    torch.float16: "F16", torch.bfloat16: "BF16", torch.float32: "F32", torch.float64: "F64",
    torch.float8_e5m2: "F8_E5M2", torch.float8_e4m3fn: "F8_E4M3",
}
_RDT = {v: k for k, v in _DT.items()}


def save_safetensors(tensors: Mapping[str, torch.Tensor], path, metadata: Optional[Mapping[str, str]] = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        if not isinstance(t, torch.Tensor):
            raise TypeError("safetensors stores a flat mapping of tensors")
        h = t.detach().to("cpu").contiguous()
        raw = h.reshape(-1).view(torch.uint8) if h.numel() else h.new_empty(0, dtype=torch.uint8)
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + raw.numel()]}
        off += raw.numel()
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b.numpy().tobytes() if b.numel() else b"")


def read_safetensors_header(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > (1 << 30):
            raise ValueError("not a safetensors file")
        header = json.loads(f.read(n).decode("utf-8"))
    return header, 8 + n


def load_safetensors(path, map_location=None, mmap: bool = False) -> Dict[str, torch.Tensor]:
    header, start = read_safetensors_header(path)
    size = os.path.getsize(path)
    whole = torch.from_file(os.fspath(path), shared=False, size=size, dtype=torch.uint8)
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        raw = whole[start + a: start + b]
        if not mmap:
            raw = raw.clone()
        t = raw.view(_RDT[rec["dtype"]]).reshape(rec["shape"]) if b > a else torch.empty(rec["shape"], dtype=_RDT[rec["dtype"]])
        out[name] = t.to(map_location) if map_location is not None else t
    return out
