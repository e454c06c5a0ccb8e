"""``.mega`` container: header building in Python, parsing and payload IO in C++ (``libtpb200rt``).

On-disk format and TensorPlay metadata keys as written by the reference
(tensorplay/serialization/mega.py:436-553 header and metadata, :323-422 layout tree escapes).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
import sys
import zlib
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from .. import _native

MAGIC = 0x4147454D
DEFAULT_ALIGNMENT = 4096
CHECKSUM_TYPES = {"none": 0, "crc32": 1, "sha256": 2}

_DT2MEGA = {
    torch.bool: "BOOL", torch.uint8: "U8", torch.int8: "I8", torch.int16: "I16", torch.uint16: "U16",
    torch.int32: "I32", torch.uint32: "U32", torch.int64: "I64", torch.uint64: "U64",
    torch.float16: "F16", torch.bfloat16: "BF16", torch.float32: "F32", torch.float64: "F64",
    torch.float8_e5m2: "F8_E5M2", torch.float8_e4m3fn: "F8_E4M3",
}
if hasattr(torch, "float8_e8m0fnu"):
    _DT2MEGA[torch.float8_e8m0fnu] = "F8_E8M0"
_MEGA2DT = {v: k for k, v in _DT2MEGA.items()}


def _rt():
    lib = _native.runtime()
    if not getattr(lib, "_mega_sigs", False):
        lib.tpb_mega_write.argtypes = [C.c_char_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int,
                                       C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_int]
        lib.tpb_mega_write.restype = C.c_int
        lib.tpb_mega_parse.argtypes = [C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_longlong)]
        lib.tpb_mega_parse.restype = C.c_int
        lib.tpb_file_read.argtypes = [C.c_char_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_int]
        lib.tpb_file_read.restype = C.c_int
        lib.tpb_crc32.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32]
        lib.tpb_crc32.restype = C.c_uint32
        lib.tpb_free.argtypes = [C.c_void_p]
        lib._mega_sigs = True
    return lib


# ------------------------------------------------------------------ tree <-> flat
_ESCAPES = ("__tensor__", "__tuple__", "__dict__")


def flatten_tree(obj) -> Tuple[Dict[str, torch.Tensor], str, Any]:
    """Returns (name -> tensor, container kind, layout or None).

    Container kinds follow the reference's writer (tensorplay/serialization/mega.py:323-398) so
    that either side reads the other's files: a bare tensor is ``"tensor"`` under the name "0";
    a flat str -> tensor mapping is ``"dict"``, a flat list / tuple of tensors ``"list"`` /
    ``"tuple"`` with names "0", "1", ... and no layout; everything else is ``"tree"`` with a JSON
    layout. A tensor object that occurs more than once is stored once and referenced by name from
    every place, so tied tensors come back tied.
    """
    if isinstance(obj, torch.Tensor):
        return {"0": obj}, "tensor", None
    flat: Dict[str, torch.Tensor] = {}
    by_id: Dict[int, str] = {}
    open_nodes = set()

    def name_for(t, path):
        known = by_id.get(id(t))
        if known is None:
            base = ".".join(str(p) for p in path) or "0"
            known, n = base, 0
            while known in flat:
                n += 1
                known = f"{base}#{n}"
            flat[known] = t
            by_id[id(t)] = known
        return {"__tensor__": known}

    def enc(x, path):
        if isinstance(x, torch.Tensor):
            return name_for(x, path)
        if x is None or isinstance(x, (bool, int, float, str)):
            return x
        if isinstance(x, (torch.dtype, torch.device, torch.Size)):
            return {"__repr__": [type(x).__name__, str(x) if not isinstance(x, torch.Size) else list(x)]}
        if not isinstance(x, (Mapping, list, tuple)):
            where = ".".join(map(str, path)) or "<root>"
            raise TypeError(f"object of type {type(x).__name__} at {where} cannot be stored in a .mega file")
        if id(x) in open_nodes:
            raise ValueError("a container that contains itself cannot be stored in a .mega file")
        open_nodes.add(id(x))
        try:
            if isinstance(x, Mapping):
                items = [(k, enc(v, path + [k])) for k, v in x.items()]
                plain = all(isinstance(k, str) for k, _ in items)
                if not plain and not all(isinstance(k, (bool, int, float, str)) for k, _ in items):
                    raise TypeError("mapping keys of a .mega tree must be strings or numbers")
                if not plain or (len(items) == 1 and items[0][0] in _ESCAPES + ("__repr__",)):
                    return {"__dict__": [[k, v] for k, v in items]}
                return dict(items)
            seq = [enc(v, path + [i]) for i, v in enumerate(x)]
            return seq if isinstance(x, list) else {"__tuple__": seq}
        finally:
            open_nodes.discard(id(x))

    layout = enc(obj, [])
    all_tensors = lambda vals: all(isinstance(v, torch.Tensor) for v in vals)  # noqa: E731
    if isinstance(obj, Mapping) and all(isinstance(k, str) for k in obj) and all_tensors(obj.values()) \
            and len(flat) == len(obj):
        return {k: obj[k] for k in obj}, "dict", None
    if isinstance(obj, (list, tuple)) and all_tensors(obj) and len(flat) == len(obj):
        return {str(i): v for i, v in enumerate(obj)}, "list" if isinstance(obj, list) else "tuple", None
    return flat, "tree", layout


def unflatten_tree(flat: Mapping[str, torch.Tensor], kind: str, layout):
    if kind == "tensor":
        if len(flat) != 1:
            raise ValueError("a .mega file of kind 'tensor' holds exactly one tensor")
        return next(iter(flat.values()))
    if kind == "list" and layout is None:
        return list(flat.values())
    if kind == "tuple" and layout is None:
        return tuple(flat.values())
    if layout is None:
        return dict(flat)

    def dec(x):
        if isinstance(x, dict):
            if len(x) == 1:
                (tag, val), = x.items()
                if tag == "__tensor__":
                    if val not in flat:
                        raise ValueError(f"the .mega layout names a tensor that the file lacks: {val!r}")
                    return flat[val]
                if tag == "__tuple__":
                    return tuple(dec(v) for v in val)
                if tag == "__dict__":
                    return {k: dec(v) for k, v in val}
                if tag == "__repr__":
                    tname, r = val
                    if tname == "dtype":
                        return getattr(torch, r.split(".")[-1])
                    return torch.device(r) if tname == "device" else torch.Size(r)
            return {k: dec(v) for k, v in x.items()}
        if isinstance(x, list):
            return [dec(v) for v in x]
        return x

    # files of earlier versions of this writer stored list / tuple roots with a layout
    return dec(layout)


# ------------------------------------------------------------------ header
def _u32(b, v): b.extend(struct.pack("<I", int(v)))
def _u64(b, v): b.extend(struct.pack("<Q", int(v)))


def _string(b, s):
    e = str(s).encode("utf-8")
    _u64(b, len(e))
    b.extend(e)


def _cstring(b, s):
    e = str(s).encode("utf-8")
    _u32(b, len(e))
    b.extend(e)


def _meta_value(b, v):
    if isinstance(v, str):
        _u32(b, 11)
        _string(b, v)
    elif isinstance(v, bool):
        _u32(b, 10)
        b.extend(struct.pack("<B", int(v)))
    elif isinstance(v, int):
        if v < 0:
            raise ValueError("MEGA metadata integers must be non-negative")
        if v <= 0xFFFFFFFF:
            _u32(b, 4)
            _u32(b, v)
        else:
            _u32(b, 6)
            _u64(b, v)
    elif isinstance(v, (list, tuple)):
        _u32(b, 12)
        _u64(b, len(v))
        if not v or isinstance(v[0], str):
            _u32(b, 11)
            for it in v:
                _string(b, it)
        else:
            _u32(b, 4)
            for it in v:
                _u32(b, it)
    else:
        _u32(b, 11)
        _string(b, json.dumps(v, ensure_ascii=False, separators=(",", ":")))


def build_header(records: List[dict], metadata: Mapping[str, Any], checksum: str) -> bytes:
    b = bytearray()
    _u32(b, MAGIC)
    _u32(b, 1)
    _u64(b, len(records))
    _u64(b, len(metadata))
    for k, v in metadata.items():
        _string(b, k)
        _meta_value(b, v)
    ctype = CHECKSUM_TYPES[checksum]
    for r in records:
        _cstring(b, r["name"])
        flags = (1 << 5) if ctype else 0
        _u32(b, flags)
        _u32(b, len(r["shape"]))
        for d in reversed(r["shape"]):
            _u64(b, d)
        _cstring(b, r["dtype"])
        _u64(b, r["offset"])
        if ctype:
            _u32(b, ctype)
            b.extend(r["digest"])
    return bytes(b)


def _digest(t: torch.Tensor, checksum: str) -> bytes:
    if checksum == "none":
        return b""
    raw = t.view(torch.uint8) if t.numel() else t.new_empty(0, dtype=torch.uint8)
    if checksum == "crc32":
        v = _rt().tpb_crc32(raw.data_ptr() if raw.numel() else None, raw.numel(), 0)
        return int(v).to_bytes(4, "little") + b"\x00" * 28
    import hashlib
    return hashlib.sha256(raw.numpy().tobytes()).digest()


def save_mega(obj, path, metadata: Optional[Mapping[str, Any]] = None, alignment: int = DEFAULT_ALIGNMENT,
              checksum: str = "crc32", workers: int = 4) -> None:
    if checksum not in CHECKSUM_TYPES:
        raise ValueError(f"checksum must be one of {sorted(CHECKSUM_TYPES)} (got {checksum!r})")
    flat, kind, layout = flatten_tree(obj)
    records, devices, host, checks = [], {}, [], {}
    off = 0
    for name, t in flat.items():
        if t.dtype not in _DT2MEGA:
            raise NotImplementedError(f"dtype {t.dtype} is not representable in MEGA")
        devices[name] = str(t.device)
        h = t.detach().to("cpu").contiguous()
        flat_bytes = h.reshape(-1).view(torch.uint8) if h.numel() else h.new_empty(0, dtype=torch.uint8)
        dg = _digest(flat_bytes, checksum)
        if checksum == "crc32":
            checks[name] = f"{int.from_bytes(dg[:4], 'little'):08x}"
        elif checksum == "sha256":
            checks[name] = dg.hex()
        records.append({"name": name, "shape": list(t.shape), "dtype": _DT2MEGA[t.dtype], "offset": off,
                        "digest": dg})
        host.append(flat_bytes)
        off += flat_bytes.numel()
    meta = {str(k): (v if isinstance(v, (str, int, bool, list, tuple)) else json.dumps(v)) for k, v in (metadata or {}).items()}
    meta.setdefault("general.architecture", "tensorplay")
    meta.setdefault("general.alignment", int(alignment))
    meta.setdefault("mega.tensor_info.format", "self_describing")
    meta["tensorplay.container"] = kind
    meta["tensorplay.byteorder"] = sys.byteorder
    meta["tensorplay.tensor_devices"] = json.dumps(devices, separators=(",", ":"))
    meta["tensorplay.checksum"] = checksum
    meta["tensorplay.tensor_checksums"] = json.dumps(checks, separators=(",", ":"))
    if layout is not None:
        meta["tensorplay.layout"] = json.dumps(layout, ensure_ascii=False, separators=(",", ":"))
    header = build_header(records, meta, checksum)
    n = len(host)
    ptrs = (C.c_void_p * max(n, 1))(*[h.data_ptr() if h.numel() else None for h in host])
    sizes = (C.c_uint64 * max(n, 1))(*[h.numel() for h in host])
    code = _rt().tpb_mega_write(os.fspath(path).encode(), header, len(header), int(alignment), n, ptrs, sizes,
                                workers)
    if code != 0:
        raise OSError(f"writing {path!r} failed (code {code})")


def parse_mega(path) -> dict:
    out = C.c_void_p()
    n = C.c_longlong()
    code = _rt().tpb_mega_parse(os.fspath(path).encode(), C.byref(out), C.byref(n))
    if code != 0:
        raise ValueError(f"{path!r} is not a readable MEGA file (code {code})")
    try:
        doc = json.loads(C.string_at(out, n.value).decode("utf-8"))
    finally:
        _rt().tpb_free(out)
    return doc


def load_mega(path, map_location=None, mmap: bool = False, verify: bool = False, workers: int = 4):
    doc = parse_mega(path)
    meta = doc["metadata"]
    start = doc["data_start"]
    flat: Dict[str, torch.Tensor] = {}
    p = os.fspath(path)
    whole = None
    if mmap:
        whole = torch.from_file(p, shared=False, size=doc["file_size"], dtype=torch.uint8)
    for rec in doc["tensors"]:
        dt = _MEGA2DT[rec["dtype"]]
        numel = 1
        for d in rec["shape"]:
            numel *= d
        nbytes = numel * torch.empty(0, dtype=dt).element_size()
        if whole is not None:
            raw = whole[start + rec["offset"]: start + rec["offset"] + nbytes]
        else:
            raw = torch.empty(nbytes, dtype=torch.uint8)
            if nbytes:
                code = _rt().tpb_file_read(p.encode(), start + rec["offset"], raw.data_ptr(), nbytes, workers)
                if code != 0:
                    raise OSError(f"reading tensor {rec['name']!r} from {p!r} failed")
        if verify and rec["checksum_type"]:
            verify_record(rec, raw)
        t = raw.view(dt).reshape(rec["shape"]) if nbytes else torch.empty(rec["shape"], dtype=dt)
        if map_location is not None:
            t = t.to(map_location)
        flat[rec["name"]] = t
    layout = json.loads(meta["tensorplay.layout"]) if "tensorplay.layout" in meta else None
    return unflatten_tree(flat, meta.get("tensorplay.container", "dict"), layout)


def verify_record(rec: dict, raw: torch.Tensor) -> None:
    if rec["checksum_type"] == 1:
        got = _rt().tpb_crc32(raw.data_ptr() if raw.numel() else None, raw.numel(), 0)
        want = int.from_bytes(bytes.fromhex(rec["checksum"])[:4], "little")
        if got != want:
            raise ValueError(f"CRC32 mismatch for tensor {rec['name']!r}")
    elif rec["checksum_type"] == 2:
        import hashlib
        if hashlib.sha256(raw.numpy().tobytes()).hexdigest() != rec["checksum"]:
            raise ValueError(f"SHA256 mismatch for tensor {rec['name']!r}")
