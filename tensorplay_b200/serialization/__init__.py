"""``serialization``: ``save`` / ``load`` with format sniffing over three containers -
``.mega`` (native C++ reader/writer), torch zip ``.pt/.pth`` (weights-only unpickling) and
safetensors - plus sharded checkpoints with an index file and ``inspect_checkpoint``.

Public surface after tensorplay/serialization/api.py:124-340; sniffing order zip -> MEGA ->
safetensors (common.py:183-196).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Any, Mapping, Optional

import torch

from .mega import DEFAULT_ALIGNMENT, load_mega, parse_mega, save_mega, verify_record
from .safetensors import load_safetensors, read_safetensors_header, save_safetensors

__all__ = ["save", "load", "inspect_checkpoint", "sniff_format", "save_sharded", "load_sharded",
           "convert_to_mega", "convert_model", "save_mega", "load_mega", "save_safetensors", "load_safetensors",
           "parse_mega_header", "resolve_map_location", "DEFAULT_ALIGNMENT", "MEGA_EXTENSION", "MEGA_INDEX_SUFFIX"]


def sniff_format(path) -> str:
    with open(path, "rb") as f:
        head = f.read(16)
    if head[:4] == b"PK\x03\x04":
        return "zip"
    if len(head) >= 4 and struct.unpack("<I", head[:4])[0] == 0x4147454D:
        return "mega"
    if len(head) >= 9 and head[8:9] == b"{" and struct.unpack("<Q", head[:8])[0] < (1 << 30):
        return "safetensors"
    return "pickle"


def _format_for_save(path, fmt: Optional[str]) -> str:
    if fmt:
        return fmt
    ext = os.path.splitext(os.fspath(path))[1].lower()
    return {".mega": "mega", ".safetensors": "safetensors"}.get(ext, "zip")


def save(obj: Any, f, *, format: Optional[str] = None, metadata: Optional[Mapping[str, Any]] = None,
         checksum: str = "crc32", alignment: int = 4096, **kwargs) -> None:
    """Save tensors / nested containers. The container is chosen by extension (``.mega``,
    ``.safetensors``, anything else = torch zip) or by ``format``."""
    if not isinstance(f, (str, os.PathLike)):
        return torch.save(obj, f, **kwargs)
    fmt = _format_for_save(f, format)
    if fmt == "mega":
        save_mega(obj, f, metadata=metadata, alignment=alignment, checksum=checksum)
    elif fmt == "safetensors":
        save_safetensors(obj, f, metadata=metadata)
    else:
        torch.save(obj, f, **kwargs)


def load(f, map_location=None, *, weights_only: bool = True, mmap: bool = False,
         verify_checksums: bool = False, **kwargs) -> Any:
    """Load any of the supported containers (sniffed from the file's first bytes). Pickled
    payloads are always read with the restricted (weights-only) unpickler unless
    ``weights_only=False`` is passed explicitly."""
    if not isinstance(f, (str, os.PathLike)):
        return torch.load(f, map_location=map_location, weights_only=weights_only, **kwargs)
    if os.path.isdir(f) or os.fspath(f).endswith(".index.json"):
        return load_sharded(f, map_location=map_location)
    fmt = sniff_format(f)
    if fmt == "mega":
        return load_mega(f, map_location=map_location, mmap=mmap, verify=verify_checksums)
    if fmt == "safetensors":
        return load_safetensors(f, map_location=map_location, mmap=mmap)
    return torch.load(f, map_location=map_location, weights_only=weights_only, mmap=mmap or None, **kwargs)


def inspect_checkpoint(path, verify_checksums: bool = False) -> dict:
    """Names, shapes, dtypes and metadata without materialising tensors (``.mega`` /
    safetensors); for zip archives the entries are loaded on the meta device."""
    fmt = sniff_format(path)
    if fmt == "mega":
        doc = parse_mega(path)
        if verify_checksums:
            load_mega(path, verify=True)
        return {"format": "mega", "metadata": doc["metadata"],
                "tensors": {r["name"]: {"shape": r["shape"], "dtype": r["dtype"]} for r in doc["tensors"]}}
    if fmt == "safetensors":
        header, _ = read_safetensors_header(path)
        meta = header.pop("__metadata__", {})
        return {"format": "safetensors", "metadata": meta,
                "tensors": {k: {"shape": v["shape"], "dtype": v["dtype"]} for k, v in header.items()}}
    obj = torch.load(path, map_location="meta", weights_only=True)
    tensors = {}

    def walk(x, prefix):
        if isinstance(x, torch.Tensor):
            tensors[prefix or "tensor"] = {"shape": list(x.shape), "dtype": str(x.dtype)}
        elif isinstance(x, Mapping):
            for k, v in x.items():
                walk(v, f"{prefix}.{k}" if prefix else str(k))
        elif isinstance(x, (list, tuple)):
            for i, v in enumerate(x):
                walk(v, f"{prefix}.{i}" if prefix else str(i))

    walk(obj, "")
    return {"format": "zip", "metadata": {}, "tensors": tensors}


def save_sharded(state: Mapping[str, torch.Tensor], directory, max_shard_bytes: int = 4 << 30,
                 format: str = "mega", prefix: str = "model") -> str:
    """Split a flat state dict into shards plus ``<prefix>.<ext>.index.json`` with a ``weight_map``."""
    os.makedirs(directory, exist_ok=True)
    ext = {"mega": ".mega", "safetensors": ".safetensors", "zip": ".pt"}[format]
    shards, cur, size = [], {}, 0
    for k, v in state.items():
        nb = v.numel() * v.element_size()
        if cur and size + nb > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v
        size += nb
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        name = f"{prefix}-{i + 1:05d}-of-{len(shards):05d}{ext}"
        save(sh, os.path.join(directory, name), format=format)
        for k in sh:
            weight_map[k] = name
    index = os.path.join(directory, f"{prefix}{ext}.index.json")
    with open(index, "w") as f:
        json.dump({"metadata": {"format": format, "total_size": sum(v.numel() * v.element_size() for v in state.values())},
                   "weight_map": weight_map}, f, indent=1)
    return index


def load_sharded(path, map_location=None) -> dict:
    if os.path.isdir(path):
        cands = [p for p in os.listdir(path) if p.endswith(".index.json")]
        if not cands:
            raise FileNotFoundError(f"no shard index in {path!r}")
        path = os.path.join(path, cands[0])
    with open(path) as f:
        index = json.load(f)
    base = os.path.dirname(path)
    out = {}
    for shard in sorted(set(index["weight_map"].values())):
        out.update(load(os.path.join(base, shard), map_location=map_location))
    return out


MEGA_EXTENSION = ".mega"
MEGA_INDEX_SUFFIX = ".mega.index.json"
_CHECKPOINT_SUFFIXES = (".safetensors", ".pt", ".pth", ".bin", ".ckpt")


def convert_to_mega(src, dst=None, **kw):
    """Re-write a loadable checkpoint file, or every checkpoint file of a model directory, as
    ``.mega`` and return the path written. A file goes to ``dst`` (a ``.mega`` path or a
    directory; default: next to the source). A directory is converted file by file into ``dst``
    (default: the directory itself); when it holds a shard index, a ``model.mega.index.json`` with the
    same ``weight_map`` pointing at the new files is written too, so ``load`` accepts the result.
    After tensorplay/serialization/mega.py:1438-1479."""
    src = os.fspath(src)
    if os.path.isfile(src):
        stem = os.path.splitext(os.path.basename(src))[0]
        if dst is None:
            target = os.path.join(os.path.dirname(src), stem + MEGA_EXTENSION)
        else:
            dst = os.fspath(dst)
            target = dst if dst.endswith(MEGA_EXTENSION) and not os.path.isdir(dst) else os.path.join(dst, stem + MEGA_EXTENSION)
        os.makedirs(os.path.dirname(os.path.abspath(target)), exist_ok=True)
        save_mega(load(src), target, **kw)
        return target
    if not os.path.isdir(src):
        raise FileNotFoundError(src)
    out_dir = os.fspath(dst) if dst is not None else src
    os.makedirs(out_dir, exist_ok=True)
    renamed = {}
    for name in sorted(os.listdir(src)):
        if name.endswith(_CHECKPOINT_SUFFIXES):
            renamed[name] = os.path.basename(convert_to_mega(os.path.join(src, name), out_dir, **kw))
    if not renamed:
        raise FileNotFoundError(f"no checkpoint file ({', '.join(_CHECKPOINT_SUFFIXES)}) in {src!r}")
    for name in os.listdir(src):
        if name.endswith(".index.json") and not name.endswith(MEGA_INDEX_SUFFIX):
            with open(os.path.join(src, name)) as f:
                index = json.load(f)
            index["weight_map"] = {k: renamed.get(v, v) for k, v in index.get("weight_map", {}).items()}
            with open(os.path.join(out_dir, "model" + MEGA_INDEX_SUFFIX), "w") as f:
                json.dump(index, f, indent=1)
    return out_dir


convert_model = convert_to_mega


def parse_mega_header(path) -> dict:
    """Metadata and tensor byte ranges of a ``.mega`` file without reading tensor data
    (the native parser's document plus the file size)."""
    doc = parse_mega(path)
    doc["file_size"] = os.path.getsize(os.fspath(path))
    return doc


def resolve_map_location(map_location, location: str, nbytes: int = 0):
    """Where one saved storage goes: ``None`` keeps the saved location (returns ``None``); a string
    or ``torch.device`` names the target; a mapping translates saved locations (missing keys keep
    theirs); a callable gets ``(storage_stub, location)`` like ``torch.load``'s and may return a
    device, a destination tensor or ``None``. After tensorplay/serialization/common.py:68-100."""
    if map_location is None:
        return None
    if isinstance(map_location, bytes):
        map_location = map_location.decode()
    if isinstance(map_location, (str, torch.device)):
        return torch.device(map_location)
    if isinstance(map_location, Mapping):
        target = map_location.get(location, location)
        return None if target is None else torch.device(target)
    if callable(map_location):
        stub = torch.empty(0, dtype=torch.uint8).untyped_storage()
        stub.saved_nbytes = nbytes
        result = map_location(stub, location)
        if result is None or isinstance(result, torch.Tensor):
            return result
        if isinstance(result, (str, torch.device)):
            return torch.device(result)
        if hasattr(result, "device"):
            return torch.device(result.device)
        raise TypeError(f"map_location returned {type(result).__name__}; expected a device, a tensor or None")
    raise TypeError(f"unsupported map_location of type {type(map_location).__name__}")


def __getattr__(name):
    """Safe-globals management, mmap / endianness / CRC options, ``skip_data`` and the pickle protocol constants resolve to ``torch.serialization`` (they govern the torch zip format handled here through ``torch.save`` / ``torch.load``)."""
    import importlib
    for mod in ['torch.serialization']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
