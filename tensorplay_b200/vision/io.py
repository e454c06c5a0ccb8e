"""``vision.io``: torchvision's image / video readers and writers plus the batch forms of the reference
(tensorplay/vision/io: ``decode_jpeg_batch``, ``decode_png_batch``, ``encode_jpeg_batch``, ``encode_png_batch``): one image
per worker thread (the codecs release the interpreter lock), results in input order."""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import List, Sequence

from torch import Tensor
from torchvision.io import *  # noqa: F401,F403
from torchvision.io import decode_jpeg, decode_png, encode_jpeg, encode_png


def _map(fn, items: Sequence, workers: int) -> List:
    items = list(items)
    if len(items) <= 1 or workers <= 1:
        return [fn(x) for x in items]
    with ThreadPoolExecutor(max_workers=min(workers, len(items))) as ex:
        return list(ex.map(fn, items))


def decode_jpeg_batch(data: Sequence[Tensor], mode=None, device="cpu", num_workers: int = 8) -> List[Tensor]:
    kw = {} if mode is None else {"mode": mode}
    if str(device) != "cpu":
        return decode_jpeg(list(data), device=device, **kw)     # the GPU decoder batches by itself
    return _map(lambda d: decode_jpeg(d, **kw), data, num_workers)


def decode_png_batch(data: Sequence[Tensor], mode=None, num_workers: int = 8) -> List[Tensor]:
    kw = {} if mode is None else {"mode": mode}
    return _map(lambda d: decode_png(d, **kw), data, num_workers)


def encode_jpeg_batch(images: Sequence[Tensor], quality: int = 75, num_workers: int = 8) -> List[Tensor]:
    return _map(lambda im: encode_jpeg(im, quality=quality), images, num_workers)


def encode_png_batch(images: Sequence[Tensor], compression_level: int = 6, num_workers: int = 8) -> List[Tensor]:
    return _map(lambda im: encode_png(im, compression_level=compression_level), images, num_workers)


def __getattr__(name):
    import torchvision.io as _io
    return getattr(_io, name)
