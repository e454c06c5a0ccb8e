"""``audio``: WAV input / output on the host runtime's native codec (``csrc/runtime/wav_codec.cpp``) - ``decode_wav``,
``encode_wav``, their batch forms (one file per OpenMP thread), ``wav_info``, ``info``, ``load``, ``save`` - and the
back-end queries (tensorplay/audio/io.py, backend.py); transforms, functional, models and datasets resolve to
torchaudio when it is installed."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Sequence, Tuple, Union

import torch
from torch import Tensor

from .. import _native

__all__ = ["AudioMetaData", "info", "load", "save", "decode_wav", "decode_wav_batch", "encode_wav", "encode_wav_batch",
           "wav_info", "list_audio_backends", "get_audio_backend", "set_audio_backend", "check_available"]

_ERRORS = {-1: "not a RIFF/WAVE stream", -2: "truncated WAV stream", -3: "WAV data chunk before the format chunk",
           -4: "unsupported WAV sample format", -5: "WAV payload over 4 GiB"}
_ENCODINGS = {1: "PCM_S", 3: "PCM_F", 6: "ALAW", 7: "ULAW"}
_backend = "native"


@dataclass
class AudioMetaData:
    sample_rate: int
    num_frames: int
    num_channels: int
    bits_per_sample: int
    encoding: str


def _rt():
    rt = _native.runtime()
    if getattr(rt, "_wav_ready", False):
        return rt
    P, LL, I = C.c_void_p, C.c_longlong, C.c_int
    rt.tpb_wav_info.restype, rt.tpb_wav_info.argtypes = I, [P, LL, P, P]
    rt.tpb_wav_decode.restype, rt.tpb_wav_decode.argtypes = I, [P, LL, LL, LL, P, LL, P]
    rt.tpb_wav_encoded_bytes.restype, rt.tpb_wav_encoded_bytes.argtypes = LL, [I, LL, I]
    rt.tpb_wav_encode.restype, rt.tpb_wav_encode.argtypes = I, [P, I, LL, LL, I, I, P]
    rt.tpb_wav_decode_batch.restype, rt.tpb_wav_decode_batch.argtypes = None, [P, P, I, LL, LL, P, P, P, P]
    rt.tpb_wav_encode_batch.restype, rt.tpb_wav_encode_batch.argtypes = None, [P, P, P, P, I, I, I, P, P]
    rt._wav_ready = True
    return rt


def _check(code: int) -> None:
    if code:
        raise ValueError(_ERRORS.get(code, f"WAV codec error {code}"))


def _bytes_tensor(data) -> Tensor:
    if isinstance(data, Tensor):
        return data.to(torch.uint8).contiguous().view(-1)
    return torch.frombuffer(bytearray(data), dtype=torch.uint8)


def wav_info(data) -> Tuple[int, int, int, int, int]:
    """``(sample_rate, frames, channels, bits, format tag)`` of WAV bytes (tag: 1 PCM, 3 float)."""
    b = _bytes_tensor(data)
    out = (C.c_int * 5)()
    frames = C.c_longlong()
    _check(_rt().tpb_wav_info(b.data_ptr(), b.numel(), out, C.byref(frames)))
    return out[0], int(frames.value), out[1], out[2], out[3]


def decode_wav(data, frame_offset: int = 0, num_frames: int = -1) -> Tuple[Tensor, int]:
    """WAV bytes (a ``uint8`` tensor or ``bytes``) -> (waveform ``[channels, time]`` float32 in [-1, 1), sample rate)."""
    b = _bytes_tensor(data)
    rate, frames, ch, _, _ = wav_info(b)
    n = max(0, frames - max(0, frame_offset))
    if num_frames >= 0:
        n = min(n, num_frames)
    wave = torch.empty(ch, n, dtype=torch.float32)
    got = C.c_longlong()
    _check(_rt().tpb_wav_decode(b.data_ptr(), b.numel(), int(frame_offset), int(num_frames), wave.data_ptr(), n,
                                C.byref(got)))
    return wave, rate


def decode_wav_batch(data: Sequence, frame_offset: int = 0, num_frames: int = -1) -> List[Tuple[Tensor, int]]:
    """Decodes several WAV byte strings, one per thread of the runtime's OpenMP team; results in input order."""
    bufs = [_bytes_tensor(d) for d in data]
    if not bufs:
        return []
    metas = [wav_info(b) for b in bufs]
    outs = []
    for (rate, frames, ch, _, _) in metas:
        n = max(0, frames - max(0, frame_offset))
        outs.append(torch.empty(ch, n if num_frames < 0 else min(n, num_frames), dtype=torch.float32))
    k = len(bufs)
    ptrs = (C.c_void_p * k)(*[b.data_ptr() for b in bufs])
    sizes = (C.c_longlong * k)(*[b.numel() for b in bufs])
    optrs = (C.c_void_p * k)(*[o.data_ptr() for o in outs])
    oframes = (C.c_longlong * k)(*[o.shape[1] for o in outs])
    decoded, codes = (C.c_longlong * k)(), (C.c_int * k)()
    _rt().tpb_wav_decode_batch(ptrs, sizes, k, int(frame_offset), int(num_frames), optrs, oframes, decoded, codes)
    for c in codes:
        _check(c)
    return [(o, m[0]) for o, m in zip(outs, metas)]


def _planar(x: Tensor) -> Tensor:
    x = x.detach().to("cpu", torch.float32)
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if x.dim() != 2:
        raise ValueError("a waveform is [channels, time] or [time]")
    return x.contiguous()


def encode_wav(data: Tensor, sample_rate: int, bits: int = 16) -> Tensor:
    """Waveform ``[channels, time]`` (or mono ``[time]``) in [-1, 1) -> WAV bytes as a 1-D ``uint8`` tensor; ``bits``:
    8, 16, 24 or 32 (PCM, rounded to nearest, saturating)."""
    x = _planar(data)
    rt = _rt()
    out = torch.empty(rt.tpb_wav_encoded_bytes(x.shape[0], x.shape[1], int(bits)), dtype=torch.uint8)
    _check(rt.tpb_wav_encode(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), int(sample_rate), int(bits), out.data_ptr()))
    return out


def encode_wav_batch(data: Sequence[Tensor], sample_rate: int, bits: int = 16) -> List[Tensor]:
    xs = [_planar(d) for d in data]
    if not xs:
        return []
    if bits not in (8, 16, 24, 32):
        _check(-4)
    rt = _rt()
    k = len(xs)
    outs = [torch.empty(rt.tpb_wav_encoded_bytes(x.shape[0], x.shape[1], int(bits)), dtype=torch.uint8) for x in xs]
    xp = (C.c_void_p * k)(*[x.data_ptr() for x in xs])
    ch = (C.c_int * k)(*[x.shape[0] for x in xs])
    fr = (C.c_longlong * k)(*[x.shape[1] for x in xs])
    st = (C.c_longlong * k)(*[x.stride(0) for x in xs])
    op = (C.c_void_p * k)(*[o.data_ptr() for o in outs])
    codes = (C.c_int * k)()
    rt.tpb_wav_encode_batch(xp, ch, fr, st, k, int(sample_rate), int(bits), op, codes)
    for c in codes:
        _check(c)
    return outs


def _read(path) -> bytes:
    if hasattr(path, "read"):
        return path.read()
    with open(os.fspath(path), "rb") as f:
        return f.read()


def info(filepath, format=None, buffer_size: int = 4096) -> AudioMetaData:
    rate, frames, ch, bits, tag = wav_info(_read(filepath))
    return AudioMetaData(rate, frames, ch, bits, _ENCODINGS.get(tag, "UNKNOWN"))


def load(filepath, frame_offset: int = 0, num_frames: int = -1, normalize: bool = True, channels_first: bool = True,
         format=None) -> Tuple[Tensor, int]:
    wave, rate = decode_wav(_read(filepath), frame_offset, num_frames)
    return (wave if channels_first else wave.t().contiguous()), rate


def save(filepath, src: Tensor, sample_rate: int, channels_first: bool = True, format=None, encoding=None,
         bits_per_sample: int = 16) -> None:
    x = src if channels_first or src.dim() == 1 else src.t()
    payload = encode_wav(x, sample_rate, bits_per_sample or 16).numpy().tobytes()
    if hasattr(filepath, "write"):
        filepath.write(payload)
    else:
        with open(os.fspath(filepath), "wb") as f:
            f.write(payload)


def list_audio_backends() -> List[str]:
    """``"native"`` (the codec of this framework's runtime: WAV), then what the installed packages add."""
    out = ["native"]
    for name in ("soundfile", "scipy"):
        try:
            __import__(name)
            out.append(name)
        except ImportError:
            pass
    return out


def check_available() -> bool:
    try:
        _rt()
        return True
    except (OSError, AttributeError):
        return False


def get_audio_backend() -> str:
    return _backend


def set_audio_backend(backend: Union[str, None]) -> None:
    global _backend
    if backend is not None and backend not in list_audio_backends():
        raise RuntimeError(f"audio backend {backend!r} is not available; have {list_audio_backends()}")
    _backend = backend or "native"


def __getattr__(name):
    import importlib
    try:
        ta = importlib.import_module("torchaudio")
    except ImportError as e:
        raise AttributeError(f"tensorplay_b200.audio.{name}: not provided here and torchaudio is not installed") from e
    try:
        return getattr(ta, name)
    except AttributeError:
        try:
            return importlib.import_module(f"torchaudio.{name}")
        except ImportError:
            raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
