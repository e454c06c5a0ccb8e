"""WAV codec of the host runtime: round trips at every PCM width, agreement with the standard library's reader and
writer, partial reads, batch forms, float payloads, error codes."""
import io
import struct
import wave

import numpy as np
import pytest
import torch

import tensorplay_b200 as tp

A = tp.audio


def _signal(n=800):
    return torch.stack((torch.sin(torch.arange(n) / 10.0) * 0.8, torch.linspace(-1, 1, n)))


@pytest.mark.parametrize("bits", [8, 16, 24, 32])
def test_round_trip_within_half_a_quantisation_step(bits):
    x = _signal()
    blob = A.encode_wav(x, 16000, bits)
    assert A.wav_info(blob) == (16000, 800, 2, bits, 1)
    y, rate = A.decode_wav(blob)
    top = 1 - 2.0 ** (1 - bits)                                     # the largest code below +1
    assert rate == 16000 and (y - x.clamp(-1, top)).abs().max() <= 2.0 ** (-bits) + 1e-9


def test_agrees_with_the_standard_library_both_ways(tmp_path):
    x = _signal()
    blob = A.encode_wav(x, 8000, 16).numpy().tobytes()
    w = wave.open(io.BytesIO(blob))
    assert (w.getnchannels(), w.getframerate(), w.getnframes(), w.getsampwidth()) == (2, 8000, 800, 2)
    raw = np.frombuffer(w.readframes(800), dtype="<i2").reshape(-1, 2).T
    assert np.abs(raw / 32768.0 - A.decode_wav(blob)[0].numpy()).max() == 0.0
    buf = io.BytesIO()
    ww = wave.open(buf, "wb")
    ww.setnchannels(1); ww.setsampwidth(2); ww.setframerate(22050)
    ww.writeframes(struct.pack("<5h", 0, 16384, -16384, 32767, -32768))
    ww.close()
    y, rate = A.decode_wav(buf.getvalue())
    assert rate == 22050 and torch.allclose(y, torch.tensor([[0.0, 0.5, -0.5, 32767 / 32768, -1.0]]))
    assert A.decode_wav(buf.getvalue(), frame_offset=1, num_frames=2)[0].tolist() == [[0.5, -0.5]]
    assert A.decode_wav(buf.getvalue(), frame_offset=9)[0].shape == (1, 0)
    # files
    path = tmp_path / "a.wav"
    A.save(path, x, 16000, bits_per_sample=24)
    meta = A.info(path)
    assert (meta.sample_rate, meta.num_frames, meta.num_channels, meta.bits_per_sample, meta.encoding) == (16000, 800, 2, 24, "PCM_S")
    y, rate = A.load(path, channels_first=False)
    assert y.shape == (800, 2) and (y.t() - x.clamp(-1, 1 - 2.0 ** -23)).abs().max() < 1e-6


def test_float_payload_extra_chunks_and_errors():
    # IEEE float format with a LIST chunk of odd length (padded) before the data
    samples = struct.pack("<4f", 0.25, -0.5, 1.5, 0.0)
    fmt = struct.pack("<HHIIHH", 3, 2, 48000, 48000 * 8, 8, 32)
    body = b"WAVE" + b"fmt " + struct.pack("<I", 16) + fmt + b"LIST" + struct.pack("<I", 3) + b"abc\x00" + \
        b"data" + struct.pack("<I", len(samples)) + samples
    blob = b"RIFF" + struct.pack("<I", len(body)) + body
    y, rate = A.decode_wav(blob)
    assert rate == 48000 and y.tolist() == [[0.25, 1.5], [-0.5, 0.0]] and A.wav_info(blob)[3:] == (32, 3)
    with pytest.raises(ValueError, match="not a RIFF"):
        A.decode_wav(b"not a wave file at all")
    with pytest.raises(ValueError, match="truncated"):
        A.decode_wav(blob[:30])
    with pytest.raises(ValueError, match="unsupported"):
        A.encode_wav(_signal(), 8000, 12)
    # saturation instead of wrap-around
    loud = torch.tensor([[2.0, -3.0]])
    assert A.decode_wav(A.encode_wav(loud, 8000, 16))[0].tolist() == [[32767 / 32768, -1.0]]


def test_batch_forms_and_backends():
    x = _signal()
    blobs = A.encode_wav_batch([x, x[0], x[:, :10]], 16000, 16)
    assert [b.numel() for b in blobs] == [44 + 800 * 2 * 2, 44 + 800 * 2, 44 + 10 * 2 * 2]
    outs = A.decode_wav_batch(blobs, frame_offset=2, num_frames=5)
    assert [o[0].shape for o in outs] == [(2, 5), (1, 5), (2, 5)] and all(o[1] == 16000 for o in outs)
    assert torch.equal(outs[0][0], A.decode_wav(blobs[0], 2, 5)[0])
    assert A.decode_wav_batch([]) == [] and A.list_audio_backends()[0] == "native" and A.check_available()
    A.set_audio_backend("native")
    assert A.get_audio_backend() == "native"
    with pytest.raises(RuntimeError):
        A.set_audio_backend("sox")
