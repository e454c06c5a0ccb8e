// RIFF/WAVE codec of the host runtime: header scan, PCM (8 / 16 / 24 / 32 bit) and IEEE float (32 / 64 bit)
// payloads to planar float32 [channels, frames] and back, plus batch entry points that spread the
// files over the OpenMP team. No allocation: the caller sizes the output from tpb_wav_info.
//
// Capability reference: the reference's native audio codec behind tensorplay/audio/io.py
// (decode_wav :125, decode_wav_batch :138, encode_wav :389, encode_wav_batch :403, wav_info :416).
#include <cmath>
#include <cstdint>
#include <cstring>

namespace {

struct WavInfo {
  int sample_rate, channels, bits, format;   // format: 1 PCM, 3 IEEE float (0xFFFE resolved to its sub-format)
  long long frames;
  long long data_off, data_bytes;
};

inline uint32_t rd32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | ((uint32_t)p[3] << 24); }
inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// 0 ok; -1 not RIFF/WAVE; -2 truncated; -3 no fmt chunk before data; -4 unsupported format.
int parse(const uint8_t* d, long long n, WavInfo* w) {
  if (n < 12 || std::memcmp(d, "RIFF", 4) || std::memcmp(d + 8, "WAVE", 4)) return -1;
  long long pos = 12;
  bool have_fmt = false;
  while (pos + 8 <= n) {
    const uint32_t sz = rd32(d + pos + 4);
    const uint8_t* body = d + pos + 8;
    if (!std::memcmp(d + pos, "fmt ", 4)) {
      if (sz < 16 || pos + 8 + 16 > n) return -2;
      w->format = rd16(body);
      w->channels = rd16(body + 2);
      w->sample_rate = (int)rd32(body + 4);
      w->bits = rd16(body + 14);
      if (w->format == 0xFFFE && sz >= 26 && pos + 8 + 26 <= n) w->format = rd16(body + 24);
      have_fmt = true;
    } else if (!std::memcmp(d + pos, "data", 4)) {
      if (!have_fmt) return -3;
      long long bytes = sz;
      if (pos + 8 + bytes > n) bytes = n - pos - 8;   // a streamed file may carry a placeholder size
      const int bps = w->bits / 8;
      if (w->channels <= 0 || bps <= 0) return -4;
      if (!((w->format == 1 && (w->bits == 8 || w->bits == 16 || w->bits == 24 || w->bits == 32)) ||
            (w->format == 3 && (w->bits == 32 || w->bits == 64))))
        return -4;
      w->data_off = pos + 8;
      w->data_bytes = bytes;
      w->frames = bytes / ((long long)bps * w->channels);
      return 0;
    }
    pos += 8 + (long long)sz + (sz & 1);
  }
  return -2;
}

inline float sample_at(const uint8_t* p, int bits, int format) {
  if (format == 3) {
    if (bits == 32) { float f; std::memcpy(&f, p, 4); return f; }
    double f; std::memcpy(&f, p, 8); return (float)f;
  }
  switch (bits) {
    case 8: return ((int)p[0] - 128) * (1.f / 128.f);
    case 16: return (int16_t)rd16(p) * (1.f / 32768.f);
    case 24: { int32_t v = (int32_t)((p[0] << 8) | (p[1] << 16) | ((uint32_t)p[2] << 24)) >> 8; return v * (1.f / 8388608.f); }
    default: return (int32_t)rd32(p) * (1.f / 2147483648.f);
  }
}

}  // namespace

extern "C" {

// out5: sample_rate, channels, bits, format tag, (unused); frames through *frames.
int tpb_wav_info(const uint8_t* data, long long n, int* out5, long long* frames) {
  WavInfo w{};
  const int r = parse(data, n, &w);
  if (r) return r;
  out5[0] = w.sample_rate; out5[1] = w.channels; out5[2] = w.bits; out5[3] = w.format; out5[4] = 0;
  *frames = w.frames;
  return 0;
}

// out: float32 [channels, count] planar, count = frames actually decoded (returned through *decoded).
int tpb_wav_decode(const uint8_t* data, long long n, long long frame_offset, long long num_frames, float* out,
                   long long out_frames, long long* decoded) {
  WavInfo w{};
  const int r = parse(data, n, &w);
  if (r) return r;
  long long f0 = frame_offset < 0 ? 0 : frame_offset;
  if (f0 > w.frames) f0 = w.frames;
  long long cnt = w.frames - f0;
  if (num_frames >= 0 && num_frames < cnt) cnt = num_frames;
  if (cnt > out_frames) cnt = out_frames;
  const int bps = w.bits / 8, ch = w.channels;
  const uint8_t* base = data + w.data_off + f0 * bps * ch;
  for (int c = 0; c < ch; ++c) {
    float* dst = out + (long long)c * out_frames;
    const uint8_t* src = base + c * bps;
    for (long long i = 0; i < cnt; ++i) dst[i] = sample_at(src + i * bps * ch, w.bits, w.format);
  }
  *decoded = cnt;
  return 0;
}

long long tpb_wav_encoded_bytes(int channels, long long frames, int bits) {
  return 44 + frames * channels * (bits / 8);
}

// x: float32 [channels, frames] planar (row stride `stride` elements); PCM of `bits` (8 / 16 / 24 / 32) with
// rounding to nearest and saturation. out: tpb_wav_encoded_bytes bytes.
int tpb_wav_encode(const float* x, int channels, long long frames, long long stride, int sample_rate, int bits,
                   uint8_t* out) {
  if (channels <= 0 || frames < 0 || !(bits == 8 || bits == 16 || bits == 24 || bits == 32)) return -4;
  const int bps = bits / 8;
  const long long data_bytes = frames * channels * bps;
  if (data_bytes > 0xFFFFFFFFll - 44) return -5;   // RIFF sizes are 32-bit
  auto w32 = [](uint8_t* p, uint32_t v) { p[0] = v; p[1] = v >> 8; p[2] = v >> 16; p[3] = v >> 24; };
  auto w16 = [](uint8_t* p, uint16_t v) { p[0] = v & 0xff; p[1] = v >> 8; };
  std::memcpy(out, "RIFF", 4); w32(out + 4, (uint32_t)(36 + data_bytes)); std::memcpy(out + 8, "WAVEfmt ", 8);
  w32(out + 16, 16); w16(out + 20, 1); w16(out + 22, (uint16_t)channels); w32(out + 24, (uint32_t)sample_rate);
  w32(out + 28, (uint32_t)((long long)sample_rate * channels * bps)); w16(out + 32, (uint16_t)(channels * bps));
  w16(out + 34, (uint16_t)bits); std::memcpy(out + 36, "data", 4); w32(out + 40, (uint32_t)data_bytes);
  uint8_t* p = out + 44;
  const double full = bits == 8 ? 128.0 : bits == 16 ? 32768.0 : bits == 24 ? 8388608.0 : 2147483648.0;
  for (long long i = 0; i < frames; ++i)
    for (int c = 0; c < channels; ++c, p += bps) {
      double v = std::nearbyint((double)x[(long long)c * stride + i] * full);
      if (v > full - 1) v = full - 1;
      if (v < -full) v = -full;
      const long long q = (long long)v;
      if (bits == 8) p[0] = (uint8_t)(q + 128);
      else for (int b = 0; b < bps; ++b) p[b] = (uint8_t)((q >> (8 * b)) & 0xff);
    }
  return 0;
}

// Batch forms: arrays of per-file arguments, one file per OpenMP iteration. codes[i] receives each file's result.
void tpb_wav_decode_batch(const uint8_t* const* data, const long long* n, int count, long long frame_offset,
                          long long num_frames, float* const* out, const long long* out_frames, long long* decoded,
                          int* codes) {
#pragma omp parallel for schedule(dynamic)
  for (int i = 0; i < count; ++i)
    codes[i] = tpb_wav_decode(data[i], n[i], frame_offset, num_frames, out[i], out_frames[i], decoded + i);
}

void tpb_wav_encode_batch(const float* const* x, const int* channels, const long long* frames, const long long* stride,
                          int count, int sample_rate, int bits, uint8_t* const* out, int* codes) {
#pragma omp parallel for schedule(dynamic)
  for (int i = 0; i < count; ++i)
    codes[i] = tpb_wav_encode(x[i], channels[i], frames[i], stride[i], sample_rate, bits, out[i]);
}

}  // extern "C"
