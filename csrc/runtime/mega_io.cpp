// Native reader / writer of the ".mega" checkpoint container.
//
// File layout (little endian): u32 magic 0x4147454D ("MEGA"), u32 version = 1, u64 n_tensors,
// u64 n_meta, then n_meta typed key/value pairs (key = u64 length + bytes; value = u32 type id
// followed by: 4 -> u32, 6 -> u64, 10 -> u8 bool, 11 -> u64-length string, 12 -> array: u64 count,
// u32 element type, elements), then per tensor: u32-length name, u32 flags (bit 1: stored size
// differs from the logical size, bit 5: checksum present), u32 ndim, ndim x u64 dims in REVERSED
// order, u32-length dtype string, u64 payload offset relative to the aligned end of the header,
// [u64 stored size if bit 1], [u32 checksum type + 32 digest bytes if bit 5]. The header is
// zero-padded to "general.alignment" (default 4096); payloads follow, raw and dense.
//
// The format is the one written by the reference's tensorplay/serialization/mega.py:455-553
// (header) and :615-618, :732-744 (padding, payload order); the reference parses it through the
// external megatensors package (:107-118), this is an independent parser.
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Cursor {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (p + sizeof(T) > end) { ok = false; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str(uint64_t n) {
    if (!ok || p + n > end) { ok = false; return {}; }
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    return s;
  }
};

void json_escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof(b), "\\u%04x", c); out += b; }
        else out.push_back((char)c);
    }
  }
  out.push_back('"');
}

bool parse_value(Cursor& c, std::string& out) {
  uint32_t t = c.get<uint32_t>();
  if (!c.ok) return false;
  switch (t) {
    case 4: out += std::to_string(c.get<uint32_t>()); break;
    case 6: out += std::to_string(c.get<uint64_t>()); break;
    case 10: out += c.get<uint8_t>() ? "true" : "false"; break;
    case 11: { uint64_t n = c.get<uint64_t>(); json_escape(c.str(n), out); } break;
    case 12: {
      uint64_t n = c.get<uint64_t>();
      uint32_t et = c.get<uint32_t>();
      out.push_back('[');
      for (uint64_t i = 0; i < n && c.ok; ++i) {
        if (i) out.push_back(',');
        if (et == 11) { uint64_t l = c.get<uint64_t>(); json_escape(c.str(l), out); }
        else if (et == 4) out += std::to_string(c.get<uint32_t>());
        else if (et == 6) out += std::to_string(c.get<uint64_t>());
        else return false;
      }
      out.push_back(']');
    } break;
    default: return false;
  }
  return c.ok;
}

uint32_t crc_table[8][256];
std::atomic<bool> crc_ready{false};
void crc_init() {
  if (crc_ready.load()) return;
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
    crc_table[0][i] = c;
  }
  for (uint32_t i = 0; i < 256; ++i)
    for (int t = 1; t < 8; ++t)
      crc_table[t][i] = (crc_table[t - 1][i] >> 8) ^ crc_table[0][crc_table[t - 1][i] & 0xFF];
  crc_ready.store(true);
}

bool pwrite_all(int fd, const char* p, size_t n, off_t off) {
  while (n) {
    ssize_t w = ::pwrite(fd, p, std::min<size_t>(n, 1u << 30), off);
    if (w <= 0) return false;
    p += w; n -= (size_t)w; off += w;
  }
  return true;
}
bool pread_all(int fd, char* p, size_t n, off_t off) {
  while (n) {
    ssize_t r = ::pread(fd, p, std::min<size_t>(n, 1u << 30), off);
    if (r <= 0) return false;
    p += r; n -= (size_t)r; off += r;
  }
  return true;
}

}  // namespace

extern "C" {

// zlib-compatible CRC-32 (slice-by-8).
uint32_t tpb_crc32(const void* data, size_t n, uint32_t seed) {
  crc_init();
  const uint8_t* p = static_cast<const uint8_t*>(data);
  uint32_t c = ~seed;
  while (n >= 8) {
    uint32_t lo, hi;
    memcpy(&lo, p, 4);
    memcpy(&hi, p + 4, 4);
    lo ^= c;
    c = crc_table[7][lo & 0xFF] ^ crc_table[6][(lo >> 8) & 0xFF] ^ crc_table[5][(lo >> 16) & 0xFF] ^
        crc_table[4][lo >> 24] ^ crc_table[3][hi & 0xFF] ^ crc_table[2][(hi >> 8) & 0xFF] ^
        crc_table[1][(hi >> 16) & 0xFF] ^ crc_table[0][hi >> 24];
    p += 8;
    n -= 8;
  }
  while (n--) c = crc_table[0][(c ^ *p++) & 0xFF] ^ (c >> 8);
  return ~c;
}

// Writes header, zero padding up to `alignment`, then the payloads back to back (threads split
// the tensors). Returns 0 on success.
int tpb_mega_write(const char* path, const void* header, uint64_t header_len, uint64_t alignment,
                   int n, const void* const* ptrs, const uint64_t* sizes, int nthreads) {
  int fd = ::open(path, O_CREAT | O_TRUNC | O_WRONLY, 0644);
  if (fd < 0) return -1;
  uint64_t data_start = (header_len + alignment - 1) / alignment * alignment;
  std::vector<uint64_t> offs(n);
  uint64_t off = data_start;
  for (int i = 0; i < n; ++i) { offs[i] = off; off += sizes[i]; }
  bool ok = ::ftruncate(fd, (off_t)off) == 0;  // also zero-fills the header padding
  ok = ok && pwrite_all(fd, static_cast<const char*>(header), header_len, 0);
  if (ok && n > 0) {
    nthreads = std::max(1, std::min(nthreads, n));
    std::atomic<int> next{0};
    std::atomic<bool> good{true};
    std::vector<std::thread> ts;
    for (int t = 0; t < nthreads; ++t)
      ts.emplace_back([&] {
        int i;
        while ((i = next.fetch_add(1)) < n)
          if (!pwrite_all(fd, static_cast<const char*>(ptrs[i]), sizes[i], (off_t)offs[i])) good.store(false);
      });
    for (auto& t : ts) t.join();
    ok = good.load();
  }
  ok = (::close(fd) == 0) && ok;
  return ok ? 0 : -2;
}

// Parses the header into a JSON document (malloc'ed; free with tpb_free):
//   {"version":1,"data_start":N,"metadata":{...},"tensors":[{"name":..,"shape":[..],"dtype":..,
//    "offset":..,"nbytes":..,"checksum_type":..,"checksum":"hex"}]}
int tpb_mega_parse(const char* path, char** json_out, long long* json_len) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -1;
  struct stat st;
  if (fstat(fd, &st) != 0) { ::close(fd); return -1; }
  // headers are small next to payloads; read up to 64 MiB and grow if the parse runs out
  size_t cap = std::min<size_t>((size_t)st.st_size, 64u << 20);
  std::vector<uint8_t> buf;
  std::string out;
  for (;;) {
    buf.resize(cap);
    if (!pread_all(fd, reinterpret_cast<char*>(buf.data()), cap, 0)) { ::close(fd); return -1; }
    Cursor c{buf.data(), buf.data() + buf.size()};
    out.clear();
    uint32_t magic = c.get<uint32_t>();
    uint32_t version = c.get<uint32_t>();
    if (!c.ok || magic != 0x4147454Du) { ::close(fd); return -3; }
    uint64_t nt = c.get<uint64_t>();
    uint64_t nm = c.get<uint64_t>();
    out += "{\"version\":" + std::to_string(version) + ",\"metadata\":{";
    uint64_t alignment = 4096;
    bool fail = false;
    for (uint64_t i = 0; i < nm && c.ok; ++i) {
      uint64_t kl = c.get<uint64_t>();
      std::string key = c.str(kl);
      if (i) out.push_back(',');
      json_escape(key, out);
      out.push_back(':');
      size_t before = out.size();
      if (!parse_value(c, out)) { fail = true; break; }
      if (key == "general.alignment") alignment = strtoull(out.c_str() + before, nullptr, 10);
    }
    out += "},\"tensors\":[";
    for (uint64_t i = 0; i < nt && c.ok && !fail; ++i) {
      uint32_t nl = c.get<uint32_t>();
      std::string name = c.str(nl);
      uint32_t flags = c.get<uint32_t>();
      uint32_t nd = c.get<uint32_t>();
      if (nd > 64) { fail = true; break; }
      std::vector<uint64_t> dims(nd);
      for (uint32_t d = 0; d < nd; ++d) dims[nd - 1 - d] = c.get<uint64_t>();
      uint32_t dl = c.get<uint32_t>();
      std::string dt = c.str(dl);
      uint64_t off = c.get<uint64_t>();
      long long stored = -1;
      if (flags & (1u << 1)) stored = (long long)c.get<uint64_t>();
      uint32_t ctype = 0;
      std::string digest;
      if (flags & (1u << 5)) {
        ctype = c.get<uint32_t>();
        digest = c.str(32);
      }
      if (!c.ok) break;
      if (i) out.push_back(',');
      out += "{\"name\":";
      json_escape(name, out);
      out += ",\"shape\":[";
      for (uint32_t d = 0; d < nd; ++d) { if (d) out.push_back(','); out += std::to_string(dims[d]); }
      out += "],\"dtype\":";
      json_escape(dt, out);
      out += ",\"offset\":" + std::to_string(off) + ",\"stored_nbytes\":" + std::to_string(stored) +
             ",\"checksum_type\":" + std::to_string(ctype) + ",\"checksum\":\"";
      static const char* hx = "0123456789abcdef";
      for (unsigned char ch : digest) { out.push_back(hx[ch >> 4]); out.push_back(hx[ch & 15]); }
      out += "\"}";
    }
    if (fail) { ::close(fd); return -3; }
    if (!c.ok) {
      if (cap >= (size_t)st.st_size) { ::close(fd); return -3; }
      cap = std::min<size_t>((size_t)st.st_size, cap * 4);
      continue;
    }
    uint64_t header_len = (uint64_t)(c.p - buf.data());
    uint64_t data_start = (header_len + alignment - 1) / alignment * alignment;
    out += "],\"data_start\":" + std::to_string(data_start) + ",\"file_size\":" +
           std::to_string((uint64_t)st.st_size) + "}";
    break;
  }
  ::close(fd);
  *json_out = static_cast<char*>(malloc(out.size() + 1));
  memcpy(*json_out, out.data(), out.size() + 1);
  *json_len = (long long)out.size();
  return 0;
}

// Parallel pread of [offset, offset + nbytes) into dst (host memory, e.g. pinned).
int tpb_file_read(const char* path, uint64_t offset, void* dst, uint64_t nbytes, int nthreads) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -1;
  nthreads = std::max(1, nthreads);
  uint64_t chunk = std::max<uint64_t>((nbytes + nthreads - 1) / nthreads, 1u << 20);
  std::vector<std::thread> ts;
  std::atomic<bool> good{true};
  for (uint64_t o = 0; o < nbytes; o += chunk) {
    uint64_t n = std::min(chunk, nbytes - o);
    ts.emplace_back([=, &good] {
      if (!pread_all(fd, static_cast<char*>(dst) + o, n, (off_t)(offset + o))) good.store(false);
    });
  }
  for (auto& t : ts) t.join();
  ::close(fd);
  return good.load() ? 0 : -2;
}

}  // extern "C"
