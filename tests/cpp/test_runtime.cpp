// Native unit test of the host runtime library (store server / client, file IO, CRC-32) through
// its C ABI, without Python. Built and run by tests/test_cpp_runtime.py.
// Counterpart in the reference: test/cpp (gloo process-group and store tests), p10/tests/*.cpp.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* tpb_store_server_start(int port, int* port_out);
void tpb_store_server_stop(void* h);
void* tpb_store_connect(const char* host, int port, int timeout_ms);
void tpb_store_close(void* h);
int tpb_store_set(void* h, const char* key, int klen, const char* val, long long vlen);
int tpb_store_get(void* h, const char* key, int klen, long long timeout_ms, char** out, long long* out_len);
int tpb_store_add(void* h, const char* key, int klen, long long amount, long long* result);
int tpb_store_cas(void* h, const char* key, int klen, const char* expected, long long elen,
                  const char* desired, long long dlen, char** out, long long* out_len);
int tpb_store_wait(void* h, const char* keys, const int* lens, int nkeys, long long timeout_ms);
int tpb_store_check(void* h, const char* keys, const int* lens, int nkeys);
int tpb_store_delete(void* h, const char* key, int klen);
long long tpb_store_num_keys(void* h);
void tpb_free(void* p);
uint32_t tpb_crc32(const void* data, size_t n, uint32_t seed);
int tpb_mega_write(const char* path, const void* header, uint64_t header_len, uint64_t alignment,
                   int n, const void* const* ptrs, const uint64_t* sizes, int nthreads);
int tpb_file_read(const char* path, uint64_t offset, void* dst, uint64_t nbytes, int nthreads);
void* tpb_reducer_create(const long long* numels, const int* elem_bytes, int n, long long cap_bytes, long long align);
void tpb_reducer_destroy(void* h);
int tpb_reducer_num_buckets(void* h);
int tpb_reducer_bucket_of(void* h, int param);
long long tpb_reducer_offset_of(void* h, int param);
long long tpb_reducer_bucket_numel(void* h, int bucket);
int tpb_reducer_mark_ready(void* h, int param);
void tpb_reducer_rearm(void* h, int bucket);
void tpb_reducer_reset(void* h);
void* tpb_loader_open(const char* path, int elem_bytes, int seq_len, int batch, int rank, int world,
                      unsigned long long seed, int shuffle, int n_workers, int depth, void** tok_slots,
                      void** tgt_slots, int* err);
long long tpb_loader_batches_per_epoch(void* h);
int tpb_loader_next(void* h, long long* batch_number);
void tpb_loader_release(void* h, int slot);
void tpb_loader_close(void* h);
}

static int failures = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                                          \
    }                                                                      \
  } while (0)

static std::string get(void* c, const std::string& k, long long timeout_ms = 2000) {
  char* out = nullptr;
  long long n = 0;
  if (tpb_store_get(c, k.data(), (int)k.size(), timeout_ms, &out, &n) != 0) return "<error>";
  std::string v(out, (size_t)n);
  tpb_free(out);
  return v;
}

static void test_store() {
  int port = 0;
  void* srv = tpb_store_server_start(0, &port);
  CHECK(srv != nullptr && port > 0);
  void* a = tpb_store_connect("127.0.0.1", port, 5000);
  void* b = tpb_store_connect("127.0.0.1", port, 5000);
  CHECK(a && b);
  CHECK(tpb_store_set(a, "k", 1, "hello", 5) == 0);
  CHECK(get(b, "k") == "hello");
  std::string blob(1 << 20, '\x7f');  // binary-safe, larger than one socket buffer
  blob[12345] = '\0';
  CHECK(tpb_store_set(a, "blob", 4, blob.data(), (long long)blob.size()) == 0);
  CHECK(get(b, "blob") == blob);

  // add is atomic across clients
  std::vector<std::thread> ts;
  for (int t = 0; t < 4; ++t)
    ts.emplace_back([port] {
      void* c = tpb_store_connect("127.0.0.1", port, 5000);
      long long r = 0;
      for (int i = 0; i < 250; ++i) tpb_store_add(c, "ctr", 3, 1, &r);
      tpb_store_close(c);
    });
  for (auto& t : ts) t.join();
  long long total = 0;
  CHECK(tpb_store_add(a, "ctr", 3, 0, &total) == 0 && total == 1000);

  // compare-and-set: only the matching expectation wins
  char* out = nullptr;
  long long n = 0;
  CHECK(tpb_store_cas(a, "lock", 4, "", 0, "A", 1, &out, &n) == 0 && std::string(out, n) == "A");
  tpb_free(out);
  CHECK(tpb_store_cas(b, "lock", 4, "", 0, "B", 1, &out, &n) == 0 && std::string(out, n) == "A");
  tpb_free(out);

  // wait blocks until another client sets the key; a missing key times out
  int len = 5;
  std::thread setter([port] {
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    void* c = tpb_store_connect("127.0.0.1", port, 5000);
    tpb_store_set(c, "later", 5, "x", 1);
    tpb_store_close(c);
  });
  CHECK(tpb_store_wait(a, "later", &len, 1, 5000) == 0);
  setter.join();
  int len2 = 5;
  CHECK(tpb_store_wait(a, "never", &len2, 1, 100) != 0);
  CHECK(tpb_store_check(a, "later", &len, 1) == 0);  // status 0: every key is present
  CHECK(tpb_store_delete(a, "later", 5) == 0);
  CHECK(tpb_store_check(a, "later", &len, 1) != 0);
  CHECK(tpb_store_num_keys(a) >= 4);
  tpb_store_close(a);
  tpb_store_close(b);
  tpb_store_server_stop(srv);
}

static void test_file_io(const char* dir) {
  // CRC-32 of "123456789" is the standard check value
  CHECK(tpb_crc32("123456789", 9, 0) == 0xCBF43926u);
  std::vector<float> t0(1000), t1(77777);
  for (size_t i = 0; i < t0.size(); ++i) t0[i] = (float)i;
  for (size_t i = 0; i < t1.size(); ++i) t1[i] = (float)i * 0.5f;
  const void* ptrs[2] = {t0.data(), t1.data()};
  uint64_t sizes[2] = {t0.size() * 4, t1.size() * 4};
  std::string path = std::string(dir) + "/cpp_runtime_test.bin";
  const char header[] = "HEADER-BYTES";
  CHECK(tpb_mega_write(path.c_str(), header, sizeof(header), 64, 2, ptrs, sizes, 4) == 0);
  std::vector<float> back(t1.size());
  CHECK(tpb_file_read(path.c_str(), 64 + sizes[0], back.data(), sizes[1], 3) == 0);
  CHECK(std::memcmp(back.data(), t1.data(), sizes[1]) == 0);
  char hdr[sizeof(header)] = {0};
  CHECK(tpb_file_read(path.c_str(), 0, hdr, sizeof(header), 1) == 0 && std::memcmp(hdr, header, sizeof(header)) == 0);
  std::remove(path.c_str());
}

static void test_reducer() {
  // 4 parameters, model order; gradients arrive last-first: buckets are filled from the end
  const long long numels[4] = {100, 200, 50, 1000};
  const int elem[4] = {2, 2, 4, 2};
  void* r = tpb_reducer_create(numels, elem, 4, /*cap_bytes=*/1000, /*align=*/256);
  CHECK(tpb_reducer_num_buckets(r) == 3);
  CHECK(tpb_reducer_bucket_of(r, 3) == 0);   // larger than the cap: alone
  CHECK(tpb_reducer_bucket_of(r, 2) == 1);   // other element size: own bucket
  CHECK(tpb_reducer_bucket_of(r, 1) == 2 && tpb_reducer_bucket_of(r, 0) == 2);
  CHECK(tpb_reducer_offset_of(r, 1) == 0 && tpb_reducer_offset_of(r, 0) == 200);  // 8-element aligned
  CHECK(tpb_reducer_bucket_numel(r, 0) == 1024 && tpb_reducer_bucket_numel(r, 2) == 512);
  CHECK(tpb_reducer_mark_ready(r, 3) == 0);
  CHECK(tpb_reducer_mark_ready(r, 1) == -1);
  CHECK(tpb_reducer_mark_ready(r, 1) == -2);  // double mark in one iteration
  CHECK(tpb_reducer_mark_ready(r, 0) == 2);
  tpb_reducer_rearm(r, 2);
  CHECK(tpb_reducer_mark_ready(r, 0) == -1);  // counts again after re-arming
  tpb_reducer_reset(r);
  CHECK(tpb_reducer_mark_ready(r, 2) == 1);
  tpb_reducer_destroy(r);
}

static void test_loader(const char* dir) {
  // token i of the file has value i: a batch row names its sample, targets are tokens + 1
  const int seq = 8, batch = 2, depth = 3, n_samples = 20;
  const std::string path = std::string(dir) + "/tokens_cpp.bin";
  {
    std::vector<int32_t> v(n_samples * seq + 1);
    for (size_t i = 0; i < v.size(); ++i) v[i] = (int32_t)i;
    FILE* f = std::fopen(path.c_str(), "wb");
    CHECK(f != nullptr);
    std::fwrite(v.data(), 4, v.size(), f);
    std::fclose(f);
  }
  std::vector<std::vector<int64_t>> tok(depth, std::vector<int64_t>(batch * seq)), tgt = tok;
  std::vector<void*> tp, gp;
  for (int i = 0; i < depth; ++i) {
    tp.push_back(tok[i].data());
    gp.push_back(tgt[i].data());
  }
  int err = 0;
  void* h = tpb_loader_open(path.c_str(), 4, seq, batch, 0, 1, 42, 1, 3, depth, tp.data(), gp.data(), &err);
  CHECK(h != nullptr && err == 0);
  if (!h) return;
  CHECK(tpb_loader_batches_per_epoch(h) == n_samples / batch);
  std::vector<int> seen(n_samples, 0);
  for (long long b = 0; b < n_samples / batch; ++b) {
    long long num = -1;
    const int slot = tpb_loader_next(h, &num);
    CHECK(slot >= 0 && slot < depth && num == b);
    for (int r = 0; r < batch; ++r) {
      const int64_t first = tok[slot][r * seq];
      CHECK(first % seq == 0 && first / seq < n_samples);
      seen[first / seq]++;
      for (int t = 0; t < seq; ++t) {
        CHECK(tok[slot][r * seq + t] == first + t);
        CHECK(tgt[slot][r * seq + t] == first + t + 1);
      }
    }
    tpb_loader_release(h, slot);
  }
  for (int i = 0; i < n_samples; ++i) CHECK(seen[i] == 1);
  tpb_loader_close(h);
  void* bad = tpb_loader_open("/nonexistent/file.bin", 4, seq, batch, 0, 1, 0, 1, 1, depth, tp.data(), gp.data(), &err);
  CHECK(bad == nullptr && err != 0);
}

int main(int argc, char** argv) {
  test_loader(argc > 1 ? argv[1] : "/tmp");
  test_store();
  test_reducer();
  test_file_io(argc > 1 ? argv[1] : "/tmp");
  if (failures) {
    std::fprintf(stderr, "%d check(s) failed\n", failures);
    return 1;
  }
  std::puts("all runtime checks passed");
  return 0;
}
