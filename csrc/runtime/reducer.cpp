// Bucket bookkeeping of the DDP reducer: assignment of parameters to flat gradient buckets (in the
// order backward produces gradients: last parameter first, a bucket closes when the next parameter
// would exceed the byte cap or has another element size) and the per-iteration ready counting that
// tells the hook when a bucket is complete. The tensors themselves and the reduction launches stay
// with the caller; this object only answers "which bucket, at which offset, is it complete now".
// Counterpart in the reference: DDPReducer in src/bindings/python/Distributed.cpp:33-247 and
// _compute_bucket_assignment_by_size (tensorplay/distributed/distributed_core.py:3173).
#include <cstdint>
#include <mutex>
#include <algorithm>
#include <vector>

namespace {

struct Reducer {
  std::vector<int> bucket_of;         // per parameter
  std::vector<long long> offset_of;   // element offset inside the bucket (8-element aligned)
  std::vector<long long> bucket_numel;
  std::vector<int> bucket_size;       // parameters per bucket
  std::vector<int> pending;           // per bucket, this iteration
  std::vector<uint8_t> marked;        // per parameter, this iteration
  std::vector<std::vector<int>> members;
  std::mutex mu;                      // hooks may fire from autograd worker threads
};

}  // namespace

extern "C" {

// numels / elem_bytes: per parameter in model order. align: the bucket length is rounded up to a
// multiple of it (the collective kernels want world * 128 elements).
void* tpb_reducer_create(const long long* numels, const int* elem_bytes, int n, long long cap_bytes,
                         long long align) {
  auto* r = new Reducer();
  r->bucket_of.assign(n, -1);
  r->offset_of.assign(n, 0);
  r->marked.assign(n, 0);
  long long bytes = 0, off = 0;
  int cur_elem = 0;
  auto close = [&]() {
    if (r->members.empty() || r->members.back().empty()) return;
    long long padded = align > 0 ? (off + align - 1) / align * align : off;
    r->bucket_numel.push_back(padded);
    r->bucket_size.push_back((int)r->members.back().size());
  };
  for (int i = n - 1; i >= 0; --i) {
    const long long nb = numels[i] * elem_bytes[i];
    const bool start = r->members.empty() || r->members.back().empty();
    if (!start && (bytes + nb > cap_bytes || elem_bytes[i] != cur_elem)) {
      close();
      r->members.emplace_back();
      bytes = 0;
      off = 0;
    }
    if (r->members.empty()) r->members.emplace_back();
    cur_elem = elem_bytes[i];
    r->bucket_of[i] = (int)r->members.size() - 1;
    r->offset_of[i] = off;
    r->members.back().push_back(i);
    off += (numels[i] + 7) / 8 * 8;
    bytes += nb;
  }
  close();
  r->pending = r->bucket_size;
  return r;
}

void tpb_reducer_destroy(void* h) { delete static_cast<Reducer*>(h); }
int tpb_reducer_num_buckets(void* h) { return (int)static_cast<Reducer*>(h)->bucket_numel.size(); }
int tpb_reducer_bucket_of(void* h, int param) { return static_cast<Reducer*>(h)->bucket_of[param]; }
long long tpb_reducer_offset_of(void* h, int param) { return static_cast<Reducer*>(h)->offset_of[param]; }
long long tpb_reducer_bucket_numel(void* h, int bucket) { return static_cast<Reducer*>(h)->bucket_numel[bucket]; }
int tpb_reducer_bucket_size(void* h, int bucket) { return static_cast<Reducer*>(h)->bucket_size[bucket]; }
// out: parameter indices of the bucket in gradient-arrival order (bucket_size entries).
void tpb_reducer_bucket_members(void* h, int bucket, int* out) {
  const auto& m = static_cast<Reducer*>(h)->members[bucket];
  for (size_t i = 0; i < m.size(); ++i) out[i] = m[i];
}

// Returns the bucket index when this gradient completes its bucket, -1 when the bucket still
// waits for others, -2 when the parameter was already marked in this iteration.
int tpb_reducer_mark_ready(void* h, int param) {
  auto* r = static_cast<Reducer*>(h);
  std::lock_guard<std::mutex> lock(r->mu);
  if (r->marked[param]) return -2;
  r->marked[param] = 1;
  const int b = r->bucket_of[param];
  return --r->pending[b] == 0 ? b : -1;
}

int tpb_reducer_pending(void* h, int bucket) {
  auto* r = static_cast<Reducer*>(h);
  std::lock_guard<std::mutex> lock(r->mu);
  return r->pending[bucket];
}

// After a bucket's reduction was launched: it waits for all of its parameters again.
void tpb_reducer_rearm(void* h, int bucket) {
  auto* r = static_cast<Reducer*>(h);
  std::lock_guard<std::mutex> lock(r->mu);
  r->pending[bucket] = r->bucket_size[bucket];
  for (int p : r->members[bucket]) r->marked[p] = 0;
}

// Start of an iteration: every bucket waits for all of its parameters again.
void tpb_reducer_reset(void* h) {
  auto* r = static_cast<Reducer*>(h);
  std::lock_guard<std::mutex> lock(r->mu);
  r->pending = r->bucket_size;
  std::fill(r->marked.begin(), r->marked.end(), 0);
}

}  // extern "C"
