// Native token-file data loader: worker threads turn a memory-mapped file of token ids into
// ready batches (tokens and next-token targets, int64) in caller-owned host buffers, typically
// pinned, a few batches ahead of the training loop.
//
//   sample i      = tokens [i * seq_len, (i + 1) * seq_len] of the file (seq_len + 1 ids: inputs and
//                   targets overlap by construction), for i in [0, (n_tokens - 1) / seq_len)
//   epoch order   = Fisher-Yates permutation of the samples seeded by (seed, epoch), the same on
//                   every rank; rank r of w takes positions r, r + w, ... (tail dropped), so ranks
//                   see disjoint samples and every rank the same number of batches
//   batch b       -> slot b % depth; slots are handed to the consumer strictly in order
//
// Plain C ABI (ctypes), no torch dependency; the reference's loader builds shared-memory batches in
// Python worker processes (tensorplay/utils/data), here the hot loop is a thread pool in C++.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

namespace {

struct Loader {
  const uint8_t* data = nullptr;
  size_t file_bytes = 0;
  int fd = -1;
  int elem = 2;  // bytes per token id in the file
  long long n_tokens = 0, n_samples = 0, per_rank = 0, batches_per_epoch = 0;
  int seq_len = 0, batch = 0, rank = 0, world = 1, depth = 0, shuffle = 1;
  uint64_t seed = 0;
  std::vector<int64_t*> tok_slots, tgt_slots;
  // slot state: 0 free, 1 being filled, 2 ready; guarded by mu
  std::vector<int> state;
  std::vector<long long> slot_batch;
  std::mutex mu;
  std::condition_variable cv_free, cv_ready;
  long long next_fill = 0;     // next global batch number a worker will take
  long long next_consume = 0;  // next global batch number the consumer gets
  bool stop = false;
  std::vector<std::thread> workers;
  // permutation cache (one epoch at a time per worker would thrash; two epochs are kept)
  std::mutex perm_mu;
  long long perm_epoch[2] = {-1, -1};
  std::vector<uint32_t> perm[2];
};

inline uint64_t splitmix(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

const std::vector<uint32_t>& epoch_perm(Loader* L, long long epoch) {
  std::lock_guard<std::mutex> g(L->perm_mu);
  const int k = (int)(epoch & 1);
  if (L->perm_epoch[k] != epoch) {
    std::vector<uint32_t>& p = L->perm[k];
    p.resize((size_t)L->n_samples);
    for (long long i = 0; i < L->n_samples; ++i) p[(size_t)i] = (uint32_t)i;
    if (L->shuffle) {
      uint64_t s = L->seed * 0x9E3779B97F4A7C15ull + (uint64_t)epoch + 1;
      for (long long i = L->n_samples - 1; i > 0; --i) {
        const uint64_t j = splitmix(s) % (uint64_t)(i + 1);
        std::swap(p[(size_t)i], p[(size_t)j]);
      }
    }
    L->perm_epoch[k] = epoch;
  }
  return L->perm[k];
}

inline int64_t token_at(const Loader* L, long long i) {
  if (L->elem == 2) {
    uint16_t v;
    memcpy(&v, L->data + (size_t)i * 2, 2);
    return (int64_t)v;
  }
  int32_t v;
  memcpy(&v, L->data + (size_t)i * 4, 4);
  return (int64_t)v;
}

void fill_batch(Loader* L, long long b, int slot) {
  const long long epoch = b / L->batches_per_epoch, in_epoch = b % L->batches_per_epoch;
  // copy of the sample ids first: the cached permutation may be replaced by another worker
  std::vector<uint32_t> ids((size_t)L->batch);
  {
    const std::vector<uint32_t>& p = epoch_perm(L, epoch);
    for (int r = 0; r < L->batch; ++r) {
      const long long pos = (in_epoch * L->batch + r) * L->world + L->rank;
      ids[(size_t)r] = p[(size_t)pos];
    }
  }
  int64_t* tok = L->tok_slots[(size_t)slot];
  int64_t* tgt = L->tgt_slots[(size_t)slot];
  for (int r = 0; r < L->batch; ++r) {
    const long long base = (long long)ids[(size_t)r] * L->seq_len;
    int64_t prev = token_at(L, base);
    for (int t = 0; t < L->seq_len; ++t) {
      const int64_t nxt = token_at(L, base + t + 1);
      tok[(size_t)r * L->seq_len + t] = prev;
      tgt[(size_t)r * L->seq_len + t] = nxt;
      prev = nxt;
    }
  }
}

void worker_main(Loader* L) {
  for (;;) {
    long long b;
    int slot;
    {
      std::unique_lock<std::mutex> lk(L->mu);
      for (;;) {
        if (L->stop) return;
        b = L->next_fill;
        slot = (int)(b % L->depth);
        // a slot is taken only for the batch that is next in line for it (keeps hand-out order)
        if (L->state[(size_t)slot] == 0 && b < L->next_consume + L->depth) break;
        L->cv_free.wait(lk);
      }
      L->state[(size_t)slot] = 1;
      L->slot_batch[(size_t)slot] = b;
      L->next_fill = b + 1;
    }
    fill_batch(L, b, slot);
    {
      std::lock_guard<std::mutex> g(L->mu);
      L->state[(size_t)slot] = 2;
    }
    L->cv_ready.notify_all();
  }
}

}  // namespace

extern "C" {

// tok_slots / tgt_slots: `depth` pointers each to int64 [batch, seq_len] host buffers owned by the
// caller. elem_bytes: 2 (uint16 ids) or 4 (int32). Returns a handle, or null with *err set.
void* tpb_loader_open(const char* path, int elem_bytes, int seq_len, int batch, int rank, int world,
                      unsigned long long seed, int shuffle, int n_workers, int depth, void** tok_slots,
                      void** tgt_slots, int* err) {
  *err = 0;
  if ((elem_bytes != 2 && elem_bytes != 4) || seq_len <= 0 || batch <= 0 || world <= 0 || rank < 0 ||
      rank >= world || n_workers <= 0 || depth < 2) {
    *err = -1;
    return nullptr;
  }
  Loader* L = new Loader();
  L->fd = open(path, O_RDONLY);
  if (L->fd < 0) {
    *err = -2;
    delete L;
    return nullptr;
  }
  struct stat st;
  if (fstat(L->fd, &st) != 0 || st.st_size < (off_t)((seq_len + 1) * elem_bytes)) {
    *err = -3;
    close(L->fd);
    delete L;
    return nullptr;
  }
  L->file_bytes = (size_t)st.st_size;
  void* m = mmap(nullptr, L->file_bytes, PROT_READ, MAP_PRIVATE, L->fd, 0);
  if (m == MAP_FAILED) {
    *err = -4;
    close(L->fd);
    delete L;
    return nullptr;
  }
  madvise(m, L->file_bytes, MADV_RANDOM);
  L->data = static_cast<const uint8_t*>(m);
  L->elem = elem_bytes;
  L->n_tokens = (long long)(L->file_bytes / (size_t)elem_bytes);
  L->n_samples = (L->n_tokens - 1) / seq_len;
  L->per_rank = L->n_samples / world;
  L->batches_per_epoch = L->per_rank / batch;
  if (L->batches_per_epoch <= 0 || L->n_samples > 0xFFFFFFFFll) {
    *err = -5;
    munmap(m, L->file_bytes);
    close(L->fd);
    delete L;
    return nullptr;
  }
  L->seq_len = seq_len;
  L->batch = batch;
  L->rank = rank;
  L->world = world;
  L->seed = seed;
  L->shuffle = shuffle;
  L->depth = depth;
  for (int i = 0; i < depth; ++i) {
    L->tok_slots.push_back(static_cast<int64_t*>(tok_slots[i]));
    L->tgt_slots.push_back(static_cast<int64_t*>(tgt_slots[i]));
  }
  L->state.assign((size_t)depth, 0);
  L->slot_batch.assign((size_t)depth, -1);
  for (int i = 0; i < n_workers; ++i) L->workers.emplace_back(worker_main, L);
  return L;
}

long long tpb_loader_batches_per_epoch(void* h) { return static_cast<Loader*>(h)->batches_per_epoch; }
long long tpb_loader_num_samples(void* h) { return static_cast<Loader*>(h)->n_samples; }

// Blocks until the next batch (in order) is ready; returns its slot and writes its global number.
int tpb_loader_next(void* h, long long* batch_number) {
  Loader* L = static_cast<Loader*>(h);
  std::unique_lock<std::mutex> lk(L->mu);
  const long long b = L->next_consume;
  const int slot = (int)(b % L->depth);
  L->cv_ready.wait(lk, [&] { return L->stop || (L->state[(size_t)slot] == 2 && L->slot_batch[(size_t)slot] == b); });
  if (L->stop) return -1;
  L->next_consume = b + 1;
  *batch_number = b;
  return slot;
}

// The consumer is done with the slot's buffers (e.g. its host-to-device copy has completed).
void tpb_loader_release(void* h, int slot) {
  Loader* L = static_cast<Loader*>(h);
  {
    std::lock_guard<std::mutex> g(L->mu);
    if (slot >= 0 && slot < L->depth) L->state[(size_t)slot] = 0;
  }
  L->cv_free.notify_all();
}

void tpb_loader_close(void* h) {
  Loader* L = static_cast<Loader*>(h);
  {
    std::lock_guard<std::mutex> g(L->mu);
    L->stop = true;
  }
  L->cv_free.notify_all();
  L->cv_ready.notify_all();
  for (auto& t : L->workers) t.join();
  munmap(const_cast<uint8_t*>(L->data), L->file_bytes);
  close(L->fd);
  delete L;
}

}  // extern "C"
