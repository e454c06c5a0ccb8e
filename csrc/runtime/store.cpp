// TCP key-value store for rendezvous: a server thread pool on one rank, blocking clients on all
// ranks. Operations: set, get (blocks until the key exists or the deadline passes), add
// (atomic counter), compare-and-set, wait, delete, check, key count.
//
// Wire format (little endian): request = u8 op | u32 nkeys | { u32 len | bytes }* | u64 vlen |
// value | u64 vlen2 | value2 | i64 arg ; reply = i32 status | u64 len | bytes.
// Plays the role of the reference's C++ TCPStore (src/distributed/store/TCPStore.cpp, 844 lines;
// Python surface tensorplay/distributed/_store.py:27-160).
#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr uint64_t kMaxValue = 256ull << 20;  // largest value a request may carry (bytes)

enum Op : uint8_t { SET = 1, GET = 2, ADD = 3, CAS = 4, WAIT = 5, DEL = 6, CHECK = 7, NKEYS = 8, PING = 9 };
enum Status : int32_t { OK = 0, TIMEOUT = 1, MISSING = 2, ERR = 3 };

bool send_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w <= 0) {
      if (w < 0 && errno == EINTR) continue;
      return false;
    }
    p += w;
    n -= (size_t)w;
  }
  return true;
}
bool recv_all(int fd, void* buf, size_t n) {
  char* p = static_cast<char*>(buf);
  while (n) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r <= 0) {
      if (r < 0 && errno == EINTR) continue;
      return false;
    }
    p += r;
    n -= (size_t)r;
  }
  return true;
}

struct Server {
  int listen_fd = -1;
  int port = 0;
  std::atomic<bool> stop{false};
  std::thread accept_thread;
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::string, std::string> kv;
  std::vector<std::thread> workers;
  std::vector<int> fds;

  void reply(int fd, int32_t st, const std::string& val) {
    uint64_t n = val.size();
    send_all(fd, &st, 4);
    send_all(fd, &n, 8);
    if (n) send_all(fd, val.data(), n);
  }

  void serve(int fd) {
    while (!stop.load()) {
      uint8_t op;
      uint32_t nkeys;
      if (!recv_all(fd, &op, 1) || !recv_all(fd, &nkeys, 4) || nkeys > 4096) break;
      std::vector<std::string> keys(nkeys);
      bool bad = false;
      for (auto& k : keys) {
        uint32_t len;
        if (!recv_all(fd, &len, 4) || len > (1u << 20)) { bad = true; break; }
        k.resize(len);
        if (len && !recv_all(fd, &k[0], len)) { bad = true; break; }
      }
      if (bad) break;
      std::string v1, v2;
      uint64_t l1, l2;
      int64_t arg;
      // Values are rendezvous blobs (addresses, handles, small pickles): a peer that announces more
      // than kMaxValue is not one of ours, and the buffer is not grown for it.
      if (!recv_all(fd, &l1, 8) || l1 > kMaxValue) break;
      v1.resize(l1);
      if (l1 && !recv_all(fd, &v1[0], l1)) break;
      if (!recv_all(fd, &l2, 8) || l2 > kMaxValue) break;
      v2.resize(l2);
      if (l2 && !recv_all(fd, &v2[0], l2)) break;
      if (!recv_all(fd, &arg, 8)) break;
      auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(arg < 0 ? 0 : arg);
      // key count must fit the operation: one key for the single-key ops, at least one for the
      // multi-key ones, none needed for NKEYS / PING
      const bool single = op == SET || op == GET || op == ADD || op == CAS || op == DEL;
      const bool multi = op == WAIT || op == CHECK;
      if ((single && nkeys != 1) || (multi && nkeys < 1)) { reply(fd, ERR, ""); continue; }
      switch (op) {
        case SET: {
          { std::lock_guard<std::mutex> g(mu); kv[keys[0]] = v1; }
          cv.notify_all();
          reply(fd, OK, "");
        } break;
        case GET: case WAIT: {
          std::unique_lock<std::mutex> g(mu);
          auto have_all = [&] {
            for (auto& k : keys) if (!kv.count(k)) return false;
            return true;
          };
          bool ok = true;
          while (!have_all() && !stop.load()) {
            if (arg < 0) { cv.wait_for(g, std::chrono::milliseconds(200)); continue; }
            if (cv.wait_until(g, deadline) == std::cv_status::timeout && !have_all()) { ok = false; break; }
          }
          if (!ok || stop.load()) { g.unlock(); reply(fd, TIMEOUT, ""); break; }
          std::string out = op == GET ? kv[keys[0]] : std::string();
          g.unlock();
          reply(fd, OK, out);
        } break;
        case ADD: {
          int64_t cur = 0;
          {
            std::lock_guard<std::mutex> g(mu);
            auto it = kv.find(keys[0]);
            if (it != kv.end()) cur = strtoll(it->second.c_str(), nullptr, 10);
            cur += arg;
            kv[keys[0]] = std::to_string(cur);
          }
          cv.notify_all();
          reply(fd, OK, std::to_string(cur));
        } break;
        case CAS: {
          std::string out;
          {
            std::lock_guard<std::mutex> g(mu);
            auto it = kv.find(keys[0]);
            if (it == kv.end()) {
              if (v1.empty()) { kv[keys[0]] = v2; out = v2; }
              else out = v1;  // absent and an expectation was given: report the expectation back
            } else if (it->second == v1) { it->second = v2; out = v2; }
            else out = it->second;
          }
          cv.notify_all();
          reply(fd, OK, out);
        } break;
        case DEL: {
          size_t n;
          { std::lock_guard<std::mutex> g(mu); n = kv.erase(keys[0]); }
          reply(fd, n ? OK : MISSING, "");
        } break;
        case CHECK: {
          bool all = true;
          { std::lock_guard<std::mutex> g(mu); for (auto& k : keys) if (!kv.count(k)) all = false; }
          reply(fd, all ? OK : MISSING, "");
        } break;
        case NKEYS: {
          size_t n;
          { std::lock_guard<std::mutex> g(mu); n = kv.size(); }
          reply(fd, OK, std::to_string(n));
        } break;
        case PING: reply(fd, OK, ""); break;
        default: reply(fd, ERR, ""); break;
      }
    }
    ::close(fd);
  }

  void accept_loop() {
    while (!stop.load()) {
      pollfd p{listen_fd, POLLIN, 0};
      int r = ::poll(&p, 1, 200);
      if (r <= 0) continue;
      int fd = ::accept(listen_fd, nullptr, nullptr);
      if (fd < 0) continue;
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::lock_guard<std::mutex> g(mu);
      fds.push_back(fd);
      workers.emplace_back([this, fd] { serve(fd); });
    }
  }
};

struct Client {
  int fd = -1;
  std::mutex mu;
};

int32_t request(Client* c, uint8_t op, const std::vector<std::string>& keys, const std::string& v1,
                const std::string& v2, int64_t arg, std::string* out) {
  std::lock_guard<std::mutex> g(c->mu);
  std::string msg;
  msg.push_back((char)op);
  uint32_t nk = (uint32_t)keys.size();
  msg.append(reinterpret_cast<const char*>(&nk), 4);
  for (auto& k : keys) {
    uint32_t len = (uint32_t)k.size();
    msg.append(reinterpret_cast<const char*>(&len), 4);
    msg.append(k);
  }
  uint64_t l1 = v1.size(), l2 = v2.size();
  msg.append(reinterpret_cast<const char*>(&l1), 8);
  msg.append(v1);
  msg.append(reinterpret_cast<const char*>(&l2), 8);
  msg.append(v2);
  msg.append(reinterpret_cast<const char*>(&arg), 8);
  if (!send_all(c->fd, msg.data(), msg.size())) return ERR;
  int32_t st;
  uint64_t n;
  if (!recv_all(c->fd, &st, 4) || !recv_all(c->fd, &n, 8)) return ERR;
  std::string val(n, '\0');
  if (n && !recv_all(c->fd, &val[0], n)) return ERR;
  if (out) *out = std::move(val);
  return st;
}

}  // namespace

extern "C" {

void* tpb_store_server_start(int port, int* port_out) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return nullptr;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  // TPB_STORE_BIND_ADDR narrows the listening interface (the single-node launcher sets loopback)
  if (const char* bind_to = getenv("TPB_STORE_BIND_ADDR")) {
    in_addr a{};
    if (*bind_to && inet_pton(AF_INET, bind_to, &a) == 1) addr.sin_addr = a;
  }
  addr.sin_port = htons((uint16_t)port);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, 512) != 0) {
    ::close(fd);
    return nullptr;
  }
  socklen_t len = sizeof(addr);
  getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  auto* s = new Server();
  s->listen_fd = fd;
  s->port = ntohs(addr.sin_port);
  if (port_out) *port_out = s->port;
  s->accept_thread = std::thread([s] { s->accept_loop(); });
  return s;
}

void tpb_store_server_stop(void* h) {
  auto* s = static_cast<Server*>(h);
  if (!s) return;
  s->stop.store(true);
  s->cv.notify_all();
  if (s->accept_thread.joinable()) s->accept_thread.join();
  {
    std::lock_guard<std::mutex> g(s->mu);
    for (int fd : s->fds) ::shutdown(fd, SHUT_RDWR);
  }
  for (auto& t : s->workers) if (t.joinable()) t.join();
  ::close(s->listen_fd);
  delete s;
}

void* tpb_store_connect(const char* host, int port, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  std::string ps = std::to_string(port);
  while (true) {
    if (getaddrinfo(host, ps.c_str(), &hints, &res) == 0 && res) {
      int fd = ::socket(res->ai_family, res->ai_socktype, res->ai_protocol);
      if (fd >= 0) {
        if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
          int one = 1;
          setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
          freeaddrinfo(res);
          auto* c = new Client();
          c->fd = fd;
          return c;
        }
        ::close(fd);
      }
      freeaddrinfo(res);
      res = nullptr;
    }
    if (std::chrono::steady_clock::now() > deadline) return nullptr;
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
  }
}

void tpb_store_close(void* h) {
  auto* c = static_cast<Client*>(h);
  if (!c) return;
  ::close(c->fd);
  delete c;
}

int tpb_store_set(void* h, const char* key, int klen, const char* val, long long vlen) {
  return request(static_cast<Client*>(h), SET, {std::string(key, klen)}, std::string(val, (size_t)vlen), "", 0, nullptr);
}

// *out is malloc'ed (free with tpb_free). timeout_ms < 0 waits forever.
int tpb_store_get(void* h, const char* key, int klen, long long timeout_ms, char** out, long long* out_len) {
  std::string v;
  int32_t st = request(static_cast<Client*>(h), GET, {std::string(key, klen)}, "", "", timeout_ms, &v);
  if (st == OK) {
    *out = static_cast<char*>(malloc(v.size() ? v.size() : 1));
    memcpy(*out, v.data(), v.size());
    *out_len = (long long)v.size();
  }
  return st;
}

int tpb_store_add(void* h, const char* key, int klen, long long amount, long long* result) {
  std::string v;
  int32_t st = request(static_cast<Client*>(h), ADD, {std::string(key, klen)}, "", "", amount, &v);
  if (st == OK && result) *result = strtoll(v.c_str(), nullptr, 10);
  return st;
}

int tpb_store_cas(void* h, const char* key, int klen, const char* expected, long long elen,
                  const char* desired, long long dlen, char** out, long long* out_len) {
  std::string v;
  int32_t st = request(static_cast<Client*>(h), CAS, {std::string(key, klen)},
                       std::string(expected, (size_t)elen), std::string(desired, (size_t)dlen), 0, &v);
  if (st == OK) {
    *out = static_cast<char*>(malloc(v.size() ? v.size() : 1));
    memcpy(*out, v.data(), v.size());
    *out_len = (long long)v.size();
  }
  return st;
}

// keys: concatenated, lens[i] bytes each.
int tpb_store_wait(void* h, const char* keys, const int* lens, int nkeys, long long timeout_ms) {
  std::vector<std::string> ks;
  const char* p = keys;
  for (int i = 0; i < nkeys; ++i) { ks.emplace_back(p, lens[i]); p += lens[i]; }
  return request(static_cast<Client*>(h), WAIT, ks, "", "", timeout_ms, nullptr);
}
int tpb_store_check(void* h, const char* keys, const int* lens, int nkeys) {
  std::vector<std::string> ks;
  const char* p = keys;
  for (int i = 0; i < nkeys; ++i) { ks.emplace_back(p, lens[i]); p += lens[i]; }
  return request(static_cast<Client*>(h), CHECK, ks, "", "", 0, nullptr);
}
int tpb_store_delete(void* h, const char* key, int klen) {
  return request(static_cast<Client*>(h), DEL, {std::string(key, klen)}, "", "", 0, nullptr);
}
long long tpb_store_num_keys(void* h) {
  std::string v;
  if (request(static_cast<Client*>(h), NKEYS, {}, "", "", 0, &v) != OK) return -1;
  return strtoll(v.c_str(), nullptr, 10);
}
void tpb_free(void* p) { free(p); }

}  // extern "C"
