// Host collectives for CPU ranks.
//  * HostCollective    — ranks are threads of one process: per-rank slots + a barrier; reductions
//                        run in fixed rank order, so results are bit-reproducible
//                        (crates/model/src/collective.rs:35-143).
//  * NetworkCollective — ranks are processes on a TCP star: rank 0 listens, gathers, reduces in
//                        rank order and scatters; frames are a little-endian u32 element count
//                        followed by f32 payload, at most 2^28 elements; a short read / closed peer
//                        is reported with the peer's rank, never ignored
//                        (crates/model/src/netcollective.rs:27-237).
// Ops (all on float32 buffers): all_reduce(sum), all_gather, reduce_scatter(sum), broadcast(root).
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint32_t MAX_MSG_ELEMS = 1u << 28;

class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  // returns false when the barrier was broken (a rank left / timed out)
  bool wait(double timeout_s) {
    std::unique_lock<std::mutex> lk(m_);
    if (broken_) return false;
    const uint64_t gen = gen_;
    if (++count_ == n_) {
      count_ = 0;
      ++gen_;
      cv_.notify_all();
      return true;
    }
    const bool ok = cv_.wait_for(lk, std::chrono::duration<double>(timeout_s),
                                 [&] { return gen_ != gen || broken_; });
    if (!ok || broken_) {
      broken_ = true;
      cv_.notify_all();
      return false;
    }
    return true;
  }
  void abort() {
    std::lock_guard<std::mutex> lk(m_);
    broken_ = true;
    cv_.notify_all();
  }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  int n_, count_ = 0;
  uint64_t gen_ = 0;
  bool broken_ = false;
};

struct HostCollective {
  int world;
  Barrier bar;
  std::vector<const float*> slots;
  std::vector<int64_t> lens;
  double timeout_s;
  HostCollective(int w, double t) : world(w), bar(w), slots(w, nullptr), lens(w, 0), timeout_s(t) {}
};

// ---------------------------------------------------------------- TCP helpers
bool send_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k <= 0) {
      if (k < 0 && errno == EINTR) continue;
      return false;
    }
    p += k;
    n -= k;
  }
  return true;
}
bool recv_all(int fd, void* buf, size_t n) {
  char* p = static_cast<char*>(buf);
  while (n) {
    ssize_t k = ::recv(fd, p, n, 0);
    if (k <= 0) {
      if (k < 0 && errno == EINTR) continue;
      return false;
    }
    p += k;
    n -= k;
  }
  return true;
}
bool send_frame(int fd, const float* data, uint32_t n) {
  return send_all(fd, &n, 4) && send_all(fd, data, static_cast<size_t>(n) * 4);
}
bool recv_frame(int fd, float* data, uint32_t expect) {
  uint32_t n = 0;
  if (!recv_all(fd, &n, 4) || n != expect || n > MAX_MSG_ELEMS) return false;
  return recv_all(fd, data, static_cast<size_t>(n) * 4);
}

struct NetCollective {
  int rank = 0, world = 1;
  int listen_fd = -1;
  std::vector<int> peers;  // rank 0: fd per rank (index 0 unused); others: peers[0] = coordinator
  int failed_peer = -1;
  std::vector<float> tmp;
};

}  // namespace

// ---------------------------------------------------------------- HostCollective ABI
BBH_API void* bbh_hc_new(int world, double timeout_s) {
  return world >= 1 ? new HostCollective(world, timeout_s > 0 ? timeout_s : 60.0) : nullptr;
}
BBH_API void bbh_hc_free(void* h) { delete static_cast<HostCollective*>(h); }
BBH_API void bbh_hc_abort(void* h) { static_cast<HostCollective*>(h)->bar.abort(); }

// All ops return 0, or -1 when a peer never arrived within the timeout (the barrier is then broken
// for everyone, so no rank waits forever on a rank that raised).
BBH_API int bbh_hc_all_reduce(void* h, int rank, float* data, int64_t n) {
  auto* c = static_cast<HostCollective*>(h);
  c->slots[rank] = data;
  c->lens[rank] = n;
  if (!c->bar.wait(c->timeout_s)) return -1;
  for (int r = 0; r < c->world; ++r)
    if (c->lens[r] != n) return -2;
  // In place, no staging copy: rank r owns the r-th slice of EVERY rank's buffer, adds the ranks'
  // values in rank order (so each element gets the same bits whichever rank computes it) and writes
  // the sum back into all of them.  No other rank touches that slice between the two barriers.
  const int64_t chunk = ((n + c->world - 1) / c->world + 15) & ~int64_t(15);
  const int64_t a = std::min<int64_t>(n, rank * chunk), b = std::min<int64_t>(n, a + chunk);
  if (c->world == 2) {
    float* p0 = const_cast<float*>(c->slots[0]);
    float* p1 = const_cast<float*>(c->slots[1]);
    for (int64_t i = a; i < b; ++i) {
      const float s = p0[i] + p1[i];
      p0[i] = s;
      p1[i] = s;
    }
  } else {
    for (int64_t i = a; i < b; ++i) {
      float s = c->slots[0][i];
      for (int r = 1; r < c->world; ++r) s += c->slots[r][i];
      for (int r = 0; r < c->world; ++r) const_cast<float*>(c->slots[r])[i] = s;
    }
  }
  if (!c->bar.wait(c->timeout_s)) return -1;  // every slice of every buffer holds the sum
  return 0;
}
BBH_API int bbh_hc_all_gather(void* h, int rank, const float* data, int64_t n, float* out) {
  auto* c = static_cast<HostCollective*>(h);
  c->slots[rank] = data;
  c->lens[rank] = n;
  if (!c->bar.wait(c->timeout_s)) return -1;
  for (int r = 0; r < c->world; ++r) {
    if (c->lens[r] != n) return -2;
    std::memcpy(out + r * n, c->slots[r], static_cast<size_t>(n) * 4);
  }
  if (!c->bar.wait(c->timeout_s)) return -1;
  return 0;
}
// data: world*n elements; out: this rank's n-element shard of the sum
BBH_API int bbh_hc_reduce_scatter(void* h, int rank, const float* data, int64_t n, float* out) {
  auto* c = static_cast<HostCollective*>(h);
  c->slots[rank] = data;
  c->lens[rank] = n;
  if (!c->bar.wait(c->timeout_s)) return -1;
  for (int64_t i = 0; i < n; ++i) out[i] = 0.f;
  for (int r = 0; r < c->world; ++r) {
    if (c->lens[r] != n) return -2;
    const float* s = c->slots[r] + rank * n;
    for (int64_t i = 0; i < n; ++i) out[i] += s[i];
  }
  if (!c->bar.wait(c->timeout_s)) return -1;
  return 0;
}
BBH_API int bbh_hc_broadcast(void* h, int rank, float* data, int64_t n, int root) {
  auto* c = static_cast<HostCollective*>(h);
  c->slots[rank] = data;
  c->lens[rank] = n;
  if (!c->bar.wait(c->timeout_s)) return -1;
  if (rank != root) std::memcpy(data, c->slots[root], static_cast<size_t>(n) * 4);
  if (!c->bar.wait(c->timeout_s)) return -1;
  return 0;
}
BBH_API int bbh_hc_barrier(void* h) {
  auto* c = static_cast<HostCollective*>(h);
  return c->bar.wait(c->timeout_s) ? 0 : -1;
}

// ---------------------------------------------------------------- NetworkCollective ABI
// Rank 0: listen on 127.0.0.1:port (port 0 picks one; *port_out gets it) — call bbh_nc_accept next.
BBH_API void* bbh_nc_listen(int world, int port, int* port_out) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return nullptr;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  a.sin_port = htons(static_cast<uint16_t>(port));
  if (bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || listen(fd, world) != 0) {
    ::close(fd);
    return nullptr;
  }
  socklen_t len = sizeof(a);
  getsockname(fd, reinterpret_cast<sockaddr*>(&a), &len);
  if (port_out) *port_out = ntohs(a.sin_port);
  auto* c = new NetCollective();
  c->rank = 0;
  c->world = world;
  c->listen_fd = fd;
  c->peers.assign(world, -1);
  return c;
}
// Accept world-1 workers; each announces its rank first.  Duplicate / out-of-range ranks fail.
BBH_API int bbh_nc_accept(void* h) {
  auto* c = static_cast<NetCollective*>(h);
  for (int i = 1; i < c->world; ++i) {
    int fd = ::accept(c->listen_fd, nullptr, nullptr);
    if (fd < 0) return -1;
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    uint32_t r = 0;
    if (!recv_all(fd, &r, 4) || r == 0 || r >= static_cast<uint32_t>(c->world) || c->peers[r] != -1) {
      ::close(fd);
      return -2;
    }
    c->peers[r] = fd;
  }
  return 0;
}
BBH_API void* bbh_nc_connect(int rank, int world, int port) {
  if (rank <= 0 || rank >= world) return nullptr;
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return nullptr;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  a.sin_port = htons(static_cast<uint16_t>(port));
  bool ok = false;
  for (int attempt = 0; attempt < 200 && !ok; ++attempt) {
    if (::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) ok = true;
    else usleep(25000);
  }
  if (!ok) {
    ::close(fd);
    return nullptr;
  }
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  uint32_t r = static_cast<uint32_t>(rank);
  if (!send_all(fd, &r, 4)) {
    ::close(fd);
    return nullptr;
  }
  auto* c = new NetCollective();
  c->rank = rank;
  c->world = world;
  c->peers.assign(1, fd);
  return c;
}
BBH_API void bbh_nc_free(void* h) {
  auto* c = static_cast<NetCollective*>(h);
  if (!c) return;
  for (int fd : c->peers)
    if (fd >= 0) ::close(fd);
  if (c->listen_fd >= 0) ::close(c->listen_fd);
  delete c;
}
BBH_API int bbh_nc_failed_peer(void* h) { return static_cast<NetCollective*>(h)->failed_peer; }

// Returns 0, -1 wire failure (see bbh_nc_failed_peer), -3 message too large.
BBH_API int bbh_nc_all_reduce(void* h, float* data, int64_t n) {
  auto* c = static_cast<NetCollective*>(h);
  if (n < 0 || static_cast<uint64_t>(n) > MAX_MSG_ELEMS) return -3;
  const uint32_t un = static_cast<uint32_t>(n);
  if (c->rank == 0) {
    c->tmp.resize(static_cast<size_t>(n));
    for (int r = 1; r < c->world; ++r) {
      if (!recv_frame(c->peers[r], c->tmp.data(), un)) {
        c->failed_peer = r;
        return -1;
      }
      for (int64_t i = 0; i < n; ++i) data[i] += c->tmp[i];
    }
    for (int r = 1; r < c->world; ++r)
      if (!send_frame(c->peers[r], data, un)) {
        c->failed_peer = r;
        return -1;
      }
    return 0;
  }
  if (!send_frame(c->peers[0], data, un) || !recv_frame(c->peers[0], data, un)) {
    c->failed_peer = 0;
    return -1;
  }
  return 0;
}
BBH_API int bbh_nc_broadcast(void* h, float* data, int64_t n, int root) {
  auto* c = static_cast<NetCollective*>(h);
  if (n < 0 || static_cast<uint64_t>(n) > MAX_MSG_ELEMS) return -3;
  const uint32_t un = static_cast<uint32_t>(n);
  if (c->rank == 0) {
    if (root != 0 && !recv_frame(c->peers[root], data, un)) {
      c->failed_peer = root;
      return -1;
    }
    for (int r = 1; r < c->world; ++r) {
      if (r == root) continue;
      if (!send_frame(c->peers[r], data, un)) {
        c->failed_peer = r;
        return -1;
      }
    }
    return 0;
  }
  const bool ok = c->rank == root ? send_frame(c->peers[0], data, un) : recv_frame(c->peers[0], data, un);
  if (!ok) {
    c->failed_peer = 0;
    return -1;
  }
  return 0;
}
// out: world*n on every rank
BBH_API int bbh_nc_all_gather(void* h, const float* data, int64_t n, float* out) {
  auto* c = static_cast<NetCollective*>(h);
  if (n < 0 || static_cast<uint64_t>(n) * c->world > MAX_MSG_ELEMS) return -3;
  const uint32_t un = static_cast<uint32_t>(n);
  if (c->rank == 0) {
    std::memcpy(out, data, static_cast<size_t>(n) * 4);
    for (int r = 1; r < c->world; ++r)
      if (!recv_frame(c->peers[r], out + r * n, un)) {
        c->failed_peer = r;
        return -1;
      }
    for (int r = 1; r < c->world; ++r)
      if (!send_frame(c->peers[r], out, un * c->world)) {
        c->failed_peer = r;
        return -1;
      }
    return 0;
  }
  if (!send_frame(c->peers[0], data, un) || !recv_frame(c->peers[0], out, un * c->world)) {
    c->failed_peer = 0;
    return -1;
  }
  return 0;
}
