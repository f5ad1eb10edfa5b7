// Host-side fixed-tree all-reduce over TCP (one call = one rank), native counterpart of
// parallel/host_collectives.py::tcp_tree_all_reduce_rank for the fp32 fixed-order sum.
//
// Semantics of the reference's multi-host proof transport (scirust-core/src/tree_allreduce.rs:33-187
// tree, :199-366 TCP): rank r's children are 2r+1 and 2r+2; a rank adds itself, then its left child,
// then its right child whatever the arrival order, sends the partial to its parent and relays the
// total down. Frames are `u32 rank | u64 length | payload`, little endian, capped at 1 GiB; a frame
// from an unexpected rank, a short read or a timeout is an error returned to the caller (no abort).
// The transport is unauthenticated, as documented upstream: use it inside a trusted network only.
#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdint.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/types.h>
#include <unistd.h>

#include <chrono>
#include <new>
#include <vector>

namespace {

constexpr uint64_t kMaxFrame = 1ull << 30;
enum { OK = 0, E_ARG = 1, E_SOCKET = 2, E_TIMEOUT = 3, E_PROTOCOL = 4, E_NOMEM = 5, E_CLOSED = 6 };

using Clock = std::chrono::steady_clock;

struct Deadline {
  Clock::time_point t;
  explicit Deadline(int ms) : t(Clock::now() + std::chrono::milliseconds(ms)) {}
  int left_ms() const {
    auto d = std::chrono::duration_cast<std::chrono::milliseconds>(t - Clock::now()).count();
    return d < 0 ? 0 : static_cast<int>(d);
  }
};

int wait_fd(int fd, short events, const Deadline& dl) {
  for (;;) {
    pollfd p{fd, events, 0};
    const int left = dl.left_ms();
    if (left == 0) return E_TIMEOUT;
    const int rc = poll(&p, 1, left);
    if (rc > 0) return OK;
    if (rc == 0) return E_TIMEOUT;
    if (errno != EINTR) return E_SOCKET;
  }
}

int send_all(int fd, const void* buf, size_t n, const Deadline& dl) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    if (int rc = wait_fd(fd, POLLOUT, dl)) return rc;
    const ssize_t k = send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return E_SOCKET;
    }
    p += k;
    n -= static_cast<size_t>(k);
  }
  return OK;
}

int recv_all(int fd, void* buf, size_t n, const Deadline& dl) {
  char* p = static_cast<char*>(buf);
  while (n) {
    if (int rc = wait_fd(fd, POLLIN, dl)) return rc;
    const ssize_t k = recv(fd, p, n, 0);
    if (k == 0) return E_CLOSED;
    if (k < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return E_SOCKET;
    }
    p += k;
    n -= static_cast<size_t>(k);
  }
  return OK;
}

int send_frame(int fd, uint32_t rank, const float* data, uint64_t n_floats, const Deadline& dl) {
  const uint64_t len = n_floats * 4;
  if (len > kMaxFrame) return E_PROTOCOL;
  unsigned char hdr[12];
  for (int i = 0; i < 4; ++i) hdr[i] = static_cast<unsigned char>(rank >> (8 * i));
  for (int i = 0; i < 8; ++i) hdr[4 + i] = static_cast<unsigned char>(len >> (8 * i));
  if (int rc = send_all(fd, hdr, 12, dl)) return rc;
  return send_all(fd, data, len, dl);   // x86-64 / aarch64 little endian: floats go as stored
}

// Reads one frame whose payload must be exactly n_floats floats; *rank_out receives the sender.
int recv_frame(int fd, uint32_t* rank_out, float* data, uint64_t n_floats, const Deadline& dl) {
  unsigned char hdr[12];
  if (int rc = recv_all(fd, hdr, 12, dl)) return rc;
  uint32_t rank = 0;
  uint64_t len = 0;
  for (int i = 0; i < 4; ++i) rank |= static_cast<uint32_t>(hdr[i]) << (8 * i);
  for (int i = 0; i < 8; ++i) len |= static_cast<uint64_t>(hdr[4 + i]) << (8 * i);
  if (len > kMaxFrame || len != n_floats * 4) return E_PROTOCOL;
  *rank_out = rank;
  return recv_all(fd, data, len, dl);
}

struct Fd {
  int fd = -1;
  ~Fd() { if (fd >= 0) close(fd); }
};

}  // namespace

extern "C" {

// One rank of the all-reduce. hosts[r] / ports[r]: listener address of rank r (only ranks with
// children listen). data: n floats, replaced by the sum over all ranks. Returns 0 or an error code
// (1 argument, 2 socket, 3 timeout, 4 protocol / unexpected rank, 5 out of memory, 6 peer closed).
int sbrt_tcp_tree_allreduce_f32(int rank, int world, const char* const* hosts, const int* ports, float* data,
                                int64_t n, int timeout_ms) {
  if (world < 1 || rank < 0 || rank >= world || n < 0 || static_cast<uint64_t>(n) * 4 > kMaxFrame || timeout_ms <= 0)
    return E_ARG;
  if (world == 1) return OK;
  const Deadline dl(timeout_ms);
  const int kids[2] = {2 * rank + 1, 2 * rank + 2};
  const int n_kids = (kids[0] < world) + (kids[1] < world);
  Fd srv, kid_fd[2], up;
  std::vector<float> part[2];
  try {
    for (int i = 0; i < n_kids; ++i) part[i].resize(static_cast<size_t>(n));
  } catch (const std::bad_alloc&) {
    return E_NOMEM;   // fallible allocation: a huge request is an error, not an abort
  }
  if (n_kids) {
    srv.fd = socket(AF_INET, SOCK_STREAM, 0);
    if (srv.fd < 0) return E_SOCKET;
    int one = 1;
    setsockopt(srv.fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(ports[rank]));
    if (inet_pton(AF_INET, hosts[rank], &addr.sin_addr) != 1) return E_ARG;
    if (bind(srv.fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0) return E_SOCKET;
    if (listen(srv.fd, n_kids) != 0) return E_SOCKET;
    bool seen[2] = {false, false};
    for (int i = 0; i < n_kids; ++i) {
      if (int rc = wait_fd(srv.fd, POLLIN, dl)) return rc;
      Fd c;
      c.fd = accept(srv.fd, nullptr, nullptr);
      if (c.fd < 0) return E_SOCKET;
      setsockopt(c.fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      // the first frame names the sender; its payload is parked in that child's slot so the sum below
      // runs in child order whatever the arrival order
      unsigned char hdr[12];
      if (int rc = recv_all(c.fd, hdr, 12, dl)) return rc;
      uint32_t r = 0;
      uint64_t len = 0;
      for (int b = 0; b < 4; ++b) r |= static_cast<uint32_t>(hdr[b]) << (8 * b);
      for (int b = 0; b < 8; ++b) len |= static_cast<uint64_t>(hdr[4 + b]) << (8 * b);
      int slot = -1;
      for (int k = 0; k < n_kids; ++k)
        if (static_cast<int>(r) == kids[k] && !seen[k]) slot = k;
      if (slot < 0 || len != static_cast<uint64_t>(n) * 4) return E_PROTOCOL;
      if (int rc = recv_all(c.fd, part[slot].data(), len, dl)) return rc;
      seen[slot] = true;
      kid_fd[slot].fd = c.fd;
      c.fd = -1;
    }
    for (int k = 0; k < n_kids; ++k)          // self, then left child, then right child
      for (int64_t i = 0; i < n; ++i) data[i] += part[k][static_cast<size_t>(i)];
  }
  if (rank != 0) {
    const int parent = (rank - 1) / 2;
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(ports[parent]));
    if (inet_pton(AF_INET, hosts[parent], &addr.sin_addr) != 1) return E_ARG;
    for (;;) {   // the parent may not be listening yet
      up.fd = socket(AF_INET, SOCK_STREAM, 0);
      if (up.fd < 0) return E_SOCKET;
      if (connect(up.fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) break;
      close(up.fd);
      up.fd = -1;
      if (dl.left_ms() == 0) return E_TIMEOUT;
      usleep(20000);
    }
    int one = 1;
    setsockopt(up.fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    if (int rc = send_frame(up.fd, static_cast<uint32_t>(rank), data, static_cast<uint64_t>(n), dl)) return rc;
    uint32_t from = 0;
    if (int rc = recv_frame(up.fd, &from, data, static_cast<uint64_t>(n), dl)) return rc;
    if (static_cast<int>(from) != parent) return E_PROTOCOL;
  }
  for (int k = 0; k < n_kids; ++k)
    if (int rc = send_frame(kid_fd[k].fd, static_cast<uint32_t>(rank), data, static_cast<uint64_t>(n), dl)) return rc;
  return OK;
}

}  // extern "C"
