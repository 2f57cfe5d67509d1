// Host (CPU) collectives over TCP: ring AllReduce / ReduceScatter / AllGather / Broadcast / Barrier and neighbour
// send / receive between the processes of a job, for tensors that live in host memory (data-parallel CPU training,
// metadata exchange before the GPU communicators exist, tests without a GPU).
//
// The reference has the same layer as "MCCL": MsCollectiveCommLib + MSCollectiveOpsImpl run ring AllGather /
// Broadcast / AllReduce over its TCP RPC stack (plugin/device/cpu/hal/hardware/ms_collective_comm_lib.cc,
// ms_collective_ops_impl.cc).  Here every rank owns one listening socket and two ring connections (to rank+1, from
// rank-1); a step of a ring algorithm sends to the right neighbour and receives from the left one at the same time
// with poll(), so that messages larger than the socket buffers cannot deadlock.  All waits have a deadline; a
// call that runs out of time returns kTimeout and leaves the communicator unusable (the caller tears it down).
//
// C ABI (ctypes): msb_hc_create / destroy, msb_hc_all_reduce, msb_hc_reduce_scatter, msb_hc_all_gather,
// msb_hc_broadcast, msb_hc_barrier, msb_hc_send_next / recv_prev.

#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {

enum : int { kOk = 0, kBadArg = 1, kSocket = 2, kTimeout = 3, kPeerClosed = 4, kBadHandle = 5 };
enum : int { kF32 = 0, kF64 = 1, kI32 = 2, kI64 = 3, kU8 = 4 };
enum : int { kSum = 0, kProd = 1, kMax = 2, kMin = 3 };

using Clock = std::chrono::steady_clock;

struct Ring {
  int rank = 0, world = 1;
  int listen_fd = -1, next_fd = -1, prev_fd = -1;
  double timeout_s = 60.0;
  std::vector<uint8_t> scratch;
};

std::mutex g_mu;
std::map<int, Ring*> g_rings;
int g_next_handle = 1;

int elem_size(int dtype) {
  switch (dtype) {
    case kF32: case kI32: return 4;
    case kF64: case kI64: return 8;
    case kU8: return 1;
    default: return 0;
  }
}

void set_nonblocking(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK));
}

void tune(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

int remaining_ms(Clock::time_point deadline) {
  auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
  return left <= 0 ? 0 : static_cast<int>(std::min<long long>(left, 1000));
}

// Sends `sn` bytes on `sfd` while receiving `rn` bytes from `rfd`; either side may be empty (fd < 0 or 0 bytes).
int send_recv(int sfd, const uint8_t* sbuf, size_t sn, int rfd, uint8_t* rbuf, size_t rn, double timeout_s) {
  const auto deadline = Clock::now() + std::chrono::duration_cast<Clock::duration>(
                                           std::chrono::duration<double>(timeout_s));
  size_t so = 0, ro = 0;
  if (sfd < 0) sn = 0;
  if (rfd < 0) rn = 0;
  while (so < sn || ro < rn) {
    pollfd fds[2];
    int n = 0, si = -1, ri = -1;
    if (so < sn) { fds[n] = {sfd, POLLOUT, 0}; si = n++; }
    if (ro < rn) { fds[n] = {rfd, POLLIN, 0}; ri = n++; }
    const int wait = remaining_ms(deadline);
    if (wait == 0) return kTimeout;
    const int rc = poll(fds, n, wait);
    if (rc < 0) {
      if (errno == EINTR) continue;
      return kSocket;
    }
    if (rc == 0) continue;
    if (si >= 0 && (fds[si].revents & (POLLOUT | POLLERR | POLLHUP))) {
      const ssize_t w = send(sfd, sbuf + so, std::min<size_t>(sn - so, 1 << 20), MSG_NOSIGNAL | MSG_DONTWAIT);
      if (w > 0) so += static_cast<size_t>(w);
      else if (w < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return kPeerClosed;
    }
    if (ri >= 0 && (fds[ri].revents & (POLLIN | POLLERR | POLLHUP))) {
      const ssize_t r = recv(rfd, rbuf + ro, rn - ro, MSG_DONTWAIT);
      if (r > 0) ro += static_cast<size_t>(r);
      else if (r == 0) return kPeerClosed;
      else if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return kPeerClosed;
    }
  }
  return kOk;
}

template <typename T>
void reduce_into(T* acc, const T* in, int64_t n, int op) {
  switch (op) {
    case kSum: for (int64_t i = 0; i < n; ++i) acc[i] += in[i]; break;
    case kProd: for (int64_t i = 0; i < n; ++i) acc[i] *= in[i]; break;
    case kMax: for (int64_t i = 0; i < n; ++i) acc[i] = std::max(acc[i], in[i]); break;
    case kMin: for (int64_t i = 0; i < n; ++i) acc[i] = std::min(acc[i], in[i]); break;
  }
}

void reduce_bytes(void* acc, const void* in, int64_t n, int dtype, int op) {
  switch (dtype) {
    case kF32: reduce_into(static_cast<float*>(acc), static_cast<const float*>(in), n, op); break;
    case kF64: reduce_into(static_cast<double*>(acc), static_cast<const double*>(in), n, op); break;
    case kI32: reduce_into(static_cast<int32_t*>(acc), static_cast<const int32_t*>(in), n, op); break;
    case kI64: reduce_into(static_cast<int64_t*>(acc), static_cast<const int64_t*>(in), n, op); break;
    case kU8: reduce_into(static_cast<uint8_t*>(acc), static_cast<const uint8_t*>(in), n, op); break;
  }
}

Ring* lookup(int h) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_rings.find(h);
  return it == g_rings.end() ? nullptr : it->second;
}

void close_ring(Ring* r) {
  for (int* fd : {&r->listen_fd, &r->next_fd, &r->prev_fd}) {
    if (*fd >= 0) { close(*fd); *fd = -1; }
  }
}

// chunk c of `count` elements split into `world` nearly equal parts: [begin, begin + len)
inline void chunk_range(int64_t count, int world, int c, int64_t* begin, int64_t* len) {
  const int64_t base = count / world, rem = count % world;
  *begin = c * base + std::min<int64_t>(c, rem);
  *len = base + (c < rem ? 1 : 0);
}

}  // namespace

// peers: "host:port,host:port,..." one entry per rank.  Returns a handle > 0, or -code.
MSB_API int msb_hc_create(int rank, int world, const char* peers, double timeout_s) {
  if (world < 1 || rank < 0 || rank >= world || peers == nullptr) return -kBadArg;
  std::vector<std::pair<std::string, int>> addr;
  {
    std::string s(peers);
    size_t pos = 0;
    while (pos <= s.size()) {
      size_t comma = s.find(',', pos);
      if (comma == std::string::npos) comma = s.size();
      std::string item = s.substr(pos, comma - pos);
      size_t colon = item.rfind(':');
      if (colon == std::string::npos) return -kBadArg;
      addr.emplace_back(item.substr(0, colon), atoi(item.c_str() + colon + 1));
      pos = comma + 1;
    }
  }
  if (static_cast<int>(addr.size()) != world) return -kBadArg;
  Ring* r = new Ring();
  r->rank = rank;
  r->world = world;
  r->timeout_s = timeout_s > 0 ? timeout_s : 60.0;
  if (world > 1) {
    const auto deadline = Clock::now() + std::chrono::duration_cast<Clock::duration>(
                                             std::chrono::duration<double>(r->timeout_s));
    r->listen_fd = socket(AF_INET, SOCK_STREAM, 0);
    if (r->listen_fd < 0) { delete r; return -kSocket; }
    int one = 1;
    setsockopt(r->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_ANY);
    sa.sin_port = htons(static_cast<uint16_t>(addr[rank].second));
    if (bind(r->listen_fd, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) != 0 || listen(r->listen_fd, 4) != 0) {
      close_ring(r);
      delete r;
      return -kSocket;
    }
    set_nonblocking(r->listen_fd, true);
    const auto& nxt = addr[(rank + 1) % world];
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(nxt.first.c_str(), std::to_string(nxt.second).c_str(), &hints, &res) != 0 || res == nullptr) {
      close_ring(r);
      delete r;
      return -kSocket;
    }
    const int expect_prev = (rank - 1 + world) % world;
    // connect to the right neighbour and accept the left one, whichever becomes possible first
    while (r->next_fd < 0 || r->prev_fd < 0) {
      if (remaining_ms(deadline) == 0) {
        freeaddrinfo(res);
        close_ring(r);
        delete r;
        return -kTimeout;
      }
      if (r->next_fd < 0) {
        int fd = socket(AF_INET, SOCK_STREAM, 0);
        if (fd >= 0 && connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
          tune(fd);
          int32_t me = rank;
          if (send(fd, &me, 4, MSG_NOSIGNAL) == 4) r->next_fd = fd;
          else close(fd);
        } else if (fd >= 0) {
          close(fd);
        }
      }
      if (r->prev_fd < 0) {
        pollfd p{r->listen_fd, POLLIN, 0};
        if (poll(&p, 1, 20) > 0) {
          int fd = accept(r->listen_fd, nullptr, nullptr);
          if (fd >= 0) {
            set_nonblocking(fd, false);
            tune(fd);
            int32_t who = -1;
            uint8_t* w = reinterpret_cast<uint8_t*>(&who);
            if (send_recv(-1, nullptr, 0, fd, w, 4, 5.0) == kOk && who == expect_prev) r->prev_fd = fd;
            else close(fd);
          }
        }
      } else {
        usleep(2000);
      }
    }
    freeaddrinfo(res);
  }
  std::lock_guard<std::mutex> lk(g_mu);
  const int h = g_next_handle++;
  g_rings[h] = r;
  return h;
}

MSB_API int msb_hc_destroy(int handle) {
  Ring* r = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_rings.find(handle);
    if (it == g_rings.end()) return kBadHandle;
    r = it->second;
    g_rings.erase(it);
  }
  close_ring(r);
  delete r;
  return kOk;
}

MSB_API int msb_hc_rank(int handle) { Ring* r = lookup(handle); return r ? r->rank : -1; }
MSB_API int msb_hc_size(int handle) { Ring* r = lookup(handle); return r ? r->world : -1; }

// In-place ring ReduceScatter over `world` chunks of buf: afterwards chunk (rank + 1) % world holds the full result.
static int ring_reduce_scatter_inplace(Ring* r, uint8_t* buf, int64_t count, int dtype, int op) {
  const int es = elem_size(dtype), W = r->world;
  int64_t max_len = count / W + 1;
  r->scratch.resize(static_cast<size_t>(max_len) * es);
  for (int step = 0; step < W - 1; ++step) {
    const int send_c = ((r->rank - step) % W + W) % W;
    const int recv_c = ((r->rank - step - 1) % W + W) % W;
    int64_t sb, sl, rb, rl;
    chunk_range(count, W, send_c, &sb, &sl);
    chunk_range(count, W, recv_c, &rb, &rl);
    const int rc = send_recv(r->next_fd, buf + sb * es, static_cast<size_t>(sl) * es, r->prev_fd, r->scratch.data(),
                             static_cast<size_t>(rl) * es, r->timeout_s);
    if (rc != kOk) return rc;
    reduce_bytes(buf + rb * es, r->scratch.data(), rl, dtype, op);
  }
  return kOk;
}

// Ring AllGather of chunks already in place: rank holds chunk `own(rank)`; passes chunks around W-1 times.
static int ring_all_gather_inplace(Ring* r, uint8_t* buf, int64_t count, int es, int own_shift) {
  const int W = r->world;
  for (int step = 0; step < W - 1; ++step) {
    const int send_c = ((r->rank + own_shift - step) % W + W) % W;
    const int recv_c = ((r->rank + own_shift - step - 1) % W + W) % W;
    int64_t sb, sl, rb, rl;
    chunk_range(count, W, send_c, &sb, &sl);
    chunk_range(count, W, recv_c, &rb, &rl);
    const int rc = send_recv(r->next_fd, buf + sb * es, static_cast<size_t>(sl) * es, r->prev_fd, buf + rb * es,
                             static_cast<size_t>(rl) * es, r->timeout_s);
    if (rc != kOk) return rc;
  }
  return kOk;
}

MSB_API int msb_hc_all_reduce(int handle, void* buf, int64_t count, int dtype, int op) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  if (elem_size(dtype) == 0 || count < 0 || op < kSum || op > kMin) return kBadArg;
  if (r->world == 1 || count == 0) return kOk;
  uint8_t* b = static_cast<uint8_t*>(buf);
  int rc = ring_reduce_scatter_inplace(r, b, count, dtype, op);
  if (rc != kOk) return rc;
  return ring_all_gather_inplace(r, b, count, elem_size(dtype), 1);
}

// send: world * count_per_rank elements; recv: count_per_rank elements (the reduced chunk `rank`).
MSB_API int msb_hc_reduce_scatter(int handle, const void* send, void* recv, int64_t count_per_rank, int dtype,
                                  int op) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  const int es = elem_size(dtype);
  if (es == 0 || count_per_rank < 0) return kBadArg;
  const int W = r->world;
  if (W == 1) {
    memcpy(recv, send, static_cast<size_t>(count_per_rank) * es);
    return kOk;
  }
  // work on a rotated copy so that the chunk this rank ends up owning ((rank + 1) % W of the copy) is chunk `rank`
  std::vector<uint8_t> work(static_cast<size_t>(count_per_rank) * es * W);
  const uint8_t* s = static_cast<const uint8_t*>(send);
  const size_t cb = static_cast<size_t>(count_per_rank) * es;
  for (int c = 0; c < W; ++c) memcpy(work.data() + static_cast<size_t>((c + 1) % W) * cb, s + static_cast<size_t>(c) * cb, cb);
  const int rc = ring_reduce_scatter_inplace(r, work.data(), count_per_rank * W, dtype, op);
  if (rc != kOk) return rc;
  memcpy(recv, work.data() + static_cast<size_t>((r->rank + 1) % W) * cb, cb);
  return kOk;
}

// send: bytes_per_rank bytes; recv: world * bytes_per_rank bytes, rank order.
MSB_API int msb_hc_all_gather(int handle, const void* send, void* recv, int64_t bytes_per_rank) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  if (bytes_per_rank < 0) return kBadArg;
  uint8_t* out = static_cast<uint8_t*>(recv);
  memcpy(out + static_cast<size_t>(r->rank) * bytes_per_rank, send, static_cast<size_t>(bytes_per_rank));
  if (r->world == 1 || bytes_per_rank == 0) return kOk;
  return ring_all_gather_inplace(r, out, bytes_per_rank * r->world, 1, 0);
}

// The root's bytes travel around the ring in pipelined segments; the rank before the root does not forward.
MSB_API int msb_hc_broadcast(int handle, void* buf, int64_t bytes, int root) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  if (bytes < 0 || root < 0 || root >= r->world) return kBadArg;
  if (r->world == 1 || bytes == 0) return kOk;
  const int W = r->world;
  const int dist = ((r->rank - root) % W + W) % W;        // hops from the root
  const bool sends = dist != W - 1, recvs = dist != 0;
  const int64_t seg = 1 << 20;
  uint8_t* b = static_cast<uint8_t*>(buf);
  const int64_t nseg = (bytes + seg - 1) / seg;
  // segment i is received in round i and forwarded in round i + 1, overlapped with the next receive
  for (int64_t i = 0; i <= nseg; ++i) {
    const bool do_recv = recvs && i < nseg;
    const int64_t fwd = recvs ? i - 1 : i;
    const bool do_send = sends && fwd >= 0 && fwd < nseg;
    if (!do_recv && !do_send) continue;
    const int64_t ro = i * seg, so = fwd * seg;
    const int rc = send_recv(do_send ? r->next_fd : -1, b + so, do_send ? std::min(seg, bytes - so) : 0,
                             do_recv ? r->prev_fd : -1, b + ro, do_recv ? std::min(seg, bytes - ro) : 0,
                             r->timeout_s);
    if (rc != kOk) return rc;
  }
  return kOk;
}

MSB_API int msb_hc_barrier(int handle) {
  int32_t token = 1;
  return msb_hc_all_reduce(handle, &token, 1, kI32, kSum);
}

MSB_API int msb_hc_send_next(int handle, const void* buf, int64_t bytes) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  if (r->world == 1) return kBadArg;
  return send_recv(r->next_fd, static_cast<const uint8_t*>(buf), static_cast<size_t>(bytes), -1, nullptr, 0,
                   r->timeout_s);
}

MSB_API int msb_hc_recv_prev(int handle, void* buf, int64_t bytes) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  if (r->world == 1) return kBadArg;
  return send_recv(-1, nullptr, 0, r->prev_fd, static_cast<uint8_t*>(buf), static_cast<size_t>(bytes), r->timeout_s);
}

MSB_API int msb_hc_set_timeout(int handle, double timeout_s) {
  Ring* r = lookup(handle);
  if (r == nullptr) return kBadHandle;
  r->timeout_s = timeout_s;
  return kOk;
}
