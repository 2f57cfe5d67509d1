// Cluster bootstrap: a scheduler (metadata server) and worker clients over TCP, with registration, rank
// assignment, heartbeats, timeout detection and a key-value metadata store - the role of the reference's
// MetaServerNode / ComputeGraphNode (ccsrc/distributed/cluster/topology/meta_server_node.cc:149-343,454-527,
// compute_graph_node.cc:49-106,158-319).  One request per connection, line-framed:
//   "REG <node_id>\n"      -> "OK <rank> <world>\n"         (same node_id re-registers to the same rank)
//   "HB <node_id>\n"       -> "OK <abnormal_count> <ready>\n"
//   "PUT <key> <len>\n<bytes>" -> "OK\n"
//   "GET <key>\n"          -> "OK <len>\n<bytes>" | "NONE\n"
//   "DEL <key>\n"          -> "OK\n"
//   "UNREG <node_id>\n"    -> "OK\n"
//   "ADD <key> <delta>\n"  -> "OK <value>\n"               (atomic counter in the store; delta 0 reads it)
// The scheduler's monitor marks a node abnormal when no heartbeat arrived within the timeout; workers learn
// the abnormal count from every heartbeat reply and can abort their next collective.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {

using Clock = std::chrono::steady_clock;

struct Scheduler {
  int listen_fd = -1;
  int port = 0;
  int expected = 0;
  double timeout_s = 30.0;
  std::atomic<bool> stop{false};
  std::thread accept_thread;
  std::mutex mu;
  std::map<std::string, int> rank_of;
  std::map<std::string, Clock::time_point> last_seen;
  std::map<std::string, bool> alive;
  std::map<std::string, std::string> kv;
};

Scheduler* g_sched = nullptr;

bool read_line(int fd, std::string* out) {
  out->clear();
  char c;
  while (true) {
    const ssize_t n = ::recv(fd, &c, 1, 0);
    if (n <= 0) return false;
    if (c == '\n') return true;
    out->push_back(c);
    if (out->size() > 4096) return false;
  }
}

bool read_exact(int fd, char* buf, size_t len) {
  size_t got = 0;
  while (got < len) {
    const ssize_t n = ::recv(fd, buf + got, len - got, 0);
    if (n <= 0) return false;
    got += static_cast<size_t>(n);
  }
  return true;
}

bool write_all(int fd, const char* buf, size_t len) {
  size_t sent = 0;
  while (sent < len) {
    const ssize_t n = ::send(fd, buf + sent, len - sent, MSG_NOSIGNAL);
    if (n <= 0) return false;
    sent += static_cast<size_t>(n);
  }
  return true;
}

int abnormal_count(Scheduler* s) {
  int bad = 0;
  const auto now = Clock::now();
  for (auto& kvp : s->last_seen) {
    const double dt = std::chrono::duration<double>(now - kvp.second).count();
    if (dt > s->timeout_s) s->alive[kvp.first] = false;
    if (!s->alive[kvp.first]) ++bad;
  }
  return bad;
}

void handle(Scheduler* s, int fd) {
  std::string line;
  if (!read_line(fd, &line)) { ::close(fd); return; }
  char cmd[16] = {0}, arg[1024] = {0};
  long len = 0;
  const int nf = std::sscanf(line.c_str(), "%15s %1023s %ld", cmd, arg, &len);
  std::string reply = "ERR\n";
  const std::string c(cmd), a(arg);
  if (nf >= 2 && c == "REG") {
    std::lock_guard<std::mutex> lk(s->mu);
    auto it = s->rank_of.find(a);
    int rank;
    if (it != s->rank_of.end()) {
      rank = it->second;           // a restarted node keeps its rank
    } else if (static_cast<int>(s->rank_of.size()) < s->expected) {
      rank = static_cast<int>(s->rank_of.size());
      s->rank_of[a] = rank;
    } else {
      rank = -1;
    }
    if (rank >= 0) {
      s->last_seen[a] = Clock::now();
      s->alive[a] = true;
    }
    reply = "OK " + std::to_string(rank) + " " + std::to_string(s->expected) + "\n";
  } else if (nf >= 2 && c == "HB") {
    std::lock_guard<std::mutex> lk(s->mu);
    if (s->rank_of.count(a)) {
      s->last_seen[a] = Clock::now();
      s->alive[a] = true;
    }
    const int ready = static_cast<int>(s->rank_of.size()) >= s->expected ? 1 : 0;
    reply = "OK " + std::to_string(abnormal_count(s)) + " " + std::to_string(ready) + "\n";
  } else if (nf >= 3 && c == "PUT") {
    std::string val(static_cast<size_t>(len), '\0');
    if (len >= 0 && read_exact(fd, &val[0], static_cast<size_t>(len))) {
      std::lock_guard<std::mutex> lk(s->mu);
      s->kv[a] = val;
      reply = "OK\n";
    }
  } else if (nf >= 2 && c == "GET") {
    std::lock_guard<std::mutex> lk(s->mu);
    auto it = s->kv.find(a);
    if (it == s->kv.end()) {
      reply = "NONE\n";
    } else {
      reply = "OK " + std::to_string(it->second.size()) + "\n" + it->second;
    }
  } else if (nf >= 2 && c == "DEL") {
    std::lock_guard<std::mutex> lk(s->mu);
    s->kv.erase(a);
    reply = "OK\n";
  } else if (nf >= 3 && c == "ADD") {
    std::lock_guard<std::mutex> lk(s->mu);
    long cur = 0;
    auto it = s->kv.find(a);
    if (it != s->kv.end()) cur = std::strtol(it->second.c_str(), nullptr, 10);
    cur += len;
    s->kv[a] = std::to_string(cur);
    reply = "OK " + std::to_string(cur) + "\n";
  } else if (nf >= 2 && c == "UNREG") {
    std::lock_guard<std::mutex> lk(s->mu);
    s->alive.erase(a);
    s->last_seen.erase(a);
    reply = "OK\n";
  }
  write_all(fd, reply.data(), reply.size());
  ::close(fd);
}

void accept_loop(Scheduler* s) {
  while (!s->stop.load()) {
    fd_set rf;
    FD_ZERO(&rf);
    FD_SET(s->listen_fd, &rf);
    timeval tv{0, 100000};
    const int r = ::select(s->listen_fd + 1, &rf, nullptr, nullptr, &tv);
    if (r <= 0) continue;
    const int fd = ::accept(s->listen_fd, nullptr, nullptr);
    if (fd < 0) continue;
    timeval to{5, 0};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &to, sizeof(to));
    handle(s, fd);
  }
}

int connect_to(const char* host, int port, double timeout_s) {
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  timeval to{static_cast<long>(timeout_s), static_cast<long>((timeout_s - static_cast<long>(timeout_s)) * 1e6)};
  ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &to, sizeof(to));
  ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &to, sizeof(to));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (::inet_pton(AF_INET, host, &addr.sin_addr) != 1 ||
      ::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0) {
    ::close(fd);
    return -1;
  }
  return fd;
}

}  // namespace

// Starts the scheduler on 127.0.0.1:port (port 0 = pick one).  Returns the bound port or -1.
MSB_API int msb_sched_start(int port, int expected_workers, double node_timeout_s) {
  if (g_sched) return -1;
  Scheduler* s = new Scheduler();
  s->expected = expected_workers;
  s->timeout_s = node_timeout_s;
  s->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (s->listen_fd < 0) { delete s; return -1; }
  int one = 1;
  ::setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (::bind(s->listen_fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(s->listen_fd, 128) != 0) {
    ::close(s->listen_fd);
    delete s;
    return -1;
  }
  socklen_t alen = sizeof(addr);
  ::getsockname(s->listen_fd, reinterpret_cast<sockaddr*>(&addr), &alen);
  s->port = ntohs(addr.sin_port);
  s->accept_thread = std::thread(accept_loop, s);
  g_sched = s;
  return s->port;
}

MSB_API void msb_sched_stop() {
  if (!g_sched) return;
  g_sched->stop.store(true);
  if (g_sched->accept_thread.joinable()) g_sched->accept_thread.join();
  ::close(g_sched->listen_fd);
  delete g_sched;
  g_sched = nullptr;
}

// Number of registered nodes that missed their heartbeat deadline (scheduler side).
MSB_API int msb_sched_abnormal_nodes() {
  if (!g_sched) return -1;
  std::lock_guard<std::mutex> lk(g_sched->mu);
  return abnormal_count(g_sched);
}

MSB_API int msb_sched_registered() {
  if (!g_sched) return -1;
  std::lock_guard<std::mutex> lk(g_sched->mu);
  return static_cast<int>(g_sched->rank_of.size());
}

// Scheduler state as text, for persistence across a scheduler restart (the reference keeps the same in a
// configuration file: cluster/topology/meta_server_node.cc:561-635):
//   "NODE <rank> <node_id>\n" per registered node, "KV <key> <hex of value>\n" per store entry.
// Returns the length, or -(needed length) when `capacity` is too small.
MSB_API int msb_sched_snapshot(char* buf, int capacity) {
  if (!g_sched) return 0;
  std::string out;
  {
    std::lock_guard<std::mutex> lk(g_sched->mu);
    for (auto& kvp : g_sched->rank_of) out += "NODE " + std::to_string(kvp.second) + " " + kvp.first + "\n";
    static const char* hex = "0123456789abcdef";
    for (auto& kvp : g_sched->kv) {
      out += "KV " + kvp.first + " ";
      for (unsigned char ch : kvp.second) { out.push_back(hex[ch >> 4]); out.push_back(hex[ch & 15]); }
      out += "\n";
    }
  }
  if (static_cast<int>(out.size()) > capacity) return -static_cast<int>(out.size());
  std::memcpy(buf, out.data(), out.size());
  return static_cast<int>(out.size());
}

// Loads a snapshot into the running scheduler: nodes get their old ranks back (and a fresh heartbeat deadline, so
// that workers that kept running have one timeout period to show up again), the store gets its entries back.
MSB_API int msb_sched_restore(const char* text, int len) {
  if (!g_sched) return -1;
  std::lock_guard<std::mutex> lk(g_sched->mu);
  std::string all(text, static_cast<size_t>(len));
  size_t pos = 0;
  int n = 0;
  while (pos < all.size()) {
    size_t e = all.find('\n', pos);
    if (e == std::string::npos) e = all.size();
    const std::string line = all.substr(pos, e - pos);
    pos = e + 1;
    if (line.compare(0, 5, "NODE ") == 0) {
      const size_t sp = line.find(' ', 5);
      if (sp == std::string::npos) continue;
      const int rank = std::atoi(line.substr(5, sp - 5).c_str());
      const std::string id = line.substr(sp + 1);
      g_sched->rank_of[id] = rank;
      g_sched->last_seen[id] = Clock::now();
      g_sched->alive[id] = true;
      ++n;
    } else if (line.compare(0, 3, "KV ") == 0) {
      const size_t sp = line.find(' ', 3);
      if (sp == std::string::npos) continue;
      const std::string key = line.substr(3, sp - 3), hx = line.substr(sp + 1);
      std::string val;
      for (size_t i = 0; i + 1 < hx.size(); i += 2) {
        auto d = [](char ch) { return ch <= '9' ? ch - '0' : ch - 'a' + 10; };
        val.push_back(static_cast<char>((d(hx[i]) << 4) | d(hx[i + 1])));
      }
      g_sched->kv[key] = val;
      ++n;
    }
  }
  return n;
}

// Atomic counter in the store: adds `delta` (0 = read) and returns the new value, or -1 on IO failure.
MSB_API long long msb_store_add(const char* host, int port, const char* key, long long delta, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("ADD ") + key + " " + std::to_string(delta) + "\n";
  std::string line;
  long long v = -1;
  if (write_all(fd, req.data(), req.size()) && read_line(fd, &line)) {
    if (std::sscanf(line.c_str(), "OK %lld", &v) != 1) v = -1;
  }
  ::close(fd);
  return v;
}

// Worker side.  Each call opens one connection.  Return: >=0 on success, -1 connect/IO failure, -2 rejected.
MSB_API int msb_worker_register(const char* host, int port, const char* node_id, int* world_out, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("REG ") + node_id + "\n";
  std::string line;
  int rank = -1, world = 0;
  const bool ok = write_all(fd, req.data(), req.size()) && read_line(fd, &line) &&
                  std::sscanf(line.c_str(), "OK %d %d", &rank, &world) == 2;
  ::close(fd);
  if (!ok) return -1;
  if (world_out) *world_out = world;
  return rank < 0 ? -2 : rank;
}

// Returns the number of abnormal nodes reported by the scheduler (>= 0), or -1 when it is unreachable.
MSB_API int msb_worker_heartbeat(const char* host, int port, const char* node_id, int* ready_out, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("HB ") + node_id + "\n";
  std::string line;
  int bad = 0, ready = 0;
  const bool ok = write_all(fd, req.data(), req.size()) && read_line(fd, &line) &&
                  std::sscanf(line.c_str(), "OK %d %d", &bad, &ready) == 2;
  ::close(fd);
  if (!ok) return -1;
  if (ready_out) *ready_out = ready;
  return bad;
}

MSB_API int msb_worker_unregister(const char* host, int port, const char* node_id, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("UNREG ") + node_id + "\n";
  std::string line;
  const bool ok = write_all(fd, req.data(), req.size()) && read_line(fd, &line);
  ::close(fd);
  return ok ? 0 : -1;
}

MSB_API int msb_store_put(const char* host, int port, const char* key, const char* value, int len, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("PUT ") + key + " " + std::to_string(len) + "\n";
  std::string line;
  const bool ok = write_all(fd, req.data(), req.size()) && write_all(fd, value, static_cast<size_t>(len)) &&
                  read_line(fd, &line) && line == "OK";
  ::close(fd);
  return ok ? 0 : -1;
}

// Returns the value length (copied into buf up to capacity), -2 if the key does not exist, -1 on IO failure.
MSB_API int msb_store_get(const char* host, int port, const char* key, char* buf, int capacity, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("GET ") + key + "\n";
  std::string line;
  if (!write_all(fd, req.data(), req.size()) || !read_line(fd, &line)) { ::close(fd); return -1; }
  if (line == "NONE") { ::close(fd); return -2; }
  long len = 0;
  if (std::sscanf(line.c_str(), "OK %ld", &len) != 1 || len < 0) { ::close(fd); return -1; }
  std::string val(static_cast<size_t>(len), '\0');
  const bool ok = read_exact(fd, &val[0], static_cast<size_t>(len));
  ::close(fd);
  if (!ok) return -1;
  std::memcpy(buf, val.data(), static_cast<size_t>(std::min<long>(len, capacity)));
  return static_cast<int>(len);
}

MSB_API int msb_store_delete(const char* host, int port, const char* key, double timeout_s) {
  const int fd = connect_to(host, port, timeout_s);
  if (fd < 0) return -1;
  const std::string req = std::string("DEL ") + key + "\n";
  std::string line;
  const bool ok = write_all(fd, req.data(), req.size()) && read_line(fd, &line);
  ::close(fd);
  return ok ? 0 : -1;
}
