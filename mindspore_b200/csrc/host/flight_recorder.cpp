// Flight recorder: a fixed-size lock-free ring of the most recent runtime events (kernel launches, collectives,
// step boundaries, checkpoint writes), cheap enough to stay on in production, written to a file when the process
// fails so that "what was the job doing" can be answered after the fact.
//
// The reference's counterpart is RDR, the "running data recorder" (ccsrc/debug/rdr/recorder_manager.cc,
// base_recorder.h, stream_exec_order_recorder.cc, mem_address_recorder.cc: recorders registered by module and
// name, snapshot on exception / signal via `MS_RDR_ENABLE`, `MS_RDR_MODE`, `MS_RDR_PATH`).  Here all recorders
// share one ring of fixed-size entries; a category id tells them apart.
//
// C ABI: msb_fr_configure(capacity), msb_fr_record(category, step, a, b, text), msb_fr_count(),
// msb_fr_snapshot(out, max) and msb_fr_dump(path).

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {

struct Entry {
  uint64_t seq;            // 0 = never written; otherwise index + 1 of the event
  int64_t t_ns;            // steady clock
  int32_t category;
  int32_t step;
  int64_t a, b;            // free-form numbers (bytes, stream id, rank, ...)
  char text[80];
};

std::vector<Entry> g_ring(4096);
std::atomic<uint64_t> g_next{0};
std::mutex g_cfg_mu;

int64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

}  // namespace

// Resizes the ring (drops what was recorded).  Not to be called while other threads record.
MSB_API int msb_fr_configure(int capacity) {
  if (capacity < 16 || capacity > (1 << 24)) return 1;
  std::lock_guard<std::mutex> lk(g_cfg_mu);
  g_ring.assign(static_cast<size_t>(capacity), Entry{});
  g_next.store(0);
  return 0;
}

MSB_API uint64_t msb_fr_record(int category, int step, int64_t a, int64_t b, const char* text) {
  const uint64_t idx = g_next.fetch_add(1, std::memory_order_relaxed);
  Entry& e = g_ring[idx % g_ring.size()];
  e.seq = 0;                                             // readers skip an entry that is being rewritten
  std::atomic_thread_fence(std::memory_order_release);
  e.t_ns = now_ns();
  e.category = category;
  e.step = step;
  e.a = a;
  e.b = b;
  if (text != nullptr) {
    strncpy(e.text, text, sizeof(e.text) - 1);
    e.text[sizeof(e.text) - 1] = 0;
  } else {
    e.text[0] = 0;
  }
  std::atomic_thread_fence(std::memory_order_release);
  e.seq = idx + 1;
  return idx;
}

MSB_API uint64_t msb_fr_count() { return g_next.load(); }
MSB_API int msb_fr_capacity() { return static_cast<int>(g_ring.size()); }

// Copies up to `max` most recent entries, oldest first, as packed records of 8 int64 + 80 bytes of text:
// [seq, t_ns, category, step, a, b, 0, 0][text].  Returns the number copied.
MSB_API int msb_fr_snapshot(uint8_t* out, int max) {
  const uint64_t end = g_next.load();
  const uint64_t cap = g_ring.size();
  uint64_t begin = end > cap ? end - cap : 0;
  if (end - begin > static_cast<uint64_t>(max)) begin = end - static_cast<uint64_t>(max);
  int n = 0;
  for (uint64_t i = begin; i < end; ++i) {
    const Entry& e = g_ring[i % cap];
    if (e.seq != i + 1) continue;                        // overwritten or in flight
    int64_t head[8] = {static_cast<int64_t>(e.seq), e.t_ns, e.category, e.step, e.a, e.b, 0, 0};
    uint8_t* dst = out + static_cast<size_t>(n) * (64 + 80);
    memcpy(dst, head, 64);
    memcpy(dst + 64, e.text, 80);
    ++n;
  }
  return n;
}

// Text dump, one event per line: seq t_ns category step a b text.  Only async-signal-unsafe in its use of stdio,
// so the Python side calls it from the exception hook, not from a signal handler.
MSB_API int msb_fr_dump(const char* path) {
  FILE* f = fopen(path, "w");
  if (f == nullptr) return 1;
  const uint64_t end = g_next.load();
  const uint64_t cap = g_ring.size();
  const uint64_t begin = end > cap ? end - cap : 0;
  fprintf(f, "# seq t_ns category step a b text\n");
  for (uint64_t i = begin; i < end; ++i) {
    const Entry& e = g_ring[i % cap];
    if (e.seq != i + 1) continue;
    fprintf(f, "%llu %lld %d %d %lld %lld %s\n", static_cast<unsigned long long>(e.seq),
            static_cast<long long>(e.t_ns), e.category, e.step, static_cast<long long>(e.a),
            static_cast<long long>(e.b), e.text);
  }
  fclose(f);
  return 0;
}
