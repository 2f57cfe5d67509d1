// Sanitizer self-test of the host library: a plain executable that drives the memory pool, the memory planner, the
// pipeline scheduler, the layout algebra and the checkpoint scanner (on well-formed and on truncated / random input)
// through their C entry points.  Built with -fsanitize=address,undefined by tests/test_host_sanitizers.py; any
// out-of-bounds access, use after free, leak or undefined behaviour fails the run.  (The reference's build has the
// same switch for its whole tree: cmake/options.cmake ENABLE_ASAN.)
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

extern "C" {
void* msb_pool_create(unsigned long long block_size, unsigned long long max_size);
void msb_pool_destroy(void* pool);
void* msb_pool_alloc(void* pool, unsigned long long size, unsigned long long stream);
unsigned long long msb_pool_free(void* pool, void* ptr);
void msb_pool_mark_synchronized(void* pool);
unsigned long long msb_pool_release_idle(void* pool);
void msb_pool_stats(void* pool, unsigned long long* out);
int64_t msb_memory_plan(int n, const int64_t* size, const int32_t* start, const int32_t* end, const int32_t* group,
                        int64_t align, int64_t* offsets_out);
int msb_memory_plan_check(int n, const int64_t* size, const int32_t* start, const int32_t* end,
                          const int64_t* offsets);
int msb_pipeline_schedule(int stages, int stage, int micro, int chunks, int scheduler, int32_t* out, int capacity);
int msb_group_ranks(const int32_t* dev_matrix, int n_dev, int rank, const int32_t* dev_dims, int n_dims,
                    int base_rank, int32_t* out, int capacity);
int msb_ckpt_scan(const uint8_t* data, uint64_t len, int max_records, int64_t* rec_out, int64_t* dims_out,
                  int max_dims, int32_t* dims_index_out, char* types_out);
uint32_t msb_crc32(uint32_t crc, const void* data, uint64_t len);
}

#define CHECK(cond)                                                       \
  do {                                                                    \
    if (!(cond)) {                                                        \
      std::fprintf(stderr, "selftest: %s failed (line %d)\n", #cond, __LINE__); \
      return 1;                                                           \
    }                                                                     \
  } while (0)

int main() {
  std::mt19937_64 rng(7);
  // ---- memory pool: random allocate / write / free over three streams, with synchronisation points
  {
    void* pool = msb_pool_create(1 << 16, 1 << 22);
    std::vector<std::pair<unsigned char*, size_t>> live;
    for (int it = 0; it < 4000; ++it) {
      const bool do_alloc = live.empty() || (rng() % 100) < 55;
      if (do_alloc) {
        const size_t size = 1 + rng() % 9000;
        auto* p = static_cast<unsigned char*>(msb_pool_alloc(pool, size, rng() % 3));
        if (p != nullptr) {
          std::memset(p, 0xAB, size);           // every byte handed out must be ours to write
          live.emplace_back(p, size);
        }
      } else {
        const size_t i = rng() % live.size();
        CHECK(msb_pool_free(pool, live[i].first) >= live[i].second);
        live[i] = live.back();
        live.pop_back();
      }
      if (it % 500 == 499) {
        msb_pool_mark_synchronized(pool);
        msb_pool_release_idle(pool);
      }
    }
    unsigned long long st[7];
    msb_pool_stats(pool, st);
    CHECK(st[1] >= st[0] && st[1] <= (1u << 22));
    for (auto& b : live) CHECK(msb_pool_free(pool, b.first) > 0);
    CHECK(msb_pool_free(pool, nullptr) == 0);
    msb_pool_destroy(pool);
  }
  // ---- memory planner: random lifetimes, the plan must verify
  for (int round = 0; round < 20; ++round) {
    const int n = 1 + static_cast<int>(rng() % 200);
    std::vector<int64_t> size(n), off(n);
    std::vector<int32_t> s(n), e(n), grp(n, -1);
    for (int i = 0; i < n; ++i) {
      size[i] = 1 + static_cast<int64_t>(rng() % 100000);
      s[i] = static_cast<int32_t>(rng() % 300);
      e[i] = s[i] + static_cast<int32_t>(rng() % 50);
    }
    const int64_t total = msb_memory_plan(n, size.data(), s.data(), e.data(), grp.data(), 256, off.data());
    CHECK(total > 0);
    CHECK(msb_memory_plan_check(n, size.data(), s.data(), e.data(), off.data()) == 0);
  }
  // ---- pipeline schedules: every (stages, stage, micro) combination fits the capacity it asks for
  for (int stages = 1; stages <= 8; ++stages)
    for (int stage = 0; stage < stages; ++stage)
      for (int micro = 1; micro <= 16; ++micro)
        for (int sched = 0; sched < 2; ++sched) {
          std::vector<int32_t> out(3 * 2 * micro + 8);
          const int steps = msb_pipeline_schedule(stages, stage, micro, 1, sched, out.data(), 2 * micro);
          CHECK(steps == 2 * micro);
          CHECK(msb_pipeline_schedule(stages, stage, micro, 1, sched, out.data(), 1) == -1 || micro == 0);
        }
  // ---- layout: group ranks inside an 8-device matrix
  {
    const int32_t dm[3] = {2, 2, 2};
    int32_t dims[2] = {0, 2}, out[8];
    for (int r = 0; r < 8; ++r) {
      const int cnt = msb_group_ranks(dm, 3, r, dims, 2, 0, out, 8);
      CHECK(cnt == 4);
      CHECK(msb_group_ranks(dm, 3, r, dims, 2, 0, out, 2) == -1);
    }
  }
  // ---- checkpoint scanner on arbitrary bytes: it may reject them, it must not read outside them
  {
    std::vector<int64_t> rec(64 * 4), dims(256);
    std::vector<int32_t> idx(64 * 2);
    std::vector<char> types(64 * 16);
    for (int round = 0; round < 2000; ++round) {
      const size_t len = rng() % 300;
      std::vector<uint8_t> buf(len);
      for (auto& b : buf) b = static_cast<uint8_t>(rng());
      if (len > 4 && round % 3 == 0) { buf[0] = 0x0A; buf[1] = static_cast<uint8_t>(len - 2); }   // a plausible header
      (void)msb_ckpt_scan(buf.data(), len, 64, rec.data(), dims.data(), 256, idx.data(), types.data());
    }
    const char msg[] = "123456789";
    CHECK(msb_crc32(0, msg, 9) == 0xCBF43926u);
  }
  std::puts("selftest ok");
  return 0;
}
