// Native batch pipeline for in-memory (or memory-mapped) columnar data: shuffle -> shard -> gather rows -> optional
// image transform (random crop + horizontal flip + per-channel normalise + HWC->CHW) -> batch, executed by a pool of
// worker threads into a ring of output slots so that the training loop only ever waits for a finished batch.  The
// slots can be caller-owned pinned memory: the host->device copy then starts straight from the slot.
//
// The reference runs the same stages as a tree of C++ dataset ops with connector queues between them
// (minddata/dataset/engine/datasetops/{batch_op,map_op,shuffle_op}.cc, engine/execution_tree.cc, device_queue_op.cc
// for the hand-over to the device).  Here the tree is collapsed: a batch is one task, a worker does every stage
// of that task on rows it reads straight from the source columns, and ordering is restored by slot number.
//
// C ABI: msb_dp_create / msb_dp_set_image_transform / msb_dp_start_epoch / msb_dp_next / msb_dp_release /
// msb_dp_destroy.

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {

struct Column {
  const uint8_t* data = nullptr;
  int64_t row_bytes = 0;        // bytes of one source row
  int64_t out_row_bytes = 0;    // bytes of one row in the batch (differs when the image transform is on)
  // image transform (uint8 HWC -> float32 CHW), off when out_h == 0
  int h = 0, w = 0, c = 0, out_h = 0, out_w = 0, flip = 0;
  float mean[4] = {0, 0, 0, 0}, inv_std[4] = {1, 1, 1, 1};
};

struct Slot {
  std::vector<uint8_t*> col;    // one buffer per column
  int64_t batch_index = -1;     // which batch of the epoch sits here
  int rows = 0;
  bool ready = false, in_use = false;
};

struct Pipeline {
  std::vector<Column> cols;
  int64_t num_rows = 0;
  int batch = 1, drop_remainder = 1, shuffle = 0, num_shards = 1, shard_id = 0;
  uint64_t seed = 0;
  std::vector<Slot> slots;
  std::vector<std::vector<uint8_t>> owned;      // backing store when the caller gave no buffers
  std::vector<int64_t> order;                   // row order of the current epoch (after shuffle + shard)
  int64_t num_batches = 0, next_task = 0, next_out = 0, epoch = -1;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv_task, cv_ready;
  bool stop = false;
};

std::mutex g_mu;
std::map<int, Pipeline*> g_pipes;
int g_next = 1;

Pipeline* lookup(int h) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_pipes.find(h);
  return it == g_pipes.end() ? nullptr : it->second;
}

void transform_image(const Column& col, const uint8_t* src, float* dst, std::mt19937_64& rng) {
  int y0 = 0, x0 = 0;
  if (col.h > col.out_h) y0 = static_cast<int>(rng() % static_cast<uint64_t>(col.h - col.out_h + 1));
  if (col.w > col.out_w) x0 = static_cast<int>(rng() % static_cast<uint64_t>(col.w - col.out_w + 1));
  const bool flip = col.flip && (rng() & 1);
  const int C = col.c, OW = col.out_w, OH = col.out_h;
  for (int ch = 0; ch < C; ++ch) {
    const float m = col.mean[ch], is = col.inv_std[ch];
    float* plane = dst + static_cast<int64_t>(ch) * OH * OW;
    for (int y = 0; y < OH; ++y) {
      const uint8_t* row = src + (static_cast<int64_t>(y0 + y) * col.w + x0) * C + ch;
      float* out = plane + static_cast<int64_t>(y) * OW;
      if (!flip) {
        for (int x = 0; x < OW; ++x) out[x] = (static_cast<float>(row[static_cast<int64_t>(x) * C]) - m) * is;
      } else {
        for (int x = 0; x < OW; ++x)
          out[x] = (static_cast<float>(row[static_cast<int64_t>(OW - 1 - x) * C]) - m) * is;
      }
    }
  }
}

void build_batch(Pipeline* p, Slot& s, int64_t b, int64_t epoch) {
  const int64_t begin = b * p->batch;
  const int64_t end = std::min<int64_t>(begin + p->batch, static_cast<int64_t>(p->order.size()));
  s.rows = static_cast<int>(end - begin);
  for (size_t ci = 0; ci < p->cols.size(); ++ci) {
    const Column& col = p->cols[ci];
    uint8_t* out = s.col[ci];
    for (int64_t i = begin; i < end; ++i) {
      const int64_t row = p->order[i];
      const uint8_t* src = col.data + row * col.row_bytes;
      uint8_t* dst = out + (i - begin) * col.out_row_bytes;
      if (col.out_h == 0) {
        memcpy(dst, src, static_cast<size_t>(col.row_bytes));
      } else {
        // the augmentation of a row depends on (seed, epoch, row) only, not on which worker runs it
        std::mt19937_64 rng(p->seed * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(epoch) * 1000003ull +
                            static_cast<uint64_t>(row));
        transform_image(col, src, reinterpret_cast<float*>(dst), rng);
      }
    }
  }
}

void worker_loop(Pipeline* p) {
  std::unique_lock<std::mutex> lk(p->mu);
  while (true) {
    // a task may start when its slot (task % n_slots) is free; tasks are claimed in order
    p->cv_task.wait(lk, [&] {
      if (p->stop) return true;
      if (p->next_task >= p->num_batches) return false;
      Slot& s = p->slots[p->next_task % p->slots.size()];
      return !s.in_use;
    });
    if (p->stop) return;
    const int64_t b = p->next_task++;
    const int64_t epoch = p->epoch;
    Slot& s = p->slots[b % p->slots.size()];
    s.in_use = true;
    s.ready = false;
    s.batch_index = b;
    lk.unlock();
    build_batch(p, s, b, epoch);
    lk.lock();
    s.ready = true;
    p->cv_ready.notify_all();
  }
}

}  // namespace

// col_ptrs / row_bytes: one entry per column.  out_bufs: n_slots * n_cols caller-owned buffers (each at least
// batch * out_row_bytes bytes; pinned memory for direct host->device copies) or null for internally owned slots.
MSB_API int msb_dp_create(int n_cols, const void* const* col_ptrs, const int64_t* row_bytes, int64_t num_rows,
                          int batch, int drop_remainder, int shuffle, uint64_t seed, int num_shards, int shard_id,
                          int n_workers, int n_slots, void* const* out_bufs) {
  if (n_cols < 1 || num_rows < 0 || batch < 1 || n_workers < 1 || n_slots < 2 || num_shards < 1 || shard_id < 0 ||
      shard_id >= num_shards)
    return -1;
  Pipeline* p = new Pipeline();
  p->cols.resize(n_cols);
  for (int i = 0; i < n_cols; ++i) {
    p->cols[i].data = static_cast<const uint8_t*>(col_ptrs[i]);
    p->cols[i].row_bytes = p->cols[i].out_row_bytes = row_bytes[i];
  }
  p->num_rows = num_rows;
  p->batch = batch;
  p->drop_remainder = drop_remainder;
  p->shuffle = shuffle;
  p->seed = seed;
  p->num_shards = num_shards;
  p->shard_id = shard_id;
  p->slots.resize(n_slots);
  for (int s = 0; s < n_slots; ++s) {
    p->slots[s].col.resize(n_cols, nullptr);
    if (out_bufs != nullptr)
      for (int c = 0; c < n_cols; ++c) p->slots[s].col[c] = static_cast<uint8_t*>(out_bufs[s * n_cols + c]);
  }
  p->workers.reserve(n_workers);
  for (int i = 0; i < n_workers; ++i) p->workers.emplace_back(worker_loop, p);
  std::lock_guard<std::mutex> lk(g_mu);
  const int h = g_next++;
  g_pipes[h] = p;
  return h;
}

// Turns column `col` (uint8, rows of h*w*c) into float32 [c, out_h, out_w] rows: random crop, optional random
// horizontal flip, (x - mean[ch]) / std[ch].  Call before the first epoch; caller-owned slots must be sized for it.
MSB_API int msb_dp_set_image_transform(int handle, int col, int h, int w, int c, int out_h, int out_w, int flip,
                                       const float* mean, const float* stdv) {
  Pipeline* p = lookup(handle);
  if (p == nullptr || col < 0 || col >= static_cast<int>(p->cols.size())) return 1;
  if (c < 1 || c > 4 || out_h < 1 || out_w < 1 || out_h > h || out_w > w) return 1;
  Column& k = p->cols[col];
  if (k.row_bytes != static_cast<int64_t>(h) * w * c) return 1;
  std::lock_guard<std::mutex> lk(p->mu);
  if (p->epoch >= 0) return 2;
  k.h = h; k.w = w; k.c = c; k.out_h = out_h; k.out_w = out_w; k.flip = flip;
  for (int i = 0; i < c; ++i) {
    k.mean[i] = mean ? mean[i] : 0.f;
    k.inv_std[i] = stdv ? 1.f / stdv[i] : 1.f;
  }
  k.out_row_bytes = static_cast<int64_t>(c) * out_h * out_w * 4;
  return 0;
}

// Starts epoch `epoch` (its number seeds the shuffle); returns the number of batches, or -1.
MSB_API int64_t msb_dp_start_epoch(int handle, int64_t epoch) {
  Pipeline* p = lookup(handle);
  if (p == nullptr || epoch < 0) return -1;
  std::unique_lock<std::mutex> lk(p->mu);
  p->num_batches = 0;                                          // no new task is claimed from here on
  p->cv_ready.wait(lk, [&] {
    for (auto& s : p->slots)
      if (s.in_use && !s.ready) return false;                  // a worker is still writing this slot
    return true;
  });
  for (auto& s : p->slots) { s.in_use = s.ready = false; s.batch_index = -1; }
  std::vector<int64_t> all(static_cast<size_t>(p->num_rows));
  for (int64_t i = 0; i < p->num_rows; ++i) all[static_cast<size_t>(i)] = i;
  if (p->shuffle) {
    std::mt19937_64 rng(p->seed + 0x632BE59BD9B4E019ull * static_cast<uint64_t>(epoch + 1));
    for (int64_t i = p->num_rows - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(rng() % static_cast<uint64_t>(i + 1));
      std::swap(all[static_cast<size_t>(i)], all[static_cast<size_t>(j)]);
    }
  }
  p->order.clear();
  for (int64_t i = p->shard_id; i < p->num_rows; i += p->num_shards) p->order.push_back(all[static_cast<size_t>(i)]);
  const int64_t n = static_cast<int64_t>(p->order.size());
  const int64_t nb = p->drop_remainder ? n / p->batch : (n + p->batch - 1) / p->batch;
  // internally owned slots are (re)sized here, when the output row size is final
  if (p->owned.empty() && !p->slots.empty() && p->slots[0].col[0] == nullptr) {
    p->owned.resize(p->slots.size() * p->cols.size());
    for (size_t s = 0; s < p->slots.size(); ++s)
      for (size_t c = 0; c < p->cols.size(); ++c) {
        auto& v = p->owned[s * p->cols.size() + c];
        v.resize(static_cast<size_t>(p->batch) * p->cols[c].out_row_bytes + 64);
        p->slots[s].col[c] = v.data();
      }
  }
  p->epoch = epoch;
  p->next_task = 0;
  p->next_out = 0;
  p->num_batches = nb;
  p->cv_task.notify_all();
  return nb;
}

// Waits for the next batch in order.  Returns the slot index (>= 0), -1 at the end of the epoch, -2 on timeout,
// -3 on a bad handle.  out_ptrs receives the slot's column buffers, rows_out the number of rows in the batch.
MSB_API int msb_dp_next(int handle, void** out_ptrs, int* rows_out, double timeout_s) {
  Pipeline* p = lookup(handle);
  if (p == nullptr) return -3;
  std::unique_lock<std::mutex> lk(p->mu);
  if (p->next_out >= p->num_batches) return -1;
  const int64_t b = p->next_out;
  Slot& s = p->slots[b % p->slots.size()];
  const bool ok = p->cv_ready.wait_for(lk, std::chrono::duration<double>(timeout_s > 0 ? timeout_s : 3600.0),
                                       [&] { return s.ready && s.batch_index == b; });
  if (!ok) return -2;
  p->next_out++;
  for (size_t c = 0; c < p->cols.size(); ++c) out_ptrs[c] = s.col[c];
  if (rows_out) *rows_out = s.rows;
  return static_cast<int>(b % p->slots.size());
}

// Hands a slot back once its batch has been consumed (copied to the device).
MSB_API int msb_dp_release(int handle, int slot) {
  Pipeline* p = lookup(handle);
  if (p == nullptr || slot < 0 || slot >= static_cast<int>(p->slots.size())) return 1;
  std::lock_guard<std::mutex> lk(p->mu);
  Slot& s = p->slots[slot];
  if (s.in_use && s.ready) { s.in_use = false; s.ready = false; }
  p->cv_task.notify_all();
  return 0;
}

MSB_API int msb_dp_destroy(int handle) {
  Pipeline* p = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_pipes.find(handle);
    if (it == g_pipes.end()) return 1;
    p = it->second;
    g_pipes.erase(it);
  }
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->stop = true;
  }
  p->cv_task.notify_all();
  for (auto& t : p->workers) t.join();
  delete p;
  return 0;
}
