// Best-fit dynamic memory pool over a backing allocator (cudaMalloc on the device, malloc in tests).
//
// Memory is taken from the backing allocator in large blocks and handed out as buffers cut from them:
//   * a request is rounded up to 512 bytes and served from the smallest idle buffer that fits (best fit); the rest
//     of that buffer stays idle if it is at least one alignment unit;
//   * when nothing fits, a new block of max(block size, request) bytes is taken, unless that would pass the limit;
//   * a freed buffer merges with idle neighbours of the same block;
//   * every buffer remembers the stream it was last used on.  A request from the same stream may reuse it at once
//     (work on one stream is ordered); a request from another stream may only take buffers that were idle at the
//     last mark_synchronized() call, i.e. whose last use is known to have finished on the device;
//   * release_idle() hands blocks that are entirely idle back to the backing allocator.
// Role of the reference's DynamicMemPoolBestFit (include/backend/mem_reuse/mem_dynamic_allocator.h:90-235:
// block / buf maps per stream, eager free, event-guarded cross-stream reuse, defrag, statistics).
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace msb {

class BestFitPool {
 public:
  using AllocFn = void* (*)(size_t);
  using FreeFn = void (*)(void*);
  static constexpr size_t kAlign = 512;

  struct Stats {
    size_t used = 0, reserved = 0, peak_used = 0, peak_reserved = 0, blocks = 0, largest_idle = 0, idle_bufs = 0;
  };

  BestFitPool(size_t block_size, size_t max_size, AllocFn alloc, FreeFn release)
      : block_size_(round_up(block_size ? block_size : (size_t(1) << 30))), max_size_(max_size), alloc_(alloc),
        release_(release) {}

  ~BestFitPool() {
    for (auto& b : blocks_) release_(b.first);
  }

  void* allocate(size_t size, uint64_t stream) {
    std::lock_guard<std::mutex> lock(mu_);
    size = round_up(size ? size : 1);
    auto it = find_idle(size, stream);
    if (it == idle_.end()) {
      if (!grow(size, stream)) return nullptr;
      it = find_idle(size, stream);
      if (it == idle_.end()) return nullptr;
    }
    char* base = it->second;
    Buf buf = bufs_[base];
    idle_.erase(it);
    if (buf.size - size >= kAlign) {                  // split: the tail stays idle with the same history
      Buf tail = buf;
      tail.size = buf.size - size;
      bufs_[base + size] = tail;
      idle_.emplace(tail.size, base + size);
      buf.size = size;
    }
    buf.idle = false;
    buf.stream = stream;
    buf.synced = false;
    bufs_[base] = buf;
    stats_.used += buf.size;
    if (stats_.used > stats_.peak_used) stats_.peak_used = stats_.used;
    return base;
  }

  // Returns the size given back, 0 if ptr is not a live buffer of this pool.
  size_t deallocate(void* ptr) {
    std::lock_guard<std::mutex> lock(mu_);
    char* base = static_cast<char*>(ptr);
    auto it = bufs_.find(base);
    if (it == bufs_.end() || it->second.idle) return 0;
    Buf buf = it->second;
    const size_t freed = buf.size;
    stats_.used -= freed;
    buf.idle = true;
    // merge with the idle neighbour after, then before (same block, same stream history)
    auto next = bufs_.find(base + buf.size);
    if (next != bufs_.end() && mergeable(buf, next->second)) {
      erase_idle(next->second.size, next->first);
      buf.size += next->second.size;
      buf.synced = buf.synced && next->second.synced;
      bufs_.erase(next);
    }
    it = bufs_.find(base);
    if (it != bufs_.begin()) {
      auto prev = std::prev(it);
      if (prev->first + prev->second.size == base && mergeable(buf, prev->second)) {
        erase_idle(prev->second.size, prev->first);
        prev->second.size += buf.size;
        prev->second.synced = prev->second.synced && buf.synced;
        prev->second.stream = buf.stream;
        bufs_.erase(it);
        idle_.emplace(prev->second.size, prev->first);
        return freed;
      }
    }
    bufs_[base] = buf;
    idle_.emplace(buf.size, base);
    return freed;
  }

  // Everything idle now has finished on the device (the caller synchronised): any stream may reuse it.
  void mark_synchronized() {
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& kv : bufs_)
      if (kv.second.idle) kv.second.synced = true;
    // neighbours that differed only in their stream can merge now
    for (auto it = bufs_.begin(); it != bufs_.end();) {
      auto next = std::next(it);
      if (next != bufs_.end() && it->second.idle && next->second.idle && it->second.block == next->second.block &&
          it->first + it->second.size == next->first) {
        erase_idle(it->second.size, it->first);
        erase_idle(next->second.size, next->first);
        it->second.size += next->second.size;
        bufs_.erase(next);
        idle_.emplace(it->second.size, it->first);
      } else {
        it = next;
      }
    }
  }

  // Gives blocks without a live buffer back to the backing allocator; returns the bytes released.
  size_t release_idle() {
    std::lock_guard<std::mutex> lock(mu_);
    size_t released = 0;
    for (auto b = blocks_.begin(); b != blocks_.end();) {
      auto it = bufs_.find(b->first);
      const bool whole = it != bufs_.end() && it->second.idle && it->second.size == b->second;
      if (whole) {
        erase_idle(it->second.size, it->first);
        bufs_.erase(it);
        release_(b->first);
        released += b->second;
        stats_.reserved -= b->second;
        b = blocks_.erase(b);
      } else {
        ++b;
      }
    }
    stats_.blocks = blocks_.size();
    return released;
  }

  Stats stats() {
    std::lock_guard<std::mutex> lock(mu_);
    Stats s = stats_;
    s.idle_bufs = idle_.size();
    s.largest_idle = idle_.empty() ? 0 : idle_.rbegin()->first;
    return s;
  }

 private:
  struct Buf {
    size_t size = 0;
    char* block = nullptr;
    uint64_t stream = 0;
    bool idle = true;
    bool synced = true;      // its last use is known to have finished on the device
  };

  static size_t round_up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

  // Idle neighbours of one block merge when a later request could take either under the same condition: both known
  // to be finished on the device, or both last used on the same stream.
  static bool mergeable(const Buf& a, const Buf& b) {
    return b.idle && a.block == b.block && ((a.synced && b.synced) || a.stream == b.stream);
  }

  std::multimap<size_t, char*>::iterator find_idle(size_t size, uint64_t stream) {
    for (auto it = idle_.lower_bound(size); it != idle_.end(); ++it) {
      const Buf& b = bufs_[it->second];
      if (b.synced || b.stream == stream) return it;
    }
    return idle_.end();
  }

  void erase_idle(size_t size, char* base) {
    auto range = idle_.equal_range(size);
    for (auto it = range.first; it != range.second; ++it)
      if (it->second == base) {
        idle_.erase(it);
        return;
      }
  }

  bool grow(size_t size, uint64_t stream) {
    size_t want = size > block_size_ ? size : block_size_;
    if (max_size_ && stats_.reserved + want > max_size_) {
      want = size;                                     // a full block does not fit under the limit: try the request
      if (stats_.reserved + want > max_size_) return false;
    }
    void* p = alloc_(want);
    if (p == nullptr && want > size) {
      want = size;
      p = alloc_(want);
    }
    if (p == nullptr) return false;
    char* base = static_cast<char*>(p);
    blocks_[base] = want;
    Buf b;
    b.size = want;
    b.block = base;
    b.stream = stream;
    b.idle = true;
    b.synced = true;
    bufs_[base] = b;
    idle_.emplace(want, base);
    stats_.reserved += want;
    if (stats_.reserved > stats_.peak_reserved) stats_.peak_reserved = stats_.reserved;
    stats_.blocks = blocks_.size();
    return true;
  }

  size_t block_size_, max_size_;
  AllocFn alloc_;
  FreeFn release_;
  std::mutex mu_;
  std::map<char*, size_t> blocks_;               // block base -> size
  std::map<char*, Buf> bufs_;                    // every buffer (live or idle), ordered by address
  std::multimap<size_t, char*> idle_;            // idle buffers by size
  Stats stats_;
};

}  // namespace msb
