// Offsets inside a rank's symmetric heap: first-fit over a coalescing free list.
//
// Every rank runs its own copy of this allocator and never talks to the others about it.  The
// offsets agree across ranks because they are a pure function of the sequence of alloc / free
// calls (lowest free offset that fits, 256-byte granules), and the collectives need exactly that:
// a tensor is addressed on every peer at the caller's own offset.  A run of allocations with no
// free in between comes out as consecutive, 256-byte aligned offsets from zero.
// The reference keeps one grow-only static staging buffer and never frees it
// (allreduce_over_mpi/mpi_mod.hpp:1489-1507).
#pragma once
#include <cstddef>
#include <cstdint>
#include <iterator>
#include <map>

namespace ft {

class HeapAllocator {
 public:
  static constexpr size_t kNone = ~(size_t)0;
  static constexpr size_t kAlign = 256;

  explicit HeapAllocator(size_t bytes = 0) { reset(bytes); }

  // Forget every allocation; the heap has `bytes` usable bytes (rounded down to the granule).
  void reset(size_t bytes) {
    size_ = bytes / kAlign * kAlign;
    used_.clear();
    free_.clear();
    if (size_) free_[0] = size_;
  }
  void reset() { reset(size_); }

  // Offset of a block of at least `bytes` (zero counts as one granule), or kNone.
  size_t alloc(size_t bytes) {
    const size_t need = round_up(bytes ? bytes : 1);
    if (need < bytes) return kNone;   // overflow
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      if (it->second < need) continue;
      const size_t off = it->first, rest = it->second - need;
      free_.erase(it);
      if (rest) free_[off + need] = rest;
      used_[off] = need;
      return off;
    }
    return kNone;
  }

  // Give back the block that starts at `offset`; false when no such block is allocated.
  bool free(size_t offset) {
    auto u = used_.find(offset);
    if (u == used_.end()) return false;
    size_t off = u->first, len = u->second;
    used_.erase(u);
    auto next = free_.lower_bound(off);
    if (next != free_.end() && off + len == next->first) {   // merge with the block after
      len += next->second;
      next = free_.erase(next);
    }
    if (next != free_.begin()) {                             // merge with the block before
      auto prev = std::prev(next);
      if (prev->first + prev->second == off) {
        prev->second += len;
        return true;
      }
    }
    free_[off] = len;
    return true;
  }

  size_t size() const { return size_; }
  size_t used_bytes() const {
    size_t n = 0;
    for (const auto& kv : used_) n += kv.second;
    return n;
  }
  size_t largest_free() const {
    size_t n = 0;
    for (const auto& kv : free_) n = kv.second > n ? kv.second : n;
    return n;
  }
  size_t live_blocks() const { return used_.size(); }
  size_t free_blocks() const { return free_.size(); }
  // size of the allocated block at `offset`, 0 if none
  size_t block_size(size_t offset) const {
    auto u = used_.find(offset);
    return u == used_.end() ? 0 : u->second;
  }

 private:
  static size_t round_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }
  size_t size_ = 0;
  std::map<size_t, size_t> free_;   // offset -> bytes, never adjacent to one another
  std::map<size_t, size_t> used_;   // offset -> bytes
};

}  // namespace ft
