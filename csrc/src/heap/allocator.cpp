#include "allocator.h"

#include <stdint.h>

#include <algorithm>

namespace bshmem {

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

void HeapAllocator::mix(uint64_t a, uint64_t b) {
  digest_ = (digest_ ^ a) * 1099511628211ull;
  digest_ = (digest_ ^ b) * 1099511628211ull;
}

void HeapAllocator::insert_free(size_t off, size_t len) {
  if (len == 0) return;
  auto next = free_.lower_bound(off);
  if (next != free_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) {  // merge with the range before
      off = prev->first;
      len += prev->second;
      free_.erase(prev);
    }
  }
  if (next != free_.end() && off + len == next->first) {  // and with the one after
    len += next->second;
    free_.erase(next);
  }
  free_[off] = len;
}

void HeapAllocator::add_chunk(size_t offset, size_t size) {
  capacity_ += size;
  insert_free(offset, size);
}

bool HeapAllocator::allocate(size_t size, size_t alignment, size_t* offset_out) {
  if (size == 0) return false;
  if (alignment < kMinAlign) alignment = kMinAlign;
  if (alignment & (alignment - 1)) return false;
  // A size whose rounding wraps around, or that no heap could hold, is refused before it turns into a
  // zero-length block that aliases the next allocation.
  if (size > SIZE_MAX - kMinAlign || round_up(size, kMinAlign) == 0 || round_up(size, kMinAlign) > capacity_) return false;
  size = round_up(size, kMinAlign);
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    size_t start = it->first, len = it->second;
    size_t aligned = round_up(start, alignment);
    if (aligned + size > start + len || aligned + size < aligned) continue;
    size_t front = aligned - start, back = start + len - (aligned + size);
    free_.erase(it);
    if (front) free_[start] = front;
    if (back) free_[aligned + size] = back;
    in_use_[aligned] = size;
    used_ += size;
    mix(1, aligned ^ (size << 1));
    *offset_out = aligned;
    return true;
  }
  return false;
}

bool HeapAllocator::release(size_t offset) {
  auto it = in_use_.find(offset);
  if (it == in_use_.end()) return false;
  size_t len = it->second;
  in_use_.erase(it);
  used_ -= len;
  insert_free(offset, len);
  mix(2, offset);
  return true;
}

size_t HeapAllocator::size_of(size_t offset) const {
  auto it = in_use_.find(offset);
  return it == in_use_.end() ? 0 : it->second;
}

size_t HeapAllocator::largest_free() const {
  size_t best = 0;
  for (auto& kv : free_) best = std::max(best, kv.second);
  return best;
}

bool HeapAllocator::check_invariants() const {
  // Merge both maps in address order; ranges must not overlap, adjacent free
  // ranges must have been coalesced, and the totals must add up.
  size_t total = 0, used = 0;
  auto f = free_.begin();
  auto u = in_use_.begin();
  size_t cursor = 0;
  bool last_free = false, first = true;
  while (f != free_.end() || u != in_use_.end()) {
    bool take_free = u == in_use_.end() || (f != free_.end() && f->first < u->first);
    size_t off = take_free ? f->first : u->first;
    size_t len = take_free ? f->second : u->second;
    if (!first && off < cursor) return false;
    if (take_free && last_free && !first && off == cursor) return false;  // uncoalesced neighbours
    cursor = off + len;
    total += len;
    if (!take_free) used += len;
    last_free = take_free;
    first = false;
    if (take_free) ++f; else ++u;
  }
  return total == capacity_ && used == used_;
}

}  // namespace bshmem
