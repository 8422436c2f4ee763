// Deterministic sub-allocator of the symmetric heap.
//
// It manages *offsets*, never pointers, so the same sequence of calls gives the
// same offsets on every PE: that is what makes the heap symmetric.  Free space
// is an address-ordered map with first-fit search and coalescing on release;
// aligned requests carve the aligned block out of the first free range that can
// hold it and return the unused front and back to the free map (no
// over-allocation is kept).  Minimum alignment and size granule: 512 bytes
// (reference behaviour: src/host/mem/custom_malloc.cpp, class mspace).
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>

namespace bshmem {

class HeapAllocator {
 public:
  static constexpr size_t kMinAlign = 512;

  // Adds [offset, offset+size) to the managed space (heap growth).
  void add_chunk(size_t offset, size_t size);
  // `alignment` must be a power of two (0 = default).  Returns false when no
  // free range fits; the caller then grows the heap and retries.
  bool allocate(size_t size, size_t alignment, size_t* offset_out);
  bool release(size_t offset);
  // Size recorded for a live allocation, 0 if `offset` is not one.
  size_t size_of(size_t offset) const;
  bool owns(size_t offset) const { return in_use_.count(offset) != 0; }

  size_t capacity() const { return capacity_; }
  size_t bytes_in_use() const { return used_; }
  size_t live_allocations() const { return in_use_.size(); }
  size_t largest_free() const;
  // Order-sensitive digest of every allocate/release so far; PEs compare it to
  // detect asymmetric call sequences (NVSHMEM_ENABLE_ERROR_CHECKS).
  uint64_t history_digest() const { return digest_; }
  // Internal consistency: free and used ranges tile the managed space exactly.
  bool check_invariants() const;

 private:
  void insert_free(size_t off, size_t len);
  void mix(uint64_t a, uint64_t b);
  std::map<size_t, size_t> free_;    // offset -> length, address ordered
  std::map<size_t, size_t> in_use_;  // offset -> length
  size_t capacity_ = 0, used_ = 0;
  uint64_t digest_ = 0xcbf29ce484222325ull;
};

}  // namespace bshmem
