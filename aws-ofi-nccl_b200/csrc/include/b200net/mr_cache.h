// Registration cache: page-rounded (base, pages) keys in a sorted vector with reference counts.
// A lookup hits when the cached entry CONTAINS the requested range; inserting an existing range
// reports EEXIST; delete returns 1 when the last reference went away and the caller must really
// deregister (reference: src/nccl_ofi_mr.cpp, include/nccl_ofi_mr.h).
//
// Keys marked `exact` stand for one device allocation (its base and size): they hit only an entry
// with the very same base and size, never by page containment. The driver packs small device
// allocations a few hundred bytes apart, so several share a page, and a handle that describes one
// of them (its IPC handle, its bounds) must not be handed out for a neighbour.
#pragma once
#include <cstddef>
#include <cstdint>
#include "b200net/pthread_wrap.h"
#include <vector>

namespace b200net {

constexpr size_t MR_CACHE_PAGE_SIZE = 4096;

enum class MrKeyKind : uint8_t { IOVEC = 0, DMABUF = 1 };

struct MrCacheKey {
  MrKeyKind kind = MrKeyKind::IOVEC;
  uintptr_t addr = 0;
  size_t len = 0;
  int fd = -1;          // dmabuf only
  uint64_t offset = 0;  // dmabuf only
  const void* ep = nullptr;  // registrations tied to an endpoint only hit for the same endpoint
  bool exact = false;        // match base and length exactly (one device allocation)
  static MrCacheKey from_allocation(const void* base, size_t len, const void* ep = nullptr) {
    MrCacheKey k{MrKeyKind::IOVEC, reinterpret_cast<uintptr_t>(base), len, -1, 0, ep};
    k.exact = true;
    return k;
  }
  static MrCacheKey from_iovec(const void* p, size_t len, const void* ep = nullptr) {
    return {MrKeyKind::IOVEC, reinterpret_cast<uintptr_t>(p), len, -1, 0, ep};
  }
  static MrCacheKey from_dmabuf(int fd, uint64_t off, const void* p, size_t len, const void* ep = nullptr) {
    return {MrKeyKind::DMABUF, reinterpret_cast<uintptr_t>(p), len, fd, off, ep};
  }
};

class MrCache {
 public:
  explicit MrCache(size_t initial_slots = 128, size_t page_size = MR_CACHE_PAGE_SIZE);
  ~MrCache();
  // Returns the cached handle and takes a reference, or nullptr on a miss.
  void* lookup(const MrCacheKey& key);
  // 0 on success, -EEXIST if an entry with the same page range exists.
  int insert(const MrCacheKey& key, void* handle);
  // 0: references remain; 1: last reference dropped, entry removed; -ENOENT: unknown handle.
  int del(void* handle);
  size_t size() const;
  uint64_t hits() const { ScopedLock g(mu_); return hits_; }
  uint64_t misses() const { ScopedLock g(mu_); return misses_; }
  void page_range(const MrCacheKey& key, uintptr_t* base, size_t* pages) const;

 private:
  struct Entry { uintptr_t addr; size_t pages; int refcnt; void* handle; const void* ep; MrKeyKind kind; int fd;
                 bool exact; uintptr_t raw_addr; size_t raw_len; };
  size_t page_size_;
  mutable Mutex mu_;
  std::vector<Entry> entries_ TSA_GUARDED_BY(mu_);  // sorted by addr
  uint64_t hits_ TSA_GUARDED_BY(mu_) = 0;
  uint64_t misses_ TSA_GUARDED_BY(mu_) = 0;
};

}  // namespace b200net
