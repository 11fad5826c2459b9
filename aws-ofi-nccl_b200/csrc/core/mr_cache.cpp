#include "b200net/mr_cache.h"

#include <algorithm>
#include <cerrno>

#include "b200net/log.h"
#include "b200net/math.h"

namespace b200net {

MrCache::MrCache(size_t initial_slots, size_t page_size) : page_size_(page_size) { entries_.reserve(initial_slots); }

MrCache::~MrCache() {
  NET_INFO(NCCL_NET, "MR cache: %lu hits, %lu misses, %zu entries left", (unsigned long)hits_, (unsigned long)misses_,
           entries_.size());
}

void MrCache::page_range(const MrCacheKey& key, uintptr_t* base, size_t* pages) const {
  const uintptr_t b = round_down<uintptr_t>(key.addr, page_size_);
  const uintptr_t e = round_up<uintptr_t>(key.addr + (key.len ? key.len : 1), page_size_);
  *base = b;
  *pages = (e - b) / page_size_;
}

void* MrCache::lookup(const MrCacheKey& key) {
  uintptr_t base;
  size_t pages;
  page_range(key, &base, &pages);
  ScopedLock g(mu_);
  // entries sorted by addr: candidates start at or before base
  auto it = std::upper_bound(entries_.begin(), entries_.end(), base,
                             [](uintptr_t v, const Entry& e) { return v < e.addr; });
  while (it != entries_.begin()) {
    --it;
    const bool contains = key.exact ? (it->exact && it->raw_addr == key.addr && it->raw_len == key.len)
                                    : (!it->exact && it->addr <= base && base + pages * page_size_ <= it->addr + it->pages * page_size_);
    const bool same_owner = it->ep == key.ep && it->kind == key.kind && (key.kind == MrKeyKind::IOVEC || it->fd == key.fd);
    if (contains && same_owner) {
      ++it->refcnt;
      ++hits_;
      return it->handle;
    }
  }
  ++misses_;
  return nullptr;
}

int MrCache::insert(const MrCacheKey& key, void* handle) {
  uintptr_t base;
  size_t pages;
  page_range(key, &base, &pages);
  ScopedLock g(mu_);
  auto it = std::lower_bound(entries_.begin(), entries_.end(), base,
                             [](const Entry& e, uintptr_t v) { return e.addr < v; });
  for (auto j = it; j != entries_.end() && j->addr == base; ++j) {
    const bool same_range = key.exact ? (j->exact && j->raw_addr == key.addr && j->raw_len == key.len) : (!j->exact && j->pages == pages);
    if (same_range && j->ep == key.ep && j->kind == key.kind && j->fd == key.fd) return -EEXIST;
  }
  entries_.insert(it, Entry{base, pages, 1, handle, key.ep, key.kind, key.fd, key.exact, key.addr, key.len});
  return 0;
}

int MrCache::del(void* handle) {
  ScopedLock g(mu_);
  for (auto it = entries_.begin(); it != entries_.end(); ++it) {
    if (it->handle == handle) {
      if (--it->refcnt > 0) return 0;
      entries_.erase(it);
      return 1;
    }
  }
  return -ENOENT;
}

size_t MrCache::size() const {
  ScopedLock g(mu_);
  return entries_.size();
}

}  // namespace b200net
