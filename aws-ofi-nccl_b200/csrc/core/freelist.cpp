#include "b200net/freelist.h"

#include <sys/mman.h>

#include <atomic>
#include <cstring>

#include "b200net/assert.h"
#include "b200net/log.h"
#include "b200net/math.h"
#include "b200net/memcheck.h"

namespace b200net {

static std::atomic<size_t> g_leaked{0};
size_t Freelist::leaked_entries_total() { return g_leaked.load(); }

Freelist::Freelist(Options opt) : opt_(std::move(opt)) {
  B200NET_ASSERT_ALWAYS(opt_.entry_size > 0);
  B200NET_ASSERT_ALWAYS(is_pow2(opt_.entry_align));
  B200NET_ASSERT_ALWAYS(is_pow2(opt_.page_size));
  if (opt_.grow_count == 0) opt_.grow_count = 1;
  // each entry: [redzone][user memory padded to alignment]
  const size_t rz = round_up(memcheck::REDZONE, opt_.entry_align);
  stride_ = round_up(rz + round_up(opt_.entry_size, memcheck::GRANULARITY), opt_.entry_align);
  if (opt_.initial_count) {
    if (grow(opt_.initial_count) != 0) throw std::bad_alloc();
  }
}

Freelist::~Freelist() {
  if (in_use_) {
    g_leaked.fetch_add(in_use_);
    NET_WARN("%s: %zu entries still allocated at destruction", opt_.name, in_use_);
  }
  for (auto& b : blocks_) {
    memcheck::make_undefined(b.mem, b.bytes);
    if (opt_.entry_fini) {
      for (size_t i = 0; i < b.count; ++i) opt_.entry_fini(b.entries[i].ptr);
    }
    if (b.mr_handle && opt_.dereg) opt_.dereg(b.mr_handle);
    munmap(b.mem, b.bytes);
    delete[] b.entries;
  }
}

int Freelist::grow(size_t count) {
  if (opt_.max_count) {
    if (total_ >= opt_.max_count) return -1;
    if (total_ + count > opt_.max_count) count = opt_.max_count - total_;
  }
  const size_t bytes = round_up(count * stride_, opt_.page_size);
  // fill the page padding with extra entries: registration is by whole pages anyway
  size_t fit = bytes / stride_;
  if (opt_.max_count && total_ + fit > opt_.max_count) fit = opt_.max_count - total_;
  void* mem = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (mem == MAP_FAILED) return -1;
  void* handle = nullptr;
  if (opt_.reg) {
    if (opt_.reg(mem, bytes, &handle) != 0) {
      munmap(mem, bytes);
      return -1;
    }
  }
  Block b{mem, bytes, handle, fit, new FreelistEntry[fit]};
  const size_t rz = round_up(memcheck::REDZONE, opt_.entry_align);
  for (size_t i = 0; i < fit; ++i) {
    char* base = static_cast<char*>(mem) + i * stride_;
    FreelistEntry& e = b.entries[i];
    e.ptr = base + rz;
    e.mr_handle = handle;
    if (opt_.entry_init && opt_.entry_init(e.ptr) != 0) {
      // roll back this block
      if (opt_.entry_fini) for (size_t j = 0; j < i; ++j) opt_.entry_fini(b.entries[j].ptr);
      if (handle && opt_.dereg) opt_.dereg(handle);
      munmap(mem, bytes);
      delete[] b.entries;
      return -1;
    }
  }
  for (size_t i = fit; i-- > 0;) {
    b.entries[i].next = free_head_;
    free_head_ = &b.entries[i];
  }
  memcheck::make_noaccess(mem, bytes);
  blocks_.push_back(b);
  total_ += fit;
  return 0;
}

FreelistEntry* Freelist::entry_alloc() {
  if (!free_head_) {
    if (grow(opt_.grow_count) != 0 || !free_head_) return nullptr;
  }
  FreelistEntry* e = free_head_;
  free_head_ = e->next;
  e->next = nullptr;
  ++in_use_;
  memcheck::make_undefined(e->ptr, opt_.entry_size);
  return e;
}

void Freelist::entry_free(FreelistEntry* e) {
  B200NET_ASSERT_ALWAYS(e != nullptr && in_use_ > 0);
  memcheck::make_noaccess(e->ptr, round_up(opt_.entry_size, memcheck::GRANULARITY));
  e->next = free_head_;
  free_head_ = e;
  --in_use_;
}

}  // namespace b200net
