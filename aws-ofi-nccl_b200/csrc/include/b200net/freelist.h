// Block-grown pool of fixed-size entries. Blocks are page-padded so an optional registration
// callback (pinning / IPC export of the block) always sees whole pages; entries can carry an
// alignment, redzones (under ASAN) and are poisoned while free. Not thread safe by itself:
// callers hold the endpoint lock (reference: src/nccl_ofi_freelist.cpp, include/nccl_ofi_freelist.h).
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <vector>

namespace b200net {

struct FreelistEntry {
  void* ptr;            // user memory
  void* mr_handle;      // registration handle of the block this entry lives in (or null)
  FreelistEntry* next;  // free-list link
};

class Freelist {
 public:
  using RegFn = std::function<int(void* base, size_t bytes, void** handle)>;
  using DeregFn = std::function<int(void* handle)>;
  using EntryInitFn = std::function<int(void* entry_mem)>;
  using EntryFiniFn = std::function<void(void* entry_mem)>;

  struct Options {
    size_t entry_size = 0;
    size_t initial_count = 0;
    size_t grow_count = 16;   // entries added per growth step
    size_t max_count = 0;     // 0 = unbounded
    size_t entry_align = 8;
    size_t page_size = 4096;
    RegFn reg;
    DeregFn dereg;
    EntryInitFn entry_init;
    EntryFiniFn entry_fini;
    const char* name = "freelist";
  };

  explicit Freelist(Options opt);
  ~Freelist();
  Freelist(const Freelist&) = delete;
  Freelist& operator=(const Freelist&) = delete;

  FreelistEntry* entry_alloc();         // nullptr when max_count is reached or growth fails
  void entry_free(FreelistEntry* e);
  size_t allocated() const { return total_; }
  size_t in_use() const { return in_use_; }
  size_t block_count() const { return blocks_.size(); }
  size_t entry_stride() const { return stride_; }
  // set at destruction when entries were still out; exposed for the leak-path test
  static size_t leaked_entries_total();

 private:
  struct Block { void* mem; size_t bytes; void* mr_handle; size_t count; FreelistEntry* entries; };
  int grow(size_t count);
  Options opt_;
  size_t stride_;
  size_t total_ = 0, in_use_ = 0;
  FreelistEntry* free_head_ = nullptr;
  std::vector<Block> blocks_;
};

}  // namespace b200net
