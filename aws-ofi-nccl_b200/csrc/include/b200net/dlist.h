// Intrusive circular doubly-linked list: the node is embedded in the element, so insert/remove
// never allocate (reference: include/nccl_ofi_dlist.h).
#pragma once
#include <cstddef>

namespace b200net {

struct DListNode {
  DListNode* prev = this;
  DListNode* next = this;
  bool linked() const { return next != this; }
};

class DList {
 public:
  bool empty() const { return head_.next == &head_; }
  void push_back(DListNode* n) { insert_between(n, head_.prev, &head_); }
  void push_front(DListNode* n) { insert_between(n, &head_, head_.next); }
  DListNode* front() { return empty() ? nullptr : head_.next; }
  DListNode* pop_front() {
    if (empty()) return nullptr;
    DListNode* n = head_.next;
    remove(n);
    return n;
  }
  static void remove(DListNode* n) {
    n->prev->next = n->next;
    n->next->prev = n->prev;
    n->prev = n->next = n;
  }
  // Visit nodes in order; `fn` may remove the node it is given.
  template <typename Fn>
  void for_each_safe(Fn&& fn) {
    DListNode* n = head_.next;
    while (n != &head_) {
      DListNode* nx = n->next;
      fn(n);
      n = nx;
    }
  }
  size_t size() const {
    size_t c = 0;
    for (const DListNode* n = head_.next; n != &head_; n = n->next) ++c;
    return c;
  }

 private:
  static void insert_between(DListNode* n, DListNode* a, DListNode* b) {
    n->prev = a; n->next = b; a->next = n; b->prev = n;
  }
  DListNode head_;
};

// Recover the element from its embedded node.
#define B200NET_CONTAINER_OF(ptr, type, member) \
  reinterpret_cast<type*>(reinterpret_cast<char*>(ptr) - offsetof(type, member))

}  // namespace b200net
