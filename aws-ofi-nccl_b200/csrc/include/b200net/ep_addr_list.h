// Tracks which peer addresses each endpoint is already connected to, to answer "give me an
// endpoint that has no connection to this address yet" (reference: src/nccl_ofi_ep_addr_list.cpp).
#pragma once
#include "b200net/pthread_wrap.h"
#include <set>
#include <string>
#include <vector>

namespace b200net {

class EpAddrList {
 public:
  // Returns an endpoint not yet paired with addr (and records the pairing), or nullptr.
  void* get(const std::string& addr);
  // Registers a new endpoint already connected to addr. Returns -EINVAL if ep is known.
  int insert(void* ep, const std::string& addr);
  int remove(void* ep);  // -ENOENT if unknown
  size_t size() const;

 private:
  struct Item { void* ep; std::set<std::string> addrs; };
  mutable Mutex mu_;
  std::vector<Item> items_ TSA_GUARDED_BY(mu_);
};

}  // namespace b200net
