#include "b200net/ep_addr_list.h"

#include <cerrno>

namespace b200net {

void* EpAddrList::get(const std::string& addr) {
  ScopedLock g(mu_);
  for (auto& it : items_) {
    if (!it.addrs.count(addr)) {
      it.addrs.insert(addr);
      return it.ep;
    }
  }
  return nullptr;
}

int EpAddrList::insert(void* ep, const std::string& addr) {
  ScopedLock g(mu_);
  for (auto& it : items_)
    if (it.ep == ep) return -EINVAL;
  items_.push_back(Item{ep, {addr}});
  return 0;
}

int EpAddrList::remove(void* ep) {
  ScopedLock g(mu_);
  for (auto it = items_.begin(); it != items_.end(); ++it) {
    if (it->ep == ep) {
      items_.erase(it);
      return 0;
    }
  }
  return -ENOENT;
}

size_t EpAddrList::size() const {
  ScopedLock g(mu_);
  return items_.size();
}

}  // namespace b200net
