#include "b200net/system.h"

#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <cstdio>
#include <string>

namespace b200net {

long current_tid() { return static_cast<long>(syscall(SYS_gettid)); }

static uint64_t fnv1a(const void* data, size_t n, uint64_t h = 1469598103934665603ull) {
  const unsigned char* p = static_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * 1099511628211ull;
  return h;
}

uint32_t system_node_id() {
  ifaddrs* ifs = nullptr;
  if (getifaddrs(&ifs) != 0) return 0;
  uint32_t id = 0;
  for (int pass = 0; pass < 2 && !id; ++pass) {  // IPv4 first, then IPv6
    for (ifaddrs* i = ifs; i; i = i->ifa_next) {
      if (!i->ifa_addr || (i->ifa_flags & IFF_LOOPBACK) || !(i->ifa_flags & IFF_UP)) continue;
      if (pass == 0 && i->ifa_addr->sa_family == AF_INET) {
        const auto* a = reinterpret_cast<const sockaddr_in*>(i->ifa_addr);
        const uint32_t v = ntohl(a->sin_addr.s_addr);
        if ((v >> 16) == 0xA9FE) continue;  // link-local 169.254/16
        id = v;
        break;
      }
      if (pass == 1 && i->ifa_addr->sa_family == AF_INET6) {
        const auto* a = reinterpret_cast<const sockaddr_in6*>(i->ifa_addr);
        if (IN6_IS_ADDR_LINKLOCAL(&a->sin6_addr)) continue;
        id = static_cast<uint32_t>(fnv1a(&a->sin6_addr, sizeof(a->sin6_addr)));
        break;
      }
    }
  }
  freeifaddrs(ifs);
  return id;
}

std::string system_product_name() {
  if (const char* f = getenv("OFI_NCCL_FORCE_PRODUCT_NAME")) return f;
  if (const char* f = getenv("B200NET_FORCE_PRODUCT_NAME")) return f;
  char buf[256] = {0};
  if (FILE* f = fopen("/sys/devices/virtual/dmi/id/product_name", "r")) {
    const bool got = fgets(buf, sizeof(buf), f) != nullptr;
    fclose(f);
    if (got) {
      std::string s(buf);
      while (!s.empty() && (s.back() == '\n' || s.back() == ' ')) s.pop_back();
      return s;
    }
  }
  return "";
}

uint64_t system_host_hash() {
  if (const char* h = getenv("NCCL_HOSTID")) return fnv1a(h, strlen(h));
  char host[256] = {0};
  gethostname(host, sizeof(host) - 1);
  uint64_t h = fnv1a(host, strlen(host));
  char boot[128] = {0};
  if (FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r")) {
    if (fgets(boot, sizeof(boot), f)) h = fnv1a(boot, strlen(boot), h);
    fclose(f);
  }
  return h;
}

}  // namespace b200net
