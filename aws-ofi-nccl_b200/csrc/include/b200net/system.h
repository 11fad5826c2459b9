// Facts about the machine: a node id, the product name (DMI or OFI_NCCL_FORCE_PRODUCT_NAME, which
// lets tests and tools impersonate hardware), the host hash NCCL uses to tell hosts apart, and the
// calling thread's id (reference: src/nccl_ofi_system.cpp, src/nccl_ofi_nccl_compat.cpp).
#pragma once
#include <cstdint>
#include <string>

namespace b200net {
uint32_t system_node_id();          // from the first routable IPv4/IPv6 address; 0 if none
std::string system_product_name();  // "" when unknown
uint64_t system_host_hash();        // hash(hostname + boot id), or hash(NCCL_HOSTID) when set
long current_tid();
}  // namespace b200net
