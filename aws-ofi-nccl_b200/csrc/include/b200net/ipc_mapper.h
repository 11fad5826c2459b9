// Opening a peer's device allocation (cuIpcOpenMemHandle) can wait for the device to go idle. The
// thread that drives the plugin is NCCL's proxy: if it waits for the device while a collective
// kernel on that device waits for the proxy's data, neither moves. So the open runs on a helper
// thread; the caller waits a short grace period (the common case finishes well within it) and
// otherwise sends through host fragments until the mapping has arrived.
//
// The reference never needs this: its peers are reached through the NIC, not through a mapping of
// their memory (registration there is fi_mr_reg, src/nccl_ofi_rdma.cpp:2655-2760, which does not
// depend on the device being idle).
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>

#include "b200net/cuda_shim.h"

namespace b200net {

// What the 64 handle bytes of a CUDA_VMM registration hold.
struct VmmShare {
  uint32_t magic;    // VMM_SHARE_MAGIC
  int32_t fd;        // descriptor number in the owner's process
  uint32_t pid;      // the owner
  uint32_t pad;
  uint64_t bytes;    // size of the mapped range the descriptor stands for
  uint64_t serial;   // unique per export in the owner: descriptor numbers are reused, mappings are cached by these bytes
};
constexpr uint32_t VMM_SHARE_MAGIC = 0x564d4d31;   // "VMM1"

struct IpcMapJob {
  bool vmm = false;                  // handle holds a VmmShare instead of a legacy IPC handle
  size_t bytes = 0;                  // of the mapping (virtual-memory API only)
  // Undoes what the helper did (state == 1 only).
  int close_mapping() const { return vmm ? cuda::vmm_unmap(mapped, bytes) : cuda::ipc_close(mapped); }
  uint8_t handle[64];
  cuda::Context ctx = nullptr;       // made current on the helper thread before the open
  std::atomic<int> state{0};         // 0 in progress, 1 mapped, 2 abandoned by its owner, negative errno
  void* mapped = nullptr;            // valid once state == 1 (acquire)
  bool waited = false;               // owner's note: the grace period has been spent on this open already
  // The owner is going away. True: the mapping exists and the caller must close it. False: it does
  // not exist (failed, or still in progress: the helper closes it when it arrives).
  bool abandon() {
    int expected = 0;
    if (state.compare_exchange_strong(expected, 2, std::memory_order_acq_rel)) return false;
    return expected == 1;
  }
};

class IpcMapper {
 public:
  static IpcMapper& instance();
  // Queues the open. Never blocks on the device. nullptr if the helper thread could not start.
  std::shared_ptr<IpcMapJob> submit(const uint8_t handle[64], cuda::Context ctx, bool vmm = false);
  // The same open on the calling thread, for set-up paths where waiting for the device is harmless
  // (collective registration). 0 or a negative errno; *bytes is the mapping's size for close_now().
  static int open_now(const uint8_t handle[64], bool vmm, void** mapped, size_t* bytes);
  static int close_now(void* mapped, bool vmm, size_t bytes);
  // Polls job->state for at most wait_us microseconds; returns the state seen last.
  static int wait(const IpcMapJob& job, uint64_t wait_us);
};

}  // namespace b200net
