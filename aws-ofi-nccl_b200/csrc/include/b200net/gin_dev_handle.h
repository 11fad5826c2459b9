// The device-visible contract of kernel-initiated GIN: what ncclGinPlugin_v14.createContext and
// regMrSym upload to the GPU and what the device API (kernels/gin_device.cuh) reads. One header,
// included by the host plugin (plain C++) and by device code, so that both sides agree on every
// field and every offset
// (reference: include/rdma/gin/nccl_ofi_gin_gdaki_dev.h:302-382 — the handle a kernel indexes to
// reach its queues and signal words; src/rdma/gin/nccl_ofi_gin_gdaki.cpp:502-906 builds it).
//
// A context owns a control pad of GIN_PAD_BYTES on every rank's GPU. All pads are mapped into
// every rank's address space; a kernel reaches a peer's signal word, barrier flag or counter by
// pad[peer] + offset with the offsets below.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace b200 {

constexpr int GIN_MAX_RANKS = 8;
constexpr int GIN_MAX_BLOCKS = 256;    // barrier slots per channel
constexpr int GIN_NUM_CHANNELS = 8;    // independent barrier sets (one per concurrently used stream)
constexpr int GIN_MAX_SIGNALS = 4096;
constexpr int GIN_MAX_COUNTERS = 1024;

// Layout of the control pad (one per rank, symmetric):
constexpr size_t GIN_PAD_FLAGS_OFF = 0;                                   // u32 [channel][block][src rank]
constexpr size_t GIN_PAD_FLAGS_BYTES = size_t(GIN_NUM_CHANNELS) * GIN_MAX_BLOCKS * GIN_MAX_RANKS * 4;
constexpr size_t GIN_PAD_EPOCH_OFF = GIN_PAD_FLAGS_OFF + GIN_PAD_FLAGS_BYTES;  // u32 [channel][block], local only
constexpr size_t GIN_PAD_EPOCH_BYTES = size_t(GIN_NUM_CHANNELS) * GIN_MAX_BLOCKS * 4;
constexpr size_t GIN_PAD_SIGNAL_OFF = GIN_PAD_EPOCH_OFF + GIN_PAD_EPOCH_BYTES;  // u64 [signal]
constexpr size_t GIN_PAD_SIGNAL_BYTES = size_t(GIN_MAX_SIGNALS) * 8;
constexpr size_t GIN_PAD_SIGBASE_OFF = GIN_PAD_SIGNAL_OFF + GIN_PAD_SIGNAL_BYTES;  // u64 [signal], local reset offsets
constexpr size_t GIN_PAD_COUNTER_OFF = GIN_PAD_SIGBASE_OFF + GIN_PAD_SIGNAL_BYTES;  // u64 [counter], local
constexpr size_t GIN_PAD_COUNTER_BYTES = size_t(GIN_MAX_COUNTERS) * 8;
constexpr size_t GIN_PAD_SCRATCH_OFF = GIN_PAD_COUNTER_OFF + GIN_PAD_COUNTER_BYTES;  // free for kernels
constexpr size_t GIN_PAD_BYTES = 2u << 20;
// The last 64 bytes of the pad hold the status word of a context that the plugin created (kernels
// of the device library keep theirs elsewhere and point `status` at it).
constexpr size_t GIN_PAD_STATUS_OFF = GIN_PAD_BYTES - 64;

struct GinDevHandle {
  int rank;
  int nranks;
  uint8_t* window[GIN_MAX_RANKS];  // data window of every rank, mapped in this GPU's address space
  uint8_t* mc_window;              // multicast alias of the data window (null without NVLS)
  uint8_t* pad[GIN_MAX_RANKS];     // control pad of every rank
  size_t window_bytes;
  int* status;                     // device status word (first error wins)
  uint64_t wait_limit_ns;
};

// One symmetric registration as a kernel sees it: where the registered range of every rank is
// mapped in this GPU's address space (regMrSym of the kernel-initiated table hands out the device
// address of one of these).
struct GinDevWindow {
  uint8_t* base[GIN_MAX_RANKS];
  size_t bytes;
};

}  // namespace b200
