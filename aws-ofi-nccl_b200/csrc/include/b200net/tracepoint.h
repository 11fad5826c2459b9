// Tracepoints: one call per protocol event, fanned out to (a) an in-process ring of trace records
// that can be dumped as Chrome trace-event JSON, (b) NVTX: a begin / end pair of events becomes a
// range in the domain of its communicator (or of its device, NVTX_TRACE_DIMENSION=PER_DEV), every
// other event a mark (NVTX 3 is header-only: with no tool attached the calls do nothing), and
// (c) per-event counters. Disabled events cost one relaxed atomic load.
// B200NET_TRACE = ring | nvtx | all switches it on when the plugin starts; B200NET_TRACE_FILE
// receives the ring as Chrome trace JSON at finalize.
// The event vocabulary follows the reference's LTTng/NVTX layer (include/nccl_ofi_tracepoint.h,
// include/tracing_impl/lttng.h, nvtx.h) so traces of the two plugins can be read side by side.
#pragma once
#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

namespace b200net::trace {

enum class Event : uint16_t {
  Send, SendEnd, SendEagerStart, SendEagerComplete, WriteCtrlStart, WriteCtrlEnd, SendWriteSegmentStart,
  SendWriteSegmentComplete, Recv, RecvEnd, RecvSegmentComplete, EagerRecv, ProcessCompletionsRdma,
  ProcessCompletionsSendRecv, Flush, Read, Write, PendingQueueInsert, PendingQueueRemove,
  CmConnect, CmAccept, CmConnResp,
  GinPutBegin, GinPutEnd, GinPutSignalBegin, GinPutSignalEnd, GinGetBegin, GinGetEnd, GinFlushBegin, GinFlushEnd,
  GinSignalDeliver, GinAckSend, GinAckRecv, GinMetadataSend, GinMetadataRecv, GinWriteBegin, GinWriteEnd,
  GinProgress, GinRegMr, GinDeregMr, GinConnect, GinClose,
  NumEvents
};
const char* event_name(Event e);

struct Record {
  uint64_t ts_ns;
  Event ev;
  uint16_t dev;
  uint32_t comm_id;
  uint32_t seq;
  uint64_t size;
  const void* req;  // request pointer, to correlate begin/end pairs
};

enum class NvtxDimension { PER_COMM, PER_DEV };

void enable(bool ring, bool nvtx);
bool enabled();
void emit(Event ev, int dev, uint32_t comm_id, uint32_t seq, uint64_t size, const void* req);
uint64_t count(Event ev);
void reset_counts();
std::vector<Record> snapshot_ring();
// Chrome "trace event" JSON (one instant event per record) for chrome://tracing / Perfetto.
std::string to_chrome_json(const std::vector<Record>& recs);
bool nvtx_available();
NvtxDimension nvtx_dimension();
// Reads B200NET_TRACE / B200NET_TRACE_FILE (plugin start), writes the file (plugin finalize).
void enable_from_params();
void write_trace_file();

// Where NVTX calls go. The default sink calls NVTX 3; tests install one that records.
struct NvtxSink {
  void* (*domain_create)(const char* name);
  uint64_t (*range_start)(void* domain, const char* message, uint32_t argb, uint64_t payload);
  void (*range_end)(void* domain, uint64_t id);
  void (*mark)(void* domain, const char* message, uint32_t argb, uint64_t payload);
};
void set_nvtx_sink(const NvtxSink* sink);   // nullptr restores the default; drops open ranges
// The event that closes the range `begin` opens, or NumEvents when `begin` opens none.
Event range_end_of(Event begin);
size_t nvtx_open_ranges();

}  // namespace b200net::trace

#define B200NET_TRACE_EVENT(ev, dev, comm, seq, size, req)                                        \
  do {                                                                                            \
    if (::b200net::trace::enabled())                                                              \
      ::b200net::trace::emit(::b200net::trace::Event::ev, (dev), (comm), (seq), (size), (req));   \
  } while (0)
