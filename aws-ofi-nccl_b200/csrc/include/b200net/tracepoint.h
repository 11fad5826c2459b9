// Tracepoints: one call per protocol event, fanned out to (a) an in-process ring of trace records
// that can be dumped as Chrome trace-event JSON, (b) NVTX ranges/marks when libnvToolsExt can be
// dlopen()ed, and (c) per-event counters. Disabled events cost one relaxed atomic load.
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

}  // namespace b200net::trace

#define B200NET_TRACE_EVENT(ev, dev, comm, seq, size, req)                                        \
  do {                                                                                            \
    if (::b200net::trace::enabled())                                                              \
      ::b200net::trace::emit(::b200net::trace::Event::ev, (dev), (comm), (seq), (size), (req));   \
  } while (0)
