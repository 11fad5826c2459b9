#include "b200net/tracepoint.h"

#include <dlfcn.h>

#include <chrono>
#include <mutex>
#include <cstdio>

#include "b200net/param.h"

namespace b200net::trace {

static const char* kNames[] = {
    "Send", "SendEnd", "Send_eager_start", "Send_eager_complete", "Write_ctrl_start", "Write_ctrl_end",
    "Send_write_segment_start", "Send_write_segment_complete", "Recv", "RecvEnd", "Recv_segment_complete",
    "Eager_recv", "ProcessCompletionsRdma", "ProcessCompletionsSendRecv", "Flush", "Read", "Write",
    "Pending_queue_insert", "Pending_queue_remove", "Cm_connect", "Cm_accept", "Cm_conn_resp",
    "gin_put_begin", "gin_put_end", "gin_put_signal_begin", "gin_put_signal_end", "gin_get_begin", "gin_get_end",
    "gin_flush_begin", "gin_flush_end", "gin_signal_deliver", "gin_ack_send", "gin_ack_recv", "gin_metadata_send",
    "gin_metadata_recv", "gin_write_begin", "gin_write_end", "gin_progress", "gin_reg_mr", "gin_dereg_mr",
    "gin_connect", "gin_close"};
static_assert(sizeof(kNames) / sizeof(kNames[0]) == static_cast<size_t>(Event::NumEvents), "name table out of date");

const char* event_name(Event e) { return kNames[static_cast<size_t>(e)]; }

static std::atomic<bool> g_ring{false}, g_nvtx{false};
static std::atomic<uint64_t> g_counts[static_cast<size_t>(Event::NumEvents)];
static constexpr size_t RING = 1 << 16;
static Record g_recs[RING];
static std::atomic<uint64_t> g_head{0};

using MarkFn = void (*)(const char*);
static MarkFn g_mark = nullptr;
static std::once_flag g_nvtx_once;

static void load_nvtx() {
  for (const char* lib : {"libnvToolsExt.so.1", "libnvToolsExt.so"}) {
    if (void* h = dlopen(lib, RTLD_NOW | RTLD_LOCAL)) {
      g_mark = reinterpret_cast<MarkFn>(dlsym(h, "nvtxMarkA"));
      if (g_mark) return;
    }
  }
}

bool nvtx_available() {
  std::call_once(g_nvtx_once, load_nvtx);
  return g_mark != nullptr;
}

NvtxDimension nvtx_dimension() {
  return params().nvtx_trace_dimension.get() == "PER_DEV" ? NvtxDimension::PER_DEV : NvtxDimension::PER_COMM;
}

void enable(bool ring, bool nvtx) {
  g_ring.store(ring);
  g_nvtx.store(nvtx && nvtx_available());
}
bool enabled() { return g_ring.load(std::memory_order_relaxed) || g_nvtx.load(std::memory_order_relaxed); }

void emit(Event ev, int dev, uint32_t comm_id, uint32_t seq, uint64_t size, const void* req) {
  g_counts[static_cast<size_t>(ev)].fetch_add(1, std::memory_order_relaxed);
  if (g_ring.load(std::memory_order_relaxed)) {
    const uint64_t i = g_head.fetch_add(1, std::memory_order_relaxed);
    const auto now = std::chrono::steady_clock::now().time_since_epoch();
    g_recs[i % RING] = Record{static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(now).count()),
                              ev, static_cast<uint16_t>(dev), comm_id, seq, size, req};
  }
  if (g_nvtx.load(std::memory_order_relaxed) && g_mark) {
    char buf[96];
    // PER_COMM names the mark after the communicator, PER_DEV after the device (rail)
    if (nvtx_dimension() == NvtxDimension::PER_COMM)
      snprintf(buf, sizeof(buf), "%s comm=%u seq=%u", event_name(ev), comm_id, seq);
    else
      snprintf(buf, sizeof(buf), "%s dev=%d seq=%u", event_name(ev), dev, seq);
    g_mark(buf);
  }
}

uint64_t count(Event ev) { return g_counts[static_cast<size_t>(ev)].load(); }
void reset_counts() {
  for (auto& c : g_counts) c.store(0);
  g_head.store(0);
}

std::vector<Record> snapshot_ring() {
  const uint64_t head = g_head.load();
  const uint64_t n = head < RING ? head : RING;
  std::vector<Record> out;
  out.reserve(n);
  for (uint64_t i = head - n; i < head; ++i) out.push_back(g_recs[i % RING]);
  return out;
}

std::string to_chrome_json(const std::vector<Record>& recs) {
  std::string o = "{\"traceEvents\":[";
  char buf[384];
  for (size_t i = 0; i < recs.size(); ++i) {
    const Record& r = recs[i];
    snprintf(buf, sizeof(buf),
             "%s{\"name\":\"%s\",\"ph\":\"i\",\"s\":\"t\",\"ts\":%.3f,\"pid\":%u,\"tid\":%u,"
             "\"args\":{\"seq\":%u,\"size\":%llu,\"req\":\"%p\"}}",
             i ? "," : "", event_name(r.ev), r.ts_ns / 1000.0, static_cast<unsigned>(r.dev), r.comm_id, r.seq,
             static_cast<unsigned long long>(r.size), r.req);
    o += buf;
  }
  o += "]}";
  return o;
}

}  // namespace b200net::trace
