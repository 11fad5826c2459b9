#include "b200net/tracepoint.h"

#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

#include <nvtx3/nvToolsExt.h>

#include "b200net/log.h"
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

// ---- NVTX -----------------------------------------------------------------------------------------
// (reference: include/tracing_impl/nvtx.h — one domain per communicator or per device, ranges for
// send / eager / control / write segment / receive / flush, colours per kind)
namespace {

void* real_domain_create(const char* name) { return nvtxDomainCreateA(name); }
nvtxEventAttributes_t attributes(const char* message, uint32_t argb, uint64_t payload) {
  nvtxEventAttributes_t a{};
  a.version = NVTX_VERSION;
  a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
  a.colorType = NVTX_COLOR_ARGB;
  a.color = argb;
  a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64;
  a.payload.ullValue = payload;
  a.messageType = NVTX_MESSAGE_TYPE_ASCII;
  a.message.ascii = message;
  return a;
}
uint64_t real_range_start(void* d, const char* message, uint32_t argb, uint64_t payload) {
  const nvtxEventAttributes_t a = attributes(message, argb, payload);
  return nvtxDomainRangeStartEx(static_cast<nvtxDomainHandle_t>(d), &a);
}
void real_range_end(void* d, uint64_t id) { nvtxDomainRangeEnd(static_cast<nvtxDomainHandle_t>(d), id); }
void real_mark(void* d, const char* message, uint32_t argb, uint64_t payload) {
  const nvtxEventAttributes_t a = attributes(message, argb, payload);
  nvtxDomainMarkEx(static_cast<nvtxDomainHandle_t>(d), &a);
}
const NvtxSink kRealSink{real_domain_create, real_range_start, real_range_end, real_mark};

struct RangePair { Event begin, end; uint32_t argb; };
constexpr RangePair kRanges[] = {
    {Event::Send, Event::SendEnd, 0xFF2E86DE},
    {Event::SendEagerStart, Event::SendEagerComplete, 0xFF54A0FF},
    {Event::WriteCtrlStart, Event::WriteCtrlEnd, 0xFFFECA57},
    {Event::SendWriteSegmentStart, Event::SendWriteSegmentComplete, 0xFF1DD1A1},
    {Event::Recv, Event::RecvEnd, 0xFFEE5253},
    {Event::GinPutBegin, Event::GinPutEnd, 0xFF5F27CD},
    {Event::GinPutSignalBegin, Event::GinPutSignalEnd, 0xFF8854D0},
    {Event::GinGetBegin, Event::GinGetEnd, 0xFF00D2D3},
    {Event::GinFlushBegin, Event::GinFlushEnd, 0xFF576574},
    {Event::GinWriteBegin, Event::GinWriteEnd, 0xFF10AC84},
};
constexpr uint32_t kMarkColour = 0xFFC8D6E5;

std::mutex g_nvtx_mu;
const NvtxSink* g_sink = &kRealSink;
std::map<uint64_t, void*> g_domains;   // (dimension, id) -> domain
// open ranges: (begin event, communicator, request or — for events without one — sequence number)
// -> ids, oldest first; the segments of one message share a key and close in the order they were
// opened
std::multimap<std::tuple<uint16_t, uint32_t, uint64_t>, std::pair<void*, uint64_t>> g_open;
uint64_t range_key(const void* req, uint32_t seq) { return req ? reinterpret_cast<uintptr_t>(req) : seq; }

void* domain_for(int dev, uint32_t comm_id) {
  const bool per_dev = nvtx_dimension() == NvtxDimension::PER_DEV;
  const uint64_t key = (static_cast<uint64_t>(per_dev) << 63) | (per_dev ? static_cast<uint32_t>(dev) : comm_id);
  auto it = g_domains.find(key);
  if (it != g_domains.end()) return it->second;
  char name[64];
  if (per_dev) snprintf(name, sizeof(name), "b200net_dev_%d", dev);
  else snprintf(name, sizeof(name), "b200net_comm_%u", comm_id);
  void* d = g_sink->domain_create(name);
  g_domains.emplace(key, d);
  return d;
}

void nvtx_emit(Event ev, int dev, uint32_t comm_id, uint32_t seq, uint64_t size, const void* req) {
  std::lock_guard<std::mutex> g(g_nvtx_mu);
  for (const RangePair& rp : kRanges) {
    if (ev == rp.begin) {
      void* d = domain_for(dev, comm_id);
      char msg[96];
      snprintf(msg, sizeof(msg), "%s seq=%u", event_name(ev), seq);
      const uint64_t id = g_sink->range_start(d, msg, rp.argb, size);
      g_open.emplace(std::make_tuple(static_cast<uint16_t>(ev), comm_id, range_key(req, seq)), std::make_pair(d, id));
      return;
    }
    if (ev == rp.end) {
      auto it = g_open.find(std::make_tuple(static_cast<uint16_t>(rp.begin), comm_id, range_key(req, seq)));
      if (it == g_open.end()) return;   // the range was opened before tracing was switched on
      g_sink->range_end(it->second.first, it->second.second);
      g_open.erase(it);
      return;
    }
  }
  char msg[96];
  snprintf(msg, sizeof(msg), "%s seq=%u", event_name(ev), seq);
  g_sink->mark(domain_for(dev, comm_id), msg, kMarkColour, size);
}

}  // namespace

Event range_end_of(Event begin) {
  for (const RangePair& rp : kRanges)
    if (rp.begin == begin) return rp.end;
  return Event::NumEvents;
}

void set_nvtx_sink(const NvtxSink* sink) {
  std::lock_guard<std::mutex> g(g_nvtx_mu);
  g_sink = sink ? sink : &kRealSink;
  g_domains.clear();
  g_open.clear();
}

size_t nvtx_open_ranges() {
  std::lock_guard<std::mutex> g(g_nvtx_mu);
  return g_open.size();
}

bool nvtx_available() { return true; }   // header-only NVTX 3: the calls do nothing without a tool

NvtxDimension nvtx_dimension() {
  return params().nvtx_trace_dimension.get() == "PER_DEV" ? NvtxDimension::PER_DEV : NvtxDimension::PER_COMM;
}

void enable(bool ring, bool nvtx) {
  g_ring.store(ring);
  g_nvtx.store(nvtx);
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
  if (g_nvtx.load(std::memory_order_relaxed)) nvtx_emit(ev, dev, comm_id, seq, size, req);
}

void enable_from_params() {
  const std::string& mode = params().trace.get();
  if (mode == "none") return;
  enable(mode == "ring" || mode == "all", mode == "nvtx" || mode == "all");
}

void write_trace_file() {
  std::string path = params().trace_file.get();
  if (path.empty() || !g_ring.load()) return;
  const size_t at = path.find("%p");
  if (at != std::string::npos) path.replace(at, 2, std::to_string(getpid()));
  if (FILE* f = fopen(path.c_str(), "w")) {
    const std::string js = to_chrome_json(snapshot_ring());
    fwrite(js.data(), 1, js.size(), f);
    fputc('\n', f);
    fclose(f);
  } else {
    NET_WARN("cannot write the trace file %s", path.c_str());
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
