// Histograms (binners, printers, registry) and tracepoints (counters, ring, Chrome JSON).
#include <cstring>
#include <string>
#include <cstdlib>
#include <vector>
#include "b200net/histogram.h"
#include "b200net/param.h"
#include "b200net/tracepoint.h"
#include "test_util.h"
using namespace b200net;
using namespace b200net::stats;
int main() {
  LinearBinner<int> lb(10, 5, 4);
  CHECK_EQ(lb.bin_of(0), 0u); CHECK_EQ(lb.bin_of(10), 0u); CHECK_EQ(lb.bin_of(14), 0u); CHECK_EQ(lb.bin_of(15), 1u);
  CHECK_EQ(lb.bin_of(29), 3u); CHECK_EQ(lb.bin_of(1000), 3u); CHECK_EQ(lb.lower_bound(2), 20);
  Log2Binner<uint64_t> l2(8);
  CHECK_EQ(l2.bin_of(0), 0u); CHECK_EQ(l2.bin_of(1), 0u); CHECK_EQ(l2.bin_of(2), 1u); CHECK_EQ(l2.bin_of(1023), 7u);
  CustomBinner<double> cb({0.0, 1.5, 10.0});
  CHECK_EQ(cb.bin_of(-3), 0u); CHECK_EQ(cb.bin_of(1.4), 0u); CHECK_EQ(cb.bin_of(1.5), 1u); CHECK_EQ(cb.bin_of(99), 2u);
  {
    Histogram<int, LinearBinner<int>> h("sizes", lb, "B");
    for (int v : {1, 12, 16, 17, 100}) h.insert(v);
    CHECK_EQ(h.samples(), 5u); CHECK_EQ(h.count(0), 2u); CHECK_EQ(h.count(1), 2u); CHECK_EQ(h.count(3), 1u);
    CHECK_EQ(h.min(), 1); CHECK_EQ(h.max(), 100);
    auto snap = h.snapshot();
    for (auto f : {PrintFormat::TEXT, PrintFormat::TABLE, PrintFormat::CSV, PrintFormat::JSON}) {
      const std::string s = format_histogram(snap, f, true);
      CHECK(s.find("sizes") != std::string::npos);
      CHECK(s.find("20") == std::string::npos || f == PrintFormat::JSON);  // empty bin [20,25) skipped
    }
    CHECK(format_histogram(snap, PrintFormat::CSV, false).find(",20,0") != std::string::npos);
    TimerHistogram<> th("lat");
    { ScopedTimer<TimerHistogram<>> t(th); }
    CHECK_EQ(th.samples(), 1u);
    FILE* devnull = fopen("/dev/null", "w");
    CHECK_EQ(print_all_histograms(devnull), 2u);
    fclose(devnull);
  }
  FILE* devnull = fopen("/dev/null", "w");
  CHECK_EQ(print_all_histograms(devnull), 0u);  // both unregistered at scope exit
  fclose(devnull);

  using namespace b200net::trace;
  CHECK(!enabled());
  B200NET_TRACE_EVENT(Send, 0, 1, 2, 3, nullptr);
  CHECK_EQ(count(Event::Send), 0u);            // disabled: nothing recorded
  enable(true, false);
  int req;
  B200NET_TRACE_EVENT(Send, 1, 7, 42, 4096, &req);
  B200NET_TRACE_EVENT(SendEnd, 1, 7, 42, 4096, &req);
  B200NET_TRACE_EVENT(GinPutSignalBegin, 0, 3, 1, 64, nullptr);
  CHECK_EQ(count(Event::Send), 1u); CHECK_EQ(count(Event::SendEnd), 1u); CHECK_EQ(count(Event::Recv), 0u);
  auto recs = snapshot_ring();
  CHECK_EQ(recs.size(), 3u);
  CHECK(recs[0].ev == Event::Send && recs[0].seq == 42 && recs[0].req == &req && recs[0].size == 4096);
  CHECK(recs[0].ts_ns <= recs[2].ts_ns);
  const std::string js = to_chrome_json(recs);
  CHECK(js.find("\"traceEvents\"") != std::string::npos && js.find("gin_put_signal_begin") != std::string::npos);
  CHECK(!strcmp(event_name(Event::EagerRecv), "Eager_recv"));
  reset_counts();
  CHECK_EQ(count(Event::Send), 0u); CHECK_EQ(snapshot_ring().size(), 0u);
  enable(false, false);

  // ---- NVTX: begin / end pairs become ranges in the domain of their communicator (or device), the
  // rest marks; a recording sink stands in for the profiler
  struct Rec {
    std::vector<std::string> domains, started, marks;
    std::vector<uint64_t> ended;
    uint64_t next = 100;
  };
  static Rec rec;
  static const NvtxSink sink{
      [](const char* name) -> void* { rec.domains.push_back(name); return reinterpret_cast<void*>(rec.domains.size()); },
      [](void* d, const char* m, uint32_t, uint64_t payload) -> uint64_t {
        rec.started.push_back(std::to_string(reinterpret_cast<uintptr_t>(d)) + ":" + m + ":" + std::to_string(payload));
        return rec.next++;
      },
      [](void*, uint64_t id) { rec.ended.push_back(id); },
      [](void*, const char* m, uint32_t, uint64_t) { rec.marks.push_back(m); }};
  set_nvtx_sink(&sink);
  enable(false, true);
  CHECK(enabled());
  B200NET_TRACE_EVENT(Send, 0, 7, 42, 4096, &req);                  // range 100 in comm 7
  B200NET_TRACE_EVENT(SendWriteSegmentStart, 0, 7, 42, 2048, &req); // two segments of one message: 101, 102
  B200NET_TRACE_EVENT(SendWriteSegmentStart, 0, 7, 42, 2048, &req);
  B200NET_TRACE_EVENT(Recv, 0, 9, 42, 1, &req);                     // same sequence number, another communicator
  B200NET_TRACE_EVENT(EagerRecv, 0, 9, 5, 64, nullptr);             // no pair: a mark
  CHECK_EQ(nvtx_open_ranges(), 4u);
  CHECK_EQ(rec.domains.size(), 2u);
  CHECK(rec.domains[0] == "b200net_comm_7" && rec.domains[1] == "b200net_comm_9");
  CHECK(rec.started[0] == "1:Send seq=42:4096");
  CHECK_EQ(rec.marks.size(), 1u);
  CHECK(rec.marks[0] == "Eager_recv seq=5");
  B200NET_TRACE_EVENT(SendWriteSegmentComplete, 0, 7, 42, 2048, &req);
  B200NET_TRACE_EVENT(SendWriteSegmentComplete, 0, 7, 42, 2048, &req);
  B200NET_TRACE_EVENT(SendEnd, 0, 7, 42, 4096, &req);
  B200NET_TRACE_EVENT(SendEnd, 0, 7, 43, 4096, &req);               // never opened: ignored
  CHECK_EQ(nvtx_open_ranges(), 1u);
  CHECK_EQ(rec.ended.size(), 3u);
  CHECK(rec.ended[0] == 101 && rec.ended[1] == 102 && rec.ended[2] == 100);   // segments close oldest first
  B200NET_TRACE_EVENT(RecvEnd, 0, 9, 42, 1, &req);
  CHECK_EQ(nvtx_open_ranges(), 0u);
  CHECK(range_end_of(Event::GinPutSignalBegin) == Event::GinPutSignalEnd);
  CHECK(range_end_of(Event::EagerRecv) == Event::NumEvents);
  // every begin event of the vocabulary has its end
  for (Event b : {Event::Send, Event::SendEagerStart, Event::WriteCtrlStart, Event::SendWriteSegmentStart, Event::Recv,
                  Event::GinPutBegin, Event::GinPutSignalBegin, Event::GinGetBegin, Event::GinFlushBegin, Event::GinWriteBegin})
    CHECK(range_end_of(b) != Event::NumEvents);
  // per-device domains
  setenv("B200NET_NVTX_TRACE_DIMENSION", "PER_DEV", 1);
  b200net::params().nvtx_trace_dimension.reset_for_testing("PER_COMM");
  set_nvtx_sink(&sink);
  rec = Rec{};
  B200NET_TRACE_EVENT(Send, 3, 7, 1, 8, &req);
  B200NET_TRACE_EVENT(Send, 3, 8, 1, 8, &req);
  CHECK_EQ(rec.domains.size(), 1u);
  CHECK(rec.domains[0] == "b200net_dev_3");
  enable(false, false);
  set_nvtx_sink(nullptr);
  // the default sink calls NVTX 3 itself: harmless with no tool attached
  enable(false, true);
  B200NET_TRACE_EVENT(Send, 0, 1, 1, 8, &req);
  B200NET_TRACE_EVENT(SendEnd, 0, 1, 1, 8, &req);
  CHECK_EQ(nvtx_open_ranges(), 0u);
  enable(false, false);
  TEST_MAIN_END();
}
