// Histograms (binners, printers, registry) and tracepoints (counters, ring, Chrome JSON).
#include <cstring>
#include <string>
#include "b200net/histogram.h"
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
  TEST_MAIN_END();
}
