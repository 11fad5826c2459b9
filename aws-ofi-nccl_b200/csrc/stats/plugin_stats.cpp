#include "b200net/plugin_stats.h"

#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <memory>

#include "b200net/histogram.h"
#include "b200net/log.h"
#include "b200net/param.h"

namespace b200net {
namespace {

using SizeHist = stats::Histogram<uint64_t, stats::Log2Binner<uint64_t>>;
using StripeHist = stats::Histogram<uint64_t, stats::LinearBinner<uint64_t>>;
using NsHist = stats::Histogram<uint64_t, stats::Log2Binner<uint64_t>>;

struct Hists {
  SizeHist send_size{"send_message_size", stats::Log2Binner<uint64_t>(36), "bytes"};
  SizeHist recv_size{"recv_message_size", stats::Log2Binner<uint64_t>(36), "bytes"};
  StripeHist stripes{"stripes_per_send", stats::LinearBinner<uint64_t>(0, 1, 18), "stripes"};
  NsHist send_ns{"send_request_latency", stats::Log2Binner<uint64_t>(40), "ns"};
  NsHist recv_ns{"recv_request_latency", stats::Log2Binner<uint64_t>(40), "ns"};
  NsHist launch_ns{"copy_kernel_launch_call", stats::Log2Binner<uint64_t>(40), "ns"};
  NsHist flag_ns{"copy_kernel_launch_to_completion_seen", stats::Log2Binner<uint64_t>(40), "ns"};
  NsHist poll_gap_ns{"interval_between_progress_calls", stats::Log2Binner<uint64_t>(40), "ns"};
};
Hists* g_hists = nullptr;   // created once, never destroyed (requests may complete during teardown)

struct Named {
  const char* name;
  const PluginStats::Counter PluginStats::*field;
};
const Named kCounters[] = {
    {"sends", &PluginStats::sends},
    {"recvs", &PluginStats::recvs},
    {"send_bytes", &PluginStats::send_bytes},
    {"recv_bytes", &PluginStats::recv_bytes},
    {"eager_sends", &PluginStats::eager_sends},
    {"rendezvous_sends", &PluginStats::rendezvous_sends},
    {"send_backoffs", &PluginStats::send_backoffs},
    {"recv_backoffs", &PluginStats::recv_backoffs},
    {"bytes_copy_kernel", &PluginStats::bytes_kernel},
    {"copy_kernel_launches", &PluginStats::copy_launches},
    {"copy_batch_launches", &PluginStats::copy_batch_launches},
    {"copy_batched_stripes", &PluginStats::copy_batched_stripes},
    {"bytes_copy_engine", &PluginStats::bytes_copy_engine},
    {"bytes_staged_through_host", &PluginStats::bytes_staged},
    {"bytes_host_writes", &PluginStats::bytes_host},
    {"bytes_eager", &PluginStats::bytes_eager},
    {"flushes", &PluginStats::flushes},
    {"requests_failed", &PluginStats::requests_failed},
    {"ipc_maps", &PluginStats::ipc_maps},
    {"ipc_map_failures", &PluginStats::ipc_map_failures},
    {"ipc_map_deferred", &PluginStats::ipc_map_deferred},
    {"connects", &PluginStats::connects},
    {"accepts", &PluginStats::accepts},
    {"endpoints_aborted", &PluginStats::endpoints_aborted},
    {"gin_puts", &PluginStats::gin_puts},
    {"gin_gets", &PluginStats::gin_gets},
    {"gin_signals_applied", &PluginStats::gin_signals_applied},
    {"gin_bytes_direct", &PluginStats::gin_bytes_direct},
    {"gin_bytes_host_writes", &PluginStats::gin_bytes_host},
    {"gin_bytes_fragments", &PluginStats::gin_bytes_fragments},
    {"gin_reads_served", &PluginStats::gin_reads_served},
};

}  // namespace

PluginStats::PluginStats() {
  histograms_ = params().stats_histograms.get() || !params().stats_file.get().empty();
  if (histograms_) g_hists = new Hists;
}

PluginStats& PluginStats::get() {
  static PluginStats* s = new PluginStats;
  return *s;
}

uint64_t PluginStats::now_ns() {
  return static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

void PluginStats::sample_send(size_t bytes, size_t stripes, uint64_t ns) {
  if (!g_hists) return;
  g_hists->send_size.insert(bytes);
  g_hists->stripes.insert(stripes);
  g_hists->send_ns.insert(ns);
}

void PluginStats::sample_launch(uint64_t ns) {
  if (g_hists) g_hists->launch_ns.insert(ns);
}
void PluginStats::sample_kernel_done(uint64_t ns) {
  if (g_hists) g_hists->flag_ns.insert(ns);
}
void PluginStats::sample_poll_gap(uint64_t ns) {
  if (g_hists) g_hists->poll_gap_ns.insert(ns);
}

void PluginStats::sample_recv(size_t bytes, uint64_t ns) {
  if (!g_hists) return;
  g_hists->recv_size.insert(bytes);
  g_hists->recv_ns.insert(ns);
}

void PluginStats::reset() {
  for (const Named& n : kCounters) const_cast<Counter&>(this->*(n.field)).store(0, std::memory_order_relaxed);
}

std::string PluginStats::to_json() const {
  std::string o = "{\"pid\":" + std::to_string(getpid()) + ",\"counters\":{";
  bool first = true;
  for (const Named& n : kCounters) {
    if (!first) o += ",";
    first = false;
    o += std::string("\"") + n.name + "\":" + std::to_string((this->*(n.field)).load(std::memory_order_relaxed));
  }
  o += "},\"histograms\":[";
  if (g_hists) {
    const stats::HistogramBase* all[] = {&g_hists->send_size, &g_hists->recv_size, &g_hists->stripes, &g_hists->send_ns,
                                         &g_hists->recv_ns, &g_hists->launch_ns, &g_hists->flag_ns, &g_hists->poll_gap_ns};
    first = true;
    for (const stats::HistogramBase* h : all) {
      const stats::HistogramSnapshot s = h->snapshot();
      if (!s.samples) continue;
      if (!first) o += ",";
      first = false;
      std::string body = stats::format_histogram(s, stats::PrintFormat::JSON, true);
      while (!body.empty() && (body.back() == '\n' || body.back() == ',')) body.pop_back();
      o += body;
    }
  }
  o += "]}";
  return o;
}

void PluginStats::report() const {
  const uint64_t s = sends.load(), r = recvs.load();
  if (s | r)
    NET_INFO(NCCL_NET,
             "totals: %llu sends (%llu eager, %llu back-offs) %llu bytes; %llu receives (%llu back-offs) %llu bytes; payload by "
             "path: copy kernel %llu, copy engine %llu, staged through host %llu, host writes %llu, eager %llu",
             static_cast<unsigned long long>(s), static_cast<unsigned long long>(eager_sends.load()),
             static_cast<unsigned long long>(send_backoffs.load()), static_cast<unsigned long long>(send_bytes.load()),
             static_cast<unsigned long long>(r), static_cast<unsigned long long>(recv_backoffs.load()),
             static_cast<unsigned long long>(recv_bytes.load()), static_cast<unsigned long long>(bytes_kernel.load()),
             static_cast<unsigned long long>(bytes_copy_engine.load()), static_cast<unsigned long long>(bytes_staged.load()),
             static_cast<unsigned long long>(bytes_host.load()), static_cast<unsigned long long>(bytes_eager.load()));
  if (gin_puts.load() | gin_gets.load())
    NET_INFO(NCCL_NET,
             "GIN totals: %llu puts, %llu gets, %llu signals applied; put payload: %llu bytes direct to device windows, %llu "
             "host writes, %llu as fragments; %llu reads served for peers",
             static_cast<unsigned long long>(gin_puts.load()), static_cast<unsigned long long>(gin_gets.load()),
             static_cast<unsigned long long>(gin_signals_applied.load()), static_cast<unsigned long long>(gin_bytes_direct.load()),
             static_cast<unsigned long long>(gin_bytes_host.load()), static_cast<unsigned long long>(gin_bytes_fragments.load()),
             static_cast<unsigned long long>(gin_reads_served.load()));
  std::string path = params().stats_file.get();
  if (path.empty()) return;
  const size_t at = path.find("%p");
  if (at != std::string::npos) path.replace(at, 2, std::to_string(getpid()));
  if (FILE* f = fopen(path.c_str(), "w")) {
    const std::string js = to_json();
    fwrite(js.data(), 1, js.size(), f);
    fputc('\n', f);
    fclose(f);
  } else {
    NET_WARN("cannot write the statistics file %s", path.c_str());
  }
}

}  // namespace b200net
