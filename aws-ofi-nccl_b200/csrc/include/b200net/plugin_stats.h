// Process-wide counters of the net plugin and, when asked for, histograms of message sizes,
// stripes per message and request latencies. Counters are relaxed atomics and always on; the
// histograms (a mutex per insert) run only with B200NET_STATS_HISTOGRAMS=1 or a stats file.
// At finalize the counters go to the log at INFO level and, with B200NET_STATS_FILE=<path>
// ("%p" becomes the process id), to that file as one JSON object together with the histograms.
//
// The reference reports an MR-cache summary, freelist leaks and its histograms at teardown
// (src/nccl_ofi_mr.cpp:34, src/nccl_ofi_freelist.cpp:141, src/nccl_ofi_api.cpp:99); this adds the
// per-path byte counts and back-off counts that explain a bandwidth number.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <string>

namespace b200net {

struct PluginStats {
  using Counter = std::atomic<uint64_t>;
  Counter sends{0}, recvs{0}, send_bytes{0}, recv_bytes{0};
  Counter eager_sends{0}, rendezvous_sends{0};
  Counter send_backoffs{0}, recv_backoffs{0};   // calls answered with "no request, call again"
  Counter bytes_kernel{0}, bytes_copy_engine{0}, bytes_staged{0}, bytes_host{0}, bytes_eager{0};
  Counter copy_launches{0}, copy_batch_launches{0}, copy_batched_stripes{0};   // kernel launches; those of the batch kernel; stripes they carried
  Counter flushes{0}, requests_failed{0};
  Counter ipc_maps{0}, ipc_map_failures{0}, ipc_map_deferred{0};
  Counter connects{0}, accepts{0}, endpoints_aborted{0};
  // GIN / RMA: operations and where their payload went
  Counter gin_puts{0}, gin_gets{0}, gin_signals_applied{0};
  Counter gin_bytes_direct{0}, gin_bytes_host{0}, gin_bytes_fragments{0}, gin_reads_served{0};

  static PluginStats& get();
  static void bump(Counter& c, uint64_t n = 1) { c.fetch_add(n, std::memory_order_relaxed); }

  bool histograms_on() const { return histograms_; }
  // One completed send / receive (bytes moved, stripes it was cut into, nanoseconds from the
  // accepted post to completion); no-ops unless histograms are on.
  void sample_send(size_t bytes, size_t stripes, uint64_t ns);
  void sample_recv(size_t bytes, uint64_t ns);
  // Where a send's time goes: the launch call itself, launch to the completion word being seen by
  // the proxy thread, and how often that thread comes round to this endpoint.
  void sample_launch(uint64_t ns);
  void sample_kernel_done(uint64_t ns);
  void sample_poll_gap(uint64_t ns);

  static uint64_t now_ns();
  // Nanoseconds since a request's post time (0 when that was not recorded).
  static uint64_t since(uint64_t t_post_ns) { return t_post_ns ? now_ns() - t_post_ns : 0; }

  std::string to_json() const;
  // Logs the counters and writes the stats file if one was asked for. Called at finalize.
  void report() const;
  void reset();   // for tests

 private:
  PluginStats();
  bool histograms_ = false;
};

}  // namespace b200net
