// Typed runtime parameters. Each parameter has a default, may be overridden by the environment
// (name OFI_NCCL_<NAME>, or B200NET_<NAME> which wins when both are set) and may be set through
// the API — but only until its first get(): after a value has been observed it is frozen, so the
// plugin never sees two different values of one knob (reference: include/nccl_ofi_param_impl.h
// :197-314, the list in include/nccl_ofi_param.h).
#pragma once
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace b200net {

enum class ParamSource { DEFAULT, ENVIRONMENT, API };

class ParamBase {
 public:
  ParamBase(const char* name, const char* doc);
  virtual ~ParamBase();   // leaves the registry
  const std::string& name() const { return name_; }
  const std::string& doc() const { return doc_; }
  virtual std::string value_string() = 0;
  virtual int load_from_env() = 0;  // 0 ok, -EINVAL on an unparsable value
  ParamSource source() const { return source_; }

 protected:
  static const char* find_env(const std::string& name);
  std::string name_, doc_;
  ParamSource source_ = ParamSource::DEFAULT;
};

// Says once per parameter that a retired setting was found in the environment.
void warn_retired(const std::string& name, const char* advice, bool removed);

// Registry of every parameter object (for init-time env parsing and for dumps).
std::vector<ParamBase*>& param_registry();
// Parse the environment for every registered parameter; returns -EINVAL if any value is malformed.
int parameters_init();

namespace detail {
bool parse_value(const char* s, bool& out);
bool parse_value(const char* s, int64_t& out);
bool parse_value(const char* s, uint64_t& out);
bool parse_value(const char* s, int& out);
bool parse_value(const char* s, unsigned& out);
bool parse_value(const char* s, float& out);
bool parse_value(const char* s, std::string& out);
std::string to_string_value(bool v);
std::string to_string_value(const std::string& v);
template <typename T>
std::string to_string_value(const T& v) { return std::to_string(v); }
}  // namespace detail

template <typename T>
class Param : public ParamBase {
 public:
  Param(const char* name, T def, const char* doc = "") : ParamBase(name, doc), value_(std::move(def)) {}

  // First get() freezes the value.
  const T& get() {
    // once read, a value can no longer change (set() refuses): later reads take no lock. Hot paths
    // read several parameters per message.
    if (fast_.load(std::memory_order_acquire)) return value_;
    std::lock_guard<std::mutex> g(mu_);
    if (!loaded_) load_locked();
    frozen_ = true;
    fast_.store(true, std::memory_order_release);
    return value_;
  }
  const T& operator()() { return get(); }

  // 0 on success; -EINVAL once the value has been read.
  int set(const T& v) {
    std::lock_guard<std::mutex> g(mu_);
    if (frozen_) return -22;
    value_ = v;
    source_ = ParamSource::API;
    loaded_ = true;
    return 0;
  }
  int load_from_env() override {
    std::lock_guard<std::mutex> g(mu_);
    return load_locked();
  }
  std::string value_string() override { return detail::to_string_value(get()); }
  // test hook: forget the frozen state and the cached value
  void reset_for_testing(const T& def) {
    std::lock_guard<std::mutex> g(mu_);
    fast_.store(false, std::memory_order_release);
    value_ = def; loaded_ = false; frozen_ = false; source_ = ParamSource::DEFAULT;
  }

 protected:
  virtual bool accept(const T&) const { return true; }
  int load_locked() {
    loaded_ = true;
    if (source_ == ParamSource::API) return 0;
    const char* e = find_env(name_);
    if (!e) return 0;
    T parsed{};
    if (!detail::parse_value(e, parsed) || !accept(parsed)) return -22;
    value_ = parsed;
    source_ = ParamSource::ENVIRONMENT;
    return 0;
  }
  std::mutex mu_;
  T value_;
  bool loaded_ = false, frozen_ = false;
  std::atomic<bool> fast_{false};   // set once frozen: value_ is immutable from then on
};

// A parameter that is on its way out (still read, with a warning) or gone (setting it is an error
// at start-up, so that a script that relies on it does not run with something else silently)
// (reference: include/nccl_ofi_param_impl.h:318-345, OFI_NCCL_PARAM_DEPRECATED / _REMOVED).
template <typename T>
class RetiredParam : public Param<T> {
 public:
  RetiredParam(const char* name, T def, const char* advice, bool error_on_use)
      : Param<T>(name, std::move(def), advice), advice_(advice), error_on_use_(error_on_use) {}
  int load_from_env() override {
    const int rc = Param<T>::load_from_env();
    if (rc != 0) return rc;
    if (this->source() == ParamSource::DEFAULT) return 0;
    warn_retired(this->name(), advice_, error_on_use_);
    return error_on_use_ ? -22 : 0;
  }

 private:
  const char* advice_;
  bool error_on_use_;
};

// String parameter restricted to a fixed set of spellings (case-insensitive), e.g. PROTOCOL.
class EnumParam : public Param<std::string> {
 public:
  EnumParam(const char* name, std::string def, std::vector<std::string> allowed, const char* doc = "")
      : Param<std::string>(name, std::move(def), doc), allowed_(std::move(allowed)) {}
  const std::vector<std::string>& allowed() const { return allowed_; }

 protected:
  bool accept(const std::string& v) const override;
  std::vector<std::string> allowed_;
};

// ---- the knobs ---------------------------------------------------------------------------------
struct Params {
  EnumParam protocol{"PROTOCOL", "", {"", "RDMA", "SENDRECV"}, "transport protocol; empty = choose by rail count"};
  Param<uint64_t> eager_max_size{"EAGER_MAX_SIZE", 8192, "largest message sent eagerly (bytes); 0 disables eager"};
  Param<std::string> fault_drop{"FAULT_DROP", "",
                                "testing: drop datagrams on send, 'type:count[,type:count]' with the numeric datagram type"};
  Param<uint64_t> host_copy_threads{"HOST_COPY_THREADS", 0,
                                    "worker threads for large host-to-host stripes (0, the default: the calling thread copies)"};
  Param<uint64_t> host_copy_min_size{"HOST_COPY_MIN_SIZE", 65536, "smallest stripe handed to a copy worker (bytes)"};
  Param<std::string> stats_file{"STATS_FILE", "",
                                "write the plugin's counters and histograms to this file as JSON at finalize (%p = process id)"};
  Param<bool> stats_histograms{"STATS_HISTOGRAMS", false,
                               "keep histograms of message sizes, stripes per send and request latencies (printed at "
                               "finalize; implied by STATS_FILE)"};
  Param<uint64_t> ipc_map_wait_us{"IPC_MAP_WAIT_US", 20000,
                                  "how long a send waits for the first mapping of a peer's device allocation (the open "
                                  "runs on a helper thread because it can wait for the device to go idle); after that "
                                  "payloads travel through host fragments until the mapping has arrived"};
  Param<bool> nccl_device_buffers{"NCCL_DEVICE_BUFFERS", true,
                                  "make NCCL hand its device buffers to the plugin (publishes NCCL_NET_GDR_LEVEL=SYS and "
                                  "NCCL_NET_GDR_READ=1 unless the user has set them): payloads then move with the copy "
                                  "kernels over NVLink instead of through host memory; 0 keeps NCCL's chunks in host memory"};
  Param<bool> copy_kernel{"COPY_KERNEL", true,
                          "move device payloads with the plugin's own copy / eager-pack kernels (0: copy engine only)"};
  Param<uint64_t> stall_report_ms{"STALL_REPORT_MS", 30000,
                                  "an endpoint with requests in flight that sees no datagram, completion or accepted post for "
                                  "this long writes one report of its queues to the log (0: never)"};
  Param<bool> shared_stream{"SHARED_STREAM", true,
                            "all device work of the plugin runs on one stream per process (0: one stream per rail and endpoint)"};
  Param<bool> copy_batch{"COPY_BATCH", true,
                         "stripes posted while earlier copy launches are still running leave together, in one launch of the "
                         "batch kernel (up to 16 transfers, each with its own completion word)"};
  Param<uint64_t> copy_batch_depth{"COPY_BATCH_DEPTH", 2, "copy launches in flight below which a stripe is launched at once"};
  Param<uint64_t> copy_batch_quiet_ns{"COPY_BATCH_QUIET_NS", 1000,
                                      "a queued stripe waits for this long without a further stripe being posted before it is "
                                      "launched (NCCL posts the chunks of all channels within a microsecond or two; they then "
                                      "leave in one launch), 0 = launch at once"};
  Param<uint64_t> copy_batch_hold_ns{"COPY_BATCH_HOLD_NS", 4000, "and for no longer than this after the first stripe of the queue"};
  Param<uint64_t> copy_batch_max_age_us{"COPY_BATCH_MAX_AGE_US", 30, "a queued stripe is launched at the latest after this long"};
  Param<bool> copy_kernel_bulk{"COPY_KERNEL_BULK", true,
                               "aligned stripes of 64 KiB and more use the bulk-copy (TMA) kernel; 0: the vector-copy kernel only"};
  Param<uint64_t> copy_kernel_ctas{"COPY_KERNEL_CTAS", 0, "CTAs per copy-kernel launch (0: chosen from the size)"};
  Param<uint64_t> min_stripe_size{"MIN_STRIPE_SIZE", 128 * 1024, "smallest stripe when a message is split over rails"};
  Param<uint64_t> sched_max_small_rr_size{"SCHED_MAX_SMALL_RR_SIZE", 64, "messages below this go to one rail round-robin"};
  Param<int> cq_read_count{"CQ_READ_COUNT", 4, "completions drained per poll of one rail"};
  Param<int> cq_size{"CQ_SIZE", 12288, "entries of a completion ring"};
  Param<bool> mr_cache_disable{"MR_CACHE_DISABLE", false, "do not cache registrations"};
  Param<int> min_posted_eager_buffers{"RDMA_MIN_POSTED_EAGER_BUFFERS", 64,
                                      "accepted for scripts written for the reference plugin and not used: this transport posts no receive buffers (its rings are sized by CQ_SIZE)"};
  Param<int> max_posted_eager_buffers{"RDMA_MAX_POSTED_EAGER_BUFFERS", 128, "see RDMA_MIN_POSTED_EAGER_BUFFERS"};
  Param<int> min_posted_control_buffers{"RDMA_MIN_POSTED_CONTROL_BUFFERS", 16, "see RDMA_MIN_POSTED_EAGER_BUFFERS"};
  Param<int> max_posted_control_buffers{"RDMA_MAX_POSTED_CONTROL_BUFFERS", 32, "see RDMA_MIN_POSTED_EAGER_BUFFERS"};
  Param<bool> early_completion{"EARLY_COMPLETION", false,
                               "report a receive whose completion NCCL calls optional (LL / LL128) as done when it is posted. "
                               "Only honoured with eager sends off (EAGER_MAX_SIZE=0): once such a receive is done NCCL stops "
                               "calling into the plugin, and an eager payload needs the receiver's progress loop to land"};
  Param<bool> disable_close_message{"DISABLE_CLOSE_MESSAGE", false, "skip the close handshake"};
  Param<bool> abort_on_error{"ABORT_ON_ERROR", false, "abort() instead of returning an error code"};
  Param<int> force_num_rails{"FORCE_NUM_RAILS", 0, "override the number of copy channels per peer (0 = from topology)"};
  EnumParam tuner_type{"TUNER_TYPE", "Measured", {"Internal", "Region", "Model", "Measured"}, "tuner back-end"};
  Param<int> tuner_force_channels{"TUNER_FORCE_CHANNELS", 0,
                                  "calibration: the transport tuner answers this channel count for every size (0 = its table)"};
  Param<int> tuner_num_channels{"TUNER_NUM_CHANNELS", 8, "channels the model tuner assumes when it prices an algorithm"};
  Param<float> tuner_net_latency{"TUNER_NET_LATENCY", 20.f, "network latency assumed by the model tuner (us)"};
  Param<bool> tuner_self_register{"TUNER_SELF_REGISTER", true,
                                  "publish NCCL_TUNER_PLUGIN=<this library> at start-up unless the user has set it"};
  Param<std::string> tuner_table{"TUNER_TABLE", "", "path of a measured-bandwidth JSON table"};
  Param<std::string> platform{"PLATFORM", "", "force a platform implementation by name"};
  EnumParam nvtx_trace_dimension{"NVTX_TRACE_DIMENSION", "PER_COMM", {"PER_COMM", "PER_DEV"},
                                 "NVTX domains: one per communicator or one per device"};
  EnumParam trace{"TRACE", "none", {"none", "ring", "nvtx", "all"},
                  "tracepoints: into the in-process ring (dumped to TRACE_FILE at finalize), as NVTX ranges and marks, or both"};
  Param<std::string> trace_file{"TRACE_FILE", "", "Chrome trace-event JSON of the ring, written at finalize (%p = process id)"};
  Param<int> cm_num_rx_buffers{"CM_NUM_RX_BUFFERS", 32, "connection-manager receive slots"};
  Param<bool> errorcheck_mutex{"ERRORCHECK_MUTEX",
#ifdef NDEBUG
                               false,
#else
                               true,
#endif
                               "use error-checking mutexes"};
  Param<bool> disable_dmabuf{"DISABLE_DMABUF", false,
                             "do not advertise dma-buf registration (peers are reached through IPC / VMM mappings, a "
                             "dma-buf descriptor adds nothing; NCCL's export of its own buffers failed with it when "
                             "NCCL_NET_GDR_LEVEL=SYS forced device buffers through)"};
  Param<bool> cuda_flush_enable{"CUDA_FLUSH_ENABLE", false, "flush with the driver instead of a fence"};
  Param<bool> disable_cma{"DISABLE_CMA", false, "never use cross-memory attach for host rendezvous writes"};
  Param<bool> nvls_enable{"NVLS_ENABLE", true, "use NVSwitch multicast where available"};
  Param<uint64_t> device_wait_limit_ms{"DEVICE_WAIT_LIMIT_MS", 20000, "bound of every device-side wait"};
  Param<int> gin_ack_interval{"GIN_ACK_INTERVAL", 64, "operations between GIN acknowledgements"};
  Param<bool> rr_ctrl_msg{"RR_CTRL_MSG", true, "rotate control messages over the control rails"};
  EnumParam progress_model{"PROGRESS_MODEL", "unspec", {"unspec", "auto", "manual"},
                           "accepted for scripts written for the reference plugin and not used: progress is always made by the "
                           "calls of the thread that owns the endpoint"};
  Param<bool> nccl_topo_inject{"NCCL_TOPO_INJECT", false, "publish the generated topology through NCCL_TOPO_FILE"};
  Param<std::string> topo_file_write{"TOPO_FILE_WRITE_PATH", "", "also write the generated NCCL topology here"};
  // settings of earlier versions of the reference plugin that scripts may still carry
  RetiredParam<uint64_t> rdma_min_posted_bounce_buffers{
      "RDMA_MIN_POSTED_BOUNCE_BUFFERS", 0,
      "removed: use RDMA_MIN_POSTED_CONTROL_BUFFERS or RDMA_MIN_POSTED_EAGER_BUFFERS", true};
  RetiredParam<uint64_t> rdma_max_posted_bounce_buffers{
      "RDMA_MAX_POSTED_BOUNCE_BUFFERS", 0,
      "removed: use RDMA_MAX_POSTED_CONTROL_BUFFERS or RDMA_MAX_POSTED_EAGER_BUFFERS", true};
  RetiredParam<bool> endpoint_per_comm{"ENDPOINT_PER_COMM", false,
                                       "deprecated and ignored: endpoints are per thread and device", false};
};
Params& params();

}  // namespace b200net
