// Tuner process configuration, decision plumbing and the exported ncclTuner tables (v2, v3, v4,
// v5, v6) (reference: src/tuner/nccl_ofi_tuner.cpp:47-279,
// include/tuner/nccl_ofi_tuner_process_config.h).
#include <cstring>
#include <mutex>

#include "b200net/cuda_shim.h"
#include "b200net/log.h"
#include "b200net/param.h"
#include "b200net/system.h"
#include "b200net/topology.h"
#include "b200net/tuner/tuner.h"

namespace b200net::tuner {

const char* platform_name(PlatformKind k) {
  switch (k) {
    case PlatformKind::P5_P5E: return "p5/p5e";
    case PlatformKind::P5EN: return "p5en";
    case PlatformKind::P6_B200: return "p6-b200";
    case PlatformKind::P6_B300: return "p6-b300";
    case PlatformKind::B200_NVSWITCH: return "b200-nvswitch";
    default: return "unknown";
  }
}

PlatformKind platform_from_product_name(const std::string& product, bool local_nvswitch_b200) {
  auto starts = [&](const char* p) { return product.rfind(p, 0) == 0; };
  if (starts("p5en.")) return PlatformKind::P5EN;
  if (starts("p5.") || starts("p5e.")) return PlatformKind::P5_P5E;
  if (starts("p6-b200.") || starts("p6e-b200.")) return PlatformKind::P6_B200;
  if (starts("p6-b300.")) return PlatformKind::P6_B300;
  if (product.find("B200") != std::string::npos || local_nvswitch_b200) return PlatformKind::B200_NVSWITCH;
  return PlatformKind::UNKNOWN;
}

// Detected once per process: the product name and whether the local GPUs are Blackwell on NVSwitch.
static PlatformKind process_platform() {
  static const PlatformKind k = [] {
    bool b200 = false;
    if (cuda::available()) {
      int major = 0;
      if (cuda::device_attribute(75, 0, &major) == 0 && major == 10) b200 = Topology::discover().all_nvlink();
    }
    return platform_from_product_name(system_product_name(), b200);
  }();
  return k;
}

TunerContext::~TunerContext() {
  delete region;
  delete model;
  delete measured;
  delete transport;
}

TransportTuner::TransportTuner(PlatformKind platform, size_t n_ranks, size_t n_nodes) : n_ranks_(n_ranks) {
  supported_ = platform == PlatformKind::B200_NVSWITCH && n_ranks >= 2 && n_nodes == n_ranks;
}

int TransportTuner::channels_for(ncclFunc_t coll, size_t bytes_per_step) {
  if (coll == ncclFuncAllReduce) {
    if (bytes_per_step <= (32u << 10)) return 1;
    if (bytes_per_step <= (1u << 20)) return 2;
    if (bytes_per_step <= (2u << 20)) return 4;
    if (bytes_per_step <= (8u << 20)) return 8;
    return 16;
  }
  if (bytes_per_step <= (64u << 10)) return 1;
  if (bytes_per_step <= (128u << 10)) return 2;
  if (bytes_per_step <= (256u << 10)) return 4;
  if (bytes_per_step <= (8u << 20)) return 8;
  return 16;
}

Decision TransportTuner::decide(ncclFunc_t coll, size_t bytes) const {
  Decision d;
  if (!supported_ || bytes == 0) return d;
  // what one ring step moves: a 1/n slice of the buffer. NCCL passes the size of the whole buffer
  // for all three (for all_gather and reduce_scatter the larger of its send and receive sides,
  // which is n times the per-rank count)
  if (coll != ncclFuncAllReduce && coll != ncclFuncAllGather && coll != ncclFuncReduceScatter) return d;   // point-to-point and rooted calls: NCCL's own
  const size_t per_step = bytes / n_ranks_;
  const int forced = params().tuner_force_channels.get();
  d.n_channels = forced > 0 ? forced : channels_for(coll, per_step);
  return d;
}

TunerContext* create_context(size_t n_ranks, size_t n_nodes) {
  parameters_init();
  std::string type = params().tuner_type.get();
  for (auto& c : type) c = static_cast<char>(tolower(c));
  if (type == "internal" || params().force_num_rails.get() > 0) return nullptr;
  const PlatformKind plat = process_platform();
  auto ctx = new TunerContext();
  ctx->platform = plat;
  ctx->n_ranks = n_ranks;
  ctx->n_nodes = n_nodes;
  // a measured table, when one is configured and loads, takes precedence
  const std::string table = params().tuner_table.get();
  if ((type == "measured") && !table.empty()) {
    auto* m = new MeasuredTuner();
    if (m->load(table) && (m->world() == 0 || m->world() == n_ranks)) {
      ctx->measured = m;
      ctx->type = TunerType::MEASURED;
      return ctx;
    }
    delete m;
  }
  {
    auto* t = new TransportTuner(plat, n_ranks, n_nodes);
    if (t->supported() && type != "model" && type != "region") {
      ctx->transport = t;
      ctx->type = TunerType::TRANSPORT;
      return ctx;
    }
    delete t;
  }
  if (type != "model") {
    auto* r = new RegionTuner(plat, n_ranks, n_nodes);
    if (r->supported()) {
      ctx->region = r;
      ctx->type = TunerType::REGION;
      return ctx;
    }
    delete r;
  }
  auto* m = new ModelTuner(plat, n_ranks, n_nodes);
  if (m->supported()) {
    ctx->model = m;
    ctx->type = TunerType::MODEL;
    return ctx;
  }
  delete m;
  delete ctx;
  return nullptr;  // unknown platform: NCCL's internal tuner decides
}

Decision get_decision(const TunerContext* ctx, ncclFunc_t coll, size_t bytes, int pipe_ops, int reg_buff) {
  if (!ctx) return Decision();
  switch (ctx->type) {
    case TunerType::MEASURED: return ctx->measured->decide(coll, bytes, reg_buff);
    case TunerType::REGION: return ctx->region->decide(coll, bytes);
    case TunerType::MODEL: return ctx->model->decide(coll, bytes, pipe_ops);
    case TunerType::TRANSPORT: return ctx->transport->decide(coll, bytes);
    default: return Decision();
  }
}

bool apply_decision(const Decision& d, float** cost_table, int num_algo, int num_proto, int* n_channels) {
  if (d.algorithm == NCCL_ALGO_UNDEF || d.protocol == NCCL_PROTO_UNDEF) {
    if (n_channels && d.n_channels > 0) *n_channels = d.n_channels;   // channel count only
    return false;
  }
  if (d.algorithm >= num_algo || d.protocol >= num_proto || !cost_table) return false;
  float(*table)[NCCL_NUM_PROTOCOLS] = reinterpret_cast<float(*)[NCCL_NUM_PROTOCOLS]>(cost_table);
  if (table[d.algorithm][d.protocol] == NCCL_ALGO_PROTO_IGNORE) return false;  // NCCL ruled it out
  table[d.algorithm][d.protocol] = 0.0f;
  if (n_channels && d.n_channels > 0) *n_channels = d.n_channels;
  return true;
}

size_t get_chunk_size(const TunerContext* ctx, ncclFunc_t coll, size_t bytes, int algo, int proto, int n_channels) {
  if (!ctx || n_channels <= 0) return 0;
  // stripes of the NVLink plugin are at least 128 KiB: keep per-channel chunks at or above that for
  // bandwidth-bound Simple-protocol transfers, smaller for the latency protocols
  if (ctx->platform == PlatformKind::B200_NVSWITCH || ctx->platform == PlatformKind::P6_B200) {
    if (proto == NCCL_PROTO_SIMPLE && (coll == ncclFuncAllGather || coll == ncclFuncReduceScatter || coll == ncclFuncAllReduce)) {
      const size_t per_channel = bytes / static_cast<size_t>(n_channels);
      if (per_channel >= (4u << 20)) return 512 * 1024;
      if (per_channel >= (512u << 10)) return 256 * 1024;
      return 128 * 1024;
    }
    if (algo == NCCL_ALGO_TREE && proto == NCCL_PROTO_LL128) return 64 * 1024;
  }
  return 0;
}

}  // namespace b200net::tuner

// ------------------------------------------------------------------------------------------------ ABI
using namespace b200net;
using namespace b200net::tuner;
#define B200NET_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

ncclResult_t tuner_init_v2(size_t n_ranks, size_t n_nodes, ncclDebugLogger_t log_fn, void** context) {
  if (!context) return ncclInvalidArgument;
  if (log_fn) set_logger(log_fn);
  *context = create_context(n_ranks, n_nodes);
  NET_INFO(NCCL_INIT | NCCL_TUNING, "tuner: %zu ranks on %zu nodes -> %s", n_ranks, n_nodes,
           *context ? "active" : "NCCL internal tuner");
  return ncclSuccess;
}
// The v2 interface returns one (algorithm, protocol) pair; a user override through NCCL_ALGO /
// NCCL_PROTO must win, so the tuner stays passive when either is set.
ncclResult_t tuner_init_v2_env(size_t n_ranks, size_t n_nodes, ncclDebugLogger_t log_fn, void** context) {
  if (getenv("NCCL_ALGO") || getenv("NCCL_PROTO")) {
    if (context) *context = nullptr;
    return ncclSuccess;
  }
  return tuner_init_v2(n_ranks, n_nodes, log_fn, context);
}
ncclResult_t tuner_init_v5(void** ctx, uint64_t, size_t n_ranks, size_t n_nodes, ncclDebugLogger_t log_fn,
                           ncclNvlDomainInfo_t*, ncclTunerConstants_t*) {
  return tuner_init_v2(n_ranks, n_nodes, log_fn, ctx);
}
ncclResult_t tuner_destroy(void* context) {
  delete static_cast<TunerContext*>(context);
  return ncclSuccess;
}

ncclResult_t get_coll_info_v3(void* context, ncclFunc_t coll, size_t bytes, int pipe_ops, float** table, int num_algo,
                              int num_proto, int* n_channels) {
  if (!context) return ncclSuccess;  // passive: leave the table untouched
  const Decision d = get_decision(static_cast<TunerContext*>(context), coll, bytes, pipe_ops);
  apply_decision(d, table, num_algo, num_proto, n_channels);
  return ncclSuccess;
}
ncclResult_t get_coll_info_v4(void* context, ncclFunc_t coll, size_t bytes, int pipe_ops, float** table, int num_algo,
                              int num_proto, int reg_buff, int* n_channels) {
  if (!context) return ncclSuccess;
  const Decision d = get_decision(static_cast<TunerContext*>(context), coll, bytes, pipe_ops, reg_buff ? 1 : 0);
  apply_decision(d, table, num_algo, num_proto, n_channels);
  return ncclSuccess;
}
ncclResult_t get_coll_info_v2(void* context, ncclFunc_t coll, size_t bytes, int collnet, int nvls, int pipe_ops,
                              int* algorithm, int* protocol, int* n_channels) {
  if (!context) return ncclSuccess;
  const Decision d = get_decision(static_cast<TunerContext*>(context), coll, bytes, pipe_ops);
  if (d.algorithm == NCCL_ALGO_UNDEF) {
    if (n_channels && d.n_channels > 0) *n_channels = d.n_channels;
    return ncclSuccess;
  }
  if ((d.algorithm == NCCL_ALGO_NVLS || d.algorithm == NCCL_ALGO_NVLS_TREE) && !nvls) return ncclSuccess;
  if ((d.algorithm == NCCL_ALGO_COLLNET_DIRECT || d.algorithm == NCCL_ALGO_COLLNET_CHAIN) && !collnet) return ncclSuccess;
  if (algorithm) *algorithm = d.algorithm;
  if (protocol) *protocol = d.protocol;
  if (n_channels && d.n_channels > 0) *n_channels = d.n_channels;
  return ncclSuccess;
}
ncclResult_t get_chunk_size_v6(void* context, ncclFunc_t coll, size_t bytes, int algo, int proto, int n_channels,
                               size_t* chunk) {
  if (!chunk) return ncclInvalidArgument;
  const size_t c = get_chunk_size(static_cast<TunerContext*>(context), coll, bytes, algo, proto, n_channels);
  if (c) *chunk = c;
  return ncclSuccess;
}

}  // namespace

B200NET_EXPORT ncclTuner_v2_t ncclTunerPlugin_v2 = {"b200net_tuner", tuner_init_v2_env, get_coll_info_v2, tuner_destroy};
B200NET_EXPORT ncclTuner_v3_t ncclTunerPlugin_v3 = {"b200net_tuner", tuner_init_v2, get_coll_info_v3, tuner_destroy};
B200NET_EXPORT ncclTuner_v4_t ncclTunerPlugin_v4 = {"b200net_tuner", tuner_init_v2, get_coll_info_v4, tuner_destroy};
B200NET_EXPORT ncclTuner_v5_t ncclTunerPlugin_v5 = {"b200net_tuner", tuner_init_v5, get_coll_info_v4, tuner_destroy};
B200NET_EXPORT ncclTuner_v6_t ncclTunerPlugin_v6 = {"b200net_tuner", tuner_init_v5, get_coll_info_v4, tuner_destroy,
                                                    get_chunk_size_v6};
