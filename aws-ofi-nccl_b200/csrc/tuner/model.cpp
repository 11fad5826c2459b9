#include <cmath>
#include <limits>

#include "b200net/param.h"
#include "b200net/tuner/tuner.h"

namespace b200net::tuner {

// Per-platform inputs of the cost model (bandwidth in GiB/s, latency in microseconds).
static void nvlink_table(ModelParams& p) {
  for (auto& row : p.nvlink_lat_us)
    for (double& v : row) v = 0.0;
  // per-step NVLink latency: {LL, LL128, Simple}
  const double tree[3] = {0.6, 1.25, 28.0}, ring[3] = {0.6, 1.9, 3.4};
  for (int pr = 0; pr < 3; ++pr) {
    p.nvlink_lat_us[NCCL_ALGO_TREE][pr] = tree[pr];
    p.nvlink_lat_us[NCCL_ALGO_RING][pr] = ring[pr];
    p.nvlink_lat_us[NCCL_ALGO_NVLS][pr] = 23.0;
    p.nvlink_lat_us[NCCL_ALGO_NVLS_TREE][pr] = 23.0;
  }
}

ModelTuner::ModelTuner(PlatformKind platform, size_t n_ranks, size_t n_nodes) : n_ranks_(n_ranks), n_nodes_(n_nodes) {
  nvlink_table(p_);
  p_.channels = b200net::params().tuner_num_channels.get();
  switch (platform) {
    case PlatformKind::P5_P5E:
      p_.net_lat_us = 20.0; p_.internode_bw_GiBs = 12.5; p_.rails = 4; p_.intranode_bw_GiBs = 20.0;
      supported_ = true;
      break;
    case PlatformKind::P5EN:
      p_.net_lat_us = 18.0; p_.internode_bw_GiBs = 25.0; p_.rails = 2; p_.intranode_bw_GiBs = 20.0;
      supported_ = true;
      break;
    default:
      supported_ = false;
  }
  if (supported_ && n_nodes <= 2) supported_ = false;  // NCCL's own choice is kept on tiny jobs
  if (b200net::params().tuner_net_latency.source() != ParamSource::DEFAULT) p_.net_lat_us = b200net::params().tuner_net_latency.get();
}

double ModelTuner::cost_us(ncclFunc_t coll, int algo, int proto, int pipe_ops, size_t bytes) const {
  if (coll != ncclFuncAllReduce) return -1;
  if (algo != NCCL_ALGO_RING && algo != NCCL_ALGO_TREE && algo != NCCL_ALGO_NVLS_TREE) return -1;
  const double ranks_per_node = static_cast<double>(n_ranks_) / static_cast<double>(n_nodes_);
  const double nodes = static_cast<double>(n_nodes_);
  double net_lat = p_.net_lat_us;
  if (proto == NCCL_PROTO_SIMPLE) net_lat += 3.0;  // completion hand-shake of the Simple protocol
  double latency = 0, bw_GiBs = 0;
  const double nv = p_.nvlink_lat_us[algo][proto];
  const double net_bw = p_.internode_bw_GiBs * p_.rails;
  switch (algo) {
    case NCCL_ALGO_RING: {
      const double net_steps = 2 * (nodes - 1), intra_steps = 2 * (n_ranks_ - 1) - net_steps;
      latency = net_steps * net_lat + intra_steps * nv;
      // every byte crosses the slowest link 2(n-1)/n times
      bw_GiBs = std::min(net_bw, p_.intranode_bw_GiBs * p_.channels) * static_cast<double>(n_ranks_) /
                (2.0 * static_cast<double>(n_ranks_ - 1));
      break;
    }
    case NCCL_ALGO_TREE: {
      const double depth = std::log2(nodes);
      latency = 2 * (depth * net_lat + (ranks_per_node - 1) * nv);
      bw_GiBs = std::min(net_bw, p_.intranode_bw_GiBs * p_.channels) / 2.0;
      break;
    }
    case NCCL_ALGO_NVLS_TREE: {
      const double depth = std::log2(nodes);
      latency = 2 * depth * net_lat + nv;
      bw_GiBs = std::min(net_bw, p_.intranode_bw_GiBs * p_.channels * 2) / 2.0;
      if (proto != NCCL_PROTO_SIMPLE) return -1;
      break;
    }
  }
  if (proto == NCCL_PROTO_LL) bw_GiBs *= 0.5;
  if (proto == NCCL_PROTO_LL128) bw_GiBs *= 0.9375;
  const double bytes_per_us = bw_GiBs * 1024.0 * 1024.0 * 1024.0 / 1e6;
  return latency * pipe_ops + static_cast<double>(bytes) / bytes_per_us;
}

Decision ModelTuner::decide(ncclFunc_t coll, size_t bytes, int pipe_ops) const {
  Decision d;
  if (!supported_) return d;
  double best = std::numeric_limits<double>::max();
  for (int a = 0; a < NCCL_NUM_ALGORITHMS; ++a) {
    for (int pr = 0; pr < NCCL_NUM_PROTOCOLS; ++pr) {
      const double c = cost_us(coll, a, pr, pipe_ops < 1 ? 1 : pipe_ops, bytes);
      if (c >= 0 && c < best) {
        best = c;
        d.algorithm = a;
        d.protocol = pr;
      }
    }
  }
  if (d.algorithm != NCCL_ALGO_UNDEF) d.n_channels = p_.channels;
  return d;
}

}  // namespace b200net::tuner
