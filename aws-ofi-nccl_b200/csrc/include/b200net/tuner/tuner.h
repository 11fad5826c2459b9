// Tuner: chooses (algorithm, protocol, channel count) per collective call for NCCL's tuner plugin
// interface. Three back-ends share one context:
//   REGION   : polygons in (log2 bytes, log2 ranks) space, first match wins
//   MODEL    : Hockney cost model  latency * pipeline_ops + bytes / bandwidth
//   MEASURED : a table of measured times per (collective, algorithm, protocol, channels, size),
//              produced by a calibration run on the machine itself; active on a single node too
// (reference: src/tuner/nccl_ofi_tuner.cpp, nccl_ofi_regions.cpp, nccl_ofi_model.cpp,
//  include/tuner/nccl_ofi_tuner_region.h).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "nccl_abi.h"

namespace b200net::tuner {

constexpr size_t TUNER_MAX_RANKS = 1024 * 1024;
constexpr size_t TUNER_MAX_SIZE = 100ull * 1024 * 1024 * 1024;
constexpr int TUNER_MAX_VERTICES = 20;

enum class PlatformKind { UNKNOWN, P5_P5E, P5EN, P6_B200, P6_B300, B200_NVSWITCH };
PlatformKind platform_from_product_name(const std::string& product, bool local_nvswitch_b200);
const char* platform_name(PlatformKind k);

// ---------------------------------------------------------------- geometry
struct Point {
  double x, y;  // log2(bytes), log2(ranks)
};
struct Region {
  int algorithm, protocol;
  std::vector<Point> vertices;  // polygon, any orientation, at most TUNER_MAX_VERTICES
};
// 1 strictly inside, 0 on the boundary, -1 outside.
int is_inside_region(Point p, const Region& r);
// Push the far edges of a polygon out to the limits of the space, so that sizes / rank counts
// beyond the measured range keep the decision of the nearest measured edge.
Region extend_region(const Region& r, Point lo, Point hi);
double distance_to_segment(Point p, Point a, Point b);
bool segments_intersect(Point a, Point b, Point c, Point d);

struct Decision {
  int algorithm = NCCL_ALGO_UNDEF;
  int protocol = NCCL_PROTO_UNDEF;
  int n_channels = 0;  // 0 = leave to NCCL
};

// ---------------------------------------------------------------- back-ends
class RegionTuner {
 public:
  RegionTuner(PlatformKind platform, size_t n_ranks, size_t n_nodes);
  bool supported() const { return !regions_[ncclFuncAllReduce].empty(); }
  Decision decide(ncclFunc_t coll, size_t bytes) const;
  const std::vector<Region>& regions(ncclFunc_t coll) const { return regions_[coll]; }

 private:
  PlatformKind platform_;
  size_t n_ranks_, n_nodes_;
  std::vector<Region> regions_[ncclNumFuncs];
};

struct ModelParams {
  double net_lat_us;              // inter-node latency
  double internode_bw_GiBs;       // per rail
  int rails;
  double intranode_bw_GiBs;       // per channel
  double nvlink_lat_us[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
  int channels;
};
class ModelTuner {
 public:
  ModelTuner(PlatformKind platform, size_t n_ranks, size_t n_nodes);
  bool supported() const { return supported_; }
  // microseconds, or <0 when the combination is not modelled
  double cost_us(ncclFunc_t coll, int algo, int proto, int pipe_ops, size_t bytes) const;
  Decision decide(ncclFunc_t coll, size_t bytes, int pipe_ops) const;
  const ModelParams& params() const { return p_; }

 private:
  ModelParams p_{};
  size_t n_ranks_, n_nodes_;
  bool supported_ = false;
};

struct MeasuredRow {
  int coll, algo, proto, n_channels;
  size_t bytes;
  double time_us;
  int reg = -1;   // 1: measured with registered user buffers, 0: without, -1: not recorded
};
class MeasuredTuner {
 public:
  // Parses the calibration JSON ({"world":N,"rows":[{"coll":..,"algo":..,"proto":..,"nchannels":..,
  // "bytes":..,"time_us":..},...]}). "algo" and "proto" of -1 mark a row that timed a channel count
  // with the algorithm and protocol left to NCCL: it decides channels only. "bytes" is the size NCCL
  // reports for the call (the whole buffer, also for all_gather and reduce_scatter). Returns false
  // (and stays unsupported) on a malformed file.
  bool load(const std::string& path);
  bool load_from_string(const std::string& json);
  bool supported() const { return !rows_.empty(); }
  size_t world() const { return world_; }
  // The (algorithm, protocol) with the least time at `bytes`, where the time of a combination is
  // interpolated on a log-log scale between the two measured sizes that bracket `bytes` (measured
  // on the nearer side only it counts with that side's time; outside the measured range the nearest
  // size decides); the channel count is the one of its best row at the nearer size. Times within
  // 3 % of the best count as tied and the fewest channels win (their SMs stay with the application). reg_buff (v4+ of the
  // tuner interface: the call's buffers are registered with the network) restricts the choice to
  // rows recorded with the same setting when the table has any ("reg": 0 / 1); -1 = not known.
  Decision decide(ncclFunc_t coll, size_t bytes, int reg_buff = -1) const;
  size_t num_rows() const { return rows_.size(); }

 private:
  std::vector<MeasuredRow> rows_;
  size_t world_ = 0;
};

// Ranks that reach each other only through this library's own net transport (one GPU per "node" in
// NCCL's eyes: its intra-node transports are off, or the ranks sit in separate containers of one
// NVSwitch box). The algorithm and protocol stay NCCL's choice; what is decided here is the number
// of channels. Every channel's chunk is a transfer of the copy kernels on the transport's single
// stream: chunks posted together share a launch (about 5 us per message at 8 in flight), a lone one
// pays about 10 us, and one channel's kernel side sustains about 20 GB/s, so small calls want few
// channels and large ones all sixteen. The table is the best channel count per size of a sweep over
// 1 / 2 / 4 / 8 / 16 / 32 forced channels on two B200 (B200NET_TUNER_FORCE_CHANNELS), smoothed to be
// monotonic: e.g. all_reduce of 8 MiB 393 / 230 / 175 / 174 / 303 us on 1 / 2 / 4 / 8 / 16 channels,
// of 64 MiB 3158 / 1678 / 894 / 498 / 363 us; all_gather of 1 MiB 233 / 143 / 107 / 67 / 84 us.
class TransportTuner {
 public:
  TransportTuner(PlatformKind platform, size_t n_ranks, size_t n_nodes);
  bool supported() const { return supported_; }
  Decision decide(ncclFunc_t coll, size_t bytes) const;
  // bytes_per_step: what one ring step moves (a 1/n slice of the buffer: of the reduced buffer for
  // all_reduce, of the gathered / scattered one for all_gather and reduce_scatter)
  static int channels_for(ncclFunc_t coll, size_t bytes_per_step);

 private:
  size_t n_ranks_;
  bool supported_ = false;
};

// ---------------------------------------------------------------- context used by the ABI shims
enum class TunerType { INTERNAL, REGION, MODEL, MEASURED, TRANSPORT };
struct TunerContext {
  TunerType type = TunerType::INTERNAL;
  PlatformKind platform = PlatformKind::UNKNOWN;
  size_t n_ranks = 0, n_nodes = 0;
  RegionTuner* region = nullptr;
  ModelTuner* model = nullptr;
  MeasuredTuner* measured = nullptr;
  TransportTuner* transport = nullptr;
  ~TunerContext();
};
// nullptr means "fall back to NCCL's internal tuner" (unknown platform, TUNER_TYPE=Internal, ...).
TunerContext* create_context(size_t n_ranks, size_t n_nodes);
// Apply a decision to NCCL's cost table: the chosen entry gets cost 0 unless NCCL marked it
// NCCL_ALGO_PROTO_IGNORE. Returns true when the table was changed. A decision that names no
// algorithm but a channel count still sets the channel count.
bool apply_decision(const Decision& d, float** cost_table, int num_algo, int num_proto, int* n_channels);
// reg_buff: 1 / 0 when the caller knows whether the call's buffers are registered, -1 otherwise
Decision get_decision(const TunerContext* ctx, ncclFunc_t coll, size_t bytes, int pipe_ops, int reg_buff = -1);
// Chunk size hint (v6 getChunkSize); 0 = no opinion.
size_t get_chunk_size(const TunerContext* ctx, ncclFunc_t coll, size_t bytes, int algo, int proto, int n_channels);

}  // namespace b200net::tuner
