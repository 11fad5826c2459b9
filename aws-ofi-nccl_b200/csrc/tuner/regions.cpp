#include <algorithm>
#include <cmath>

#include "b200net/math.h"
#include "b200net/tuner/tuner.h"

namespace b200net::tuner {

static double cross(Point o, Point a, Point b) { return (a.x - o.x) * (b.y - o.y) - (a.y - o.y) * (b.x - o.x); }
static bool on_segment(Point p, Point a, Point b) {
  return std::fabs(cross(a, b, p)) < 1e-12 && p.x >= std::min(a.x, b.x) - 1e-12 && p.x <= std::max(a.x, b.x) + 1e-12 &&
         p.y >= std::min(a.y, b.y) - 1e-12 && p.y <= std::max(a.y, b.y) + 1e-12;
}

bool segments_intersect(Point a, Point b, Point c, Point d) {
  const double d1 = cross(c, d, a), d2 = cross(c, d, b), d3 = cross(a, b, c), d4 = cross(a, b, d);
  if (((d1 > 0 && d2 < 0) || (d1 < 0 && d2 > 0)) && ((d3 > 0 && d4 < 0) || (d3 < 0 && d4 > 0))) return true;
  return on_segment(a, c, d) || on_segment(b, c, d) || on_segment(c, a, b) || on_segment(d, a, b);
}

double distance_to_segment(Point p, Point a, Point b) {
  const double dx = b.x - a.x, dy = b.y - a.y;
  const double len2 = dx * dx + dy * dy;
  double t = len2 > 0 ? ((p.x - a.x) * dx + (p.y - a.y) * dy) / len2 : 0.0;
  t = std::max(0.0, std::min(1.0, t));
  return std::hypot(p.x - (a.x + t * dx), p.y - (a.y + t * dy));
}

// Ray casting along +x with the boundary reported separately.
int is_inside_region(Point p, const Region& r) {
  const size_t n = r.vertices.size();
  if (n < 3) return -1;
  bool inside = false;
  for (size_t i = 0, j = n - 1; i < n; j = i++) {
    const Point a = r.vertices[i], b = r.vertices[j];
    if (on_segment(p, a, b)) return 0;
    if ((a.y > p.y) != (b.y > p.y)) {
      const double xint = a.x + (p.y - a.y) * (b.x - a.x) / (b.y - a.y);
      if (p.x < xint) inside = !inside;
    }
  }
  return inside ? 1 : -1;
}

Region extend_region(const Region& r, Point lo, Point hi) {
  if (r.vertices.empty()) return r;
  double minx = r.vertices[0].x, maxx = minx, miny = r.vertices[0].y, maxy = miny;
  for (const Point& v : r.vertices) {
    minx = std::min(minx, v.x); maxx = std::max(maxx, v.x);
    miny = std::min(miny, v.y); maxy = std::max(maxy, v.y);
  }
  Region out = r;
  for (Point& v : out.vertices) {
    if (v.x == maxx) v.x = hi.x;
    if (v.y == maxy) v.y = hi.y;
    if (v.x == minx) v.x = lo.x;
    if (v.y == miny) v.y = lo.y;
  }
  return out;
}

// ---------------------------------------------------------------- region tables
// Coordinates are (log2 bytes, log2 ranks). The multi-node Blackwell table encodes the crossover
// points between Tree/LL, Tree/LL128, NVLS-Tree/Simple and Ring/Simple as straight boundaries in
// log-log space between the 16-rank and the 2048-rank measurements.
static double lg(double v) { return std::log2(v); }

static void add(std::vector<Region>& v, int algo, int proto, std::vector<Point> pts) { v.push_back(Region{algo, proto, std::move(pts)}); }

static void p6_b200_tables(std::vector<Region>* regions) {
  const double xmax = lg(static_cast<double>(TUNER_MAX_SIZE)), ymax = lg(static_cast<double>(TUNER_MAX_RANKS));
  const double y16 = lg(16), y32 = lg(32), y2k = lg(2048);
  const double ll_end = lg(384.0 * 1024);
  const double ll128_end_16 = lg(4.5 * 1024 * 1024), ll128_end_2k = lg(101.0 * 1024 * 1024);
  const double ring_start_32 = lg(415.0 * 1024 * 1024);
  auto& ar = regions[ncclFuncAllReduce];
  add(ar, NCCL_ALGO_TREE, NCCL_PROTO_LL, {{0, y16}, {ll_end, y16}, {ll_end, ymax}, {0, ymax}});
  add(ar, NCCL_ALGO_TREE, NCCL_PROTO_LL128, {{ll_end, y16}, {ll128_end_16, y16}, {ll128_end_2k, y2k}, {ll128_end_2k, ymax}, {ll_end, ymax}});
  // large messages on few ranks: ring wins over NVLS-tree
  add(ar, NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, {{ring_start_32, y16}, {xmax, y16}, {xmax, y32 + 1.0}, {ring_start_32 + 1.0, y32 + 1.0}, {ring_start_32, y32}});
  add(ar, NCCL_ALGO_NVLS_TREE, NCCL_PROTO_SIMPLE, {{ll128_end_16, y16}, {xmax, y16}, {xmax, ymax}, {ll128_end_2k, ymax}, {ll128_end_2k, y2k}});
  // all-gather / reduce-scatter: PAT for small, ring for large
  for (ncclFunc_t f : {ncclFuncAllGather, ncclFuncReduceScatter}) {
    auto& r = regions[f];
    const double pat_end_16 = lg(1.0 * 1024 * 1024), pat_end_2k = lg(64.0 * 1024 * 1024);
    add(r, NCCL_ALGO_PAT, NCCL_PROTO_SIMPLE, {{0, y16}, {pat_end_16, y16}, {pat_end_2k, y2k}, {pat_end_2k, ymax}, {0, ymax}});
    add(r, NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, {{pat_end_16, y16}, {xmax, y16}, {xmax, ymax}, {pat_end_2k, ymax}, {pat_end_2k, y2k}});
  }
}

// One NVSwitch box (the ranks of a single node): latency-bound sizes on Ring/LL, then NVLS.
static void b200_nvswitch_tables(std::vector<Region>* regions, size_t n_ranks) {
  const double xmax = lg(static_cast<double>(TUNER_MAX_SIZE)), y0 = 0, ymax = lg(static_cast<double>(TUNER_MAX_RANKS));
  (void)n_ranks;
  auto& ar = regions[ncclFuncAllReduce];
  const double ll_end = lg(64.0 * 1024), ll128_end = lg(1.0 * 1024 * 1024);
  add(ar, NCCL_ALGO_RING, NCCL_PROTO_LL, {{0, y0}, {ll_end, y0}, {ll_end, ymax}, {0, ymax}});
  add(ar, NCCL_ALGO_RING, NCCL_PROTO_LL128, {{ll_end, y0}, {ll128_end, y0}, {ll128_end, ymax}, {ll_end, ymax}});
  add(ar, NCCL_ALGO_NVLS, NCCL_PROTO_SIMPLE, {{ll128_end, y0}, {xmax, y0}, {xmax, ymax}, {ll128_end, ymax}});
  for (ncclFunc_t f : {ncclFuncAllGather, ncclFuncReduceScatter}) {
    auto& r = regions[f];
    add(r, NCCL_ALGO_RING, NCCL_PROTO_LL, {{0, y0}, {ll_end, y0}, {ll_end, ymax}, {0, ymax}});
    add(r, NCCL_ALGO_RING, NCCL_PROTO_LL128, {{ll_end, y0}, {ll128_end, y0}, {ll128_end, ymax}, {ll_end, ymax}});
    add(r, NCCL_ALGO_NVLS, NCCL_PROTO_SIMPLE, {{ll128_end, y0}, {xmax, y0}, {xmax, ymax}, {ll128_end, ymax}});
  }
}

// Hopper-generation instance types (p5 / p5e / p5en): the regions are cut out of the cost model of
// model.cpp rather than measured: for every power-of-two node count from 4 to 256 (8 ranks each)
// the all-reduce decision is evaluated at quarter-octave steps of the size, and every run of equal
// decisions becomes a rectangle that spans half an octave of ranks around that node count. The
// tables therefore agree with the model at the sampled rank counts and keep its crossovers between
// them, which is what a region tuner is for: a cheap look-up at run time.
static void hopper_tables_from_model(PlatformKind platform, std::vector<Region>* regions) {
  auto& ar = regions[ncclFuncAllReduce];
  const double xmax = lg(static_cast<double>(TUNER_MAX_SIZE));
  for (size_t nodes = 4; nodes <= 256; nodes *= 2) {
    const size_t ranks = nodes * 8;
    ModelTuner model(platform, ranks, nodes);
    if (!model.supported()) return;
    const double y = lg(static_cast<double>(ranks));
    const double ylo = nodes == 4 ? lg(24.0) : y - 0.5, yhi = nodes == 256 ? lg(static_cast<double>(TUNER_MAX_RANKS)) : y + 0.5;
    Decision cur;
    double start = 0;
    for (double x = 3.0; x <= 36.0 + 1e-9; x += 0.25) {
      const Decision d = model.decide(ncclFuncAllReduce, static_cast<size_t>(std::exp2(x)), 1);
      const bool same = d.algorithm == cur.algorithm && d.protocol == cur.protocol;
      if (!same) {
        if (cur.algorithm != NCCL_ALGO_UNDEF) add(ar, cur.algorithm, cur.protocol, {{start, ylo}, {x, ylo}, {x, yhi}, {start, yhi}});
        cur = d;
        start = x <= 3.0 ? 0 : x;
      }
    }
    if (cur.algorithm != NCCL_ALGO_UNDEF) add(ar, cur.algorithm, cur.protocol, {{start, ylo}, {xmax, ylo}, {xmax, yhi}, {start, yhi}});
  }
}

RegionTuner::RegionTuner(PlatformKind platform, size_t n_ranks, size_t n_nodes)
    : platform_(platform), n_ranks_(n_ranks), n_nodes_(n_nodes) {
  switch (platform) {
    case PlatformKind::P5_P5E:
    case PlatformKind::P5EN:
      if (n_nodes > 2 && n_ranks == 8 * n_nodes) hopper_tables_from_model(platform, regions_);
      break;
    case PlatformKind::P6_B200:
    case PlatformKind::P6_B300:
      // tables were taken with 8 ranks per node
      if (n_nodes > 2 && n_ranks == 8 * n_nodes) p6_b200_tables(regions_);
      break;
    case PlatformKind::B200_NVSWITCH:
      if (n_nodes == 1) b200_nvswitch_tables(regions_, n_ranks);
      break;
    default:
      break;
  }
}

Decision RegionTuner::decide(ncclFunc_t coll, size_t bytes) const {
  Decision d;
  if (coll >= ncclNumFuncs || bytes == 0) return d;
  const Point p{std::log2(static_cast<double>(std::min(bytes, TUNER_MAX_SIZE))), std::log2(static_cast<double>(n_ranks_))};
  for (const Region& r : regions_[coll]) {
    if (is_inside_region(p, r) >= 0) {  // boundary counts; first match wins
      d.algorithm = r.algorithm;
      d.protocol = r.protocol;
      break;
    }
  }
  // channel heuristics of the multi-node Blackwell tables
  if ((platform_ == PlatformKind::P6_B200 || platform_ == PlatformKind::P6_B300) && d.algorithm != NCCL_ALGO_UNDEF) {
    if (d.algorithm == NCCL_ALGO_TREE && d.protocol == NCCL_PROTO_LL128 && bytes >= (4u << 20) && bytes <= (32u << 20)) {
      // enough channels that each moves at least ~256 KiB, from the set the pipeline likes
      const size_t per = 256 * 1024;
      const size_t want = div_ceil<size_t>(bytes, per);
      d.n_channels = want <= 16 ? 16 : want <= 24 ? 24 : 32;
    } else if (d.algorithm == NCCL_ALGO_PAT) {
      if (bytes <= 64 * 1024 * n_nodes_) d.n_channels = 1;
      else if (bytes <= 128 * 1024 * n_nodes_) d.n_channels = 2;
    }
  }
  return d;
}

}  // namespace b200net::tuner
