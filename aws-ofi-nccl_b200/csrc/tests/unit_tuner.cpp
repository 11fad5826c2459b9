// Tuner: polygon geometry (inside / boundary / outside, extension), region decisions per platform,
// cost-model ordering, measured-table lookup, cost-table mutation rules, platform mapping.
#include <cmath>
#include <cstring>
#include "b200net/platform.h"
#include "b200net/tuner/tuner.h"
#include <cstdlib>
#include "test_util.h"
using namespace b200net;
using namespace b200net::tuner;

int main() {
  // ---- geometry
  Region sq{NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, {{0, 0}, {4, 0}, {4, 4}, {0, 4}}};
  CHECK_EQ(is_inside_region({2, 2}, sq), 1);
  CHECK_EQ(is_inside_region({4, 2}, sq), 0);   // on an edge
  CHECK_EQ(is_inside_region({0, 0}, sq), 0);   // on a vertex
  CHECK_EQ(is_inside_region({5, 2}, sq), -1);
  CHECK_EQ(is_inside_region({2, -0.1}, sq), -1);
  Region tri{0, 0, {{0, 0}, {10, 0}, {0, 10}}};
  CHECK_EQ(is_inside_region({1, 1}, tri), 1);
  CHECK_EQ(is_inside_region({5, 5}, tri), 0);   // on the hypotenuse
  CHECK_EQ(is_inside_region({6, 6}, tri), -1);
  Region concave{0, 0, {{0, 0}, {6, 0}, {6, 6}, {3, 2}, {0, 6}}};
  CHECK_EQ(is_inside_region({3, 1}, concave), 1);
  CHECK_EQ(is_inside_region({3, 4}, concave), -1);  // in the notch
  CHECK(segments_intersect({0, 0}, {2, 2}, {0, 2}, {2, 0}));
  CHECK(!segments_intersect({0, 0}, {1, 1}, {2, 2}, {3, 3}));
  CHECK(std::fabs(distance_to_segment({1, 1}, {0, 0}, {2, 0}) - 1.0) < 1e-12);
  CHECK(std::fabs(distance_to_segment({5, 0}, {0, 0}, {2, 0}) - 3.0) < 1e-12);
  Region ext = extend_region(sq, {0, 0}, {40, 20});
  CHECK_EQ(is_inside_region({30, 15}, ext), 1);
  CHECK_EQ(is_inside_region({30, 15}, sq), -1);
  CHECK_EQ(is_inside_region({2, 2}, ext), 1);

  // ---- region tuner: multi-node Blackwell table, 8 ranks per node
  {
    RegionTuner t(PlatformKind::P6_B200, 128, 16);
    CHECK(t.supported());
    Decision d = t.decide(ncclFuncAllReduce, 64 * 1024);
    CHECK_EQ(d.algorithm, NCCL_ALGO_TREE); CHECK_EQ(d.protocol, NCCL_PROTO_LL);
    d = t.decide(ncclFuncAllReduce, 2u << 20);
    CHECK_EQ(d.algorithm, NCCL_ALGO_TREE); CHECK_EQ(d.protocol, NCCL_PROTO_LL128);
    d = t.decide(ncclFuncAllReduce, 8u << 20);   // still LL128 at 128 ranks, with a channel choice
    CHECK_EQ(d.protocol, NCCL_PROTO_LL128); CHECK(d.n_channels == 16 || d.n_channels == 24 || d.n_channels == 32);
    d = t.decide(ncclFuncAllReduce, 1ull << 30);
    CHECK_EQ(d.algorithm, NCCL_ALGO_NVLS_TREE); CHECK_EQ(d.protocol, NCCL_PROTO_SIMPLE);
    RegionTuner small(PlatformKind::P6_B200, 16, 2);   // two nodes: NCCL decides
    CHECK(!small.supported());
    CHECK_EQ(small.decide(ncclFuncAllReduce, 1 << 20).algorithm, NCCL_ALGO_UNDEF);
    RegionTuner t32(PlatformKind::P6_B200, 32, 4);
    d = t32.decide(ncclFuncAllReduce, 1ull << 30);     // few ranks, huge message: ring
    CHECK_EQ(d.algorithm, NCCL_ALGO_RING);
    d = t.decide(ncclFuncAllGather, 256 * 1024);
    CHECK_EQ(d.algorithm, NCCL_ALGO_PAT); CHECK_EQ(d.n_channels, 1);
    RegionTuner odd(PlatformKind::P6_B200, 100, 16);   // not 8 ranks per node: no table
    CHECK(!odd.supported());
  }
  {  // one NVSwitch box: active on a single node
    RegionTuner t(PlatformKind::B200_NVSWITCH, 8, 1);
    CHECK(t.supported());
    CHECK_EQ(t.decide(ncclFuncAllReduce, 1024).protocol, NCCL_PROTO_LL);
    CHECK_EQ(t.decide(ncclFuncAllReduce, 256 << 10).protocol, NCCL_PROTO_LL128);
    CHECK_EQ(t.decide(ncclFuncAllReduce, 64u << 20).algorithm, NCCL_ALGO_NVLS);
    CHECK_EQ(t.decide(ncclFuncAllReduce, 0).algorithm, NCCL_ALGO_UNDEF);
  }
  // ---- model tuner
  {
    ModelTuner m(PlatformKind::P5EN, 256, 32);
    CHECK(m.supported());
    CHECK(m.cost_us(ncclFuncAllGather, NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, 1, 1 << 20) < 0);
    const double small_ll = m.cost_us(ncclFuncAllReduce, NCCL_ALGO_TREE, NCCL_PROTO_LL, 1, 1024);
    const double small_simple = m.cost_us(ncclFuncAllReduce, NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, 1, 1024);
    CHECK(small_ll > 0 && small_ll < small_simple);         // latency bound: tree/LL wins
    Decision d = m.decide(ncclFuncAllReduce, 1024, 1);
    CHECK_EQ(d.algorithm, NCCL_ALGO_TREE);
    d = m.decide(ncclFuncAllReduce, 4ull << 30, 1);           // bandwidth bound: not LL
    CHECK(d.protocol != NCCL_PROTO_LL);
    const double c1 = m.cost_us(ncclFuncAllReduce, NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, 1, 1 << 20);
    const double c2 = m.cost_us(ncclFuncAllReduce, NCCL_ALGO_RING, NCCL_PROTO_SIMPLE, 2, 1 << 20);
    CHECK(c2 > c1);                                          // more pipeline ops cost more latency
    ModelTuner tiny(PlatformKind::P5EN, 16, 2);
    CHECK(!tiny.supported());
    ModelTuner unk(PlatformKind::UNKNOWN, 256, 32);
    CHECK(!unk.supported());
  }
  // ---- measured tuner
  {
    MeasuredTuner mt;
    CHECK(!mt.load_from_string("{}"));
    CHECK(!mt.load_from_string("{\"rows\": [ {\"coll\": 4} ]}"));
    const char* js =
        "{\"world\": 8, \"rows\": ["
        "{\"coll\":4,\"algo\":1,\"proto\":0,\"nchannels\":4,\"bytes\":1024,\"time_us\":9.0},"
        "{\"coll\":4,\"algo\":4,\"proto\":2,\"nchannels\":16,\"bytes\":1024,\"time_us\":14.0},"
        "{\"coll\":4,\"algo\":1,\"proto\":0,\"nchannels\":4,\"bytes\":67108864,\"time_us\":900.0},"
        "{\"coll\":4,\"algo\":4,\"proto\":2,\"nchannels\":24,\"bytes\":67108864,\"time_us\":210.0},"
        "{\"coll\":2,\"algo\":1,\"proto\":2,\"nchannels\":8,\"bytes\":1048576,\"time_us\":30.0}]}";
    CHECK(mt.load_from_string(js));
    CHECK_EQ(mt.num_rows(), 5u); CHECK_EQ(mt.world(), 8u);
    Decision d = mt.decide(ncclFuncAllReduce, 2000);
    CHECK_EQ(d.algorithm, NCCL_ALGO_RING); CHECK_EQ(d.protocol, NCCL_PROTO_LL); CHECK_EQ(d.n_channels, 4);
    d = mt.decide(ncclFuncAllReduce, 32u << 20);
    CHECK_EQ(d.algorithm, NCCL_ALGO_NVLS); CHECK_EQ(d.n_channels, 24);
    CHECK_EQ(mt.decide(ncclFuncReduceScatter, 1 << 20).algorithm, NCCL_ALGO_UNDEF);  // nothing measured
    CHECK_EQ(mt.decide(ncclFuncAllGather, 1 << 10).algorithm, NCCL_ALGO_RING);
    // between two measured sizes every combination's time is interpolated (log-log): ring LL goes
    // 9 -> 900 us over 16 octaves, NVLS simple 14 -> 210 us; they cross near 2^(10 + 16 * 0.23)
    CHECK_EQ(mt.decide(ncclFuncAllReduce, 8u << 10).algorithm, NCCL_ALGO_RING);     // 3 octaves up: 21 vs 23 us
    CHECK_EQ(mt.decide(ncclFuncAllReduce, 64u << 10).algorithm, NCCL_ALGO_NVLS);    // 6 octaves up: 51 vs 39 us
    // ties within 3 %: the fewer channels; registered-buffer rows only for calls that say so
    const char* js2 =
        "{\"world\": 8, \"rows\": ["
        "{\"coll\":4,\"algo\":1,\"proto\":2,\"nchannels\":16,\"bytes\":1048576,\"time_us\":100.0},"
        "{\"coll\":4,\"algo\":1,\"proto\":2,\"nchannels\":8,\"bytes\":1048576,\"time_us\":102.0},"
        "{\"coll\":4,\"algo\":1,\"proto\":2,\"nchannels\":4,\"bytes\":1048576,\"time_us\":110.0},"
        "{\"coll\":3,\"algo\":1,\"proto\":2,\"nchannels\":8,\"bytes\":1048576,\"time_us\":50.0,\"reg\":0},"
        "{\"coll\":3,\"algo\":6,\"proto\":2,\"nchannels\":8,\"bytes\":1048576,\"time_us\":30.0,\"reg\":1}]}";
    MeasuredTuner m2;
    CHECK(m2.load_from_string(js2));
    CHECK_EQ(m2.decide(ncclFuncAllReduce, 1u << 20).n_channels, 8);
    CHECK_EQ(m2.decide(ncclFuncReduceScatter, 1u << 20, 0).algorithm, NCCL_ALGO_RING);
    CHECK_EQ(m2.decide(ncclFuncReduceScatter, 1u << 20, 1).algorithm, NCCL_ALGO_PAT);
    CHECK_EQ(m2.decide(ncclFuncReduceScatter, 1u << 20).algorithm, NCCL_ALGO_PAT);   // not known: the fastest row
    CHECK_EQ(m2.decide(ncclFuncAllReduce, 1u << 20, 1).n_channels, 8);               // table silent about registration
    // rows that timed channel counts only (algorithm and protocol -1): the shipped sweep of two B200
    MeasuredTuner sweep;
    const char* path = getenv("B200NET_TEST_CHANNEL_TABLE");
    if (path && sweep.load(path)) {
      CHECK_EQ(sweep.world(), 2u);
      Decision c = sweep.decide(ncclFuncAllReduce, 64u << 10);
      CHECK_EQ(c.algorithm, NCCL_ALGO_UNDEF); CHECK_EQ(c.protocol, NCCL_PROTO_UNDEF); CHECK_EQ(c.n_channels, 1);
      CHECK_EQ(sweep.decide(ncclFuncAllReduce, 64u << 20).n_channels, 16);
      CHECK_EQ(sweep.decide(ncclFuncAllGather, 1u << 20).n_channels, 8);
      CHECK_EQ(sweep.decide(ncclFuncReduceScatter, 8u << 20).n_channels, 8);
      int nch = 0;
      float table[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
      for (auto& row : table) for (float& v : row) v = 5.0f;
      CHECK(!apply_decision(c, reinterpret_cast<float**>(table), NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, &nch));
      CHECK_EQ(nch, 1); CHECK_EQ(table[NCCL_ALGO_RING][NCCL_PROTO_SIMPLE], 5.0f);   // channels only, NCCL's costs untouched
    } else if (path) {
      CHECK(false);   // the table named by the test did not load
    }
  }
  // ---- cost table mutation
  {
    float table[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
    for (auto& row : table) for (float& v : row) v = 100.0f;
    table[NCCL_ALGO_NVLS][NCCL_PROTO_SIMPLE] = NCCL_ALGO_PROTO_IGNORE;
    int nch = 7;
    Decision d{NCCL_ALGO_NVLS, NCCL_PROTO_SIMPLE, 16};
    CHECK(!apply_decision(d, reinterpret_cast<float**>(table), NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, &nch));
    CHECK_EQ(nch, 7); CHECK(table[NCCL_ALGO_NVLS][NCCL_PROTO_SIMPLE] == NCCL_ALGO_PROTO_IGNORE);
    d = Decision{NCCL_ALGO_TREE, NCCL_PROTO_LL128, 24};
    CHECK(apply_decision(d, reinterpret_cast<float**>(table), NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, &nch));
    CHECK(table[NCCL_ALGO_TREE][NCCL_PROTO_LL128] == 0.0f); CHECK_EQ(nch, 24);
    CHECK(table[NCCL_ALGO_RING][NCCL_PROTO_SIMPLE] == 100.0f);
    d = Decision{NCCL_ALGO_PAT, NCCL_PROTO_SIMPLE, 0};
    CHECK(!apply_decision(d, reinterpret_cast<float**>(table), 6, NCCL_NUM_PROTOCOLS, &nch));  // older NCCL: fewer algorithms
    CHECK(!apply_decision(Decision(), reinterpret_cast<float**>(table), NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, &nch));
  }
  // ---- platform mapping (instance names and regexes; kernel-initiated GIN only where offered)
  CHECK(platform_from_product_name("p5en.48xlarge", false) == PlatformKind::P5EN);
  CHECK(platform_from_product_name("p5.48xlarge", false) == PlatformKind::P5_P5E);
  CHECK(platform_from_product_name("p5e.48xlarge", false) == PlatformKind::P5_P5E);
  CHECK(platform_from_product_name("p6-b200.48xlarge", false) == PlatformKind::P6_B200);
  CHECK(platform_from_product_name("p6-b300.48xlarge", false) == PlatformKind::P6_B300);
  CHECK(platform_from_product_name("m5.large", false) == PlatformKind::UNKNOWN);
  CHECK(platform_from_product_name("DGX B200", false) == PlatformKind::B200_NVSWITCH);
  CHECK(platform_from_product_name("", true) == PlatformKind::B200_NVSWITCH);
  CHECK(find_instance("p4d.24xlarge") && !find_instance("p4d.24xlarge")->gdaki && find_instance("p4d.24xlarge")->latency_us == 75.f);
  CHECK(find_instance("p5e.48xlarge") && !strcmp(find_instance("p5e.48xlarge")->name, "p5.48xlarge"));
  CHECK(find_instance("p5en.48xlarge")->gdaki && find_instance("p5en.48xlarge")->latency_us == 35.f);
  CHECK(find_instance("p6-b200.48xlarge")->gdaki && find_instance("p6e-b200.36xlarge") != nullptr);
  CHECK(find_instance("p3dn.24xlarge")->latency_us == 150.f && !find_instance("p3dn.24xlarge")->gdaki);
  CHECK(find_instance("c5.large") == nullptr && find_instance("") == nullptr);
  // p5 / p5en region tables are cut out of the cost model: they must agree with it at the sampled rank counts
  for (PlatformKind plat : {PlatformKind::P5_P5E, PlatformKind::P5EN}) {
    for (size_t nodes : {4, 16, 64, 256}) {
      RegionTuner r(plat, nodes * 8, nodes);
      ModelTuner m(plat, nodes * 8, nodes);
      CHECK(r.supported() && m.supported());
      int disagreements = 0, checked = 0;
      for (double x = 4.1; x < 35.0; x += 0.9) {   // between the sampled sizes too
        const size_t bytes = static_cast<size_t>(std::exp2(x));
        const Decision a = r.decide(ncclFuncAllReduce, bytes), b = m.decide(ncclFuncAllReduce, bytes, 1);
        ++checked;
        if (a.algorithm != b.algorithm || a.protocol != b.protocol) ++disagreements;
      }
      CHECK(checked > 30);
      CHECK(disagreements <= 2);   // only within a quarter octave of a crossover
    }
    CHECK(!RegionTuner(plat, 16, 2).supported());    // two nodes: NCCL's own choice
    CHECK(!RegionTuner(plat, 40, 8).supported());    // not 8 ranks per node
  }
  // ranks that only reach each other through the plugin's own transport: channel counts by size, algorithm left to NCCL
  {
    TransportTuner t(PlatformKind::B200_NVSWITCH, 8, 8);
    CHECK(t.supported());
    CHECK(!TransportTuner(PlatformKind::B200_NVSWITCH, 8, 1).supported());   // one node: NVLink transports, not this one
    CHECK(!TransportTuner(PlatformKind::P5EN, 8, 8).supported());
    Decision d = t.decide(ncclFuncAllReduce, 256u << 10);   // 32 KiB per step
    CHECK_EQ(d.algorithm, NCCL_ALGO_UNDEF);
    CHECK_EQ(d.n_channels, 1);
    CHECK_EQ(t.decide(ncclFuncAllReduce, 8u << 20).n_channels, 2);     // 1 MiB per step
    CHECK_EQ(t.decide(ncclFuncAllReduce, 64u << 20).n_channels, 8);    // 8 MiB per step
    CHECK_EQ(t.decide(ncclFuncAllGather, 512u << 10).n_channels, 1);   // 64 KiB per rank
    CHECK_EQ(t.decide(ncclFuncAllGather, 2u << 20).n_channels, 4);      // 256 KiB per rank
    CHECK_EQ(t.decide(ncclFuncAllGather, 8u << 20).n_channels, 8);      // 1 MiB per rank
    CHECK_EQ(t.decide(ncclFuncReduceScatter, 8u << 20).n_channels, 8);
    // never fewer channels for a larger call of the same kind
    for (ncclFunc_t f : {ncclFuncAllReduce, ncclFuncAllGather, ncclFuncReduceScatter}) {
      int prev = 0;
      for (size_t b = 8; b <= (size_t{1} << 33); b *= 2) {
        const int n = t.decide(f, b).n_channels;
        CHECK(n >= prev && n >= 1 && n <= 16);
        prev = n;
      }
    }
    CHECK_EQ(t.decide(ncclFuncReduceScatter, 256u << 20).n_channels, 16);  // 32 MiB per rank
    CHECK_EQ(t.decide(ncclFuncAllReduce, 256u << 20).n_channels, 16);
    CHECK_EQ(t.decide(ncclFuncSendRecv, 1u << 20).n_channels, 0);
    int nch = 0;
    float table[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
    for (auto& row : table) for (float& c : row) c = 1.0f;
    CHECK(!apply_decision(d, reinterpret_cast<float**>(table), NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, &nch));
    CHECK_EQ(nch, 1);                 // the channel count is applied although no table entry was chosen
    CHECK_EQ(table[0][0], 1.0f);      // and the table is untouched
  }
  TEST_MAIN_END();
}
