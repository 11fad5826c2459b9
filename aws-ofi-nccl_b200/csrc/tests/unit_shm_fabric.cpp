// Shared-memory fabric endpoint: datagrams between two endpoints of one process (small and large
// cells, ring-full back-pressure, ordering flag), remote host writes and reads, the MR table, drop
// injection, a closed peer, and collection of segments left behind by dead processes.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

#include "b200net/shm_fabric.h"
#include "test_util.h"

using namespace b200net;

int main() {
  FabricEndpoint a, b;
  CHECK(a.name() != b.name());
  PeerMapping* to_b = a.av_insert(b.name());
  PeerMapping* to_a = b.av_insert(a.name());
  CHECK(to_b != nullptr && to_a != nullptr);
  CHECK(a.av_insert("/b200net.no-such-endpoint") == nullptr);
  CHECK(a.av_insert(b.name()) == to_b);   // cached

  // ---- datagrams: small and large cells, two-part payloads, arrival order per ring
  std::vector<std::pair<uint16_t, std::string>> got;
  auto handler = [&](const DgramHdr& h, const void* p) { got.emplace_back(h.type, std::string(static_cast<const char*>(p), h.len)); };
  CHECK_EQ(a.send(to_b, DgramType::USER, 0, "hello", 5), 0);
  std::string big(6000, 'x');
  CHECK_EQ(a.send(to_b, DgramType::USER, 0, "hdr:", 4, big.data(), big.size()), 0);
  CHECK_EQ(b.poll(16, handler), 2);
  CHECK_EQ(got.size(), 2u);
  bool saw_small = false, saw_big = false;
  for (auto& g : got) {
    saw_small |= g.second == "hello";
    saw_big |= g.second == "hdr:" + big;
  }
  CHECK(saw_small && saw_big);
  CHECK_EQ(a.send(to_b, DgramType::USER, 0, big.data(), FAB_LARGE_CELL + 1), -EMSGSIZE);

  // ---- back-pressure: the ring fills up, -EAGAIN, and drains again
  int accepted = 0;
  while (a.send(to_b, DgramType::USER, 0, "p", 1) == 0) ++accepted;
  CHECK(accepted >= 1024);
  CHECK(a.eagain_count() > 0);
  got.clear();
  int drained = 0;
  while (int n = b.poll(256, handler)) drained += n;
  CHECK_EQ(drained, accepted);
  CHECK_EQ(a.send(to_b, DgramType::USER, 0, "again", 5), 0);
  CHECK_EQ(b.poll(4, handler), 1);

  // ---- drop injection counts down and reports
  a.inject_drop(DgramType::USER, 2);
  got.clear();
  for (int i = 0; i < 3; ++i) CHECK_EQ(a.send(to_b, DgramType::USER, 0, "d", 1), 0);
  CHECK_EQ(b.poll(8, handler), 1);
  CHECK_EQ(a.dropped(), 2u);

  // ---- remote write / read of host memory (same process: cross-memory attach or fragments)
  std::vector<uint8_t> src(300000), dst(300000, 0), back(300000, 0);
  for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint8_t>(i * 7 + 3);
  size_t done = 0;
  int rc;
  while ((rc = a.write_host(to_b, reinterpret_cast<uint64_t>(dst.data()), src.data(), src.size(), &done)) == -EAGAIN)
    b.poll(64, handler);
  CHECK_EQ(rc, 0);
  while (b.poll(64, handler)) {}
  CHECK(dst == src);
  rc = a.read_host(to_b, reinterpret_cast<uint64_t>(dst.data()), back.data(), back.size());
  CHECK(rc == 0 || rc == -ENOTSUP);
  if (rc == 0) CHECK(back == src);

  // ---- MR table: publish, look up from the peer's mapping, unpublish
  MrTableEntry e{};
  e.key = 0xABCD;
  e.base = 0x1000;
  e.size = 4096;
  CHECK_EQ(b.mr_publish(e), 0);
  const MrTableEntry* f = FabricEndpoint::mr_lookup(to_b, 0xABCD);
  CHECK(f != nullptr && f->base == 0x1000 && f->size == 4096);
  b.mr_unpublish(0xABCD);
  CHECK(FabricEndpoint::mr_lookup(to_b, 0xABCD) == nullptr);

  // ---- a closed peer is reported, not written to
  {
    FabricEndpoint c;
    PeerMapping* to_c = a.av_insert(c.name());
    CHECK(to_c != nullptr);
    CHECK_EQ(a.send(to_c, DgramType::USER, 0, "x", 1), 0);
    a.av_remove(c.name());
  }

  // ---- segments of dead processes are collected, those of live ones are kept
  const pid_t child = fork();
  if (child == 0) _exit(0);
  int status = 0;
  waitpid(child, &status, 0);   // the pid is now free: nobody owns a segment named after it
  char stale[64], stale_mb[64];
  snprintf(stale, sizeof(stale), "/b200net.%d.0", static_cast<int>(child));
  snprintf(stale_mb, sizeof(stale_mb), "/b200net.mb.%d.0.1", static_cast<int>(child));
  for (const char* n : {stale, stale_mb}) {
    const int fd = shm_open(n, O_CREAT | O_RDWR, 0600);
    CHECK(fd >= 0);
    if (fd >= 0) {
      CHECK_EQ(ftruncate(fd, 4096), 0);
      close(fd);
    }
  }
  CHECK(FabricEndpoint::collect_stale_segments() >= 2);
  CHECK(shm_open(stale, O_RDWR, 0600) < 0);
  CHECK(shm_open(stale_mb, O_RDWR, 0600) < 0);
  const int own = shm_open(a.name().c_str(), O_RDWR, 0600);   // ours is alive and must survive
  CHECK(own >= 0);
  if (own >= 0) close(own);
  TEST_MAIN_END();
}
