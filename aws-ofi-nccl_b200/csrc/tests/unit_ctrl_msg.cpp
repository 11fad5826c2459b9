// Control mailbox entries of the RDMA-style protocol: layout (one cache line, ready word last),
// the ready word over the 10-bit sequence wrap, and the sender's tag-matching rule for grouped
// receives (bounded by the group size, skipping entries already taken).
#include <cstddef>
#include <cstring>

#include "b200net/rdma_proto.h"
#include "test_util.h"

using namespace b200net::rdma;

static void post_group(CtrlMsg& slot, uint16_t seq, int n, const int* tags) {
  for (int i = 0; i < n; ++i) {
    CtrlEntry& e = slot.entries[i];
    e.buff_addr = 0x1000u * (i + 1);
    e.mr_key = 7;
    e.buff_len = 4096;
    e.tag = tags[i];
    e.num_recvs = static_cast<uint8_t>(n);
    e.recv_idx = static_cast<uint8_t>(i);
    e.ready.store(static_cast<uint16_t>(CTRL_READY | (seq & SEQ_MASK)), std::memory_order_release);
  }
}

int main() {
  // ---- layout
  CHECK_EQ(sizeof(CtrlEntry), 64u);
  CHECK_EQ(offsetof(CtrlEntry, buff_addr), 0u);
  CHECK_EQ(offsetof(CtrlEntry, ready), 62u);   // written last: a reader that sees it sees the entry
  CHECK_EQ(sizeof(CtrlMsg), 512u);
  CHECK_EQ(MAILBOX_BYTES, 512u * 256u);
  CHECK_EQ(sizeof(EagerHdr), 24u);

  // ---- ready word and the sequence wrap
  CtrlMsg slot;
  memset(static_cast<void*>(&slot), 0, sizeof(slot));
  int n = 0;
  CHECK_EQ(match_entry(slot, 5, 0, 1, &n), -1);   // nothing posted
  const int one_tag[1] = {1};
  post_group(slot, 5, 1, one_tag);
  CHECK_EQ(match_entry(slot, 5, 0, 1, &n), 0);
  CHECK_EQ(n, 1);
  // the same mailbox slot serves seq 5 and seq 5 + 256: an old entry must not match the new lap
  CHECK_EQ(match_entry(slot, 5 + MAILBOX_SLOTS, 0, 1, &n), -1);
  post_group(slot, 5 + MAILBOX_SLOTS, 1, one_tag);
  CHECK_EQ(match_entry(slot, 5 + MAILBOX_SLOTS, 0, 1, &n), 0);
  CHECK_EQ(match_entry(slot, 5, 0, 1, &n), -1);
  // 10-bit wrap: sequence 1023 + 1 is 0, and only the low ten bits are compared
  post_group(slot, 1023, 1, one_tag);
  CHECK(entry_ready(slot.entries[0], 1023));
  CHECK(entry_ready(slot.entries[0], 1023 + 1024));   // same number modulo 2^10
  CHECK(!entry_ready(slot.entries[0], 0));
  CHECK(seq_before(1023, 0) && seq_before(1000, 10) && !seq_before(10, 1000) && !seq_before(7, 7));

  // ---- grouped receive: all entries must be there, matching is bounded by the group size
  memset(static_cast<void*>(&slot), 0, sizeof(slot));
  const int tags[4] = {3, 9, 3, 4};
  post_group(slot, 40, 4, tags);
  slot.entries[2].ready.store(0);                     // third entry has not landed yet
  CHECK_EQ(match_entry(slot, 40, 0, 3, &n), -1);
  slot.entries[2].ready.store(static_cast<uint16_t>(CTRL_READY | 40));
  CHECK_EQ(match_entry(slot, 40, 0, 3, &n), 0);
  CHECK_EQ(n, 4);
  CHECK_EQ(match_entry(slot, 40, 0x1, 3, &n), 2);     // first taken: the second entry with tag 3
  CHECK_EQ(match_entry(slot, 40, 0x5, 3, &n), -2);    // both taken: present, but nothing free with this tag
  CHECK_EQ(match_entry(slot, 40, 0, 9, &n), 1);
  CHECK_EQ(match_entry(slot, 40, 0, 77, &n), -2);
  // stale entries beyond the group size are never looked at
  slot.entries[5].tag = 77;
  slot.entries[5].ready.store(static_cast<uint16_t>(CTRL_READY | 40));
  CHECK_EQ(match_entry(slot, 40, 0, 77, &n), -2);
  // a corrupt group size is refused
  slot.entries[0].num_recvs = MAX_RECVS + 1;
  CHECK_EQ(match_entry(slot, 40, 0, 3, &n), -1);
  TEST_MAIN_END();
}
