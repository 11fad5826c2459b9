// Wire formats of the RDMA-style protocol: control mailbox entries, eager header, the immediate
// data that accompanies a write completion, and the connect payloads
// (reference: include/nccl_ofi_rdma.h:50-125 imm-data fields, :217-228 eager header, :235-311
// control entries and mailbox, doc/multi-recv.md).
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>

namespace b200net::rdma {

constexpr int SEQ_BITS = 10;
constexpr uint16_t SEQ_MASK = (1u << SEQ_BITS) - 1;
constexpr int MAILBOX_SLOTS = 256;
constexpr int MAX_RECVS = 8;
constexpr int MAX_EAGER_PENDING = 32;
constexpr uint16_t CTRL_READY = 0x8000;

enum CtrlFlags : uint16_t { CTRL_FLAG_NO_COMPLETION = 1 };  // receiver does not wait for write completions

// One receive buffer advertised to the sender. 64 bytes; `ready` is written last (release).
struct CtrlEntry {
  uint64_t buff_addr;
  uint64_t mr_key;
  uint64_t buff_len;
  int32_t tag;
  uint16_t flags;
  uint8_t num_recvs;   // size of the group this entry belongs to (same in all its entries)
  uint8_t recv_idx;    // position inside the group
  uint8_t pad[30];
  std::atomic<uint16_t> ready;  // CTRL_READY | (msg_seq_num & SEQ_MASK)
};
static_assert(sizeof(CtrlEntry) == 64, "control entries are one cache line");
static_assert(offsetof(CtrlEntry, ready) == 62, "ready word closes the entry");

struct CtrlMsg {
  CtrlEntry entries[MAX_RECVS];
};
static_assert(sizeof(CtrlMsg) == 512, "a control message is 8 entries");
constexpr size_t MAILBOX_BYTES = sizeof(CtrlMsg) * MAILBOX_SLOTS;

// An entry is valid for sequence number `seq` when its ready word carries exactly that number:
// a slot still holding the group of 256 sequence numbers ago does not match.
inline bool entry_ready(const CtrlEntry& e, uint16_t seq) {
  return e.ready.load(std::memory_order_acquire) == static_cast<uint16_t>(CTRL_READY | (seq & SEQ_MASK));
}

// The sender's matching rule for one receive group (mailbox slot): the whole group must have
// arrived; among its entries not yet taken (`consumed` bit mask) the first with the send's tag
// wins. Returns the entry index, -1 when the group is not (completely) there yet, -2 when it is
// there but holds no free entry with this tag. *num_recvs receives the group size.
inline int match_entry(const CtrlMsg& slot, uint16_t seq, uint8_t consumed, int tag, int* num_recvs) {
  if (!entry_ready(slot.entries[0], seq)) return -1;
  const int n = slot.entries[0].num_recvs;
  if (n < 1 || n > MAX_RECVS) return -1;
  for (int i = 1; i < n; ++i)
    if (!entry_ready(slot.entries[i], seq)) return -1;
  *num_recvs = n;
  for (int i = 0; i < n; ++i)
    if (!(consumed & (1u << i)) && slot.entries[i].tag == tag) return i;
  return -2;
}

inline bool seq_before(uint16_t a, uint16_t b) {  // a strictly before b in the wrapping 10-bit space
  return a != b && (((b - a) & SEQ_MASK) < (1u << (SEQ_BITS - 1)));
}

// Eager message: [EagerHdr][payload]. base_seq / base_mask record which receive group the sender
// was on and which of its entries earlier sends had already taken, so the receiver can repeat
// the sender's matching decision no matter how datagrams of different rings interleave.
struct EagerHdr {
  uint32_t remote_comm_id;
  uint16_t eager_seq;
  uint16_t base_seq;
  uint8_t base_mask;
  uint8_t pad[3];
  int32_t tag;
  uint64_t size;
};
static_assert(sizeof(EagerHdr) == 24, "eager header");

// "Immediate data" of a write: sent as a small datagram once the stripe has landed.
struct WriteCompletion {
  uint32_t remote_comm_id;
  uint16_t seq;
  uint8_t recv_idx;
  uint8_t seg_cnt;     // stripes of this message
  uint64_t len;        // bytes of this stripe
};

struct CloseMsg {
  uint32_t remote_comm_id;
  uint32_t nonce;      // identifies the connection: ids are recycled, a late close must not hit a new comm
};

// Connect payloads carried by the connection manager.
struct ConnPayload {          // connector -> acceptor
  uint32_t comm_id;           // sender's local id
  uint32_t num_rails;
  uint32_t nonce;             // random per connection
  char mailbox_name[48];      // shared window holding the sender's control mailbox
};
struct ConnRespPayload {      // acceptor -> connector
  uint32_t comm_id;           // receiver's local id
  uint32_t num_rails;
};

}  // namespace b200net::rdma
