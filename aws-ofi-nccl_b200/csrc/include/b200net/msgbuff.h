// Message buffer: a circular window over a wrapping sequence-number space that remembers, for
// each in-flight message, whether it has not started, is in progress (with the request or the
// bounce buffer that holds it) or has completed. Sequence numbers wrap at 2^bits, and the window
// may hold at most 2^bits / 2 messages so "before" and "after" stay distinguishable
// (reference: src/nccl_ofi_msgbuff.cpp, include/nccl_ofi_msgbuff.h).
#pragma once
#include <cstdint>
#include "b200net/pthread_wrap.h"
#include <vector>

namespace b200net {

enum class MsgStatus : uint8_t { COMPLETED, INPROGRESS, NOTSTARTED, UNAVAILABLE };
enum class MsgElemType : uint8_t { REQ, BUFF };
enum class MsgResult : uint8_t { SUCCESS, INVALID_IDX };

class MsgBuff {
 public:
  // max_inprogress entries; sequence numbers are `bit_width` bits wide; next expected seq = start_seq.
  MsgBuff(uint16_t max_inprogress, uint16_t bit_width, uint16_t start_seq);
  MsgResult insert(uint16_t seq, void* elem, MsgElemType type, MsgStatus* status);
  MsgResult replace(uint16_t seq, void* elem, MsgElemType type, MsgStatus* status);
  MsgResult retrieve(uint16_t seq, void** elem, MsgElemType* type, MsgStatus* status);
  MsgResult complete(uint16_t seq, MsgStatus* status);
  uint16_t field_size() const { return field_size_; }
  uint16_t last_incomplete() const { return last_incomplete_; }

 private:
  struct Slot { MsgStatus stat; MsgElemType type; void* elem; };
  uint16_t distance(uint16_t front, uint16_t back) const;  // (front - back) mod field
  MsgStatus status_of(uint16_t seq) const TSA_REQUIRES(mu_);
  Slot& slot(uint16_t seq) TSA_REQUIRES(mu_) { return buff_[seq % max_inprogress_]; }
  const Slot& slot(uint16_t seq) const TSA_REQUIRES(mu_) { return buff_[seq % max_inprogress_]; }
  uint16_t max_inprogress_, field_size_, field_mask_;
  mutable Mutex mu_;
  uint16_t last_incomplete_ TSA_GUARDED_BY(mu_);  // oldest sequence number not yet completed
  uint16_t next_ TSA_GUARDED_BY(mu_);             // one past the newest sequence number ever inserted
  std::vector<Slot> buff_ TSA_GUARDED_BY(mu_);
};

}  // namespace b200net
