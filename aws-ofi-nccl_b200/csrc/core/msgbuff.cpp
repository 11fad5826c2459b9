#include "b200net/msgbuff.h"

#include "b200net/assert.h"

namespace b200net {

MsgBuff::MsgBuff(uint16_t max_inprogress, uint16_t bit_width, uint16_t start_seq)
    : max_inprogress_(max_inprogress), field_size_(static_cast<uint16_t>(1u << bit_width)),
      field_mask_(static_cast<uint16_t>((1u << bit_width) - 1)), last_incomplete_(start_seq), next_(start_seq),
      buff_(max_inprogress) {
  B200NET_ASSERT_ALWAYS(max_inprogress > 0 && bit_width > 0 && bit_width < 16);
  // the window must be smaller than half the sequence space
  B200NET_ASSERT_ALWAYS(static_cast<unsigned>(field_size_) > 2u * max_inprogress);
  for (auto& s : buff_) s = Slot{MsgStatus::NOTSTARTED, MsgElemType::REQ, nullptr};
}

uint16_t MsgBuff::distance(uint16_t front, uint16_t back) const {
  return static_cast<uint16_t>((front - back) & field_mask_);
}

// Classify seq relative to the window [last_incomplete_, last_incomplete_ + max_inprogress_).
MsgStatus MsgBuff::status_of(uint16_t seq) const {
  const uint16_t ahead = distance(seq, last_incomplete_);
  if (ahead < max_inprogress_) return slot(seq).stat;           // inside the window
  if (ahead >= field_size_ - max_inprogress_) return MsgStatus::COMPLETED;  // just behind it
  return MsgStatus::UNAVAILABLE;                                 // too far ahead
}

MsgResult MsgBuff::insert(uint16_t seq, void* elem, MsgElemType type, MsgStatus* status) {
  ScopedLock g(mu_);
  seq &= field_mask_;
  *status = status_of(seq);
  if (*status != MsgStatus::NOTSTARTED) return MsgResult::INVALID_IDX;
  slot(seq) = Slot{MsgStatus::INPROGRESS, type, elem};
  if (distance(seq, last_incomplete_) >= distance(next_, last_incomplete_)) next_ = (seq + 1) & field_mask_;
  return MsgResult::SUCCESS;
}

MsgResult MsgBuff::replace(uint16_t seq, void* elem, MsgElemType type, MsgStatus* status) {
  ScopedLock g(mu_);
  seq &= field_mask_;
  *status = status_of(seq);
  if (*status != MsgStatus::INPROGRESS) return MsgResult::INVALID_IDX;
  slot(seq).elem = elem;
  slot(seq).type = type;
  return MsgResult::SUCCESS;
}

MsgResult MsgBuff::retrieve(uint16_t seq, void** elem, MsgElemType* type, MsgStatus* status) {
  ScopedLock g(mu_);
  seq &= field_mask_;
  *status = status_of(seq);
  if (*status != MsgStatus::INPROGRESS) return MsgResult::INVALID_IDX;
  *elem = slot(seq).elem;
  *type = slot(seq).type;
  return MsgResult::SUCCESS;
}

MsgResult MsgBuff::complete(uint16_t seq, MsgStatus* status) {
  ScopedLock g(mu_);
  seq &= field_mask_;
  *status = status_of(seq);
  if (*status != MsgStatus::INPROGRESS) return MsgResult::INVALID_IDX;
  slot(seq).stat = MsgStatus::COMPLETED;
  slot(seq).elem = nullptr;
  // slide the window past every leading completed message, recycling their slots
  while (slot(last_incomplete_).stat == MsgStatus::COMPLETED) {
    slot(last_incomplete_) = Slot{MsgStatus::NOTSTARTED, MsgElemType::REQ, nullptr};
    last_incomplete_ = (last_incomplete_ + 1) & field_mask_;
    if (last_incomplete_ == next_) break;
  }
  return MsgResult::SUCCESS;
}

}  // namespace b200net
