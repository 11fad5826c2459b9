// MsgBuff: insert / retrieve / replace / complete across sequence wrap-around, window limits.
#include "b200net/msgbuff.h"
#include "test_util.h"
using namespace b200net;
int main() {
  const uint16_t W = 4, BITS = 4;  // 16 sequence numbers, 4 in flight
  for (uint16_t start : {0, 5, 13, 15}) {
    MsgBuff mb(W, BITS, start);
    int elems[64];
    MsgStatus st; MsgElemType ty; void* out;
    uint16_t seq = start;
    for (int round = 0; round < 40; ++round) {  // crosses the wrap several times
      const uint16_t s = seq & 15;
      CHECK(mb.retrieve(s, &out, &ty, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::NOTSTARTED);
      CHECK(mb.insert(s, &elems[round], MsgElemType::REQ, &st) == MsgResult::SUCCESS);
      CHECK(mb.insert(s, &elems[round], MsgElemType::REQ, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::INPROGRESS);
      CHECK(mb.retrieve(s, &out, &ty, &st) == MsgResult::SUCCESS); CHECK(out == &elems[round]); CHECK(ty == MsgElemType::REQ);
      CHECK(mb.replace(s, &elems[63], MsgElemType::BUFF, &st) == MsgResult::SUCCESS);
      CHECK(mb.retrieve(s, &out, &ty, &st) == MsgResult::SUCCESS); CHECK(out == &elems[63]); CHECK(ty == MsgElemType::BUFF);
      CHECK(mb.complete(s, &st) == MsgResult::SUCCESS);
      CHECK(mb.complete(s, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::COMPLETED);
      ++seq;
    }
  }
  {  // out-of-order completion keeps the window pinned at the oldest incomplete message
    MsgBuff mb(W, BITS, 14);
    int e; MsgStatus st;
    for (uint16_t s : {14, 15, 0, 1}) CHECK(mb.insert(s, &e, MsgElemType::REQ, &st) == MsgResult::SUCCESS);
    CHECK(mb.insert(2, &e, MsgElemType::REQ, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::UNAVAILABLE);
    CHECK(mb.complete(15, &st) == MsgResult::SUCCESS);
    CHECK(mb.complete(0, &st) == MsgResult::SUCCESS);
    CHECK(mb.insert(2, &e, MsgElemType::REQ, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::UNAVAILABLE);
    CHECK_EQ(mb.last_incomplete(), 14);
    CHECK(mb.complete(14, &st) == MsgResult::SUCCESS);  // window slides past 14, 15, 0
    CHECK_EQ(mb.last_incomplete(), 1);
    CHECK(mb.insert(2, &e, MsgElemType::REQ, &st) == MsgResult::SUCCESS);
    CHECK(mb.insert(4, &e, MsgElemType::REQ, &st) == MsgResult::SUCCESS);
    CHECK(mb.insert(5, &e, MsgElemType::REQ, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::UNAVAILABLE);
    void* out; MsgElemType ty;
    CHECK(mb.retrieve(15, &out, &ty, &st) == MsgResult::INVALID_IDX); CHECK(st == MsgStatus::COMPLETED);
  }
  CHECK_THROWS(MsgBuff(8, 4, 0));  // window must be smaller than half the sequence space
  TEST_MAIN_END();
}
