// Per-rank mailbox of the peer-to-peer exchange and its mapping into every peer (CUDA IPC).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "hctr_kernels.h"

namespace hetuCTR {

class Transport;

class P2PMailbox {
 public:
  P2PMailbox(int rank, int nrank, int device_id, size_t width, Transport *bootstrap);
  ~P2PMailbox();
  // True when every rank can map every other rank's memory (decided collectively at construction).
  bool usable() const { return usable_; }
  // Collective: (re)allocates mailboxes for `cap` rows per source and exchanges the IPC handles.
  // Every rank must call it with the same cap at the same point of the step sequence.
  void reserve(size_t cap, cudaStream_t stream);
  size_t capacity() const { return cap_; }
  const hctr_p2p_ctx &ctx() const { return ctx_; }
  const hctr_p2p_box &mine() const { return mine_box_; }  // this rank's own mailbox (host copy of the pointers)
  uint32_t nextSeq() { return ++seq_; }
  void setTimeoutNs(unsigned long long ns) { ctx_.timeout_ns = ns; }

 private:
  void releaseMappings();
  hctr_p2p_box carve(char *base) const;
  size_t bytesFor(size_t cap) const;

  int rank_, nrank_, device_id_;
  size_t width_, cap_ = 0;
  Transport *bootstrap_;
  bool usable_ = false;
  char *mine_ = nullptr;               // this rank's mailbox
  std::vector<char *> mapped_;         // peers' mailboxes as mapped here (mapped_[rank_] == mine_)
  hctr_p2p_box *d_boxes_ = nullptr;    // device copy of the box table
  uint32_t *d_cnt_in_ = nullptr;
  hctr_p2p_ctx ctx_{};
  hctr_p2p_box mine_box_{};
  uint32_t seq_ = 0;
};

}  // namespace hetuCTR
