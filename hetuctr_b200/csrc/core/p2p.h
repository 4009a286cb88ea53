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
  // True when all ranks are threads of one process on one GPU: peers' mailboxes are plain pointers of the shared
  // context, and no kernel may wait for a peer's kernel (nothing guarantees that two launches on one GPU run at the
  // same time).  The table then publishes with hctr_p2p_signal, drains its stream, meets the peers at a host
  // barrier and only afterwards launches hctr_p2p_wait, which finds every sequence number already in place.
  bool sameContext() const { return same_context_; }
  void hostBarrier();
  // Collective: (re)allocates mailboxes for `cap` rows per source and exchanges the IPC handles.
  // Every rank must call it with the same cap at the same point of the step sequence.
  void reserve(size_t cap, cudaStream_t stream);
  size_t capacity() const { return cap_; }
  const hctr_p2p_ctx &ctx() const { return ctx_; }
  const hctr_p2p_box &mine() const { return mine_box_; }  // this rank's own mailbox (host copy of the pointers)
  uint32_t nextSeq() { return ++seq_; }
  void setTimeoutNs(unsigned long long ns) { ctx_.timeout_ns = ns; }
  void setErr(uint32_t *err) { ctx_.err = err; }  // the device error word the kernels report through

 private:
  void releaseMappings();
  hctr_p2p_box carve(char *base) const;
  size_t bytesFor(size_t cap) const;

  int rank_, nrank_, device_id_;
  size_t width_, cap_ = 0;
  Transport *bootstrap_;
  bool usable_ = false;
  bool same_context_ = false;
  char *mine_ = nullptr;               // this rank's mailbox
  std::vector<char *> mapped_;         // peers' mailboxes as mapped here (mapped_[rank_] == mine_)
  hctr_p2p_box *d_boxes_ = nullptr;    // device copy of the box table
  uint32_t *d_cnt_in_ = nullptr;
  hctr_p2p_ctx ctx_{};
  hctr_p2p_box mine_box_{};
  uint32_t seq_ = 0;
};

}  // namespace hetuCTR
