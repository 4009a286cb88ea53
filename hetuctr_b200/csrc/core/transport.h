// Variable-size all-to-all behind the three exchanges of a step (keys, gradients, embeddings).
//
// A group is a list of items {peer, send range, receive range}.  Items addressed to the same peer are
// matched in order with that peer's items addressed to this rank, exactly like grouped
// ncclSend/ncclRecv (the reference's scheme, csrc/core/all2all.cu:18-130).  Two implementations:
//   * NcclTransport    one process per GPU, NCCL communicator bootstrapped over TCP  (production)
//   * InprocTransport  all ranks are threads of ONE process (ip == "inproc"); copies are
//                      cudaMemcpyAsync between the ranks' buffers, ordered by host barriers.  It lets
//                      every multi-rank kernel run and be checked on a single GPU.
#pragma once
#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <vector>

namespace hetuCTR {

struct XferItem {
  int peer;
  const void *send;
  size_t send_bytes;
  void *recv;
  size_t recv_bytes;
};

class Transport {
 public:
  virtual ~Transport() {}
  // Enqueues the group on `stream`; on return the operation is ordered in the stream (NCCL) or complete
  // (in-process).
  virtual void exchange(const std::vector<XferItem> &items, cudaStream_t stream) = 0;
  virtual const char *name() const = 0;
  // Host-memory all-gather of `bytes` per rank (set-up paths only); acts as a barrier.
  virtual void allgatherHost(const void *mine, void *all, size_t bytes) = 0;
  // True when ranks are separate processes that each drive their own GPU.
  virtual bool multiProcess() const = 0;
  // Waits until `stream` has drained.  The NCCL transport does not block inside the driver: it polls the stream
  // and the communicator's asynchronous error state, and after HCTR_NCCL_TIMEOUT_MS (default 120 s; a peer that
  // never joins a group leaves the stream stuck for ever) aborts the communicator and throws.
  virtual void waitStream(cudaStream_t stream);
};

// ip == "inproc" selects the in-process transport (all ranks of the job must use the same port value,
// which names the job).  Collective: returns when all ranks of the job have called it.
std::unique_ptr<Transport> make_transport(int rank, int nrank, const std::string &ip, int port, int verbose);

}  // namespace hetuCTR
