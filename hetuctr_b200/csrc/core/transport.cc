#include "core/transport.h"

#include <nccl.h>

#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <mutex>

#include "utils/errors.h"
#include "utils/rendezvous.h"

namespace hetuCTR {

void Transport::waitStream(cudaStream_t stream) { HCTR_CUDA(cudaStreamSynchronize(stream)); }

namespace {

// ------------------------------------------------------------------------------------------------
class NcclTransport : public Transport {
 public:
  NcclTransport(int rank, int nrank, const std::string &ip, int port, int verbose) {
    int version = 0;
    HCTR_NCCL(ncclGetVersion(&version));
    if (version < 20800)
      throw std::runtime_error("NCCL version error, required 2.8 but get " + std::to_string(version));
    if (verbose >= 1)
      std::cout << "HetuTable rank " << rank << ": Start TCP rendezvous at " << ip << ":" << port
                << " NCCL VERSION=" << version << std::endl;
    ncclUniqueId uid;
    std::memset(&uid, 0, sizeof(uid));
    if (rank == 0) HCTR_NCCL(ncclGetUniqueId(&uid));
    TCPRendezvous tcp(rank, nrank, ip, port);
    tcp.broadcast(&uid, sizeof(uid));
    HCTR_NCCL(ncclCommInitRank(&comm_, nrank, uid, rank));
    nrank_ = nrank;
    if (const char *e = std::getenv("HCTR_NCCL_TIMEOUT_MS")) {
      char *end = nullptr;
      const long ms = std::strtol(e, &end, 10);
      HCTR_CHECK(end != e && *end == 0 && ms >= 100 && ms <= 3600000, "HCTR_NCCL_TIMEOUT_MS must be in [100, 3600000]");
      timeout_ms_ = ms;
    }
  }
  void waitStream(cudaStream_t stream) override {
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned spins = 0;; spins++) {
      const cudaError_t q = cudaStreamQuery(stream);
      if (q == cudaSuccess) return;
      if (q != cudaErrorNotReady) HCTR_CUDA(q);
      if ((spins & 1023u) != 1023u) continue;  // look at the clock and the communicator now and then only
      ncclResult_t async = ncclSuccess;
      HCTR_NCCL(ncclCommGetAsyncError(comm_, &async));
      const bool late = std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms_);
      if (async != ncclSuccess && async != ncclInProgress || late) {
        ncclCommAbort(comm_);  // unblocks the kernels of the stuck group
        comm_ = nullptr;
        throw std::runtime_error(late ? "NCCL exchange did not finish in time (is every rank calling the same step?)"
                                      : std::string("NCCL reported an asynchronous error: ") + ncclGetErrorString(async));
      }
    }
  }
  ~NcclTransport() override {
    if (comm_) ncclCommDestroy(comm_);
  }
  void exchange(const std::vector<XferItem> &items, cudaStream_t stream) override {
    HCTR_NCCL(ncclGroupStart());
    for (const XferItem &it : items) {
      if (it.send_bytes) HCTR_NCCL(ncclSend(it.send, it.send_bytes, ncclChar, it.peer, comm_, stream));
      if (it.recv_bytes) HCTR_NCCL(ncclRecv(it.recv, it.recv_bytes, ncclChar, it.peer, comm_, stream));
    }
    HCTR_NCCL(ncclGroupEnd());
  }
  const char *name() const override { return "nccl"; }
  bool multiProcess() const override { return true; }
  void allgatherHost(const void *mine, void *all, size_t bytes) override {
    char *d = nullptr;
    HCTR_CUDA(cudaMalloc(reinterpret_cast<void **>(&d), bytes * (nrank_ + 1)));
    HCTR_CUDA(cudaMemcpy(d, mine, bytes, cudaMemcpyHostToDevice));
    HCTR_NCCL(ncclAllGather(d, d + bytes, bytes, ncclChar, comm_, nullptr));
    HCTR_CUDA(cudaStreamSynchronize(nullptr));
    HCTR_CUDA(cudaMemcpy(all, d + bytes, bytes * nrank_, cudaMemcpyDeviceToHost));
    cudaFree(d);
  }

 private:
  ncclComm_t comm_ = nullptr;
  int nrank_ = 1;
  long timeout_ms_ = 120000;
};

// ------------------------------------------------------------------------------------------------
// All ranks of a job share one InprocWorld, found by (port, nrank).
struct InprocWorld {
  int nrank;
  std::mutex mu;
  std::condition_variable cv;
  int arrived = 0;
  long generation = 0;
  int attached = 0;
  std::vector<std::vector<XferItem>> posted;

  explicit InprocWorld(int n) : nrank(n), posted(n) {}

  void barrier() {
    std::unique_lock<std::mutex> lk(mu);
    const long gen = generation;
    if (++arrived == nrank) {
      arrived = 0;
      generation++;
      cv.notify_all();
      return;
    }
    // a rank that never arrives must not hang the others forever
    if (!cv.wait_for(lk, std::chrono::seconds(120), [&] { return generation != gen; }))
      throw std::runtime_error("inproc transport: a rank did not reach the exchange within 120 s");
  }
};

std::mutex g_worlds_mu;
std::map<std::pair<int, int>, std::shared_ptr<InprocWorld>> g_worlds;

class InprocTransport : public Transport {
 public:
  InprocTransport(int rank, int nrank, int port) : rank_(rank) {
    {
      std::lock_guard<std::mutex> g(g_worlds_mu);
      auto key = std::make_pair(port, nrank);
      auto it = g_worlds.find(key);
      if (it == g_worlds.end() || it->second->attached >= nrank) {
        world_ = std::make_shared<InprocWorld>(nrank);
        g_worlds[key] = world_;
      } else {
        world_ = it->second;
      }
      world_->attached++;
    }
    world_->barrier();
  }
  void exchange(const std::vector<XferItem> &items, cudaStream_t stream) override {
    HCTR_CUDA(cudaStreamSynchronize(stream));  // my send ranges are final
    {
      std::lock_guard<std::mutex> g(world_->mu);
      world_->posted[rank_] = items;
    }
    world_->barrier();
    // my k-th receive from peer p pairs with p's k-th send addressed to me
    std::vector<size_t> cursor(world_->nrank, 0);
    for (const XferItem &it : items) {
      const std::vector<XferItem> &theirs = world_->posted[it.peer];
      size_t &c = cursor[it.peer];
      while (c < theirs.size() && theirs[c].peer != rank_) c++;
      HCTR_CHECK(c < theirs.size(), "inproc transport: unmatched exchange item");
      const XferItem &src = theirs[c++];
      HCTR_CHECK(src.send_bytes == it.recv_bytes, "inproc transport: send/receive sizes differ");
      if (it.recv_bytes)
        HCTR_CUDA(cudaMemcpyAsync(it.recv, src.send, it.recv_bytes, cudaMemcpyDefault, stream));
    }
    HCTR_CUDA(cudaStreamSynchronize(stream));
    world_->barrier();  // nobody reuses a send range before every reader is done
  }
  const char *name() const override { return "inproc"; }
  bool multiProcess() const override { return false; }
  void allgatherHost(const void *mine, void *all, size_t bytes) override {
    std::vector<XferItem> items;
    items.push_back({rank_, mine, bytes, nullptr, 0});
    {
      std::lock_guard<std::mutex> g(world_->mu);
      world_->posted[rank_] = items;
    }
    world_->barrier();
    for (int p = 0; p < world_->nrank; p++)
      std::memcpy(static_cast<char *>(all) + (size_t)p * bytes, world_->posted[p][0].send, bytes);
    world_->barrier();
  }

 private:
  int rank_;
  std::shared_ptr<InprocWorld> world_;
};

}  // namespace

std::unique_ptr<Transport> make_transport(int rank, int nrank, const std::string &ip, int port, int verbose) {
  if (ip == "inproc") return std::make_unique<InprocTransport>(rank, nrank, port);
  return std::make_unique<NcclTransport>(rank, nrank, ip, port, verbose);
}

}  // namespace hetuCTR
