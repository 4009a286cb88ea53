#include "core/p2p.h"

#include <cstdlib>
#include <cstring>

#include "core/transport.h"
#include "utils/errors.h"

namespace hetuCTR {

namespace {
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
constexpr size_t kHdrBytes = 64;
}  // namespace

P2PMailbox::P2PMailbox(int rank, int nrank, int device_id, size_t width, Transport *bootstrap)
    : rank_(rank), nrank_(nrank), device_id_(device_id), width_(width), bootstrap_(bootstrap), mapped_(nrank, nullptr) {
  // Every rank tells the others which device it drives; the exchange is usable only if every rank can
  // map every other rank's device memory (same NVLink domain, peer access possible).
  std::vector<int> devs(nrank_, -1);
  bootstrap_->allgatherHost(&device_id_, devs.data(), sizeof(int));
  same_context_ = !bootstrap_->multiProcess();
  int ok = 1;
  for (int p = 0; p < nrank_; p++) {
    if (p == rank_) continue;
    if (same_context_) {
      if (devs[p] != device_id_) ok = 0;  // thread ranks share mailboxes by plain pointer: one device only
      continue;
    }
    if (devs[p] == device_id_) {
      ok = 0;  // two processes on one GPU: their wait kernels could starve each other
      continue;
    }
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, device_id_, devs[p]) != cudaSuccess || !can) ok = 0;
  }
  std::vector<int> oks(nrank_, 0);
  bootstrap_->allgatherHost(&ok, oks.data(), sizeof(int));
  usable_ = true;
  for (int v : oks) usable_ = usable_ && v != 0;
  ctx_.nrank = nrank_;
  ctx_.rank = rank_;
  ctx_.width = width_;
  ctx_.timeout_ns = 10ull * 1000 * 1000 * 1000;
  if (const char *e = std::getenv("HCTR_P2P_TIMEOUT_MS")) {
    // an unparsable value must not turn into 0 (every wait would give up at once) and a huge one must not make the
    // device-side poll unbounded in practice
    char *end = nullptr;
    const unsigned long long ms = std::strtoull(e, &end, 10);
    HCTR_CHECK(end != e && *end == 0 && ms >= 1 && ms <= 60000, "HCTR_P2P_TIMEOUT_MS must be a number of milliseconds in [1, 60000]");
    ctx_.timeout_ns = ms * 1000000ull;
  }
}

void P2PMailbox::hostBarrier() {
  int token = 0;
  std::vector<int> tokens(nrank_);
  bootstrap_->allgatherHost(&token, tokens.data(), sizeof(int));
}

size_t P2PMailbox::bytesFor(size_t cap) const {
  const size_t n = nrank_, rows = n * cap;
  size_t b = align_up(n * kHdrBytes, 256);
  b += 4 * align_up(rows * 8, 256);            // qkey qver pkey pupd
  b += align_up(rows * width_ * 4, 256);       // pval
  b += align_up(rows, 256);                    // flag
  b += align_up(rows * 8, 256);                // rver
  b += align_up(rows * width_ * 4, 256);       // rval
  return b;
}

hctr_p2p_box P2PMailbox::carve(char *base) const {
  const size_t n = nrank_, rows = n * cap_;
  hctr_p2p_box b;
  char *p = base;
  b.hdr = reinterpret_cast<uint32_t *>(p);
  p += align_up(n * kHdrBytes, 256);
  b.qkey = reinterpret_cast<int64_t *>(p);
  p += align_up(rows * 8, 256);
  b.qver = reinterpret_cast<int64_t *>(p);
  p += align_up(rows * 8, 256);
  b.pkey = reinterpret_cast<int64_t *>(p);
  p += align_up(rows * 8, 256);
  b.pupd = reinterpret_cast<int64_t *>(p);
  p += align_up(rows * 8, 256);
  b.pval = reinterpret_cast<float *>(p);
  p += align_up(rows * width_ * 4, 256);
  b.flag = reinterpret_cast<uint8_t *>(p);
  p += align_up(rows, 256);
  b.rver = reinterpret_cast<int64_t *>(p);
  p += align_up(rows * 8, 256);
  b.rval = reinterpret_cast<float *>(p);
  return b;
}

void P2PMailbox::releaseMappings() {
  for (int p = 0; p < nrank_; p++) {
    if (p != rank_ && mapped_[p] && !same_context_) cudaIpcCloseMemHandle(mapped_[p]);
    mapped_[p] = nullptr;
  }
  if (mine_) cudaFree(mine_);
  mine_ = nullptr;
}

void P2PMailbox::reserve(size_t cap, cudaStream_t stream) {
  if (cap <= cap_) return;
  HCTR_CHECK(usable_, "peer-to-peer exchange is not usable on this set of devices");
  HCTR_CHECK(cap < (size_t)1 << 31, "batch too large for the peer-to-peer exchange");
  HCTR_CUDA(cudaStreamSynchronize(stream));
  if (same_context_) hostBarrier();  // thread ranks: nobody frees a mailbox while a peer's last step still runs
  // Every rank has finished the step that last used the old mailboxes before it gets here (a step only
  // ends after all peers' rows for it have arrived), so they can be unmapped and freed.
  releaseMappings();
  cap_ = cap;
  const size_t bytes = bytesFor(cap);
  HCTR_CUDA(cudaMalloc(reinterpret_cast<void **>(&mine_), bytes));
  HCTR_CUDA(cudaMemset(mine_, 0, bytes));  // sequence numbers start at 0
  HCTR_CUDA(cudaDeviceSynchronize());
  std::vector<hctr_p2p_box> boxes(nrank_);
  if (same_context_) {
    std::vector<char *> all(nrank_);
    bootstrap_->allgatherHost(&mine_, all.data(), sizeof(char *));  // also a barrier: every mailbox is zeroed by now
    for (int p = 0; p < nrank_; p++) mapped_[p] = all[p];
  } else {
    cudaIpcMemHandle_t h;
    HCTR_CUDA(cudaIpcGetMemHandle(&h, mine_));
    std::vector<cudaIpcMemHandle_t> all(nrank_);
    bootstrap_->allgatherHost(&h, all.data(), sizeof(h));  // also a barrier: every mailbox is zeroed by now
    for (int p = 0; p < nrank_; p++) {
      if (p == rank_) {
        mapped_[p] = mine_;
      } else {
        void *ptr = nullptr;
        HCTR_CUDA(cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess));
        mapped_[p] = static_cast<char *>(ptr);
      }
    }
  }
  for (int p = 0; p < nrank_; p++) boxes[p] = carve(mapped_[p]);
  if (!d_boxes_) HCTR_CUDA(cudaMalloc(reinterpret_cast<void **>(&d_boxes_), nrank_ * sizeof(hctr_p2p_box)));
  if (!d_cnt_in_) {
    HCTR_CUDA(cudaMalloc(reinterpret_cast<void **>(&d_cnt_in_), HCTR_P2P_CNT_WORDS(nrank_) * sizeof(uint32_t)));
    HCTR_CUDA(cudaMemset(d_cnt_in_, 0, HCTR_P2P_CNT_WORDS(nrank_) * sizeof(uint32_t)));
  }
  HCTR_CUDA(cudaMemcpy(d_boxes_, boxes.data(), nrank_ * sizeof(hctr_p2p_box), cudaMemcpyHostToDevice));
  mine_box_ = boxes[rank_];
  ctx_.cap = (uint32_t)cap;
  ctx_.box = d_boxes_;
  ctx_.cnt_in = d_cnt_in_;
  seq_ = 0;
  // nobody may write into a mailbox before its owner has finished zeroing it and everyone has mapped it
  int token = 0;
  std::vector<int> tokens(nrank_);
  bootstrap_->allgatherHost(&token, tokens.data(), sizeof(int));
}

P2PMailbox::~P2PMailbox() {
  cudaSetDevice(device_id_);
  cudaDeviceSynchronize();
  releaseMappings();
  if (d_boxes_) cudaFree(d_boxes_);
  if (d_cnt_in_) cudaFree(d_cnt_in_);
}

}  // namespace hetuCTR
