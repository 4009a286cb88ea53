// Peer-to-peer exchange kernels: queries, pushed rows and returned rows are written straight into the
// destination rank's mailbox (plain stores to peer memory over NVLink); a release-store of a sequence
// number publishes them, a bounded acquire-poll on the receiver's own memory consumes them.
// No multicast, no TMA on peer memory: ordinary ld/st only.
#include "p2p.cuh"
#include "rowops.cuh"

namespace hctr {

constexpr int kThreads = 256;
constexpr long long kInvalidVersion = INT64_MIN;

// Requester: (key, local version) of every unique key goes into its owner's mailbox; the thread block that
// finishes last then publishes this rank's counts (queries per owner from the batch's segment starts, pushed rows
// per owner from `push_counts`, null = none) and releases sequence number `seq` to every peer.  The pushed rows
// themselves were written by the gradient reduction, an earlier kernel.
// (Publishing kernels run at most one thread block per SM: every block ends with a system-scope fence, and an SM
// works through the fences of its resident blocks one after the other - with 832 small blocks this kernel took 25 us
// for 77 k keys, most of it fences.)
constexpr int kPubThreads = 1024;

__global__ void __launch_bounds__(kPubThreads) p2p_query_send(hctr_p2p_ctx c, const u32 *__restrict__ meta,
                                                           const long long *__restrict__ uniq,
                                                           const uint8_t *__restrict__ uniq_owner,
                                                           const int32_t *__restrict__ uniq_row,
                                                           const long long *__restrict__ version, u32 seq,
                                                           const u32 *__restrict__ push_counts) {
  const size_t U = meta[HCTR_META_UNIQUE];
  const u32 *seg = meta + HCTR_META_SEG;
  for (size_t u = (size_t)blockIdx.x * kPubThreads + threadIdx.x; u < U; u += (size_t)gridDim.x * kPubThreads) {
    const unsigned p = uniq_owner[u];
    const u32 j = (u32)u - seg[p];
    if (j >= c.cap) {
      atomicOr(c.err, HCTR_ERR_CAPACITY);
      continue;
    }
    const hctr_p2p_box b = c.box[p];
    const size_t slot = (size_t)c.rank * c.cap + j;
    const int32_t row = uniq_row[u];
    b.qkey[slot] = uniq[u];
    b.qver[slot] = row >= 0 ? version[row] : kInvalidVersion;
  }
  if (!last_block_of_launch(c.cnt_in + HCTR_P2P_TICKET0(c.nrank))) return;
  for (int p = threadIdx.x; p < c.nrank; p += kPubThreads) {
    __threadfence_system();
    u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
    hdr[1] = seg[p + 1] - seg[p];
    hdr[2] = push_counts ? push_counts[p] : 0u;
    st_release_sys(hdr + 0, seq);
  }
}

// One thread per peer.  Runs after the kernels that filled the peers' mailboxes (stream order); the
// system-scope fence + release store make those rows visible before the sequence number.
__global__ void p2p_signal(hctr_p2p_ctx c, int phase, u32 seq, const u32 *__restrict__ meta,
                           const u32 *__restrict__ counts) {
  const int p = threadIdx.x;
  if (p >= c.nrank) return;
  __threadfence_system();
  u32 *hdr = c.box[p].hdr + (size_t)c.rank * kHdrWords;
  if (phase == 0) {
    const u32 *seg = meta + HCTR_META_SEG;
    hdr[1] = seg[p + 1] - seg[p];
    hdr[2] = counts ? counts[p] : 0u;
    st_release_sys(hdr + 0, seq);
  } else {
    hdr[9] = counts[p];
    st_release_sys(hdr + 8, seq);
  }
}

// One thread block; thread s waits for source s (bounded) and the counts land in c.cnt_in.
__global__ void __launch_bounds__(kMaxRanks) p2p_wait(hctr_p2p_ctx c, int phase, u32 seq) {
  __shared__ u32 a[kMaxRanks + 1], b[kMaxRanks + 1];
  if (phase == 0) wait_queries(c, seq, a, b, true);
  else wait_returns(c, seq, a, true, true);
}

}  // namespace hctr

using namespace hctr;

extern "C" int hctr_p2p_query_send(const hctr_p2p_ctx *c, const uint32_t *meta, size_t u_max, const int64_t *uniq,
                                   const uint8_t *uniq_owner, const int32_t *uniq_row, const int64_t *version,
                                   uint32_t seq, const uint32_t *push_counts, void *stream) {
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  size_t g = (u_max + kPubThreads - 1) / kPubThreads;
  if (g > (size_t)kSMs) g = kSMs;
  p2p_query_send<<<(unsigned)(g ? g : 1), kPubThreads, 0, (cudaStream_t)stream>>>(
      *c, meta, (const long long *)uniq, uniq_owner, uniq_row, (const long long *)version, seq, push_counts);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_signal(const hctr_p2p_ctx *c, int phase, uint32_t seq, const uint32_t *meta,
                               const uint32_t *counts, void *stream) {
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  p2p_signal<<<1, kMaxRanks, 0, (cudaStream_t)stream>>>(*c, phase, seq, meta, counts);
  count_launches(1);
  return launch_status();
}

extern "C" int hctr_p2p_wait(const hctr_p2p_ctx *c, int phase, uint32_t seq, void *stream) {
  if (c->nrank > kMaxRanks) return (int)cudaErrorInvalidValue;
  p2p_wait<<<1, kMaxRanks, 0, (cudaStream_t)stream>>>(*c, phase, seq);
  count_launches(1);
  return launch_status();
}

