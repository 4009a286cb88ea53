// HetuTable: one rank of a distributed GPU embedding table (host orchestration).
//
// Mirrors the reference's class of the same name (csrc/core/hetu_gpu_table.h:21-145): same
// constructor arguments, same preprocess()/pushPull() call pattern and semantics, one table per
// process/GPU.  The implementation underneath is new: all GPU work goes through the C-ABI launchers
// of hctr_kernels.h, the key->row map is a dense array instead of a managed-memory hash map, and the
// exchanges are packed into three NCCL groups per step with one mid-step host synchronisation.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <limits>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "hctr_kernels.h"

namespace hetuCTR {

class Transport;
class P2PMailbox;

// csrc/core/types.h:12-28
typedef float embed_t;
typedef long long version_t;
typedef long long index_t;
typedef unsigned char worker_t;
const index_t kInvalidIndex = -1;
const version_t kInvalidVersion = std::numeric_limits<version_t>::min();

// csrc/utils/initializer.h:8-25
enum class InitType { kZero, kNormal, kUniform, kTruncatedNormal, kNone };
struct Initializer {
  Initializer(InitType _type, float a, float b) : type(_type), param(a, b) {}
  InitType type;
  std::pair<float, float> param;  // (mean, stddev) or (a, b)
};

// Process-wide seed used by tables constructed afterwards (hetuCTR.seed, csrc/pybind/pybind.cu:77).
void set_seed(unsigned long seed);
unsigned long get_seed();

// Growable device allocation.
struct DevBuf {
  void *p = nullptr;
  size_t bytes = 0;
  void ensure(size_t want);  // grows (contents are NOT preserved); never shrinks
  void release();
  template <class T>
  T *as() const { return static_cast<T *>(p); }
};

// Device-side description of one preprocessed batch (the reference's PreprocessData,
// csrc/core/preprocess_struct.h:7-24, with 32-bit indices).
struct BatchDesc {
  size_t batch_size = 0;
  size_t unique_size = 0;
  size_t capacity = 0;
  size_t n_heavy = 0;  // runs longer than HCTR_LIGHT_RUN
  bool pending = false;  // sizes not yet read back from the device (single-rank tables defer this)
  cudaEvent_t ev_order = nullptr;  // completion of the ordering of this batch's long runs (on the ordering stream)
  bool order_recorded = false;
  cudaEvent_t ev_scatter = nullptr;  // this batch's positions are in their runs (end of the dedupe pipeline)
  bool scatter_recorded = false;
  bool light_ordered = false;        // runs of up to HCTR_LIGHT_RUN positions have been put in ascending order
  bool decided = false;            // the push decision for this batch has been enqueued
  bool order_pending = false;      // the run-ordering kernels of this batch are not enqueued yet
  bool dedupe_pending = false;     // single-rank tables: the dedupe pipeline of this batch is not enqueued yet
  hctr_dedupe_args order_args;     // what both will be launched with
  DevBuf keys, idx_map, sorted_pos, uniq, uniq_owner, uniq_row, run_start, meta, pos_row, heavy;
  // Push decision of this batch (multi-rank tables): flag and send slot per unique key.  They belong to the batch
  // because the decision is taken at the end of the batch's own push_pull and consumed by the next one; a larger
  // batch arriving in between must not move them.
  DevBuf need_push, push_slot;
  // rank of every position inside its run; later the staging area of the batch's run ordering (its own buffer, so
  // that the ordering of one batch can overlap the dedupe of the next)
  DevBuf rank;
  uint32_t *h_meta = nullptr;      // pinned: the batch's meta words (sizes, segment starts, error bits) as read back
  std::vector<size_t> seg;         // [n+1] first unique of each owner
  std::vector<size_t> query_send;  // [n] unique keys addressed to each owner
  std::vector<size_t> query_recv;  // [n] keys each requester sends to me
  std::vector<size_t> push_send;   // [n] rows of this batch's gradient pushed to each owner
  std::vector<size_t> push_recv;   // [n]
  std::vector<size_t> ret_send;    // [n] rows I return to each requester
  std::vector<size_t> ret_recv;    // [n] rows each owner returns to me
};

struct StepStats {  // sizes of the last push_pull, for roofline arithmetic
  size_t batch = 0, unique = 0, prev_batch = 0, prev_unique = 0;
  size_t pushed_rows = 0, received_push_rows = 0, queried_keys = 0, returned_rows = 0, received_rows = 0;
  // peer-to-peer exchange: longest in-kernel wait of the step for a peer's queries / returned rows (peer skew)
  size_t wait_queries_us = 0, wait_returns_us = 0;
};

// Phases timed with CUDA events on the table's stream when profiling is enabled.
enum Phase {
  kPhDedupe = 0,      // hctr_dedupe_map
  kPhPushDecide,      // hctr_push_decide
  kPhReduce,          // hctr_grad_reduce_apply_pack
  kPhQuery,           // hctr_query_versions
  kPhExchange,        // transport groups (all of a step)
  kPhOwnerUpdate,     // hctr_owner_update (all sources); peer-to-peer: wait for the peers + sources and versions
  kPhStaleGather,     // hctr_stale_check + hctr_gather_rows; peer-to-peer: hctr_p2p_stale_gather
  kPhRefresh,         // hctr_recv_slots + hctr_cache_refresh; peer-to-peer: wait for the owners + hctr_p2p_refresh_index
  kPhExpand,          // hctr_expand_rows
  kPhOwnerApply,      // peer-to-peer: row pass of the owner update
  kPhCount
};

class HetuTable {
 public:
  const int rank_;
  const int nrank_;
  const int device_id_;
  const size_t kEmbeddingIDMax;
  const size_t kEmbeddingWidth;
  const size_t kStorageMax;
  size_t kNonLocalStorageMax = 0;
  const embed_t learning_rate_;
  const version_t pull_bound_, push_bound_;
  int verbose_;

  HetuTable(const int rank, const int nrank, const int device_id, const std::string &ip, const int port,
            const size_t embedding_length, const size_t embedding_width, const version_t pull_bound,
            const version_t push_bound, const worker_t *root_id_arr, const size_t root_id_len,
            const index_t *storage_id_arr, const size_t storage_id_len, const Initializer &init,
            const embed_t learning_rate, const int verbose);
  HetuTable(const HetuTable &) = delete;
  HetuTable &operator=(const HetuTable &) = delete;
  ~HetuTable();

  // csrc/core/hetu_gpu_table.h:127-141.  data_ptr: host or device memory; grad/dst: device memory
  // (host memory is also accepted and staged).  Both calls return after the stream has drained.
  void preprocess(index_t *data_ptr, size_t batch_size);
  void pushPull(embed_t *grad, embed_t *dst);

  std::string debugString();
  std::string debugStringFull();

  // ---- extensions used by tests, benchmarks and tools -----------------------------------------
  // Copies a named internal array to host memory as int64 (or float for "embedding"/"gradient");
  // returns the element count; out may be null to query the size.  Names follow the reference's
  // members: unique_idx, idx_map, sorted_arg, run_length, root, offset, shape, shape_exchanged,
  // version, updates, stored_keys, need_update; prev selects the previous batch descriptor.
  long long dump(const std::string &what, bool prev, void *out);
  // Overwrites the local rows (local row order) from host memory.
  void setEmbedding(const embed_t *host_rows);
  // Writes / reads the learned state (rows, versions, pending gradients and counts of cached rows) to a file.
  // The importing table must have been constructed with the same rank, nrank, length, width and storage_arr.
  // Import is only legal between steps (not between preprocess and push_pull); batches preprocessed before
  // it are dropped, so the next push_pull behaves like the first one of a fresh table.
  void exportState(const std::string &path);
  void importState(const std::string &path);
  // (A single-rank table learns the unique count of its current batch only when the dedupe, which runs behind the
  // step, has finished: asking waits for it.)
  const StepStats &stats() {
    if (cur_batch_.pending || prev_batch_.pending) quiesce();
    stats_.unique = stats_.batch ? cur_batch_.unique_size : 0;
    stats_.prev_unique = stats_.prev_batch ? prev_batch_.unique_size : 0;
    return stats_;
  }
  // "none" (single rank), "nccl", "inproc" or "p2p"
  const char *exchangeName() const;
  // Per-phase device time.  While enabled, every phase is bracketed by two events on the table's
  // stream; times are summed when the call that recorded them has drained the stream.
  // every = 0: off; 1: every step; k: every k-th step (the timing events cost a few microseconds per phase)
  void setProfile(int every);
  void phaseTimes(double ms[kPhCount], long long calls[kPhCount], bool reset);
  // The most recent spans as (phase, start ms, end ms) triples, oldest first; times count from the moment
  // profiling was enabled.  Returns the number of triples written (at most max_spans).
  size_t timeline(double *out, size_t max_spans);
  cudaStream_t stream() const { return stream_main_; }

 private:
  void initComm(const std::string &ip, int port);
  void initTable(const worker_t *root, const index_t *storage);
  void reserveBatch(BatchDesc &b, size_t batch);
  void reserveShared(size_t batch);
  void exchangeCounts();
  void releaseAll();
  void finalizeBatch();
  void finalizePending();
  void finalizePrev();   // single-rank tables: sizes of the previous batch, read back on demand
  uint32_t readSizes(BatchDesc &b);  // copies b's meta words into the descriptor; returns the error bits
  int expandRows(size_t batch, size_t width, const int32_t *pos_row, const int32_t *idx_map, const uint32_t *recv_slot,
                 const float *recv_val, const float *embedding, float *dst, uint32_t *err, cudaStream_t stream);
  void launchPushDecide(BatchDesc &b);
  void flushOrdering(BatchDesc &b);  // enqueues a batch's deferred run ordering
  void flushDedupe(BatchDesc &b);    // enqueues a batch's deferred dedupe pipeline (single-rank tables)
  void orderLightRuns(BatchDesc &b, cudaStream_t s);  // the short-run half of the ordering, where somebody needs it
  void quiesce();  // every stream drained, pending batch sizes read back
  void exchangeP2P(embed_t *dst_dev);
  const void *stageIn(const void *ptr, size_t bytes, DevBuf &buf, cudaStream_t s);

  cudaStream_t stream_main_ = nullptr;
  cudaStream_t stream_side_ = nullptr;  // overlaps the long-run kernels with their short-run twins
  // The gradient reduction of the PREVIOUS batch runs here, concurrently with the dedupe of the current
  // batch on stream_main_ (they touch disjoint data); stream_main_ joins it before the first kernel that
  // reads updated rows or versions.
  cudaStream_t stream_reduce_ = nullptr;
  cudaStream_t stream_reduce_side_ = nullptr;  // long-run reduce kernel, forked from stream_reduce_
  cudaEvent_t ev_decide_ = nullptr, ev_reduce_ = nullptr, ev_rfork_ = nullptr, ev_rjoin_ = nullptr;
  cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr, ev_keys_ = nullptr;
  cudaEvent_t ev_early_ = nullptr;   // end of the gradient-independent half of a split row expansion
  bool split_host_expand_ = true;    // HCTR_SPLIT_HOST_EXPAND=0 switches the split off
  bool fused_refresh_expand_ = true; // HCTR_P2P_FUSED_EXPAND=0: cache refresh and row expansion as two launches
  std::unique_ptr<Transport> transport_;
  std::unique_ptr<P2PMailbox> p2p_;  // device-driven exchange (one process per GPU, peer access); else NCCL groups
  bool use_p2p_ = false;
  bool p2p_counts_pending_ = false;
  bool p2p_pushed_valid_ = false;    // the push counts read back with the step describe a real previous batch
  bool expand_bulk_ = false;         // HCTR_EXPAND=bulk
  // Field count of the (sample-major) key batches, used to give every warp of the dedupe kernels one field of
  // 32 consecutive samples: HCTR_KEY_STRIDE = auto (default: found from the first large batch) or a number
  // (0 or 1 = off).
  uint32_t key_stride_ = 0;
  bool key_stride_known_ = false;
  void detectKeyStride(const BatchDesc &b);
  bool batch_open_ = false;          // preprocess done, push_pull not yet
  bool prev_push_valid_ = false;     // d_push_count_/d_push_base_ describe prev_batch_

  // table state
  DevBuf d_embedding_, d_gradient_, d_updates_, d_version_, d_root_, d_row_of_, d_stored_keys_;
  size_t length_pad_ = 0;

  // dedupe scratch (persistent, all-zero between calls) and per-step scratch
  DevBuf d_bits_, d_blk_cnt_, d_blk_flag_, d_chain_, d_chain3_, d_ent_row_, d_ent_next_, d_row_mask_, d_row_head_, d_src_off_, d_src_cnt_, d_word_base_, d_scan_, d_sk_, d_cnt_;
  DevBuf d_push_count_, d_push_base_, d_recv_idx_, d_err_;
  size_t shared_capacity_ = 0;
  uint32_t dedupe_epoch_ = 0;
  uint32_t nextEpoch() { return ++dedupe_epoch_ ? dedupe_epoch_ : ++dedupe_epoch_; }  // never 0

  // exchange buffers: *_s = send side, *_r = receive side
  DevBuf d_cnt_s_, d_cnt_r_;                      // packed per-peer counts
  DevBuf d_qver_s_, d_qkey_r_, d_qver_r_;         // query (keys are sent straight from the batch)
  DevBuf d_pkey_s_, d_pupd_s_, d_pval_s_, d_pkey_r_, d_pupd_r_, d_pval_r_;  // pushed gradients
  DevBuf d_flag_s_, d_flag_r_, d_flag32_, d_ret_slot_, d_recv_slot_, d_seg_r_;
  DevBuf d_retcnt_s_, d_retcnt_r_;
  DevBuf d_rver_s_, d_rval_s_, d_rver_r_, d_rval_r_;  // returned rows
  DevBuf d_stage_grad_, d_stage_dst_;

  void *h_src_ = nullptr;         // pinned staging of the per-source list descriptors
  size_t p2p_off_cap_ = 0;        // mailbox capacity d_src_off_ was filled for
  uint32_t *h_pinned_ = nullptr;  // pinned mirror for counts read back from the device
  // Mapped pinned word the key ingest reports an out-of-range key through: the host reads it right after the
  // ingest without a copy.
  uint32_t *h_ingest_err_ = nullptr, *d_ingest_err_ = nullptr;
  size_t h_pinned_words_ = 0;

  BatchDesc cur_batch_, prev_batch_;
  StepStats stats_;

  // profiling
  struct Span { int phase; cudaEvent_t a, b; };
  int tic(int phase, cudaStream_t s = nullptr);
  void toc(int span, cudaStream_t s = nullptr);
  void collectSpans();
  void resolveSpans();
  static constexpr size_t kMaxDeferredSpans = 1 << 15;
  bool profile_ = false;   // this step is being timed
  int profile_every_ = 0;
  size_t profile_step_ = 0;
  std::vector<Span> spans_;
  size_t spans_used_ = 0;
  cudaEvent_t ev_epoch_ = nullptr;          // recorded on stream_main_ when profiling is enabled
  std::vector<double> timeline_;            // ring of (phase, start, end), kTimelineSpans entries
  size_t timeline_next_ = 0, timeline_count_ = 0;
  static constexpr size_t kTimelineSpans = 256;
  double phase_ms_[kPhCount] = {};
  long long phase_calls_[kPhCount] = {};
};

}  // namespace hetuCTR
