#include "core/hetu_table.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

#include "core/p2p.h"
#include "core/transport.h"
#include "hctr_kernels.h"
#include "utils/errors.h"

namespace hetuCTR {

namespace {
unsigned long g_seed = 0;

template <class... Args>
void info(const HetuTable &t, Args... args) {
  if (t.verbose_ >= 1) {
    std::cout << "HetuTable rank " << t.rank_ << ": ";
    (void)std::initializer_list<int>{(std::cout << args, 0)...};
    std::cout << std::endl;
  }
}

size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }
}  // namespace

void set_seed(unsigned long seed) { g_seed = seed; }
unsigned long get_seed() { return g_seed; }

void DevBuf::ensure(size_t want) {
  if (want <= bytes) return;
  release();
  // round to 256 B so every buffer base keeps 16-byte (and TMA-friendly) alignment
  want = round_up(want, 256);
  HCTR_CUDA(cudaMalloc(&p, want));
  bytes = want;
}

void DevBuf::release() {
  if (p) cudaFree(p);
  p = nullptr;
  bytes = 0;
}

// ------------------------------------------------------------------------------------------------
// Construction.  Same order as the reference (csrc/core/table_initialize.cu:116-164): device check,
// communicator, table layout, value init, batch descriptors.
// ------------------------------------------------------------------------------------------------
HetuTable::HetuTable(const int rank, const int nrank, const int device_id, const std::string &ip, const int port,
                     const size_t embedding_length, const size_t embedding_width, const version_t pull_bound,
                     const version_t push_bound, const worker_t *root_id_arr, const size_t root_id_len,
                     const index_t *storage_id_arr, const size_t storage_id_len, const Initializer &init,
                     const embed_t learning_rate, const int verbose)
    : rank_(rank),
      nrank_(nrank),
      device_id_(device_id),
      kEmbeddingIDMax(embedding_length),
      kEmbeddingWidth(embedding_width),
      kStorageMax(storage_id_len),
      learning_rate_(learning_rate),
      pull_bound_(pull_bound),
      push_bound_(push_bound),
      verbose_(verbose) {
  HCTR_CHECK(nrank >= 1 && nrank <= 256, "nrank must be in [1, 256] (owner ids are one byte)");
  HCTR_CHECK(rank >= 0 && rank < nrank, "rank out of range");
  HCTR_CHECK(embedding_width >= 1, "width must be positive");
  HCTR_CHECK(root_id_len == embedding_length, "root_arr must have `length` entries");
  HCTR_CHECK(embedding_length < (size_t)1 << 40, "length too large");
  HCTR_CHECK(storage_id_len < (size_t)1 << 31, "at most 2^31-1 rows can be stored per rank");
  int num_gpus = 0;
  HCTR_CUDA(cudaGetDeviceCount(&num_gpus));
  HCTR_CHECK(device_id >= 0 && device_id < num_gpus, "InCorrect device number.");
  HCTR_CUDA(cudaSetDevice(device_id_));
  {
    const char *env = std::getenv("HCTR_EXPAND");
    const std::string mode = env ? env : "default";
    HCTR_CHECK(mode == "default" || mode == "bulk", "HCTR_EXPAND must be default or bulk");
    expand_bulk_ = mode == "bulk";
    const char *ks = std::getenv("HCTR_KEY_STRIDE");
    if (ks && std::string(ks) != "auto") {
      const long v = std::strtol(ks, nullptr, 10);
      HCTR_CHECK(v >= 0 && v <= 4096, "HCTR_KEY_STRIDE must be auto or a number of fields (0..4096)");
      key_stride_ = (uint32_t)v;
      key_stride_known_ = true;
    }
  }
  {
    // Multi-rank tables: stream_main_ carries the step's chain of short, latency-bound kernels and gets the highest
    // priority, so that their thread blocks are placed ahead of the bulk gradient reduction that runs concurrently on
    // stream_reduce_.  A single-rank table is the other way round: the row expansion does not need the dedupe
    // pipeline (every key is stored here and the key ingest resolves the rows), so reduction + expansion on
    // stream_reduce_ are the step's critical path and the dedupe on stream_main_ - whose results only the NEXT
    // step's reduction reads - fills in behind them.
    int lo = 0, hi = 0;
    HCTR_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    const bool single = nrank == 1;
    HCTR_CUDA(cudaStreamCreateWithPriority(&stream_main_, cudaStreamNonBlocking, single ? lo : hi));
    // the side stream carries the few long-run CTAs that should start ahead of the bulk kernels
    HCTR_CUDA(cudaStreamCreateWithPriority(&stream_side_, cudaStreamNonBlocking, single ? lo : hi));
    HCTR_CUDA(cudaStreamCreateWithPriority(&stream_reduce_, cudaStreamNonBlocking, single ? hi : lo));
    HCTR_CUDA(cudaStreamCreateWithPriority(&stream_reduce_side_, cudaStreamNonBlocking, hi));
  }
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_rfork_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_rjoin_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_decide_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_reduce_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_keys_, cudaEventDisableTiming));
  HCTR_CUDA(cudaEventCreateWithFlags(&ev_early_, cudaEventDisableTiming));
  if (const char *e = std::getenv("HCTR_SPLIT_HOST_EXPAND")) split_host_expand_ = std::atoi(e) != 0;
  if (const char *e = std::getenv("HCTR_P2P_FUSED_EXPAND")) fused_refresh_expand_ = std::atoi(e) != 0;

  try {
    initComm(ip, port);
    info(*this, "communicator ready");
    initTable(root_id_arr, storage_id_arr);
    if (p2p_) p2p_->setErr(d_err_.as<uint32_t>());

    int kind;
    switch (init.type) {
      case InitType::kZero: kind = 0; break;
      case InitType::kNormal: kind = 1; break;
      case InitType::kUniform: kind = 2; break;
      case InitType::kTruncatedNormal: kind = 3; break;
      default: throw std::runtime_error("Unknown initializer.");
    }
    HCTR_LAUNCH(hctr_initialize(d_embedding_.as<float>(), kStorageMax * kEmbeddingWidth, kind, init.param.first,
                                init.param.second, (unsigned int)g_seed, stream_main_));
    HCTR_CUDA(cudaStreamSynchronize(stream_main_));
    info(*this, "Table Init Successfully");

    for (BatchDesc *b : {&cur_batch_, &prev_batch_}) {
      b->seg.assign(nrank_ + 1, 0);
      b->query_send.assign(nrank_, 0);
      b->query_recv.assign(nrank_, 0);
      b->push_send.assign(nrank_, 0);
      b->push_recv.assign(nrank_, 0);
      b->ret_send.assign(nrank_, 0);
      b->ret_recv.assign(nrank_, 0);
      HCTR_CUDA(cudaMallocHost(&b->h_meta, (HCTR_META_WORDS + (size_t)nrank_ + 1) * sizeof(uint32_t)));
      reserveBatch(*b, 1);
    }
    HCTR_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&h_ingest_err_), 64, cudaHostAllocMapped));
    h_ingest_err_[0] = h_ingest_err_[1] = 0;
    HCTR_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&d_ingest_err_), h_ingest_err_, 0));
    reserveShared(1);
    h_pinned_words_ = HCTR_META_WORDS + (size_t)nrank_ + 1 + 12 * (size_t)nrank_ + 16;
    HCTR_CUDA(cudaMallocHost(&h_pinned_, h_pinned_words_ * sizeof(uint32_t)));
    HCTR_CUDA(cudaMallocHost(&h_src_, (size_t)nrank_ * 16 + 32));
  } catch (...) {
    releaseAll();
    throw;
  }
}

void HetuTable::initComm(const std::string &ip, int port) {
  if (nrank_ == 1) return;  // a single-rank table has nobody to talk to
  transport_ = make_transport(rank_, nrank_, ip, port, verbose_);
  // Exchange flavour: HCTR_EXCHANGE = auto (default) | p2p | nccl.  The peer-to-peer exchange needs one
  // process per GPU and peer access between all of them; all ranks take the same decision.
  const char *env = std::getenv("HCTR_EXCHANGE");
  const std::string mode = env ? env : "auto";
  HCTR_CHECK(mode == "auto" || mode == "p2p" || mode == "nccl", "HCTR_EXCHANGE must be auto, p2p or nccl");
  // Thread ranks of one process (in-process transport) use their memcpy exchange unless p2p is asked for by name:
  // the mailbox kernels then run on one GPU with a host barrier between publishing and consuming.
  if (mode != "nccl" && (transport_->multiProcess() || mode == "p2p")) {
    p2p_ = std::make_unique<P2PMailbox>(rank_, nrank_, device_id_, kEmbeddingWidth, transport_.get());
    use_p2p_ = p2p_->usable();
    if (!use_p2p_) p2p_.reset();
  }
  HCTR_CHECK(mode != "p2p" || use_p2p_, "HCTR_EXCHANGE=p2p but the ranks cannot map each other's memory");
  info(*this, "exchange: ", exchangeName());
}

const char *HetuTable::exchangeName() const {
  if (nrank_ == 1) return "none";
  return use_p2p_ ? "p2p" : transport_->name();
}

// csrc/core/table_initialize.cu:66-114 — owner array, storage layout (cached rows first, stable),
// key -> row table, versions, pending gradient state.
void HetuTable::initTable(const worker_t *root, const index_t *storage) {
  const size_t N = kEmbeddingIDMax, S = kStorageMax, W = kEmbeddingWidth;
  length_pad_ = round_up(std::max<size_t>(N, 1), HCTR_BLOCK_KEYS);
  d_root_.ensure(std::max<size_t>(N, 1));
  HCTR_CUDA(cudaMemcpyAsync(d_root_.p, root, N, cudaMemcpyHostToDevice, stream_main_));
  d_row_of_.ensure(std::max<size_t>(N, 1) * sizeof(int32_t));
  d_err_.ensure(256);
  HCTR_CUDA(cudaMemsetAsync(d_err_.p, 0, 256, stream_main_));
  uint32_t *err = d_err_.as<uint32_t>();
  unsigned long long *owned_cnt = reinterpret_cast<unsigned long long *>(d_err_.as<char>() + 64);

  DevBuf raw, flags, before, scratch;
  raw.ensure(std::max<size_t>(S, 1) * sizeof(index_t));
  flags.ensure((S + 1) * sizeof(uint32_t));
  before.ensure((S + 1) * sizeof(uint32_t));
  scratch.ensure(hctr_scan_scratch_words(S + 1) * sizeof(uint32_t));
  d_stored_keys_.ensure(std::max<size_t>(S, 1) * sizeof(index_t));
  HCTR_CUDA(cudaMemcpyAsync(raw.p, storage, S * sizeof(index_t), cudaMemcpyHostToDevice, stream_main_));
  HCTR_LAUNCH(hctr_storage_flags(raw.as<int64_t>(), S, N, d_root_.as<uint8_t>(), rank_, flags.as<uint32_t>(), err,
                                 stream_main_));
  HCTR_LAUNCH(hctr_scan_exclusive_u32(flags.as<uint32_t>(), before.as<uint32_t>(), S, nullptr,
                                      scratch.as<uint32_t>(), stream_main_));
  HCTR_LAUNCH(hctr_storage_layout(raw.as<int64_t>(), S, flags.as<uint32_t>(), before.as<uint32_t>(),
                                  d_stored_keys_.as<int64_t>(), stream_main_));
  uint32_t n_cached = 0;
  HCTR_CUDA(cudaMemcpyAsync(&n_cached, before.as<uint32_t>() + S, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                            stream_main_));
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));
  kNonLocalStorageMax = n_cached;

  d_version_.ensure(std::max<size_t>(S, 1) * sizeof(version_t));
  d_updates_.ensure(std::max<size_t>(kNonLocalStorageMax, 1) * sizeof(version_t));
  d_embedding_.ensure(std::max<size_t>(S * W, 1) * sizeof(embed_t));
  d_gradient_.ensure(std::max<size_t>(kNonLocalStorageMax * W, 1) * sizeof(embed_t));
  HCTR_CUDA(cudaMemsetAsync(d_gradient_.p, 0, d_gradient_.bytes, stream_main_));
  HCTR_CUDA(cudaMemsetAsync(d_updates_.p, 0, d_updates_.bytes, stream_main_));
  HCTR_LAUNCH(hctr_table_build(d_stored_keys_.as<int64_t>(), S, kNonLocalStorageMax, N, d_row_of_.as<int32_t>(),
                               d_version_.as<int64_t>(), err, stream_main_));
  HCTR_LAUNCH(hctr_count_owned(d_root_.as<uint8_t>(), N, rank_, owned_cnt, stream_main_));
  uint32_t h_err = 0;
  unsigned long long h_owned = 0;
  HCTR_CUDA(cudaMemcpyAsync(&h_err, err, sizeof(h_err), cudaMemcpyDeviceToHost, stream_main_));
  HCTR_CUDA(cudaMemcpyAsync(&h_owned, owned_cnt, sizeof(h_owned), cudaMemcpyDeviceToHost, stream_main_));
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));
  raw.release();
  flags.release();
  before.release();
  scratch.release();
  HCTR_CUDA(cudaMemsetAsync(d_err_.p, 0, 256, stream_main_));
  HCTR_CHECK(!(h_err & HCTR_ERR_KEY_RANGE), "storage_arr holds a key outside [0, length)");
  HCTR_CHECK(!(h_err & HCTR_ERR_CAPACITY), "storage_arr lists a key twice");
  // The owner answers every query for its rows (csrc/core/handle_query.cu:12-15 asserts it), so a
  // rank must store all rows it owns.
  HCTR_CHECK(h_owned == S - kNonLocalStorageMax, "storage_arr must contain every key whose root_arr entry is this rank");

  if (nrank_ > 1) {
    // owner-side apply: one source-mask word per owned row, and the per-source list descriptors
    d_row_mask_.ensure(std::max<size_t>(S - kNonLocalStorageMax, 1) * sizeof(unsigned long long));
    HCTR_CUDA(cudaMemsetAsync(d_row_mask_.p, 0, d_row_mask_.bytes, stream_main_));
    d_row_head_.ensure(std::max<size_t>(S - kNonLocalStorageMax, 1) * sizeof(unsigned long long));
    HCTR_CUDA(cudaMemsetAsync(d_row_head_.p, 0, d_row_head_.bytes, stream_main_));
    d_src_off_.ensure((size_t)nrank_ * sizeof(unsigned long long));
    d_src_cnt_.ensure(((size_t)nrank_ + 1) * sizeof(uint32_t));
  }

  // dedupe scratch over the (owner, key) space: all-zero at rest
  const size_t words = (size_t)nrank_ * length_pad_ / HCTR_WORD_BITS;
  const size_t blocks = (size_t)nrank_ * length_pad_ / HCTR_BLOCK_KEYS;
  d_bits_.ensure(words * sizeof(unsigned long long));
  d_word_base_.ensure(words * sizeof(uint32_t));
  d_blk_cnt_.ensure((2 * (blocks / 8 + 2)) * sizeof(uint32_t));  // chain scratch of the block-rank kernel
  HCTR_CUDA(cudaMemsetAsync(d_bits_.p, 0, d_bits_.bytes, stream_main_));
  d_blk_flag_.ensure(blocks + 1);
  HCTR_CUDA(cudaMemsetAsync(d_blk_cnt_.p, 0, d_blk_cnt_.bytes, stream_main_));
  HCTR_CUDA(cudaMemsetAsync(d_blk_flag_.p, 0, d_blk_flag_.bytes, stream_main_));
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));
}

void HetuTable::reserveBatch(BatchDesc &b, size_t batch) {
  if (batch <= b.capacity) return;
  if (b.capacity) info(*this, "ReAllocate cuda memory for batch ", b.capacity, "->", batch);
  HCTR_CHECK(batch < (size_t)1 << 31, "batch too large");
  b.keys.ensure(batch * sizeof(index_t));
  b.idx_map.ensure(batch * sizeof(int32_t));
  b.sorted_pos.ensure(batch * sizeof(uint32_t));
  b.uniq.ensure(batch * sizeof(index_t));
  b.uniq_owner.ensure(batch);
  b.uniq_row.ensure(batch * sizeof(int32_t));
  b.run_start.ensure((batch + 1) * sizeof(uint32_t));
  b.meta.ensure((HCTR_META_WORDS + nrank_ + 1) * sizeof(uint32_t));
  b.pos_row.ensure(batch * sizeof(int32_t));
  b.heavy.ensure((batch / 32 + 2) * sizeof(uint32_t));
  b.rank.ensure(batch * sizeof(uint32_t));
  if (nrank_ > 1) {
    b.need_push.ensure((batch + 1) * sizeof(uint32_t));
    b.push_slot.ensure((batch + 1) * sizeof(uint32_t));
  }
  b.capacity = batch;
}

void HetuTable::reserveShared(size_t batch) {
  if (batch <= shared_capacity_) return;
  const size_t blocks = (size_t)nrank_ * length_pad_ / HCTR_BLOCK_KEYS;
  // receive side of a step can hold up to batch keys from every rank
  const size_t scan_n = std::max(blocks, batch * (size_t)nrank_) + 2;
  d_scan_.ensure(hctr_scan_scratch_words(scan_n) * sizeof(uint32_t));
  d_chain_.ensure(hctr_scan_chained_scratch_words(batch + 1) * sizeof(uint32_t));
  HCTR_CUDA(cudaMemsetAsync(d_chain_.p, 0, d_chain_.bytes, stream_main_));
  d_chain3_.ensure(hctr_scan_chained_scratch_words(batch + 1) * sizeof(uint32_t));
  HCTR_CUDA(cudaMemsetAsync(d_chain3_.p, 0, d_chain3_.bytes, stream_main_));
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));  // the scratch is used from other streams as well
  d_sk_.ensure(batch * sizeof(unsigned long long));
  d_cnt_.ensure((batch + 1) * sizeof(uint32_t));  // all-zero between calls, like the bitmap
  HCTR_CUDA(cudaMemsetAsync(d_cnt_.p, 0, d_cnt_.bytes, stream_main_));
  d_push_count_.ensure((size_t)nrank_ * sizeof(uint32_t));
  d_push_base_.ensure((size_t)nrank_ * sizeof(uint32_t));
  d_recv_idx_.ensure((batch + 1) * sizeof(uint32_t));
  if (nrank_ > 1) {
    const size_t n = nrank_;
    d_cnt_s_.ensure(2 * n * sizeof(uint32_t));
    d_cnt_r_.ensure(2 * n * sizeof(uint32_t));
    d_retcnt_s_.ensure(n * sizeof(uint32_t));
    d_retcnt_r_.ensure(n * sizeof(uint32_t));
    d_seg_r_.ensure((n + 1) * sizeof(uint32_t));
    d_qver_s_.ensure(batch * sizeof(version_t));
    d_pkey_s_.ensure(batch * sizeof(index_t));
    d_pupd_s_.ensure(batch * sizeof(version_t));
    d_pval_s_.ensure(batch * kEmbeddingWidth * sizeof(embed_t));
    d_flag_r_.ensure(batch + 16);
    d_recv_slot_.ensure((batch + 1) * sizeof(uint32_t));
  }
  shared_capacity_ = batch;
}

// ------------------------------------------------------------------------------------------------
// preprocess — csrc/core/hetu_gpu_table.cu:43-65
// ------------------------------------------------------------------------------------------------
void HetuTable::preprocess(index_t *data_ptr, size_t batch_size) {
  HCTR_CUDA(cudaSetDevice(device_id_));
  // A single-rank table never waits for its dedupe here: the next reduction reads the batch's sizes on the device.
  if (nrank_ == 1) flushDedupe(cur_batch_);  // two preprocess calls in a row: the first one's dedupe is still due
  else finalizePending();
  batch_open_ = true;
  profile_ = profile_every_ > 0 && (profile_step_++ % (size_t)profile_every_) == 0;
  flushOrdering(cur_batch_);  // normally done by push_pull already; two preprocess calls in a row get here
  std::swap(cur_batch_, prev_batch_);
  BatchDesc &cur = cur_batch_, &prev = prev_batch_;
  cur.decided = false;
  reserveBatch(cur, std::max<size_t>(batch_size, 1));
  reserveShared(std::max<size_t>(batch_size, 1));
  if (use_p2p_) p2p_->reserve(std::max<size_t>(batch_size, 1), stream_main_);  // collective when it grows
  cur.batch_size = batch_size;
  const int n = nrank_;
  const size_t meta_words = HCTR_META_WORDS + n + 1;

  bool keys_on_device = false;
  if (batch_size > 0) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, data_ptr) == cudaSuccess)
      keys_on_device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    else
      cudaGetLastError();
  }
  // One launch in front of the pipeline: private copy of the keys (host keys are copied first, then taken in place),
  // cleared meta words, and the local row of every batch position - which is all the row expansion needs for keys
  // that are stored here, so a single-rank table starts it without waiting for the dedupe.
  // A single-rank table ingests on the (idle) stream of its reduction: stream_main_ may still hold the previous
  // batch's dedupe, which nothing here has to wait for.  The dedupe of this batch waits for ev_keys_.
  cudaStream_t ks = n == 1 ? stream_reduce_ : stream_main_;
  const int64_t *key_src = reinterpret_cast<const int64_t *>(data_ptr);
  if (!keys_on_device) {
    HCTR_CUDA(cudaMemcpyAsync(cur.keys.p, data_ptr, sizeof(index_t) * batch_size, cudaMemcpyDefault, ks));
    key_src = cur.keys.as<int64_t>();
  }
  HCTR_LAUNCH(hctr_ingest_keys_rows(key_src, cur.keys.as<int64_t>(), batch_size, cur.meta.as<uint32_t>(),
                                    (unsigned)meta_words, d_row_of_.as<int32_t>(), kEmbeddingIDMax,
                                    cur.pos_row.as<int32_t>(), d_ingest_err_, ks));
  HCTR_CUDA(cudaEventRecord(ev_keys_, ks));
  if (n == 1) HCTR_CUDA(cudaStreamWaitEvent(stream_main_, ev_keys_, 0));

  if (!key_stride_known_ && batch_size >= 4096) detectKeyStride(cur);  // once per table
  hctr_dedupe_args a;
  a.stride = key_stride_;
  a.keys = cur.keys.as<int64_t>();
  a.batch = batch_size;
  a.length = kEmbeddingIDMax;
  a.length_pad = length_pad_;
  a.nrank = n;
  a.owner_of = d_root_.as<uint8_t>();
  a.row_of = d_row_of_.as<int32_t>();
  a.bits = d_bits_.as<unsigned long long>();
  a.chain_scratch = d_blk_cnt_.as<uint32_t>();
  a.epoch = nextEpoch();
  a.blk_flag = d_blk_flag_.as<uint8_t>();
  a.word_base = d_word_base_.as<uint32_t>();
  a.scan_scratch = d_chain_.as<uint32_t>();
  a.sk = d_sk_.as<unsigned long long>();
  a.rank_in_run = cur.rank.as<uint32_t>();
  a.heavy_list = cur.heavy.as<uint32_t>();
  a.pos_row = nullptr;  // resolved by the key ingest above
  a.uniq = cur.uniq.as<int64_t>();
  a.uniq_owner = cur.uniq_owner.as<uint8_t>();
  a.uniq_row = cur.uniq_row.as<int32_t>();
  a.cnt = d_cnt_.as<uint32_t>();
  a.run_start = cur.run_start.as<uint32_t>();
  a.sorted_pos = cur.sorted_pos.as<uint32_t>();
  a.idx_map = cur.idx_map.as<int32_t>();
  a.meta = cur.meta.as<uint32_t>();
  // run ordering happens on stream_side_, off this stream's critical path; the reduction of this batch
  // (next step) waits on the batch's own event.  The ordering stages through the batch's own rank buffer, so the
  // ordering of the previous batch may still run while this batch is deduplicated; only the descriptor being
  // recycled (two batches old) must be out of use.
  if (cur.order_recorded) HCTR_CUDA(cudaStreamWaitEvent(stream_main_, cur.ev_order, 0));
  if (!cur.ev_order) HCTR_CUDA(cudaEventCreateWithFlags(&cur.ev_order, cudaEventDisableTiming));
  if (!cur.ev_scatter) HCTR_CUDA(cudaEventCreateWithFlags(&cur.ev_scatter, cudaEventDisableTiming));
  a.side_stream = stream_side_;
  a.fork_event = cur.ev_scatter;
  // The ordering kernels are not even enqueued here: push_pull enqueues them after the gradient reduction,
  // which brings the reduction (it only starts once push_pull is called) several launches forward.
  a.join_event = nullptr;
  cur.order_recorded = false;
  cur.scatter_recorded = false;
  cur.light_ordered = false;
  cur.order_pending = true;
  cur.order_args = a;
  // The push decision for the previous batch goes first: the gradient reduction (on its own stream, started
  // by the next push_pull) only needs this, not the dedupe of the new batch that follows.

  // Push decision for the previous batch (csrc/core/preprocess.cu:167-182).  With one rank every
  // row is owned, nothing is ever pushed.
  const bool decide = n > 1 && prev.unique_size > 0;
  if (decide && !prev.decided) launchPushDecide(prev);  // normally done at the end of the previous push_pull
  HCTR_CUDA(cudaEventRecord(ev_decide_, stream_reduce_));
  prev_push_valid_ = decide;
  cur.dedupe_pending = true;
  cur.pending = true;
  if (n == 1) {
    // Single rank: nothing of this step reads what the dedupe produces (the expansion has the rows from the key
    // ingest), so its launches are left to push_pull, AFTER the reduction and the expansion have been enqueued: the
    // host reaches those sooner.  Wait only until the caller's key buffer has been consumed.
    HCTR_CUDA(cudaEventSynchronize(ev_keys_));
    if (*h_ingest_err_) {
      // a key outside the table: drop the batch (its dedupe is not enqueued yet) and report right away
      *h_ingest_err_ = 0;
      cur.dedupe_pending = cur.order_pending = cur.pending = false;
      cur.batch_size = cur.unique_size = cur.n_heavy = 0;
      throw std::runtime_error("preprocess: a key is outside [0, length)");
    }
    return;
  }
  *h_ingest_err_ = 0;  // multi-rank tables learn about bad keys from the dedupe (which also checks the owners)
  flushDedupe(cur);
  int sp;
  uint32_t *h_cnt_s = h_pinned_ + meta_words;
  uint32_t *h_cnt_r = h_cnt_s + 2 * n;
  if (n > 1 && !use_p2p_) {
    // One packed count exchange instead of the reference's two all2allExchangeShape rounds
    // (csrc/core/preprocess.cu:135,176): per peer {keys I will query, rows I will push}.
    if (decide) HCTR_CUDA(cudaStreamWaitEvent(stream_main_, ev_decide_, 0));  // push counts come from the other stream
    HCTR_LAUNCH(hctr_pack_counts(cur.meta.as<uint32_t>(), decide ? d_push_count_.as<uint32_t>() : nullptr, n,
                                 d_cnt_s_.as<uint32_t>(), stream_main_));
    std::vector<XferItem> items;
    for (int p = 0; p < n; p++)
      items.push_back({p, d_cnt_s_.as<uint32_t>() + 2 * p, 8, d_cnt_r_.as<uint32_t>() + 2 * p, 8});
    sp = tic(kPhExchange);
    transport_->exchange(items, stream_main_);
    toc(sp);
    HCTR_CUDA(cudaMemcpyAsync(h_cnt_s, d_cnt_s_.p, 2 * n * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
    HCTR_CUDA(cudaMemcpyAsync(h_cnt_r, d_cnt_r_.p, 2 * n * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
  }
  if (use_p2p_) {
    // (The device-driven exchange, where counts never visit the host.)
    // Nothing on the host depends on the result before push_pull: wait only until the caller's key
    // buffer has been consumed and let the rest of the pipeline run under the next call's launches.
    // The batch's sizes (and a key-range error, if any) are picked up at the next synchronisation.
    HCTR_CUDA(cudaEventSynchronize(ev_keys_));
    return;
  }
  transport_->waitStream(stream_main_);  // an NCCL group is in the stream: wait with a deadline
  collectSpans();
  finalizeBatch();
}

// The row expansion: the register kernel, or (HCTR_EXPAND=bulk) the bulk-copy engine variant.
int HetuTable::expandRows(size_t batch, size_t width, const int32_t *pos_row, const int32_t *idx_map,
                          const uint32_t *recv_slot, const float *recv_val, const float *embedding, float *dst,
                          uint32_t *err, cudaStream_t stream) {
  if (expand_bulk_)
    return hctr_expand_rows_bulk(batch, width, pos_row, idx_map, recv_slot, recv_val, embedding, dst, err, stream);
  return hctr_expand_rows(batch, width, pos_row, idx_map, recv_slot, recv_val, embedding, dst, stream);
}

// Looks at the first large batch (already in the table's private key buffer) for the period at which keys
// repeat: in a sample-major batch of F fields the hot keys of a field recur at distances F, 2F, ..., and never
// at other distances because fields use disjoint key ranges.  Costs one small kernel and one synchronisation,
// once.  A batch without such structure (uniform keys, a single field) leaves the positions in order.
void HetuTable::detectKeyStride(const BatchDesc &b) {
  key_stride_known_ = true;
  DevBuf scores;
  scores.ensure(65 * sizeof(uint32_t));
  uint32_t h[65] = {};
  HCTR_LAUNCH(hctr_detect_key_stride(b.keys.as<int64_t>(), b.batch_size, scores.as<uint32_t>(), stream_main_));
  HCTR_CUDA(cudaMemcpyAsync(h, scores.p, sizeof(h), cudaMemcpyDeviceToHost, stream_main_));
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));
  scores.release();
  uint32_t best = 0;
  for (int d = 1; d <= 64; d++) best = std::max(best, h[d]);
  key_stride_ = 0;
  if (best >= 64) {  // enough repeats to tell
    for (int d = 1; d <= 64; d++)
      if (2 * (uint64_t)h[d] >= best) {
        key_stride_ = (uint32_t)d;
        break;
      }
  }
  info(*this, "key batches look sample-major with ", key_stride_, " fields (0/1: no structure found)");
}

// Push decision for batch b (csrc/core/preprocess.cu:167-182), on the reduction's stream: only the reduction of
// b's gradient (and the counts published after it) need the result.  It depends on the pending-update counts as
// the previous reduction left them, so it can run as soon as b's own push_pull is over.
void HetuTable::launchPushDecide(BatchDesc &b) {
  int spd = tic(kPhPushDecide, stream_reduce_);
  HCTR_LAUNCH(hctr_push_decide_fused(b.meta.as<uint32_t>(), nrank_, rank_, b.unique_size, b.uniq_owner.as<uint8_t>(),
                                     b.uniq_row.as<int32_t>(), b.run_start.as<uint32_t>(), d_updates_.as<int64_t>(),
                                     push_bound_, b.need_push.as<uint32_t>(), b.push_slot.as<uint32_t>(),
                                     d_chain3_.as<uint32_t>(), nextEpoch(), d_push_count_.as<uint32_t>(),
                                     d_push_base_.as<uint32_t>(), d_err_.as<uint32_t>(), stream_reduce_));
  toc(spd, stream_reduce_);
  b.decided = true;
}

// Enqueues the dedupe pipeline of batch b on stream_main_ (behind the batch's key ingest) and the copy of its
// meta words to pinned memory.
void HetuTable::flushDedupe(BatchDesc &b) {
  if (!b.dedupe_pending) return;
  b.dedupe_pending = false;
  int sp = tic(kPhDedupe);
  HCTR_LAUNCH(hctr_dedupe_map(&b.order_args, stream_main_));  // records b.ev_scatter behind its last kernel
  b.scatter_recorded = true;
  toc(sp);
  const size_t meta_words = HCTR_META_WORDS + nrank_ + 1;
  HCTR_CUDA(cudaMemcpyAsync(b.h_meta, b.meta.p, meta_words * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
}

// The long runs (hot keys) are ordered on stream_side_; only the long-run kernel of the next reduction waits for
// that.  The short runs are ordered by the reduction itself where its kernel can (orderLightRuns otherwise).
void HetuTable::flushOrdering(BatchDesc &b) {
  if (!b.order_pending) return;
  b.order_pending = false;
  flushDedupe(b);
  HCTR_CUDA(cudaStreamWaitEvent(stream_side_, b.ev_scatter, 0));
  HCTR_LAUNCH(hctr_dedupe_order_heavy(&b.order_args, stream_side_));
  HCTR_CUDA(cudaEventRecord(b.ev_order, stream_side_));
  b.order_recorded = true;
}

void HetuTable::orderLightRuns(BatchDesc &b, cudaStream_t s) {
  if (b.light_ordered || !b.scatter_recorded) return;
  HCTR_CUDA(cudaStreamWaitEvent(s, b.ev_scatter, 0));
  HCTR_LAUNCH(hctr_dedupe_order_light(&b.order_args, s));
  b.light_ordered = true;
}

// Reads the counts the preprocess pipeline copied to pinned memory into the batch descriptors.
// The stream must have drained.
uint32_t HetuTable::readSizes(BatchDesc &b) {
  const int n = nrank_;
  const uint32_t *h_meta = b.h_meta;
  b.pending = false;
  b.unique_size = h_meta[HCTR_META_UNIQUE];
  b.n_heavy = h_meta[HCTR_META_NHEAVY];
  for (int p = 0; p <= n; p++) b.seg[p] = h_meta[HCTR_META_SEG + p];
  for (int p = 0; p < n; p++) b.query_send[p] = b.seg[p + 1] - b.seg[p];
  return h_meta[HCTR_META_ERR];
}

void HetuTable::finalizeBatch() {
  BatchDesc &cur = cur_batch_, &prev = prev_batch_;
  const int n = nrank_;
  const size_t meta_words = HCTR_META_WORDS + n + 1;
  const uint32_t *h_cnt_s = h_pinned_ + meta_words;
  const uint32_t *h_cnt_r = h_cnt_s + 2 * n;
  const uint32_t err = readSizes(cur);
  for (int p = 0; p < n; p++) {
    const bool host_counts = n > 1 && !use_p2p_;  // the device-driven exchange keeps counts on the device
    cur.query_recv[p] = host_counts ? h_cnt_r[2 * p] : cur.query_send[p];
    prev.push_send[p] = host_counts ? h_cnt_s[2 * p + 1] : 0;
    prev.push_recv[p] = host_counts ? h_cnt_r[2 * p + 1] : 0;
  }
  if (err & HCTR_ERR_TIMEOUT)
    throw std::runtime_error("preprocess: a chained scan gave up waiting for an earlier thread block");
  if (err & HCTR_ERR_KEY_RANGE) {
    // leave a consistent (empty) batch behind, then report
    cur.batch_size = 0;
    cur.unique_size = 0;
    cur.n_heavy = 0;
    throw std::runtime_error("preprocess: a key is outside [0, length) or its root_arr entry is >= nrank");
  }
}

// Single-rank tables hand a batch on to the next step without ever reading its sizes on the host; whoever wants
// them for the previous batch (dump, stats) gets them here.  stream_main_ must have drained.
void HetuTable::finalizePrev() {
  if (!prev_batch_.pending) return;
  const uint32_t err = readSizes(prev_batch_);
  if (err & HCTR_ERR_TIMEOUT)
    throw std::runtime_error("preprocess: a chained scan gave up waiting for an earlier thread block");
}

void HetuTable::finalizePending() {
  if (!cur_batch_.pending && !prev_batch_.pending) return;
  flushDedupe(cur_batch_);
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));
  collectSpans();
  finalizePrev();  // (the dedupe of the previous batch sits in front of this one's on the same stream)
  if (cur_batch_.pending) finalizeBatch();
}

const void *HetuTable::stageIn(const void *ptr, size_t bytes, DevBuf &buf, cudaStream_t st) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    attr.type = cudaMemoryTypeUnregistered;
  }
  if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) return ptr;
  buf.ensure(bytes);
  HCTR_CUDA(cudaMemcpyAsync(buf.p, ptr, bytes, cudaMemcpyHostToDevice, st));
  return buf.p;
}

// ------------------------------------------------------------------------------------------------
// pushPull — csrc/core/hetu_gpu_table.cu:9-41
// ------------------------------------------------------------------------------------------------
void HetuTable::pushPull(embed_t *grad, embed_t *dst) {
  HCTR_CUDA(cudaSetDevice(device_id_));
  batch_open_ = false;
  BatchDesc &cur = cur_batch_, &prev = prev_batch_;
  const int n = nrank_;
  const size_t W = kEmbeddingWidth;

  // No gradient = inference step: the previous batch is dropped (all ranks must do this together).
  if (grad == nullptr) {
    prev.batch_size = 0;
    prev.unique_size = 0;
    prev.n_heavy = 0;
    std::fill(prev.push_send.begin(), prev.push_send.end(), 0);
    std::fill(prev.push_recv.begin(), prev.push_recv.end(), 0);
  }

  // dst (and grad) are normally device memory; host buffers are staged
  embed_t *dst_dev = dst, *dst_mapped = nullptr;
  bool dst_staged = false;
  if (cur.batch_size > 0) {
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, dst);
    if (e != cudaSuccess) {
      cudaGetLastError();
      attr.type = cudaMemoryTypeUnregistered;
    }
    if (!(attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged)) {
      dst_mapped = attr.type == cudaMemoryTypeHost ? static_cast<embed_t *>(attr.devicePointer) : nullptr;
      dst_staged = true;
    }
  }
  const embed_t *grad_dev = grad;
  if (grad != nullptr && prev.batch_size > 0)
    grad_dev = static_cast<const embed_t *>(stageIn(grad, prev.batch_size * W * sizeof(embed_t), d_stage_grad_, stream_reduce_));

  // Single rank, gradients arriving from host memory and dst in pinned host memory: the step is two transfers over
  // the host link with a short computation between them.  The rows of dst whose keys the previous batch did not
  // contain do not depend on the gradients, so they are written (by the kernel, straight into dst) while the
  // gradients are still coming in, and only the other rows after the update: the two directions of the link overlap.
  const bool split_expand = n == 1 && dst_mapped != nullptr && grad_dev != grad && prev.scatter_recorded &&
                            cur.batch_size > 0 && split_host_expand_;
  if (split_expand) {
    dst_dev = dst_mapped;
    dst_staged = false;
    // stream_main_ is idle here (the previous batch's dedupe ended long ago; this batch's is enqueued below) and
    // already waits for the key ingest
    HCTR_CUDA(cudaStreamWaitEvent(stream_main_, prev.ev_scatter, 0));
    HCTR_LAUNCH(hctr_expand_rows_subset(cur.batch_size, W, cur.pos_row.as<int32_t>(), cur.keys.as<int64_t>(),
                                        prev.uniq.as<int64_t>(), prev.meta.as<uint32_t>(), 0,
                                        d_embedding_.as<float>(), dst_dev, stream_main_));
    HCTR_CUDA(cudaEventRecord(ev_early_, stream_main_));
  } else if (dst_staged) {
    d_stage_dst_.ensure(cur.batch_size * W * sizeof(embed_t));
    dst_dev = d_stage_dst_.as<embed_t>();
  }

  size_t pushed = 0, push_recv = 0, q_recv = 0;
  for (int p = 0; p < n; p++) {
    pushed += prev.push_send[p];
    push_recv += prev.push_recv[p];
    q_recv += cur.query_recv[p];
  }
  stats_ = StepStats();
  stats_.batch = cur.batch_size;
  stats_.unique = cur.unique_size;
  stats_.prev_batch = prev.batch_size;
  stats_.prev_unique = prev.unique_size;
  stats_.pushed_rows = pushed;
  stats_.received_push_rows = push_recv;
  stats_.queried_keys = q_recv;

  // A. duplicate-gradient reduction + local apply + pack (generateGradient)
  // A single-rank table has not read the previous batch's sizes (that would mean waiting for its dedupe on the
  // host): the kernels take them from the batch's meta words on the device, the host passes upper bounds.
  const bool sizes_on_device = n == 1 && prev.pending;
  if (sizes_on_device ? prev.batch_size > 0 : prev.unique_size > 0) {
    hctr_reduce_args r;
    r.meta = sizes_on_device ? prev.meta.as<uint32_t>() : nullptr;
    r.n_unique = sizes_on_device ? prev.batch_size : prev.unique_size;
    r.width = W;
    r.n_cached = kNonLocalStorageMax;
    r.neg_lr = -learning_rate_;
    r.grad = grad_dev;
    r.run_start = prev.run_start.as<uint32_t>();
    r.sorted_pos = prev.sorted_pos.as<uint32_t>();
    r.heavy_list = prev.heavy.as<uint32_t>();
    r.n_heavy = sizes_on_device ? prev.batch_size / (HCTR_LIGHT_RUN + 1) + 1 : prev.n_heavy;
    r.uniq = prev.uniq.as<int64_t>();
    r.uniq_row = prev.uniq_row.as<int32_t>();
    r.need_push = n > 1 ? prev.need_push.as<uint32_t>() : nullptr;
    r.push_slot = n > 1 ? prev.push_slot.as<uint32_t>() : nullptr;
    r.embedding = d_embedding_.as<float>();
    r.version = d_version_.as<int64_t>();
    r.pending = d_gradient_.as<float>();
    r.pending_cnt = d_updates_.as<int64_t>();
    r.push_key = d_pkey_s_.as<int64_t>();
    r.push_updates = d_pupd_s_.as<int64_t>();
    r.push_val = d_pval_s_.as<float>();
    r.work_counter = d_err_.as<uint32_t>() + 32;
    r.p2p = use_p2p_ ? &p2p_->ctx() : nullptr;
    r.uniq_owner = prev.uniq_owner.as<uint8_t>();
    r.push_base = d_push_base_.as<uint32_t>();
    r.side_stream = stream_reduce_side_;
    r.fork_event = ev_rfork_;
    r.join_event = ev_rjoin_;
    // Own stream: overlaps the (still running) dedupe of the current batch.  It needs the push decision of
    // the previous batch (ev_decide_) and nothing else from stream_main_.
    HCTR_CUDA(cudaStreamWaitEvent(stream_reduce_, ev_decide_, 0));
    // the batch's runs must exist (end of its dedupe); the ordering of its long runs only concerns the long-run
    // kernel, and the short runs are ordered by the streaming kernel as it loads them (or here, for the row
    // widths and gradient buffers that kernel does not take)
    if (prev.scatter_recorded) HCTR_CUDA(cudaStreamWaitEvent(stream_reduce_, prev.ev_scatter, 0));
    if (!prev.light_ordered && !hctr_reduce_orders_short_runs(W, grad_dev)) orderLightRuns(prev, stream_reduce_);
    r.short_runs_unordered = prev.light_ordered ? 0 : 1;
    r.long_wait_event = prev.order_recorded ? prev.ev_order : nullptr;
    int sp = tic(kPhReduce, stream_reduce_);
    HCTR_LAUNCH(hctr_grad_reduce_apply_pack(&r, stream_reduce_));
    toc(sp, stream_reduce_);
    HCTR_CUDA(cudaEventRecord(ev_reduce_, stream_reduce_));
    // everything below reads rows / versions the reduction updates (a single-rank table runs it on the reduction's
    // own stream instead, and its dedupe on stream_main_ needs nothing from here)
    if (n > 1) HCTR_CUDA(cudaStreamWaitEvent(stream_main_, ev_reduce_, 0));
  }
  if (n > 1) flushOrdering(cur);  // the current batch's run ordering, deferred by preprocess

  // the stream the step ends on
  cudaStream_t tail = n == 1 ? stream_reduce_ : stream_main_;
  if (n == 1) {
    // Single rank: every key is owned and stored here; the pull is a local gather that only needs the rows the
    // key ingest resolved (ev_keys_) and the reduction in front of it on this stream.  The dedupe of this batch
    // keeps running on stream_main_; nothing of this step reads its results.
    HCTR_CUDA(cudaStreamWaitEvent(tail, ev_keys_, 0));
    int sp = tic(kPhExpand, tail);
    if (split_expand) {
      HCTR_LAUNCH(hctr_expand_rows_subset(cur.batch_size, W, cur.pos_row.as<int32_t>(), cur.keys.as<int64_t>(),
                                          prev.uniq.as<int64_t>(), prev.meta.as<uint32_t>(), 1,
                                          d_embedding_.as<float>(), dst_dev, tail));
      HCTR_CUDA(cudaStreamWaitEvent(tail, ev_early_, 0));  // the step ends when both halves are in dst
    } else {
      HCTR_LAUNCH(expandRows(cur.batch_size, W, cur.pos_row.as<int32_t>(), cur.idx_map.as<int32_t>(), nullptr,
                                   nullptr, d_embedding_.as<float>(), dst_dev, d_ingest_err_ + 1, tail));
    }
    toc(sp, tail);
    // The dedupe of this batch goes behind the step's critical path on stream_main_ (low priority): only the next
    // step's reduction needs it.  (Holding it back until the reduction has ended was measured and is slower: the
    // dedupe then ends after the expansion and the next reduction waits for it.)
    flushDedupe(cur);
    flushOrdering(cur);
  } else if (use_p2p_) {
    exchangeP2P(dst_dev);
  } else {
    const size_t U = cur.unique_size;
    // B. query = (key, local version) for every unique key (generateQuery)
    int sp = tic(kPhQuery);
    HCTR_LAUNCH(hctr_query_versions(U, cur.uniq_row.as<int32_t>(), d_version_.as<int64_t>(),
                                    d_qver_s_.as<int64_t>(), stream_main_));
    toc(sp);

    // exchange 1 (keys + versions) and exchange 3 (pushed ids, update counts, rows) in ONE group
    d_qkey_r_.ensure(std::max<size_t>(q_recv, 1) * sizeof(index_t));
    d_qver_r_.ensure(std::max<size_t>(q_recv, 1) * sizeof(version_t));
    d_pkey_r_.ensure(std::max<size_t>(push_recv, 1) * sizeof(index_t));
    d_pupd_r_.ensure(std::max<size_t>(push_recv, 1) * sizeof(version_t));
    d_pval_r_.ensure(std::max<size_t>(push_recv * W, 1) * sizeof(embed_t));
    d_flag_s_.ensure(q_recv + 16);
    d_flag32_.ensure((std::max(q_recv, U) + 1) * sizeof(uint32_t));
    d_ret_slot_.ensure((q_recv + 1) * sizeof(uint32_t));
    {
      size_t so = 0, ro = 0, pso = 0, pro = 0;
      std::vector<XferItem> items;
      for (int p = 0; p < n; p++) {
        const size_t qs = cur.query_send[p], qr = cur.query_recv[p];
        const size_t ps = prev.push_send[p], pr = prev.push_recv[p];
        items.push_back({p, cur.uniq.as<int64_t>() + so, qs * 8, d_qkey_r_.as<int64_t>() + ro, qr * 8});
        items.push_back({p, d_qver_s_.as<int64_t>() + so, qs * 8, d_qver_r_.as<int64_t>() + ro, qr * 8});
        items.push_back({p, d_pkey_s_.as<int64_t>() + pso, ps * 8, d_pkey_r_.as<int64_t>() + pro, pr * 8});
        items.push_back({p, d_pupd_s_.as<int64_t>() + pso, ps * 8, d_pupd_r_.as<int64_t>() + pro, pr * 8});
        items.push_back({p, d_pval_s_.as<float>() + pso * W, ps * W * 4, d_pval_r_.as<float>() + pro * W, pr * W * 4});
        so += qs;
        ro += qr;
        pso += ps;
        pro += pr;
      }
      sp = tic(kPhExchange);
      transport_->exchange(items, stream_main_);
      toc(sp);
    }

    // C. owner applies pushed rows in source order (handleGradient)
    {
      sp = tic(kPhOwnerUpdate);
      if (n >= 4 && n <= 32) {
        // all sources in two launches, same per-row order as source-by-source (with fewer than three remote
        // sources a launch per source is cheaper)
        unsigned long long *h_off = reinterpret_cast<unsigned long long *>(h_src_);
        uint32_t *h_start = reinterpret_cast<uint32_t *>(h_off + n);
        size_t off = 0;
        for (int p = 0; p < n; p++) {
          h_off[p] = off;
          h_start[p] = (uint32_t)off;
          off += prev.push_recv[p];
        }
        h_start[n] = (uint32_t)off;
        HCTR_CUDA(cudaMemcpyAsync(d_src_off_.p, h_off, n * sizeof(unsigned long long), cudaMemcpyHostToDevice, stream_main_));
        HCTR_CUDA(cudaMemcpyAsync(d_src_cnt_.p, h_start, (n + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_main_));
        d_ent_row_.ensure((push_recv + 1) * sizeof(int32_t));
        d_ent_next_.ensure((push_recv + 1) * sizeof(uint32_t));
        HCTR_LAUNCH(hctr_owner_update_merged(n, push_recv, W, d_pkey_r_.as<int64_t>(),
                                             d_pupd_r_.as<int64_t>(), d_pval_r_.as<float>(),
                                             d_src_off_.as<unsigned long long>(), d_src_cnt_.as<uint32_t>(),
                                             d_row_of_.as<int32_t>(), kEmbeddingIDMax, kNonLocalStorageMax,
                                             d_row_mask_.as<unsigned long long>(),
                                             d_row_head_.as<unsigned long long>(), nextEpoch(),
                                             d_ent_row_.as<int32_t>(), d_ent_next_.as<uint32_t>(), d_embedding_.as<float>(),
                                             d_version_.as<int64_t>(), d_err_.as<uint32_t>(), stream_main_));
      } else {
        size_t off = 0;
        for (int p = 0; p < n; p++) {
          const size_t c = prev.push_recv[p];
          HCTR_LAUNCH(hctr_owner_update(c, W, d_pkey_r_.as<int64_t>() + off, d_pupd_r_.as<int64_t>() + off,
                                        d_pval_r_.as<float>() + off * W, d_row_of_.as<int32_t>(), kEmbeddingIDMax,
                                        kNonLocalStorageMax, d_embedding_.as<float>(), d_version_.as<int64_t>(),
                                        d_err_.as<uint32_t>(), stream_main_));
          off += c;
        }
      }
      toc(sp);
    }

    // D. owner decides staleness, counts per requester, gathers rows (handleQuery)
    uint32_t *h_seg = h_pinned_ + HCTR_META_WORDS + n + 1 + 4 * n;  // [n+1] receive-side segment starts
    {
      size_t acc = 0;
      for (int p = 0; p <= n; p++) {
        h_seg[p] = (uint32_t)acc;
        if (p < n) acc += cur.query_recv[p];
      }
    }
    HCTR_CUDA(cudaMemcpyAsync(d_seg_r_.p, h_seg, (n + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_main_));
    sp = tic(kPhStaleGather);
    HCTR_LAUNCH(hctr_stale_check(q_recv, n, rank_, d_seg_r_.as<uint32_t>(), d_qkey_r_.as<int64_t>(),
                                 d_qver_r_.as<int64_t>(), d_row_of_.as<int32_t>(), kEmbeddingIDMax,
                                 kNonLocalStorageMax, d_version_.as<int64_t>(), pull_bound_, d_flag_s_.as<uint8_t>(),
                                 d_flag32_.as<uint32_t>(), d_ret_slot_.as<uint32_t>(), d_scan_.as<uint32_t>(),
                                 d_retcnt_s_.as<uint32_t>(), d_err_.as<uint32_t>(), stream_main_));
    // the number of rows to return is only known on the device; the return buffer is sized for the
    // worst case (every queried key stale)
    d_rver_s_.ensure(std::max<size_t>(q_recv, 1) * sizeof(version_t));
    d_rval_s_.ensure(std::max<size_t>(q_recv * W, 1) * sizeof(embed_t));
    HCTR_LAUNCH(hctr_gather_rows(q_recv, W, d_qkey_r_.as<int64_t>(), d_flag_s_.as<uint8_t>(),
                                 d_ret_slot_.as<uint32_t>(), d_row_of_.as<int32_t>(), d_embedding_.as<float>(),
                                 d_version_.as<int64_t>(), d_rval_s_.as<float>(), d_rver_s_.as<int64_t>(),
                                 stream_main_));
    toc(sp);

    // flags travel back along the query route (one byte per key instead of the reference's int64,
    // csrc/core/all2all.cu:89-101) together with the per-requester row counts
    {
      size_t so = 0, ro = 0;
      std::vector<XferItem> items;
      for (int p = 0; p < n; p++) {
        const size_t qs = cur.query_send[p], qr = cur.query_recv[p];
        items.push_back({p, d_flag_s_.as<uint8_t>() + ro, qr, d_flag_r_.as<uint8_t>() + so, qs});
        items.push_back({p, d_retcnt_s_.as<uint32_t>() + p, 4, d_retcnt_r_.as<uint32_t>() + p, 4});
        so += qs;
        ro += qr;
      }
      sp = tic(kPhExchange);
      transport_->exchange(items, stream_main_);
      toc(sp);
    }
    uint32_t *h_ret_s = h_pinned_ + HCTR_META_WORDS + n + 1 + 5 * n + 1;
    uint32_t *h_ret_r = h_ret_s + n;
    uint32_t *h_err = h_ret_r + n;
    HCTR_CUDA(cudaMemcpyAsync(h_ret_s, d_retcnt_s_.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
    HCTR_CUDA(cudaMemcpyAsync(h_ret_r, d_retcnt_r_.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
    HCTR_CUDA(cudaMemcpyAsync(h_err, d_err_.p, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
    // meanwhile: slots of the rows this rank will receive (scan of the flags it got back)
    sp = tic(kPhRefresh);
    HCTR_LAUNCH(hctr_recv_slots(U, d_flag_r_.as<uint8_t>(), d_flag32_.as<uint32_t>(), d_recv_slot_.as<uint32_t>(),
                                d_scan_.as<uint32_t>(), stream_main_));
    toc(sp);
    transport_->waitStream(stream_main_);  // the one mid-step host sync: NCCL needs the row counts

    if (*h_err) {
      HCTR_CUDA(cudaMemsetAsync(d_err_.p, 0, sizeof(uint32_t), stream_main_));
      // keep the collective pattern intact on every rank, then report
    }
    size_t ret_total = 0, recv_total = 0;
    for (int p = 0; p < n; p++) {
      cur.ret_send[p] = h_ret_s[p];
      cur.ret_recv[p] = h_ret_r[p];
      ret_total += h_ret_s[p];
      recv_total += h_ret_r[p];
    }
    stats_.returned_rows = ret_total;
    stats_.received_rows = recv_total;
    info(*this, "Total gradient update receive/push = ", push_recv, "/", pushed);
    info(*this, "Total embedding fetching serve/query = ", ret_total, "/", recv_total);

    // exchange 2: versions + rows of the stale keys (all2allReturnValue)
    d_rver_r_.ensure(std::max<size_t>(recv_total, 1) * sizeof(version_t));
    d_rval_r_.ensure(std::max<size_t>(recv_total * W, 1) * sizeof(embed_t));
    {
      size_t so = 0, ro = 0;
      std::vector<XferItem> items;
      for (int p = 0; p < n; p++) {
        const size_t sn = cur.ret_send[p], rn = cur.ret_recv[p];
        items.push_back({p, d_rver_s_.as<int64_t>() + so, sn * 8, d_rver_r_.as<int64_t>() + ro, rn * 8});
        items.push_back({p, d_rval_s_.as<float>() + so * W, sn * W * 4, d_rval_r_.as<float>() + ro * W, rn * W * 4});
        so += sn;
        ro += rn;
      }
      sp = tic(kPhExchange);
      transport_->exchange(items, stream_main_);
      toc(sp);
    }

    // E. requester: refresh cached replicas, expand to batch order (writeBack)
    sp = tic(kPhRefresh);
    HCTR_LAUNCH(hctr_cache_refresh(U, W, d_flag_r_.as<uint8_t>(), d_recv_slot_.as<uint32_t>(),
                                   cur.uniq_row.as<int32_t>(), d_rval_r_.as<float>(), d_rver_r_.as<int64_t>(),
                                   d_gradient_.as<float>(), d_embedding_.as<float>(), d_version_.as<int64_t>(),
                                   stream_main_));
    toc(sp);
    sp = tic(kPhExpand);
    HCTR_LAUNCH(expandRows(cur.batch_size, W, cur.pos_row.as<int32_t>(), cur.idx_map.as<int32_t>(),
                                 d_recv_slot_.as<uint32_t>(), d_rval_r_.as<float>(), d_embedding_.as<float>(), dst_dev,
                                 d_ingest_err_ + 1, stream_main_));
    toc(sp);
    if (*h_err) {
      HCTR_CUDA(cudaStreamSynchronize(stream_main_));
      throw std::runtime_error("push_pull: a peer addressed a key to a rank that does not own it (root_arr differs between ranks?)");
    }
  }

  if (dst_staged)
    HCTR_CUDA(cudaMemcpyAsync(dst, dst_dev, cur.batch_size * W * sizeof(embed_t), cudaMemcpyDeviceToHost, tail));
  // the expand kernel reports a bounded wait that ran out through a mapped pinned word: nothing to copy back
  if (transport_ && !use_p2p_) transport_->waitStream(tail);
  else HCTR_CUDA(cudaStreamSynchronize(tail));
  collectSpans();
  if (h_ingest_err_[1]) {
    h_ingest_err_[1] = 0;
    throw std::runtime_error("push_pull: the row expansion gave up waiting for a bulk copy");
  }
  if (cur.pending && n > 1) {
    finalizeBatch();
    stats_.unique = cur.unique_size;
  }

  uint32_t p2p_err = 0;
  if (p2p_counts_pending_) {
    p2p_counts_pending_ = false;
    const uint32_t *h_cnt = h_pinned_ + HCTR_META_WORDS + n + 1 + 4 * n;
    stats_.queried_keys = stats_.received_push_rows = stats_.received_rows = stats_.pushed_rows = 0;
    for (int p = 0; p < n; p++) {
      cur.query_recv[p] = h_cnt[p];
      prev.push_recv[p] = h_cnt[n + p];
      cur.ret_recv[p] = h_cnt[2 * n + p];
      prev.push_send[p] = p2p_pushed_valid_ ? h_cnt[5 * n + 7 + p] : 0;
      stats_.queried_keys += h_cnt[p];
      stats_.received_push_rows += h_cnt[n + p];
      stats_.received_rows += h_cnt[2 * n + p];
      stats_.pushed_rows += prev.push_send[p];
    }
    stats_.wait_queries_us = h_cnt[HCTR_P2P_WAIT0(n)];
    stats_.wait_returns_us = h_cnt[HCTR_P2P_WAIT1(n)];
    stats_.returned_rows = h_cnt[HCTR_P2P_SERVED(n)];
    p2p_err = h_cnt[6 * n + 7];
    if (p2p_err) HCTR_CUDA(cudaMemsetAsync(d_err_.p, 0, sizeof(uint32_t), stream_main_));
  }
  // The push decision for the batch just pulled runs now, while the caller computes its gradient: everything it
  // reads is final, and the next step's reduction no longer has to wait for it.
  if (n > 1 && p2p_err == 0 && cur.unique_size > 0 && !cur.decided) launchPushDecide(cur);
  if (p2p_err & HCTR_ERR_TIMEOUT)
    throw std::runtime_error("push_pull: a peer's message did not arrive in time (is every rank calling push_pull?)");
  if (p2p_err & HCTR_ERR_NOT_OWNER)
    throw std::runtime_error("push_pull: a peer addressed a key to a rank that does not own it (root_arr differs between ranks?)");
  if (p2p_err & HCTR_ERR_CAPACITY)
    throw std::runtime_error("push_pull: a peer sent more rows than the mailbox holds (ranks must use the same batch size)");
}

// ------------------------------------------------------------------------------------------------
// Steps B-E of pushPull with the device-driven peer-to-peer exchange: no NCCL call and no host
// synchronisation inside the step; every count stays on the device.
// ------------------------------------------------------------------------------------------------
void HetuTable::exchangeP2P(embed_t *dst_dev) {
  BatchDesc &cur = cur_batch_;
  const int n = nrank_;
  const size_t W = kEmbeddingWidth;
  const hctr_p2p_ctx *c = &p2p_->ctx();
  const uint32_t seq = p2p_->nextSeq();
  const size_t cap = p2p_->capacity();
  const size_t slots = (size_t)n * cap;
  const size_t u_max = cur.batch_size;  // U is only known on the device here
  const uint32_t *meta = cur.meta.as<uint32_t>();
  const bool split = p2p_->sameContext();  // thread ranks on one GPU: no kernel may wait for a peer's kernel
  d_ent_row_.ensure((slots + 1) * sizeof(int32_t));
  d_ent_next_.ensure((slots + 1) * sizeof(uint32_t));
  d_flag_r_.ensure(u_max + 16);
  // In split mode every rank drains its stream after publishing and meets the others at a host barrier, so the
  // kernel that consumes finds every sequence number in place and never polls.
  auto meet = [&] {
    if (!split) return;
    HCTR_CUDA(cudaStreamSynchronize(stream_main_));
    p2p_->hostBarrier();
  };

  // B. queries straight into the owners' mailboxes; the last thread block publishes counts + sequence number
  int sp = tic(kPhQuery);
  HCTR_LAUNCH(hctr_p2p_query_send(c, meta, u_max, cur.uniq.as<int64_t>(), cur.uniq_owner.as<uint8_t>(),
                                  cur.uniq_row.as<int32_t>(), d_version_.as<int64_t>(), seq,
                                  prev_push_valid_ && prev_batch_.unique_size > 0 ? d_push_count_.as<uint32_t>()
                                                                                   : nullptr,
                                  stream_main_));
  toc(sp);
  meet();

  // C. owner applies the pushed rows of each source in rank order
  const hctr_p2p_box mine = p2p_->mine();
  sp = tic(kPhOwnerUpdate);
  if (n <= 32) {
    // pass A waits for the peers' counts, then marks sources, chains the entries of every row and finishes the
    // versions; pass B adds the rows
    HCTR_LAUNCH(hctr_p2p_owner_mark(c, &mine, seq, d_row_of_.as<int32_t>(), kEmbeddingIDMax, kNonLocalStorageMax,
                                    d_row_mask_.as<unsigned long long>(), d_row_head_.as<unsigned long long>(),
                                    nextEpoch(), d_ent_row_.as<int32_t>(), d_ent_next_.as<uint32_t>(),
                                    d_version_.as<int64_t>(), stream_main_));
    toc(sp);
    sp = tic(kPhOwnerApply);
    HCTR_LAUNCH(hctr_p2p_owner_apply(c, &mine, kNonLocalStorageMax, d_ent_row_.as<int32_t>(),
                                     d_row_mask_.as<unsigned long long>(), d_row_head_.as<unsigned long long>(),
                                     d_ent_next_.as<uint32_t>(), d_embedding_.as<float>(), stream_main_));
    toc(sp);
  } else {
    // more sources than a mask word holds: one cooperative launch with a grid-wide barrier between sources
    HCTR_LAUNCH(hctr_p2p_wait(c, 0, seq, stream_main_));
    HCTR_LAUNCH(hctr_p2p_owner_update(c, d_row_of_.as<int32_t>(), kEmbeddingIDMax, kNonLocalStorageMax,
                                      d_embedding_.as<float>(), d_version_.as<int64_t>(), stream_main_));
    toc(sp);
  }

  // D. staleness test and rows of the stale keys, straight into the requesters' mailboxes (one launch, no scan:
  // the row for a requester's j-th query goes to row j of this rank's sub-region in its mailbox)
  sp = tic(kPhStaleGather);
  HCTR_LAUNCH(hctr_p2p_stale_gather(c, seq, d_row_of_.as<int32_t>(), kEmbeddingIDMax, kNonLocalStorageMax,
                                    d_embedding_.as<float>(), d_version_.as<int64_t>(), pull_bound_, stream_main_));
  toc(sp);
  meet();

  // E. requester: wait for the owners, cache refresh and row expansion in one launch; or (HCTR_P2P_FUSED_EXPAND=0,
  // HCTR_EXPAND=bulk) in two: row index + flag of every unique key and cache refresh, then the expansion
  if (fused_refresh_expand_ && !expand_bulk_) {
    sp = tic(kPhExpand);
    HCTR_LAUNCH(hctr_p2p_refresh_expand(c, seq, meta, cur.uniq_owner.as<uint8_t>(), cur.uniq_row.as<int32_t>(),
                                        kNonLocalStorageMax, d_gradient_.as<float>(), d_embedding_.as<float>(),
                                        d_version_.as<int64_t>(), cur.batch_size, cur.pos_row.as<int32_t>(),
                                        cur.idx_map.as<int32_t>(), dst_dev, stream_main_));
    toc(sp);
  } else {
    sp = tic(kPhRefresh);
    HCTR_LAUNCH(hctr_p2p_refresh_index(c, seq, meta, u_max, cur.uniq_owner.as<uint8_t>(), cur.uniq_row.as<int32_t>(),
                                       kNonLocalStorageMax, d_gradient_.as<float>(), d_embedding_.as<float>(),
                                       d_version_.as<int64_t>(), d_flag_r_.as<uint8_t>(), d_recv_idx_.as<uint32_t>(),
                                       stream_main_));
    toc(sp);
    sp = tic(kPhExpand);
    HCTR_LAUNCH(expandRows(cur.batch_size, W, cur.pos_row.as<int32_t>(), cur.idx_map.as<int32_t>(),
                           d_recv_idx_.as<uint32_t>(), mine.rval, d_embedding_.as<float>(), dst_dev,
                           d_ingest_err_ + 1, stream_main_));
    toc(sp);
  }

  // counts, wait times and the error word come back with the step's final synchronisation
  uint32_t *h_cnt = h_pinned_ + HCTR_META_WORDS + n + 1 + 4 * n;  // [5n+7] + [n] push counts + error word
  HCTR_CUDA(cudaMemcpyAsync(h_cnt, c->cnt_in, (5 * n + 7) * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
  HCTR_CUDA(cudaMemcpyAsync(h_cnt + 5 * n + 7, d_push_count_.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
  HCTR_CUDA(cudaMemcpyAsync(h_cnt + 6 * n + 7, d_err_.p, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_main_));
  p2p_counts_pending_ = true;
  p2p_pushed_valid_ = prev_push_valid_ && prev_batch_.unique_size > 0;
}

// ------------------------------------------------------------------------------------------------
// Profiling spans
// ------------------------------------------------------------------------------------------------
void HetuTable::setProfile(int every) {
  if (every < 0) every = 0;
  if (every > 0 && profile_every_ == 0) {
    HCTR_CUDA(cudaSetDevice(device_id_));
    if (!ev_epoch_) HCTR_CUDA(cudaEventCreate(&ev_epoch_));
    HCTR_CUDA(cudaEventRecord(ev_epoch_, stream_main_));
    timeline_.assign(3 * kTimelineSpans, 0.0);
    timeline_next_ = timeline_count_ = 0;
  }
  profile_every_ = every;
  profile_step_ = 0;
  profile_ = every > 0;
}

size_t HetuTable::timeline(double *out, size_t max_spans) {
  if (spans_used_) {
    quiesce();
    resolveSpans();
  }
  const size_t n = std::min(max_spans, timeline_count_);
  for (size_t i = 0; i < n; i++) {
    const size_t slot = (timeline_next_ + kTimelineSpans - n + i) % kTimelineSpans;
    for (int j = 0; j < 3; j++) out[3 * i + j] = timeline_[3 * slot + j];
  }
  return n;
}

int HetuTable::tic(int phase, cudaStream_t st) {
  if (!profile_) return -1;
  if (!st) st = stream_main_;
  if (spans_used_ == spans_.size()) {
    Span s{phase, nullptr, nullptr};
    HCTR_CUDA(cudaEventCreate(&s.a));
    HCTR_CUDA(cudaEventCreate(&s.b));
    spans_.push_back(s);
  }
  Span &s = spans_[spans_used_];
  s.phase = phase;
  HCTR_CUDA(cudaEventRecord(s.a, st));
  return (int)spans_used_++;
}

void HetuTable::toc(int span, cudaStream_t st) {
  if (span < 0) return;
  HCTR_CUDA(cudaEventRecord(spans_[span].b, st ? st : stream_main_));
}

// Called at the synchronisation points of a step.  Reading the event times costs several microseconds of
// host time per span, so the spans of many steps are left to pile up and are only read when somebody
// asks for the result (phaseTimes / timeline) or when the pile is large.
void HetuTable::collectSpans() {
  if (spans_used_ >= kMaxDeferredSpans) resolveSpans();
}

// Every recorded span must have completed: call after the streams have drained.
void HetuTable::resolveSpans() {
  for (size_t i = 0; i < spans_used_; i++) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, spans_[i].a, spans_[i].b) == cudaSuccess) {
      phase_ms_[spans_[i].phase] += ms;
      phase_calls_[spans_[i].phase]++;
      float t0 = 0.f;
      if (ev_epoch_ && cudaEventElapsedTime(&t0, ev_epoch_, spans_[i].a) == cudaSuccess) {
        double *slot = &timeline_[3 * timeline_next_];
        slot[0] = spans_[i].phase, slot[1] = t0, slot[2] = t0 + ms;
        timeline_next_ = (timeline_next_ + 1) % kTimelineSpans;
        if (timeline_count_ < kTimelineSpans) timeline_count_++;
      } else {
        cudaGetLastError();
      }
    } else {
      cudaGetLastError();
    }
  }
  spans_used_ = 0;
}

void HetuTable::phaseTimes(double ms[kPhCount], long long calls[kPhCount], bool reset) {
  if (spans_used_) {
    quiesce();
    resolveSpans();
  }
  for (int i = 0; i < kPhCount; i++) {
    ms[i] = phase_ms_[i];
    calls[i] = phase_calls_[i];
    if (reset) phase_ms_[i] = 0, phase_calls_[i] = 0;
  }
}

// ------------------------------------------------------------------------------------------------
// Introspection
// ------------------------------------------------------------------------------------------------
namespace {
template <class T>
long long copy_widen(const void *dev, size_t n, void *out, cudaStream_t s) {
  if (!out) return (long long)n;
  std::vector<T> tmp(n);
  if (n) {
    HCTR_CUDA(cudaMemcpyAsync(tmp.data(), dev, n * sizeof(T), cudaMemcpyDeviceToHost, s));
    HCTR_CUDA(cudaStreamSynchronize(s));
  }
  long long *o = static_cast<long long *>(out);
  for (size_t i = 0; i < n; i++) o[i] = (long long)tmp[i];
  return (long long)n;
}
long long copy_sizes(const std::vector<size_t> &v, size_t n, void *out) {
  if (out)
    for (size_t i = 0; i < n; i++) static_cast<long long *>(out)[i] = (long long)v[i];
  return (long long)n;
}
}  // namespace

long long HetuTable::dump(const std::string &what, bool prev, void *out) {
  quiesce();  // also enqueues and completes a deferred run ordering
  BatchDesc &b = prev ? prev_batch_ : cur_batch_;
  const size_t B = b.batch_size, U = b.unique_size;
  cudaStream_t s = stream_main_;
  if (what == "unique_idx") return copy_widen<long long>(b.uniq.p, U, out, s);
  if (what == "idx_map") return copy_widen<int32_t>(b.idx_map.p, B, out, s);
  if (what == "sorted_arg") return copy_widen<uint32_t>(b.sorted_pos.p, B, out, s);
  if (what == "run_length") return copy_widen<uint32_t>(b.run_start.p, B ? U + 1 : 1, out, s);
  if (what == "root") return copy_widen<uint8_t>(b.uniq_owner.p, U, out, s);
  if (what == "offset") return copy_widen<int32_t>(b.uniq_row.p, U, out, s);
  if (what == "shape") return copy_sizes(b.query_send, nrank_, out);
  if (what == "shape_exchanged") {
    if (use_p2p_ && !prev) {
      // The device-driven exchange never brings the peers' counts to the host before push_pull, so this
      // view is assembled on demand with a host all-gather: COLLECTIVE in that mode (every rank must ask).
      std::vector<unsigned long long> mine(nrank_), all((size_t)nrank_ * nrank_);
      for (int p = 0; p < nrank_; p++) mine[p] = b.query_send[p];
      transport_->allgatherHost(mine.data(), all.data(), nrank_ * sizeof(unsigned long long));
      for (int p = 0; p < nrank_; p++) b.query_recv[p] = (size_t)all[(size_t)p * nrank_ + rank_];
    }
    return copy_sizes(b.query_recv, nrank_, out);
  }
  if (what == "push_shape") return copy_sizes(b.push_send, nrank_, out);
  if (what == "push_shape_exchanged") return copy_sizes(b.push_recv, nrank_, out);
  if (what == "return_shape") return copy_sizes(b.ret_send, nrank_, out);
  if (what == "return_shape_exchanged") return copy_sizes(b.ret_recv, nrank_, out);
  if (what == "need_update") return copy_widen<uint32_t>(prev_batch_.need_push.p, nrank_ > 1 ? prev_batch_.unique_size : 0, out, s);
  if (what == "version") return copy_widen<long long>(d_version_.p, kStorageMax, out, s);
  if (what == "updates") return copy_widen<long long>(d_updates_.p, kNonLocalStorageMax, out, s);
  if (what == "stored_keys") return copy_widen<long long>(d_stored_keys_.p, kStorageMax, out, s);
  if (what == "embedding" || what == "gradient") {
    const size_t n = (what == "embedding" ? kStorageMax : kNonLocalStorageMax) * kEmbeddingWidth;
    if (out && n) {
      HCTR_CUDA(cudaMemcpyAsync(out, what == "embedding" ? d_embedding_.p : d_gradient_.p, n * sizeof(embed_t),
                                cudaMemcpyDeviceToHost, s));
      HCTR_CUDA(cudaStreamSynchronize(s));
    }
    return (long long)n;
  }
  throw std::runtime_error("dump: unknown array " + what);
}

void HetuTable::setEmbedding(const embed_t *host_rows) {
  HCTR_CUDA(cudaSetDevice(device_id_));
  HCTR_CUDA(cudaMemcpyAsync(d_embedding_.p, host_rows, kStorageMax * kEmbeddingWidth * sizeof(embed_t),
                            cudaMemcpyHostToDevice, stream_main_));
  HCTR_CUDA(cudaStreamSynchronize(stream_main_));
}

// csrc/core/debug.cu:5-24 — same text formats
std::string HetuTable::debugString() {
  char buffer[1024];
  std::snprintf(buffer, sizeof(buffer), "<HetuTable root/store/all=%ld/%ld/%ld>",
                (long)(kStorageMax - kNonLocalStorageMax), (long)kStorageMax, (long)kEmbeddingIDMax);
  return buffer;
}

std::string HetuTable::debugStringFull() {
  char buffer[1024];
  std::snprintf(buffer, sizeof(buffer),
                "<HetuTable root/store/all=%ld/%ld/%ld rank=%d nrank=%d device_id=%d width=%ld push/pull=%lld/%lld>",
                (long)(kStorageMax - kNonLocalStorageMax), (long)kStorageMax, (long)kEmbeddingIDMax, rank_, nrank_,
                device_id_, (long)kEmbeddingWidth, push_bound_, pull_bound_);
  return buffer;
}

HetuTable::~HetuTable() { releaseAll(); }

void HetuTable::releaseAll() {
  cudaSetDevice(device_id_);
  if (stream_side_) cudaStreamSynchronize(stream_side_);
  if (stream_reduce_side_) cudaStreamSynchronize(stream_reduce_side_);
  if (stream_reduce_) cudaStreamSynchronize(stream_reduce_);
  if (stream_main_) cudaStreamSynchronize(stream_main_);
  p2p_.reset();
  transport_.reset();
  DevBuf *all[] = {&d_embedding_, &d_gradient_, &d_updates_, &d_version_, &d_root_, &d_row_of_, &d_stored_keys_,
                   &d_bits_, &d_blk_cnt_, &d_blk_flag_, &d_chain_, &d_chain3_, &d_ent_row_, &d_ent_next_, &d_row_mask_, &d_row_head_, &d_src_off_, &d_src_cnt_, &d_word_base_, &d_scan_, &d_sk_, &d_cnt_,
                   &d_push_count_, &d_push_base_, &d_recv_idx_, &d_err_, &d_cnt_s_, &d_cnt_r_, &d_qver_s_,
                   &d_qkey_r_, &d_qver_r_, &d_pkey_s_, &d_pupd_s_, &d_pval_s_, &d_pkey_r_, &d_pupd_r_, &d_pval_r_,
                   &d_flag_s_, &d_flag_r_, &d_flag32_, &d_ret_slot_, &d_recv_slot_, &d_seg_r_, &d_retcnt_s_,
                   &d_retcnt_r_, &d_rver_s_, &d_rval_s_, &d_rver_r_, &d_rval_r_, &d_stage_grad_, &d_stage_dst_};
  for (DevBuf *b : all) b->release();
  for (BatchDesc *b : {&cur_batch_, &prev_batch_}) {
    if (b->ev_order) cudaEventDestroy(b->ev_order);
    b->ev_order = nullptr;
    if (b->ev_scatter) cudaEventDestroy(b->ev_scatter);
    b->ev_scatter = nullptr;
    if (b->h_meta) cudaFreeHost(b->h_meta);
    b->h_meta = nullptr;
  }
  if (h_ingest_err_) cudaFreeHost(h_ingest_err_);
  h_ingest_err_ = d_ingest_err_ = nullptr;
  for (BatchDesc *b : {&cur_batch_, &prev_batch_})
    for (DevBuf *d : {&b->keys, &b->idx_map, &b->sorted_pos, &b->uniq, &b->uniq_owner, &b->uniq_row,
                      &b->run_start, &b->meta, &b->pos_row, &b->heavy, &b->need_push, &b->push_slot, &b->rank})
      d->release();
  for (Span &sp : spans_) {
    cudaEventDestroy(sp.a);
    cudaEventDestroy(sp.b);
  }
  spans_.clear();
  if (h_pinned_) cudaFreeHost(h_pinned_);
  h_pinned_ = nullptr;
  if (h_src_) cudaFreeHost(h_src_);
  h_src_ = nullptr;
  if (ev_epoch_) cudaEventDestroy(ev_epoch_);
  ev_epoch_ = nullptr;
  if (ev_fork_) cudaEventDestroy(ev_fork_);
  if (ev_join_) cudaEventDestroy(ev_join_);
  if (ev_keys_) cudaEventDestroy(ev_keys_);
  if (ev_early_) cudaEventDestroy(ev_early_);
  ev_early_ = nullptr;
  if (ev_decide_) cudaEventDestroy(ev_decide_);
  if (ev_reduce_) cudaEventDestroy(ev_reduce_);
  if (ev_rfork_) cudaEventDestroy(ev_rfork_);
  if (ev_rjoin_) cudaEventDestroy(ev_rjoin_);
  ev_decide_ = ev_reduce_ = ev_rfork_ = ev_rjoin_ = nullptr;
  if (stream_reduce_side_) cudaStreamDestroy(stream_reduce_side_);
  stream_reduce_side_ = nullptr;
  if (stream_reduce_) cudaStreamDestroy(stream_reduce_);
  stream_reduce_ = nullptr;
  ev_fork_ = ev_join_ = ev_keys_ = nullptr;
  if (stream_side_) cudaStreamDestroy(stream_side_);
  stream_side_ = nullptr;
  if (stream_main_) cudaStreamDestroy(stream_main_);
  stream_main_ = nullptr;
}

}  // namespace hetuCTR
