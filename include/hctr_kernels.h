/*
 * hctr_kernels.h — C-ABI launchers for the sm_100a kernels of the HetuTable hot path.
 *
 * Every function takes raw DEVICE pointers, sizes and a CUDA stream (passed as void*, it is a
 * cudaStream_t), enqueues its kernels on that stream and returns 0 or a cudaError_t value.  Nothing
 * here allocates, synchronises or touches host memory unless stated.  The host class (HetuTable)
 * calls the GPU only through these entry points.
 *
 * Citations name the reference code each launcher replaces (paths inside the reference project).
 *
 * Conventions
 *   key / version types : int64   (csrc/core/types.h:16,19)
 *   owner               : uint8   (csrc/core/types.h:28)
 *   values              : float   (csrc/core/types.h:12)
 *   local row ids, batch positions, unique indices, counts : 32-bit on the device
 *   HCTR_INVALID_ROW (-1)  = key not stored here    (kInvalidIndex,   csrc/core/types.h:22)
 *   HCTR_INVALID_VERSION   = INT64_MIN              (kInvalidVersion, csrc/core/types.h:25)
 */
#ifndef HCTR_KERNELS_H_
#define HCTR_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HCTR_INVALID_ROW (-1)
#define HCTR_INVALID_VERSION INT64_MIN

/* bits of the device error word */
#define HCTR_ERR_KEY_RANGE 1u    /* a batch key is <0, >= length, or its owner id is >= nrank          */
#define HCTR_ERR_NOT_OWNER 2u    /* an owner-side kernel met a key this rank does not store as owned   */
#define HCTR_ERR_CAPACITY 4u     /* an internal list overflowed its reserved capacity                  */
#define HCTR_ERR_TIMEOUT 8u      /* a peer's message did not arrive within the wait limit              */

/* Keys of the dedupe bitmap are sort keys  sk = key + length_pad * owner  with length_pad = length
 * rounded up to HCTR_BLOCK_KEYS, so every owner's range starts on a bitmap-block boundary. */
#define HCTR_WORD_BITS 64
#define HCTR_BLOCK_WORDS 64
#define HCTR_BLOCK_KEYS 4096
#define HCTR_SCAN_TILE 4096
#define HCTR_LIGHT_RUN 32 /* runs up to this many positions are "short" */

/* Kernels this library has enqueued since it was loaded (all launchers, all streams). */
unsigned long long hctr_launch_count(void);

/* Number of 32-bit scratch words hctr_scan_exclusive_u32 needs for n_max inputs. */
size_t hctr_scan_scratch_words(size_t n_max);

/* Exclusive prefix sum of 32-bit counts: out[i] = sum(in[0..i)), for i in [0, n]; out has n+1 entries.
 * n = *n_dev when n_dev is non-null (a count that only exists on the device), else n_max; grids are
 * sized from n_max.  `scratch` holds hctr_scan_scratch_words(n_max) words.  in == out is allowed.
 * Replaces cub::DeviceScan::ExclusiveSum at csrc/core/preprocess.cu:124-125,173-174,
 * csrc/core/handle_query.cu:56-57 and csrc/core/writeback.cu:45-46. */
int hctr_scan_exclusive_u32(const uint32_t *in, uint32_t *out, size_t n_max, const uint32_t *n_dev,
                            uint32_t *scratch, void *stream);

/* Same result in ONE launch: tile-local scans chained through per-tile totals that later tiles pick up
 * with bounded acquire-polls (HCTR_ERR_TIMEOUT in *err if a tile never publishes).  `scratch` holds
 * hctr_scan_chained_scratch_words(n_max) words, 8-byte aligned, and needs no initialisation provided
 * `epoch` is non-zero and differs from the epoch of the previous launch that used the same scratch. */
size_t hctr_scan_chained_scratch_words(size_t n_max);
int hctr_scan_exclusive_u32_chained(const uint32_t *in, uint32_t *out, size_t n_max, const uint32_t *n_dev,
                                    uint32_t *scratch, uint32_t epoch, uint32_t *err, void *stream);

/* Exclusive prefix sum for callers that cannot allocate device memory.  (No counterpart in the
 * reference: it sizes and allocates cub temp storage itself, csrc/core/table_initialize.cu:166-177.)
 *
 * Same result as hctr_scan_exclusive_u32 for n <= HCTR_NOALLOC_SCAN_MAX elements (out has n+1 entries,
 * in == out allowed), but the scratch is a fixed array inside the library, so the call performs no
 * cudaMalloc/cudaFree.  It is meant for callers such as allocator callbacks of a host framework,
 * latency-critical loops that must stay clear of the driver's allocation lock, or plugins that only
 * receive input and output buffers.
 *  - Larger n is refused: returns cudaErrorInvalidValue and hctr_noalloc_last_error() says why.
 *  - The first call on each device looks up the array's device address (with that device current); make
 *    that first call before any stream capture starts.
 *  - All calls on one device share the one array: calls that may overlap on the GPU (different streams
 *    without ordering between them) race on it.  Nothing in it needs clearing between calls.
 *  - Every GPU that loads the library holds the array (64 KB) until the process exits. */
#define HCTR_NOALLOC_SCAN_MAX (1u << 26)
int hctr_scan_exclusive_u32_noalloc(const uint32_t *in, uint32_t *out, size_t n, void *stream);
const char *hctr_noalloc_last_error(void);

/* ---------------------------------------------------------------------------------------------
 * Table build (set-up side of the path).
 * ------------------------------------------------------------------------------------------- */

/* row_of[key] = local row of every stored key, HCTR_INVALID_ROW elsewhere; version[row] = INT64_MIN for
 * cached rows (row < n_cached), 0 for owned rows.  `stored_keys` is the storage list already put in
 * layout order (cached rows first, each group in caller order).  Sets HCTR_ERR_KEY_RANGE for a key outside
 * [0,length) and HCTR_ERR_CAPACITY for a key listed twice.
 * Replaces the hash-map build and version fill of csrc/core/table_initialize.cu:84-87,108-112. */
int hctr_table_build(const int64_t *stored_keys, size_t n_stored, size_t n_cached, size_t length,
                     int32_t *row_of, int64_t *version, uint32_t *err, void *stream);

/* Stable partition flags for the storage list: is_cached[i] = owner_of[storage[i]] != rank, and
 * dst[i] = final local row (cached keys first, both groups in input order), given the exclusive scan
 * `cached_before` of is_cached (n_stored+1 entries).  Replaces thrust::stable_partition at
 * csrc/core/table_initialize.cu:76-81. */
int hctr_storage_flags(const int64_t *storage, size_t n_stored, size_t length, const uint8_t *owner_of,
                       int rank, uint32_t *is_cached, uint32_t *err, void *stream);
int hctr_storage_layout(const int64_t *storage, size_t n_stored, const uint32_t *is_cached,
                        const uint32_t *cached_before, int64_t *stored_keys, void *stream);

/* Counts keys with owner_of[key]==rank (into *n_owned, a device word that must be zero on entry).
 * Used to check that a rank stores every row it owns. */
int hctr_count_owned(const uint8_t *owner_of, size_t length, int rank, unsigned long long *n_owned,
                     void *stream);

/* Fill `data[0..len)`: kind 0 = zeros, 1 = normal(a=mean,b=stddev), 2 = uniform[a,b),
 * 3 = normal truncated to mean +- 2 stddev.  Element i is drawn from a minstd engine seeded with `seed` and
 * advanced i steps, so values depend on the local element index only.
 * Replaces csrc/utils/initializer.cu:11-103. */
int hctr_initialize(float *data, size_t len, int kind, float a, float b, unsigned int seed, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Preprocess: dedupe + key -> (owner, local row) + batch -> unique map.
 * Replaces preprocessIndex, csrc/core/preprocess.cu:11-141 (radix sort, run-length encode, scans,
 * hash probes, binary searches) with bitmap ranking over the dense (owner, key) space.
 * ------------------------------------------------------------------------------------------- */

typedef struct hctr_dedupe_args {
  /* inputs */
  const int64_t *keys;      /* [B] batch keys (device) */
  size_t batch;             /* B */
  size_t length;            /* table length N */
  size_t length_pad;        /* N rounded up to HCTR_BLOCK_KEYS */
  int nrank;
  const uint8_t *owner_of;  /* [N] */
  const int32_t *row_of;    /* [N] */
  /* persistent scratch, all-zero between calls */
  unsigned long long *bits; /* [nrank*length_pad/64] */
  uint8_t *blk_flag;        /* [nrank*length_pad/4096] block touched by this batch */
  uint32_t *cnt;            /* [B+1] occurrences per unique key (consumed by the run-start scan) */
  /* epoch-tagged scratch: zero-initialised ONCE, never cleared afterwards */
  uint32_t *chain_scratch;  /* [2 * (nblocks / 8 + 2)] words, 8-byte aligned: CTA totals of the block-rank kernel */
  uint32_t *scan_scratch;   /* hctr_scan_chained_scratch_words(B + 1) words, 8-byte aligned */
  uint32_t epoch;           /* non-zero, different from every earlier call's on the same scratch */
  /* scratch that needs no initial value */
  uint32_t *word_base;      /* [nrank*length_pad/64] */
  unsigned long long *sk;   /* [B] sort keys */
  uint32_t *rank_in_run;    /* [B] (also staging of the long-run ordering kernel) */
  /* outputs */
  int64_t *uniq;            /* [B] unique keys, owner-major, key ascending */
  uint8_t *uniq_owner;      /* [B] */
  int32_t *uniq_row;        /* [B] local row or HCTR_INVALID_ROW */
  uint32_t *run_start;      /* [B+1] first slot of each unique key's run in sorted_pos; entry U = batch */
  uint32_t *sorted_pos;     /* [B] batch positions grouped by unique, ascending inside a group */
  int32_t *idx_map;         /* [B] batch position -> unique index */
  int32_t *pos_row;         /* [B] batch position -> local row or HCTR_INVALID_ROW; null = not wanted (see hctr_ingest_keys_rows) */
  uint32_t *heavy_list;     /* [B/32 + 2] unique indices whose run is longer than HCTR_LIGHT_RUN */
  uint32_t *meta;           /* [HCTR_META_WORDS + nrank + 1]: see HCTR_META_* */
  /* optional: a second stream (cudaStream_t) and two events (cudaEvent_t).  When given, the two
   * run-ordering kernels (the only consumers/producers of the final order inside sorted_pos) run on
   * side_stream after the rest of the pipeline, and join_event is recorded there when they are done:
   * the call's stream does NOT wait for them, whoever reads sorted_pos must wait on join_event.
   * side_stream and fork_event given but join_event null: the ordering kernels are NOT enqueued; fork_event
   * is recorded when their inputs are ready and the caller enqueues them later with hctr_dedupe_order.
   * All null = everything on the call's stream */
  void *side_stream;
  void *fork_event;
  void *join_event;
  /* optional: the number of fields of a sample-major batch (position = sample * stride + field).  With a
   * stride > 1 a warp works on one field of 32 consecutive samples, which turns the scattered accesses of
   * small-vocabulary fields into shared cache lines and merged atomics.  0 or 1 = positions in order.  The
   * outputs do not depend on it.  hctr_detect_key_stride finds it from a batch. */
  uint32_t stride;
} hctr_dedupe_args;

#define HCTR_META_UNIQUE 0   /* number of unique keys U                         */
#define HCTR_META_ERR 1      /* error word (HCTR_ERR_*)                         */
#define HCTR_META_NHEAVY 2   /* number of runs longer than HCTR_LIGHT_RUN       */
#define HCTR_META_SEG 4      /* seg_start[0..nrank]: first unique of each owner */
#define HCTR_META_WORDS 4

/* Enqueues the whole dedupe pipeline.  On completion meta[HCTR_META_UNIQUE] = U, meta[HCTR_META_SEG+p]
 * = index of the first unique key owned by p (entry nrank = U), and the bitmap scratch is all-zero
 * again.  Keys out of range set HCTR_ERR_KEY_RANGE in meta[HCTR_META_ERR] and get idx_map = -1. */
int hctr_dedupe_map(const hctr_dedupe_args *a, void *stream);

/* Finds the field count of a sample-major batch: scores[d] (d = 1..64, 65 words, scores[0] unused) = number of
 * positions i among the first 32768 with keys[i] == keys[i + d].  Keys of different fields never coincide and hot
 * keys of one field repeat from sample to sample, so the smallest d with a large score is the field count. */
int hctr_detect_key_stride(const int64_t *keys, size_t n, uint32_t *scores, void *stream);

/* Front of the pipeline for keys that already live in device memory: dst[0..n) = src[0..n) (the table's private
 * copy, so that the caller may reuse its buffer) and meta[0..meta_words) = 0, in one launch. */
int hctr_ingest_keys(const int64_t *src, int64_t *dst, size_t n, uint32_t *meta, unsigned meta_words, void *stream);
/* hctr_ingest_keys plus pos_row[i] = row_of[keys[i]] (HCTR_INVALID_ROW for a key that is not stored here or lies
 * outside [0, length); the latter also sets HCTR_ERR_KEY_RANGE in *err).  With pos_row known this early the row
 * expansion of a batch whose keys are all stored locally does not depend on the dedupe pipeline at all.  src may
 * equal dst.  Part of what cvt_embedding_idx_2_offset did, csrc/core/preprocess.cu:62-76. */
int hctr_ingest_keys_rows(const int64_t *src, int64_t *dst, size_t n, uint32_t *meta, unsigned meta_words,
                          const int32_t *row_of, size_t length, int32_t *pos_row, uint32_t *err, void *stream);

/* The run-ordering half of the pipeline alone (positions of every unique key's run in ascending batch order
 * inside sorted_pos), for callers that deferred it: same args as the hctr_dedupe_map call it completes, on a
 * stream that has waited for that call's fork_event.  Nothing but the next gradient reduction (and a reader
 * of sorted_pos) needs it. */
int hctr_dedupe_order(const hctr_dedupe_args *a, void *stream);
/* The two halves of hctr_dedupe_order: runs of 2..HCTR_LIGHT_RUN positions (one warp per run) and longer runs
 * (a thread block per run).  The short-run half is not needed when the consumer orders short runs itself, see
 * hctr_reduce_orders_short_runs. */
int hctr_dedupe_order_light(const hctr_dedupe_args *a, void *stream);
int hctr_dedupe_order_heavy(const hctr_dedupe_args *a, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Gradient push decision (previous batch).  Replaces decide_update_kernel + scan,
 * csrc/core/preprocess.cu:148-182.
 * ------------------------------------------------------------------------------------------- */

/* need_push[u] = 0 if owner==rank; 1 if not stored; else pending_cnt[row] + occurrences(u) > push_bound,
 * with occurrences(u) = run_start[u+1] - run_start[u].
 * Then push_slot = exclusive scan of need_push (U+1 entries) and push_count[p] = pushes to owner p.
 * U is read from meta (device). */
/* push_base[p] (optional output, device [nrank]) = push_slot at the first unique key of owner p. */
int hctr_push_decide(const uint32_t *meta, int nrank, int rank, size_t u_max, const uint8_t *uniq_owner,
                     const int32_t *uniq_row, const uint32_t *run_start, const int64_t *pending_cnt,
                     int64_t push_bound, uint32_t *need_push, uint32_t *push_slot,
                     uint32_t *scan_scratch, uint32_t *push_count, uint32_t *push_base, void *stream);

/* Packs the per-peer counts a rank announces after preprocess: out[2p] = unique keys of the current
 * batch owned by p (from meta's segment starts), out[2p+1] = push_count[p] (0 when push_count is null).
 * Feeds the count exchange that replaces all2allExchangeShape, csrc/core/all2all.cu:6-16. */
int hctr_pack_counts(const uint32_t *meta, const uint32_t *push_count, int nrank, uint32_t *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Gradient aggregation + local SGD apply + pack of pushed rows (previous batch).
 * Replaces gradient_index_kernel and gradient_reduction_kernel, csrc/core/generate_query.cu:8-89.
 * ------------------------------------------------------------------------------------------- */

/* Same result in two launches instead of four (decision, scan and slot assignment fused; tile totals
 * chained with bounded waits, HCTR_ERR_TIMEOUT in *err).  chain_scratch: hctr_scan_chained_scratch_words(u_max)
 * words, 8-byte aligned, zero-initialised once; epoch: non-zero, different from the previous call's. */
int hctr_push_decide_fused(const uint32_t *meta, int nrank, int rank, size_t u_max, const uint8_t *uniq_owner,
                           const int32_t *uniq_row, const uint32_t *run_start, const int64_t *pending_cnt,
                           int64_t push_bound, uint32_t *need_push, uint32_t *push_slot, uint32_t *chain_scratch,
                           uint32_t epoch, uint32_t *push_count, uint32_t *push_base, uint32_t *err, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Peer-to-peer exchange (one process per GPU, all GPUs of one NVLink domain).
 *
 * Every rank owns a MAILBOX in its own device memory, mapped into every peer through CUDA IPC.  Each
 * region of a mailbox holds nrank sub-regions of `cap` rows; sub-region s is written only by source
 * rank s (plain peer stores from that rank's kernels) and read only by the owner of the mailbox.
 * A 64-byte header per source carries the counts and a sequence number written last with release
 * semantics; the receiver's wait kernel polls its own memory with acquire loads, for at most
 * `timeout_ns`, and reports HCTR_ERR_TIMEOUT instead of hanging.  This replaces the grouped
 * ncclSend/ncclRecv rounds of csrc/core/all2all.cu:6-130 and the host synchronisations between them
 * (csrc/core/hetu_gpu_table.cu:33,64): counts never leave the device.
 * ------------------------------------------------------------------------------------------- */
typedef struct hctr_p2p_box { /* one rank's mailbox as mapped into the calling GPU's address space */
  uint32_t *hdr;  /* [nrank][16] words: 0 query seq, 1 query count, 2 push count, 8 return seq, 9 return count */
  int64_t *qkey;  /* [nrank*cap]   queried keys                      (requester -> owner) */
  int64_t *qver;  /* [nrank*cap]   requester's version of each key                        */
  int64_t *pkey;  /* [nrank*cap]   ids of pushed rows                (requester -> owner) */
  int64_t *pupd;  /* [nrank*cap]   update counts of pushed rows                           */
  float *pval;    /* [nrank*cap*W] pushed rows                                            */
  uint8_t *flag;  /* [nrank*cap]   stale flag per queried key        (owner -> requester) */
  int64_t *rver;  /* [nrank*cap]   versions of returned rows                              */
  float *rval;    /* [nrank*cap*W] returned rows                                          */
} hctr_p2p_box;

typedef struct hctr_p2p_ctx {
  int nrank, rank;
  uint32_t cap;             /* rows per (mailbox, source) sub-region */
  size_t width;
  const hctr_p2p_box *box;  /* device array [nrank]; box[rank] is this rank's own mailbox */
  uint32_t *cnt_in;         /* device [HCTR_P2P_CNT_WORDS(nrank)], zero-initialised once: query, push and return counts
                               received from each peer ([0,n), [n,2n), [2n,3n)), the exclusive prefixes of the query
                               counts ([3n,4n]) and of the push counts ([4n+1,5n+1]; word 2n is reused as the number
                               of keys the owners flagged for this rank), the longest wait of the last step
                               for a peer's queries and for a peer's returned rows in microseconds (5n+2, 5n+3), and
                               two arrival counters of the publishing kernels */
  uint32_t *err;            /* device error word */
  unsigned long long timeout_ns;
} hctr_p2p_ctx;
#define HCTR_P2P_CNT_WORDS(n) (5 * (size_t)(n) + 8)
#define HCTR_P2P_WAIT0(n) (5 * (n) + 2)   /* index in cnt_in: longest wait for a peer's queries, microseconds */
#define HCTR_P2P_WAIT1(n) (5 * (n) + 3)   /* longest wait for a peer's returned rows */
#define HCTR_P2P_TICKET0(n) (5 * (n) + 4) /* arrival counters of the two publishing kernels */
#define HCTR_P2P_TICKET1(n) (5 * (n) + 5)
#define HCTR_P2P_SERVED(n) (5 * (n) + 6)  /* rows this rank returned to its peers in the last step */

/* Requester: (key, local version) of every unique key, written into its owner's mailbox; the thread block that
 * finishes last then publishes this rank's counts for the step (queries per owner from the batch's meta words,
 * pushed rows per owner from push_counts, null = none) and releases sequence number `seq` to every peer.
 * Replaces generateQuery + the first half of all2allExchangeQuery, csrc/core/generate_query.cu:91-106,
 * csrc/core/all2all.cu:18-44.  nrank <= 256. */
int hctr_p2p_query_send(const hctr_p2p_ctx *c, const uint32_t *meta, size_t u_max, const int64_t *uniq,
                        const uint8_t *uniq_owner, const int32_t *uniq_row, const int64_t *version, uint32_t seq,
                        const uint32_t *push_counts, void *stream);

/* Publishes this rank's counts to every peer and releases sequence number `seq` (what the last thread block of
 * hctr_p2p_query_send / hctr_p2p_stale_gather does, as a launch of its own).
 * phase 0: query count (from meta's segments) + push_count (null = zeros); phase 1: ret_count. */
int hctr_p2p_signal(const hctr_p2p_ctx *c, int phase, uint32_t seq, const uint32_t *meta,
                    const uint32_t *counts, void *stream);

/* Waits (bounded by c->timeout_ns) until every peer has released `seq` for `phase`; copies the announced counts
 * into c->cnt_in.  On timeout sets HCTR_ERR_TIMEOUT in *c->err, records zero counts for the silent peers and
 * returns normally.  hctr_p2p_owner_mark (phase 0) and hctr_p2p_refresh_index (phase 1) do the same wait in their
 * first instructions; this launch is for the paths that do not use them. */
int hctr_p2p_wait(const hctr_p2p_ctx *c, int phase, uint32_t seq, void *stream);

/* Owner: applies the pushed rows of every source, source after source in rank order, in one cooperative
 * launch (grid-wide barrier between sources).  Same arithmetic as hctr_owner_update.  For more than 32 ranks. */
int hctr_p2p_owner_update(const hctr_p2p_ctx *c, const int32_t *row_of, size_t length, size_t n_cached,
                          float *embedding, int64_t *version, void *stream);

/* Owner, up to 32 ranks: hctr_owner_update_merged split in its two passes, on the pushed rows in this rank's own
 * mailbox (`mine` = host copy of box[rank]).  hctr_p2p_owner_mark first waits (bounded) for the peers' phase-0
 * counts of step `seq` and records them in c->cnt_in, then marks sources, resolves rows (ent_row, nrank * cap
 * entries) and adds the update counts to the versions: versions are final when it ends.  hctr_p2p_owner_apply adds
 * the rows. */
int hctr_p2p_owner_mark(const hctr_p2p_ctx *c, const hctr_p2p_box *mine, uint32_t seq, const int32_t *row_of,
                        size_t length, size_t n_cached, unsigned long long *row_mask, unsigned long long *row_head,
                        uint32_t epoch, int32_t *ent_row, uint32_t *ent_next, int64_t *version, void *stream);
int hctr_p2p_owner_apply(const hctr_p2p_ctx *c, const hctr_p2p_box *mine, size_t n_cached, const int32_t *ent_row,
                         const unsigned long long *row_mask, unsigned long long *row_head, uint32_t *ent_next,
                         float *embedding, void *stream);

/* Pull side.  Nothing is compacted: the row returned for the j-th query requester s sent to this owner goes to row
 * (owner * cap + j) of s's mailbox - a place s can compute for each of its unique keys without knowing what the
 * owner decided - so neither side scans flags.
 * hctr_p2p_stale_gather (owner; after the pushed rows have been applied): for every received query, indexed FLAT
 * (q in [0, Q) runs over the queries of source 0, then source 1, ...; Q and the per-source starts are in c->cnt_in),
 * stale = (requester's version is INT64_MIN or version + pull_bound < owner's version) and the requester is not
 * this rank.  Flag bytes, and rows + versions of the stale keys, go straight into the requesters' mailboxes; the
 * thread block that finishes last releases `seq` (phase 1).  Replaces decide_outdated_kernel, the scan, the
 * segmented reduce, the select and write_return_value_kernel of csrc/core/handle_query.cu:7-78 and
 * all2allReturnOutdated / all2allReturnValue, csrc/core/all2all.cu:89-130.
 * hctr_p2p_refresh_index (requester): waits (bounded) for the owners' phase-1 release of `seq`; then for every
 * unique key u: recv_index[u] = its row in box[rank].rval / rver, flags[u] = the owner's decision, and for a
 * flagged key cached here embedding[row] = returned row + pending[row], version[row] = returned version.
 * Replaces the scan and update_cache_kernel of csrc/core/writeback.cu:8-50. */
int hctr_p2p_stale_gather(const hctr_p2p_ctx *c, uint32_t seq, const int32_t *row_of, size_t length, size_t n_cached,
                          const float *embedding, const int64_t *version, int64_t pull_bound, void *stream);
int hctr_p2p_refresh_index(const hctr_p2p_ctx *c, uint32_t seq, const uint32_t *meta, size_t u_max,
                           const uint8_t *uniq_owner, const int32_t *uniq_row, size_t n_cached, const float *pending,
                           float *embedding, int64_t *version, uint8_t *flags, uint32_t *recv_index, void *stream);

/* hctr_p2p_refresh_index followed by hctr_expand_rows as ONE launch, without the flag / row-index arrays between
 * them: after the (bounded) wait for the owners' phase-1 release the kernel refreshes the flagged cached rows and
 * writes dst[i] for every batch position - from the table (key owned, or cached and not flagged), from the mailbox
 * (key not stored here) or as mailbox row + pending row (key cached and flagged: the value the refresh stores).
 * Replaces update_cache_kernel, the scan and write_back_kernel of csrc/core/writeback.cu:8-71. */
int hctr_p2p_refresh_expand(const hctr_p2p_ctx *c, uint32_t seq, const uint32_t *meta, const uint8_t *uniq_owner,
                            const int32_t *uniq_row, size_t n_cached, const float *pending, float *embedding,
                            int64_t *version, size_t batch, const int32_t *pos_row, const int32_t *idx_map,
                            float *dst, void *stream);

typedef struct hctr_reduce_args {
  size_t n_unique;            /* U of the previous batch (host value) */
  size_t width;               /* W */
  size_t n_cached;            /* rows [0,n_cached) are cached replicas */
  float neg_lr;               /* -learning_rate */
  const float *grad;          /* [B_prev, W] caller's gradients */
  const uint32_t *run_start;  /* [U+1] */
  const uint32_t *sorted_pos; /* [B_prev] */
  const uint32_t *heavy_list; /* unique indices whose run is longer than HCTR_LIGHT_RUN */
  size_t n_heavy;             /* entries in heavy_list (host value) */
  const int64_t *uniq;        /* [U] */
  const int32_t *uniq_row;    /* [U] */
  const uint32_t *need_push;  /* [U] or null when nrank==1 */
  const uint32_t *push_slot;  /* [U+1] or null */
  float *embedding;           /* [S, W] */
  int64_t *version;           /* [S] */
  float *pending;             /* [n_cached, W] */
  int64_t *pending_cnt;       /* [n_cached] */
  int64_t *push_key;          /* [P] packed ids of pushed rows */
  int64_t *push_updates;      /* [P] update counts */
  float *push_val;            /* [P, W] */
  uint32_t *work_counter;     /* three device words of scratch (work queues of the kernels) */
  /* optional peer-to-peer routing of pushed rows: when p2p is non-null, a pushed row of a key owned by
   * rank p goes to slot (push_slot[u] - push_base[p]) of this rank's sub-region in p's mailbox instead
   * of push_key / push_updates / push_val */
  const hctr_p2p_ctx *p2p;    /* host pointer, copied into the launch */
  const uint8_t *uniq_owner;  /* [U] */
  const uint32_t *push_base;  /* device [nrank]: push_slot at the first unique key of each owner */
  /* optional: a second stream (cudaStream_t) and two events (cudaEvent_t, timing disabled) that let
   * the long-run kernel overlap the short-run kernel; null = everything on the call's stream */
  void *side_stream;
  void *fork_event;
  void *join_event;
  /* optional: the batch's meta words on the device.  When non-null the kernels read the number of unique keys and
   * of long runs from meta[HCTR_META_UNIQUE] / meta[HCTR_META_NHEAVY] - the host need not have seen them - and
   * n_unique / n_heavy are only upper bounds that size the grids. */
  const uint32_t *meta;
  /* runs of up to HCTR_LIGHT_RUN positions are in arbitrary order in sorted_pos (hctr_dedupe_order_light has not
   * run): the kernel puts each of them in ascending order as it loads them.  Only legal when
   * hctr_reduce_orders_short_runs(width, grad) is non-zero. */
  int short_runs_unordered;
  /* optional cudaEvent_t the long-run kernel waits for before it starts (the ordering of the long runs, when that
   * runs on another stream); the short-run kernel does not wait for it */
  void *long_wait_event;
} hctr_reduce_args;

int hctr_grad_reduce_apply_pack(const hctr_reduce_args *a, void *stream);
/* Non-zero when, for rows of `width` floats and this gradient buffer, the short-run kernel is the one that can
 * order its runs itself (short_runs_unordered). */
int hctr_reduce_orders_short_runs(size_t width, const float *grad);

/* ---------------------------------------------------------------------------------------------
 * Query generation.  Replaces lookup_version_kernel, csrc/core/generate_query.cu:91-106.
 * ------------------------------------------------------------------------------------------- */
int hctr_query_versions(size_t n_unique, const int32_t *uniq_row, const int64_t *version,
                        int64_t *query_version, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Owner side.
 * ------------------------------------------------------------------------------------------- */

/* Apply `n_rows` pushed rows of ONE source rank: row = row_of[key]; version[row] += updates;
 * embedding[row] += val.  Called once per source in rank order, which keeps the reference's
 * conflict-free, deterministic apply order.  Replaces cvt_embedding_idx_2_offset and
 * table_update_remote_kernel, csrc/core/handle_query.cu:81-116. */
int hctr_owner_update(size_t n_rows, size_t width, const int64_t *key, const int64_t *updates,
                      const float *val, const int32_t *row_of, size_t length, size_t n_cached,
                      float *embedding, int64_t *version, uint32_t *err, void *stream);
/* All sources at once, in two launches (mark sources + versions, then rows), with the same per-row apply order
 * (ascending source rank) and therefore the same bits as calling hctr_owner_update once per source.  ent_row and
 * ent_next are scratch for one 32-bit word per pushed row; row_head is a second array like row_mask (one 64-bit
 * word per owned row, zero-initialised once, epoch-tagged): the mark pass chains the entries that push the same
 * row through row_head / ent_next, the row pass walks the chain instead of searching the sources' lists.  Source s's rows start at entry
 * src_off[s] of key/updates/val and number flat_start[s+1] - flat_start[s] (device arrays of nsrc and nsrc+1
 * entries; the counts may only exist on the device); every source's list must be sorted by key, as the
 * slices of a unique list are.  row_mask: one 64-bit word per OWNED row (row - n_cached), zero-initialised once; `epoch` must be
 * non-zero and differ from every earlier call's on the same row_mask (no clearing between calls).
 * rows_hint sizes the grids (an upper bound of the total number of rows is fine).  nsrc <= 32. */
int hctr_owner_update_merged(int nsrc, size_t rows_hint, size_t width, const int64_t *key,
                             const int64_t *updates, const float *val, const unsigned long long *src_off,
                             const uint32_t *flat_start, const int32_t *row_of, size_t length, size_t n_cached,
                             unsigned long long *row_mask, unsigned long long *row_head, uint32_t epoch,
                             int32_t *ent_row, uint32_t *ent_next, float *embedding, int64_t *version, uint32_t *err,
                             void *stream);

/* Same, with the row count read from device memory (at most n_rows_max). */
int hctr_owner_update_dev(size_t n_rows_max, const uint32_t *n_rows_dev, size_t width, const int64_t *key,
                          const int64_t *updates, const float *val, const int32_t *row_of, size_t length,
                          size_t n_cached, float *embedding, int64_t *version, uint32_t *err, void *stream);

/* Staleness decision for `n_query` received (key, version) pairs, laid out as nrank consecutive
 * segments whose starts are seg_start[0..nrank] (device, 32-bit).  stale = (v == INT64_MIN or
 * v + pull_bound < version[row]) and the requester is not this rank.  Writes flags (one byte per key),
 * ret_slot = exclusive scan of flags (n_query+1 entries) and ret_count[p] = rows to return to p.
 * Replaces decide_outdated_kernel + scan + segmented reduce, csrc/core/handle_query.cu:7-61. */
int hctr_stale_check(size_t n_query, int nrank, int rank, const uint32_t *seg_start, const int64_t *key,
                     const int64_t *req_version, const int32_t *row_of, size_t length, size_t n_cached,
                     const int64_t *version, int64_t pull_bound, uint8_t *flags, uint32_t *flags32,
                     uint32_t *ret_slot, uint32_t *scan_scratch, uint32_t *ret_count, uint32_t *err,
                     void *stream);

/* Gather the flagged rows (+ versions) into the return buffer at ret_slot.  Replaces the compaction and
 * write_return_value_kernel, csrc/core/handle_query.cu:24-40,74-77. */
int hctr_gather_rows(size_t n_query, size_t width, const int64_t *key, const uint8_t *flags,
                     const uint32_t *ret_slot, const int32_t *row_of, const float *embedding,
                     const int64_t *version, float *ret_val, int64_t *ret_version, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Requester side.  Replaces writeBack, csrc/core/writeback.cu:8-56.
 * ------------------------------------------------------------------------------------------- */

/* recv_slot = exclusive scan of the flags this rank got back for its unique keys (U+1 entries). */
int hctr_recv_slots(size_t n_unique, const uint8_t *flags, uint32_t *flags32, uint32_t *recv_slot,
                    uint32_t *scan_scratch, void *stream);

/* For every flagged unique key that is cached here: embedding[row] = returned + pending[row];
 * version[row] = returned version. */
int hctr_cache_refresh(size_t n_unique, size_t width, const uint8_t *flags, const uint32_t *recv_slot,
                       const int32_t *uniq_row, const float *recv_val, const int64_t *recv_version,
                       const float *pending, float *embedding, int64_t *version, void *stream);

/* dst[i] = row of keys[i]: from the local table when stored (pos_row[i] >= 0), else from the receive
 * buffer at recv_slot[idx_map[i]].  recv_slot / recv_val may be null when every key is stored locally
 * (single-rank tables). */
int hctr_expand_rows(size_t batch, size_t width, const int32_t *pos_row, const int32_t *idx_map,
                     const uint32_t *recv_slot, const float *recv_val, const float *embedding,
                     float *dst, void *stream);

/* Half of hctr_expand_rows for a table that stores every key itself: only the positions whose key is
 * (in_prev != 0) / is not (in_prev == 0) among prev_uniq[0 .. prev_meta[HCTR_META_UNIQUE]), the ascending unique
 * keys of the previous batch.  The two halves together write every row of dst exactly once; the "is not" half
 * reads no row the previous batch's gradients change. */
int hctr_expand_rows_subset(size_t batch, size_t width, const int32_t *pos_row, const int64_t *keys,
                            const int64_t *prev_uniq, const uint32_t *prev_meta, int in_prev,
                            const float *embedding, float *dst, void *stream);

/* Same result through the bulk-copy engine (cp.async.bulk row -> shared memory -> dst, double-buffered per warp,
 * mbarrier completion with bounded waits: a wait that runs out sets HCTR_ERR_TIMEOUT in *err).  Needs 16-byte
 * aligned buffers, width % 4 == 0 and rows of at most 4 KB; anything else goes to hctr_expand_rows. */
int hctr_expand_rows_bulk(size_t batch, size_t width, const int32_t *pos_row, const int32_t *idx_map,
                          const uint32_t *recv_slot, const float *recv_val, const float *embedding, float *dst,
                          uint32_t *err, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* HCTR_KERNELS_H_ */
