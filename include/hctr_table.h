/*
 * hctr_table.h — C-ABI of the table object: what a foreign-function binding of the reference's
 * HetuTable would bind.  One handle = one rank of a distributed embedding table on one GPU.
 *
 * Each entry point mirrors a member of the reference's Python-facing class
 * (csrc/pybind/pybind.cu:42-79, csrc/pybind/container.h:10-37, csrc/core/hetu_gpu_table.h:109-144);
 * argument meaning and call protocol are the reference's.  Functions return 0 on success and -1 on
 * error; hctr_last_error() then describes the failure (thread-local).
 */
#ifndef HCTR_TABLE_H_
#define HCTR_TABLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hctr_table hctr_table;  /* opaque */
typedef struct hctr_wait hctr_wait;    /* opaque handle of an asynchronous call */

/* InitType, csrc/utils/initializer.h:8-14 and csrc/pybind/pybind.cu:53-57 */
enum { HCTR_INIT_ZERO = 0, HCTR_INIT_NORMAL = 1, HCTR_INIT_UNIFORM = 2, HCTR_INIT_TRUNCATED_NORMAL = 3 };

const char *hctr_last_error(void);

/* hetuCTR.seed(n), csrc/pybind/pybind.cu:77: seed for tables created afterwards in this process. */
void hctr_seed(unsigned long seed);

/* hetuCTR.HetuTable(...), csrc/pybind/pybind.cu:9-36,62-69.  Collective over all `nrank` processes
 * when nrank > 1 (TCP rendezvous on ip:port, then an NCCL communicator).  root_arr has `length`
 * entries (owner of every key), storage_arr lists the keys this rank stores (owned + cached); both are
 * host arrays read during construction only.  init_a/init_b are (mean, stddev) or (a, b).
 * Returns NULL on error. */
hctr_table *hctr_table_create(int rank, int nrank, int device_id, const char *ip, int port, size_t length,
                              size_t width, int64_t pull_bound, int64_t push_bound, const uint8_t *root_arr,
                              const int64_t *storage_arr, size_t storage_len, int init_type, float init_a,
                              float init_b, float learning_rate, int verbose);

/* ~HetuTable, csrc/core/table_initialize.cu:231-245 */
void hctr_table_destroy(hctr_table *t);

/* HetuTable.preprocess(data_ptr, n_keys), csrc/pybind/container.h:19-22: `keys` is host or device
 * memory holding n_keys int64 keys.  Returns when the batch is ready. */
int hctr_table_preprocess(hctr_table *t, const int64_t *keys, size_t n_keys);

/* HetuTable.push_pull(grad_ptr, dst_ptr), csrc/pybind/container.h:14-17: grad = [n_keys_prev, width]
 * gradients of the PREVIOUS batch (NULL = inference step, on all ranks together), dst = [n_keys_cur,
 * width] output.  Device memory; host memory is accepted and staged.  Returns when dst is written. */
int hctr_table_push_pull(hctr_table *t, const float *grad, float *dst);

/* async_preprocess / async_push_pull / _waittype.wait(), csrc/pybind/container.h:24-34,
 * csrc/pybind/pybind.cu:46-51: the same calls queued on the table's single worker thread, in order.
 * hctr_wait_finish blocks, frees the handle and returns the call's status. */
hctr_wait *hctr_table_preprocess_async(hctr_table *t, const int64_t *keys, size_t n_keys);
hctr_wait *hctr_table_push_pull_async(hctr_table *t, const float *grad, float *dst);
int hctr_wait_finish(hctr_wait *w);

/* __repr__ / debug(), csrc/core/debug.cu:5-24.  Writes a NUL-terminated string, returns its length. */
int hctr_table_repr(hctr_table *t, int full, char *buf, size_t buf_len);

/* ---- extensions (no counterpart in the reference; used by parity tests and benchmarks) ---------- */

/* Copies an internal array to host memory: as int64 for index/version arrays, float for "embedding"
 * and "gradient".  Returns the element count (call with out = NULL to size the buffer), -1 on error.
 * Names: unique_idx idx_map sorted_arg run_length root offset shape shape_exchanged push_shape
 * push_shape_exchanged return_shape return_shape_exchanged need_update version updates stored_keys
 * embedding gradient.  prev != 0 selects the previous batch. */
long long hctr_table_dump(hctr_table *t, const char *what, int prev, void *out);

/* Overwrites all local rows from host memory ([stored rows, width], local row order). */
int hctr_table_set_embedding(hctr_table *t, const float *rows);

/* Checkpoint (no counterpart in the reference, which cannot save a table at all): writes / reads the rows,
 * versions and, for cached rows, pending gradients and pending-update counts of this rank to `path`.  The
 * importing table must have been created with the same rank, nrank, length, width and storage_arr; a file of
 * another shape, with other keys, truncated or with a wrong checksum is refused before anything is changed.
 * Import is legal between steps only; batches preprocessed earlier are dropped.  Export writes `path`.tmp and
 * renames it over `path` once complete.  In a multi-rank job both calls are COLLECTIVE in the sense of the step
 * protocol: every rank exports / imports (its own file) at the same point between two steps, because an import
 * drops the batches preprocessed so far on the rank that does it. */
int hctr_table_export(hctr_table *t, const char *path);
int hctr_table_import(hctr_table *t, const char *path);

/* Sizes of the last push_pull: {batch, unique, prev_batch, prev_unique, pushed_rows,
 * received_push_rows, queried_keys, returned_rows, received_rows, stored_rows, cached_rows, wait_queries_us,
 * wait_returns_us}; the last two are the longest in-kernel waits of the step for a peer's queries and for a
 * peer's returned rows (peer-to-peer exchange; 0 otherwise). */
int hctr_table_stats(hctr_table *t, long long out[13]);

/* Per-phase device time.  hctr_table_profile(t, k): k = 0 off, 1 every step, k > 1 every k-th step (the
 * timing events cost the step a few microseconds per phase, sampling keeps that out of a benchmark).  In a
 * timed step each phase of preprocess/push_pull is bracketed by two CUDA events on the stream it runs on; hctr_table_phase_times returns the accumulated milliseconds and
 * call counts per phase (and clears them when reset != 0).  Phase order: dedupe, push_decide, reduce,
 * query, exchange, owner_update, stale_gather, refresh, expand, owner_apply (the row pass of the owner update in
 * the peer-to-peer exchange; there owner_update is the wait for the peers' queries + source marking + versions, and
 * refresh includes the wait for the owners' rows). */
#define HCTR_N_PHASES 10
int hctr_table_profile(hctr_table *t, int enable);
int hctr_table_phase_times(hctr_table *t, double ms[HCTR_N_PHASES], long long calls[HCTR_N_PHASES], int reset);
/* The most recent timed phases (up to 256 are kept) as triples {phase index, start ms, end ms}, oldest first,
 * in milliseconds since profiling was enabled: shows which phases overlap and where the device idles.
 * Writes at most max_spans triples to out and returns how many. */
int hctr_table_timeline(hctr_table *t, double *out, int max_spans);

/* The bootstrap broadcast used when a multi-rank table is constructed, exposed for tests and tools: copies
 * `len` bytes at `data` from rank 0 to every rank over TCP (rank 0 listens on ip:port).  Returns -1 with a
 * message in hctr_last_error() if a rank does not show up within timeout_s seconds.  Same role as the
 * reference's TCPRendezvous::broadcast, csrc/utils/rendezvous.cc:42-64 (which blocks forever instead). */
int hctr_rendezvous_broadcast(int rank, int nrank, const char *ip, int port, void *data, size_t len,
                              double timeout_s);

/* How this table exchanges data with its peers: "none" (single rank), "p2p" (device-driven mailboxes
 * in peer memory; one process per GPU with peer access, the default when possible), "nccl" (grouped
 * send/receive; forced with HCTR_EXCHANGE=nccl) or "inproc" (thread ranks of one process, tests). */
const char *hctr_table_exchange_name(hctr_table *t);

/* The CUDA stream (cudaStream_t) the table enqueues its work on. */
void *hctr_table_stream(hctr_table *t);

#ifdef __cplusplus
}
#endif
#endif /* HCTR_TABLE_H_ */
