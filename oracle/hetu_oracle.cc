// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT.
//
// CPU restatement of the HetuCTR distributed embedding table hot path
// (preprocess -> query -> gradient push -> writeback/update).  All `n` ranks of
// a job live in ONE host process and advance in lockstep; the three exchanges
// become plain array moves.  Only tests, the smoke check and the benchmark's CPU
// baseline may link or load this file; the product library never does.
//
// Every function cites the reference source (paths relative to the reference
// project root) whose behaviour it restates.  Nothing here is copied from the
// reference: the reference is CUDA kernels + cub + NCCL, this is sequential
// loops over the same arrays with the same arithmetic in the same order.
//
// Parity pinning: the reference ships no golden vectors for this path.  The
// restatement is pinned by (1) the reference's three known-answer scripts
// (tests/test_update.py:17-70, tests/check.py:14-46) re-run against this file,
// and (2) dumps of the reference's own build (oracle/_ref, run on a GPU box)
// committed under tests/golden/.
//
// Build: g++ -O2 -shared -fPIC hetu_oracle.cc -o _build/libhetu_oracle.so
//        (add -fopenmp -DHO_PARALLEL for the multithreaded CPU baseline build)

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>
#include <limits>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

#ifdef HO_PARALLEL
#include <omp.h>
#include <parallel/algorithm>
#define HO_PFOR _Pragma("omp parallel for schedule(static)")
#define HO_PFOR_DYN _Pragma("omp parallel for schedule(dynamic, 256)")
#else
#define HO_PFOR
#define HO_PFOR_DYN
#endif

namespace {

// csrc/core/types.h:12-28
using embed_t = float;
using version_t = long long;
using index_t = long long;
using worker_t = unsigned char;
constexpr index_t kInvalidIndex = -1;
constexpr version_t kInvalidVersion = std::numeric_limits<version_t>::min();

// wrap-around add: the reference adds update counts to versions that may still be
// kInvalidVersion (csrc/core/generate_query.cu:68-77); keep that defined in C++.
inline version_t wadd(version_t a, version_t b) {
  return (version_t)((unsigned long long)a + (unsigned long long)b);
}

// Zero-initialised array whose pages are only touched when used (calloc): a 17 GB table of which a
// benchmark sample touches a few hundred MB costs nothing to create.
template <class T>
struct ZeroBuf {
  T *p = nullptr;
  size_t n = 0;
  ZeroBuf() {}
  ZeroBuf(const ZeroBuf &) = delete;
  ZeroBuf &operator=(const ZeroBuf &) = delete;
  ~ZeroBuf() { std::free(p); }
  void assign_zero(size_t count) {
    std::free(p);
    p = count ? static_cast<T *>(std::calloc(count, sizeof(T))) : nullptr;
    if (count && !p) throw std::bad_alloc();
    n = count;
  }
  size_t size() const { return n; }
  T *begin() { return p; }
  T &operator[](size_t i) { return p[i]; }
  const T &operator[](size_t i) const { return p[i]; }
};

// csrc/core/preprocess_struct.h:7-24 — one batch descriptor.
struct Batch {
  size_t batch_size = 0;
  size_t unique_size = 0;
  std::vector<index_t> idx;         // d_idx
  std::vector<index_t> unique_idx;  // d_unique_idx
  std::vector<index_t> sorted_arg;  // d_sorted_arg
  std::vector<index_t> run_length;  // d_run_length (after the exclusive scan)
  std::vector<index_t> idx_map;     // d_idx_map
  std::vector<worker_t> root;       // d_root
  std::vector<index_t> offset;      // d_offset
  std::vector<size_t> shape;            // h_shape / u_shape            (n+1)
  std::vector<size_t> shape_exchanged;  // h_shape_exchanged            (n+1)
};

struct Rank {
  int rank = 0;
  size_t storage = 0;    // kStorageMax
  size_t nonlocal = 0;   // kNonLocalStorageMax
  std::vector<int32_t> row_of;       // dense stand-in for the key->row hash map; -1 = not stored
  std::vector<index_t> stored_keys;  // key of each local row
  ZeroBuf<embed_t> emb;              // d_embedding_
  ZeroBuf<embed_t> pend;             // d_gradient_ (cached rows only)
  std::vector<version_t> pend_cnt;   // d_updates_  (cached rows only)
  std::vector<version_t> ver;        // d_version_
  Batch cur, prev;
  std::vector<index_t> need_update;    // d_need_update_
  std::vector<index_t> update_prefix;  // d_update_prefix_ (push slots, then reused as compacted ids)
  // exchange buffers, [0] = send side, [1] = receive side
  std::vector<index_t> q_idx_s, q_idx_r, q_grad_idx_s, q_grad_idx_r;
  std::vector<version_t> q_ver_s, q_ver_r, q_upd_s, q_upd_r;
  std::vector<embed_t> q_val_s, q_val_r;
  std::vector<index_t> ret_outdated_s, ret_outdated_r;
  std::vector<embed_t> ret_val_s, ret_val_r;
  std::vector<version_t> ret_ver_s, ret_ver_r;
  size_t received = 0, grad_received = 0;  // all2all_received_, all2all_gradient_received_
  size_t stat_push_rows = 0, stat_query_keys = 0, stat_return_rows = 0, stat_recv_rows = 0;
};

struct World {
  int n = 1;
  size_t length = 0, width = 0;
  version_t pull_bound = 0, push_bound = 0;
  embed_t lr = 0;
  std::vector<worker_t> owner;  // d_root_
  std::vector<Rank> ranks;
  std::string err;
};

// csrc/core/table_initialize.cu:66-114 — storage layout and version init.
// Local row of a stored key = its position after a STABLE partition of storage_arr
// that puts keys owned by another rank first (:76-81,91).  Cached rows start at
// kInvalidVersion, owned rows at 0 (:108-112); pending gradient/update count = 0 (:102-105).
void set_storage(World &w, int r, const index_t *storage, size_t S) {
  Rank &k = w.ranks[r];
  k.rank = r;
  k.storage = S;
  k.stored_keys.clear();
  k.stored_keys.reserve(S);
  for (size_t i = 0; i < S; i++) {
    if (storage[i] < 0 || (size_t)storage[i] >= w.length) throw std::runtime_error("storage key out of range");
    if (w.owner[storage[i]] != r) k.stored_keys.push_back(storage[i]);
  }
  k.nonlocal = k.stored_keys.size();
  for (size_t i = 0; i < S; i++)
    if (w.owner[storage[i]] == r) k.stored_keys.push_back(storage[i]);
  k.row_of.assign(w.length, -1);
  for (size_t i = 0; i < S; i++) k.row_of[k.stored_keys[i]] = (int32_t)i;
  k.emb.assign_zero(S * w.width);
  k.pend.assign_zero(k.nonlocal * w.width);
  k.pend_cnt.assign(k.nonlocal, 0);
  k.ver.assign(S, 0);
  std::fill(k.ver.begin(), k.ver.begin() + k.nonlocal, kInvalidVersion);
  k.cur = Batch();
  k.prev = Batch();
  k.cur.shape.assign(w.n + 1, 0);
  k.cur.shape_exchanged.assign(w.n + 1, 0);
  k.prev.shape.assign(w.n + 1, 0);
  k.prev.shape_exchanged.assign(w.n + 1, 0);
}

// csrc/core/preprocess.cu:92-141 (preprocessIndex) minus the count exchange.
//  * sort key = id + length*owner, value = position, stable sort   (:11-20,105-109)
//  * run-length encode the sorted ids -> unique ids + counts        (:34-41,115-117)
//  * exclusive scan of counts over batch_size+1 entries             (:124-125)
//  * owner, local row (or -1) and per-owner segment starts          (:45-69)
//  * batch position -> index of its key in the unique list          (:71-90)
//  * segment starts -> per-owner counts                             (:22-32)
void preprocess_index(World &w, Rank &k, const index_t *data, size_t B) {
  Batch &b = k.cur;
  const int n = w.n;
  b.batch_size = B;
  b.idx.assign(data, data + B);
  for (size_t i = 0; i < B; i++)
    if (data[i] < 0 || (size_t)data[i] >= w.length) throw std::runtime_error("key out of range");
  std::vector<std::pair<unsigned long long, index_t>> kv(B);
  HO_PFOR
  for (size_t i = 0; i < B; i++)
    kv[i] = {(unsigned long long)data[i] + (unsigned long long)w.length * w.owner[data[i]], (index_t)i};
  // positions are distinct and ascending, so an ordinary sort of (key, position) pairs
  // is the stable argsort the reference gets from a radix sort.
#ifdef HO_PARALLEL
  __gnu_parallel::sort(kv.begin(), kv.end());
#else
  std::sort(kv.begin(), kv.end());
#endif
  b.sorted_arg.resize(B);
  HO_PFOR
  for (size_t i = 0; i < B; i++) b.sorted_arg[i] = kv[i].second;
  b.unique_idx.clear();
  std::vector<index_t> counts;
  for (size_t i = 0; i < B; i++) {
    index_t id = data[kv[i].second];
    if (i == 0 || id != b.unique_idx.back()) {
      b.unique_idx.push_back(id);
      counts.push_back(1);
    } else {
      counts.back()++;
    }
  }
  const size_t U = b.unique_idx.size();
  b.unique_size = U;
  // exclusive scan; entries past U repeat the total, as scanning zero-length runs would.
  b.run_length.assign(B + 1, 0);
  index_t acc = 0;
  for (size_t i = 0; i <= B; i++) {
    b.run_length[i] = acc;
    if (i < U) acc += counts[i];
  }
  b.root.resize(U);
  b.offset.resize(U);
  b.shape.assign(n + 1, 0);
  std::vector<size_t> start(n + 2, U);
  HO_PFOR
  for (size_t u = 0; u < U; u++) {
    index_t id = b.unique_idx[u];
    b.root[u] = w.owner[id];
    int32_t row = k.row_of[id];
    b.offset[u] = row < 0 ? kInvalidIndex : (index_t)row;
  }
  {
    // segment start of owner p = first unique index whose owner >= p
    size_t u = 0;
    for (int p = 0; p <= n; p++) {
      while (u < U && b.root[u] < p) u++;
      start[p] = u;
    }
  }
  b.idx_map.resize(B);
  HO_PFOR
  for (size_t i = 0; i < B; i++) {
    index_t id = data[i];
    int p = w.owner[id];
    auto first = b.unique_idx.begin() + start[p], last = b.unique_idx.begin() + start[p + 1];
    b.idx_map[i] = std::lower_bound(first, last, id) - b.unique_idx.begin();
  }
  for (int p = 0; p < n; p++) b.shape[p] = start[p + 1] - start[p];
  b.shape[n] = 0;
}

// csrc/core/preprocess.cu:148-182 (decide_update_kernel + exclusive scan), on the PREVIOUS batch:
// owned -> never pushed; not stored -> always pushed; cached -> pushed once the pending
// update count plus this batch's occurrences exceeds push_bound.
void preprocess_gradient(World &w, Rank &k) {
  Batch &p = k.prev;
  const size_t U = p.unique_size;
  std::fill(p.shape.begin(), p.shape.begin() + w.n, 0);
  k.need_update.assign(U, 0);
  k.update_prefix.assign(U, 0);
  index_t slot = 0;
  for (size_t u = 0; u < U; u++) {
    version_t update_new = p.run_length[u + 1] - p.run_length[u];
    index_t off = p.offset[u];
    index_t need;
    if (p.root[u] == k.rank) need = 0;
    else if (off == kInvalidIndex) need = 1;
    else need = (k.pend_cnt[off] + update_new <= w.push_bound) ? 0 : 1;
    k.need_update[u] = need;
    k.update_prefix[u] = slot;
    slot += need;
    if (need) p.shape[p.root[u]]++;
  }
}

// all2allExchangeShape, csrc/core/all2all.cu:6-16.
void exchange_shape(World &w, bool prev) {
  for (auto &dst : w.ranks)
    for (auto &src : w.ranks) {
      Batch &bd = prev ? dst.prev : dst.cur;
      Batch &bs = prev ? src.prev : src.cur;
      bd.shape_exchanged[src.rank] = bs.shape[dst.rank];
    }
}

// csrc/core/hetu_gpu_table.cu:43-65
void world_preprocess(World &w, const index_t *const *keys, const size_t *nkeys) {
#ifdef HO_PARALLEL
#pragma omp parallel for if (w.n > 1) schedule(static, 1)
#endif
  for (int r = 0; r < w.n; r++) {
    Rank &k = w.ranks[r];
    std::swap(k.cur, k.prev);
    try {
      preprocess_index(w, k, keys[r], nkeys[r]);
      preprocess_gradient(w, k);
    } catch (std::exception &e) {
#ifdef HO_PARALLEL
#pragma omp critical
#endif
      w.err = e.what();
    }
  }
  if (!w.err.empty()) {
    std::string e = w.err;
    w.err.clear();
    throw std::runtime_error(e);
  }
  exchange_shape(w, false);
  exchange_shape(w, true);
}

inline int update_type(const Rank &k, index_t off, bool need) {
  if (off == kInvalidIndex) return 0;          // not stored
  if ((size_t)off >= k.nonlocal) return 1;     // owned
  return need ? 2 : 3;                         // cached: push / hold
}

// csrc/core/generate_query.cu:51-83 (gradient_index_kernel) then :8-49 (gradient_reduction_kernel).
void generate_gradient(World &w, Rank &k, const embed_t *grad) {
  Batch &p = k.prev;
  const size_t U = p.unique_size, W = w.width;
  size_t pushed = 0;
  for (int i = 0; i < w.n; i++) pushed += p.shape[i];
  k.q_grad_idx_s.assign(pushed, 0);
  k.q_upd_s.assign(pushed, 0);
  k.q_val_s.assign(pushed * W, 0.f);
  k.stat_push_rows = pushed;
  for (size_t u = 0; u < U; u++) {
    bool need = k.need_update[u];
    index_t off = p.offset[u];
    int t = update_type(k, off, need);
    version_t c = p.run_length[u + 1] - p.run_length[u];
    if (t == 1) k.ver[off] = wadd(k.ver[off], c);
    else if (t >= 2) {
      k.pend_cnt[off] += c;
      if (t == 2) {
        c = k.pend_cnt[off];
        k.pend_cnt[off] = 0;
        k.ver[off] = wadd(k.ver[off], c);
      }
    }
    if (need) {
      k.q_grad_idx_s[k.update_prefix[u]] = p.unique_idx[u];
      k.q_upd_s[k.update_prefix[u]] = c;
    }
  }
  const embed_t neg_lr = -w.lr;
  HO_PFOR_DYN
  for (size_t u = 0; u < U; u++) {
    bool need = k.need_update[u];
    index_t off = p.offset[u];
    int t = update_type(k, off, need);
    index_t l = p.run_length[u], r = p.run_length[u + 1];
    embed_t *dq = need ? &k.q_val_s[k.update_prefix[u] * W] : nullptr;
    for (size_t d = 0; d < W; d++) {
      embed_t sum = 0;
      for (index_t j = l; j < r; j++) sum += grad[p.sorted_arg[j] * W + d];
      sum *= neg_lr;
      if (t != 0) k.emb[off * W + d] += sum;
      else dq[d] = sum;
      if (t >= 2) k.pend[off * W + d] += sum;
      if (t == 2) {
        dq[d] = k.pend[off * W + d];
        k.pend[off * W + d] = 0;
      }
    }
  }
}

// csrc/core/generate_query.cu:91-106
void generate_query(Rank &k) {
  Batch &c = k.cur;
  const size_t U = c.unique_size;
  k.q_idx_s.assign(c.unique_idx.begin(), c.unique_idx.begin() + U);
  k.q_ver_s.resize(U);
  for (size_t u = 0; u < U; u++)
    k.q_ver_s[u] = c.offset[u] != kInvalidIndex ? k.ver[c.offset[u]] : kInvalidVersion;
}

// Generic all-to-all-v (csrc/core/all2all.cu:18-130): destination d receives, from each source s
// in rank order, the segment of s's send buffer addressed to d.  Send offsets advance by the
// sender's counts, so the receive buffer is the concatenation over sources.
//   snd/rcv : accessors for the send / receive vectors of a rank
//   cnt     : cnt(src_rank_struct, dst_rank_id) = items src sends to dst
template <class Snd, class Rcv, class Cnt>
void move_segments(World &w, Snd snd, Rcv rcv, Cnt cnt, size_t per_item) {
  for (auto &d : w.ranks) {
    auto &out = rcv(d);
    out.clear();
    for (auto &s : w.ranks) {
      size_t off = 0;
      for (int i = 0; i < d.rank; i++) off += cnt(s, i);
      const auto &in = snd(s);
      out.insert(out.end(), in.begin() + off * per_item, in.begin() + (off + cnt(s, d.rank)) * per_item);
    }
  }
}

// csrc/core/handle_query.cu:81-116 — owner applies pushed gradients source by source.
void handle_gradient(World &w, Rank &k) {
  const size_t W = w.width;
  const size_t G = k.q_grad_idx_r.size();
  k.grad_received = G;
  for (size_t g = 0; g < G; g++) {
    index_t id = k.q_grad_idx_r[g];
    int32_t row = k.row_of[id];
    if (row < 0 || w.owner[id] != k.rank) throw std::runtime_error("pushed gradient for a row this rank does not own");
    k.ver[row] = wadd(k.ver[row], k.q_upd_r[g]);
    for (size_t d = 0; d < W; d++) k.emb[(size_t)row * W + d] += k.q_val_r[g * W + d];
  }
}

// csrc/core/handle_query.cu:7-78 — staleness decision, per-requester counts, compaction, gather.
void handle_query(World &w, Rank &k) {
  const size_t W = w.width;
  Batch &c = k.cur;
  const size_t Q = k.q_idx_r.size();
  k.received = Q;
  k.stat_query_keys = Q;
  size_t self_start = 0;
  for (int i = 0; i < k.rank; i++) self_start += c.shape_exchanged[i];
  size_t self_end = self_start + c.shape_exchanged[k.rank];
  k.ret_outdated_s.assign(Q, 0);
  k.update_prefix.clear();
  k.ret_ver_s.clear();
  k.ret_val_s.clear();
  std::vector<size_t> counts(w.n + 1, 0);
  size_t q = 0;
  for (int src = 0; src < w.n; src++) {
    for (size_t j = 0; j < c.shape_exchanged[src]; j++, q++) {
      version_t lv = k.q_ver_r[q];
      index_t id = k.q_idx_r[q];
      int32_t row = k.row_of[id];
      if (row < 0 || w.owner[id] != k.rank) throw std::runtime_error("query for a row this rank does not own");
      version_t gv = k.ver[row];
      bool self = q >= self_start && q < self_end;
      bool outdated = lv == kInvalidVersion || wadd(lv, w.pull_bound) < gv;
      bool flag = outdated && !self;
      k.ret_outdated_s[q] = flag;
      if (flag) {
        counts[src]++;
        k.update_prefix.push_back(id);
        k.ret_ver_s.push_back(gv);
        k.ret_val_s.insert(k.ret_val_s.end(), k.emb.p + (size_t)row * W, k.emb.p + (size_t)(row + 1) * W);
      }
    }
  }
  k.stat_return_rows = k.ret_ver_s.size();
  // the batch's shape arrays are reused for the return counts (handle_query.cu:59-71)
  for (int i = 0; i < w.n; i++) c.shape[i] = counts[i];
}

// csrc/core/writeback.cu:8-56 — refresh cached replicas, then expand unique rows to batch order.
void write_back(World &w, Rank &k, embed_t *dst) {
  const size_t W = w.width;
  Batch &c = k.cur;
  const size_t U = c.unique_size;
  // exclusive scan of the received flags -> slot in the receive buffer; flagged ids in order
  std::vector<index_t> prefix(U);
  std::vector<index_t> ids;
  index_t acc = 0;
  for (size_t u = 0; u < U; u++) {
    prefix[u] = acc;
    if (k.ret_outdated_r[u]) {
      acc++;
      ids.push_back(c.unique_idx[u]);
    }
  }
  const size_t R = k.ret_ver_r.size();
  k.stat_recv_rows = R;
  for (size_t i = 0; i < R; i++) {
    int32_t row = k.row_of[ids[i]];
    if (row >= 0) {
      k.ver[row] = k.ret_ver_r[i];
      for (size_t d = 0; d < W; d++)
        k.emb[(size_t)row * W + d] = k.ret_val_r[i * W + d] + k.pend[(size_t)row * W + d];
    }
  }
  HO_PFOR
  for (size_t i = 0; i < c.batch_size; i++) {
    index_t m = c.idx_map[i];
    index_t off = c.offset[m];
    const embed_t *val = off == kInvalidIndex ? &k.ret_val_r[prefix[m] * W] : &k.emb[off * W];
    std::memcpy(dst + i * W, val, W * sizeof(embed_t));
  }
  k.ret_outdated_s = prefix;  // the reference leaves the scan in d_return_outdated_[0]
}

// csrc/core/hetu_gpu_table.cu:9-41
void world_push_pull(World &w, const embed_t *const *grads, embed_t *const *dsts) {
  bool any_null = false, all_null = true;
  for (int r = 0; r < w.n; r++) {
    bool isnull = grads == nullptr || grads[r] == nullptr;
    any_null |= isnull;
    all_null &= isnull;
  }
  if (any_null && !all_null) throw std::runtime_error("inference steps must be taken by all ranks together");
  for (auto &k : w.ranks) {
    if (all_null) {
      k.prev.batch_size = 0;
      k.prev.unique_size = 0;
      std::fill(k.prev.shape.begin(), k.prev.shape.end(), 0);
      std::fill(k.prev.shape_exchanged.begin(), k.prev.shape_exchanged.end(), 0);
    }
  }
#ifdef HO_PARALLEL
#pragma omp parallel for if (w.n > 1) schedule(static, 1)
#endif
  for (int r = 0; r < w.n; r++) {
    generate_gradient(w, w.ranks[r], all_null ? nullptr : grads[r]);
    generate_query(w.ranks[r]);
  }

  const size_t W = w.width;
  // all2allExchangeQuery, csrc/core/all2all.cu:18-87: keys + versions of the current batch,
  // then ids + update counts + values of the previous batch's pushed rows.
  auto cur_cnt = [](Rank &s, int d) { return s.cur.shape[d]; };
  auto prev_cnt = [](Rank &s, int d) { return s.prev.shape[d]; };
  move_segments(w, [](Rank &r) -> auto & { return r.q_idx_s; }, [](Rank &r) -> auto & { return r.q_idx_r; }, cur_cnt, 1);
  move_segments(w, [](Rank &r) -> auto & { return r.q_ver_s; }, [](Rank &r) -> auto & { return r.q_ver_r; }, cur_cnt, 1);
  move_segments(w, [](Rank &r) -> auto & { return r.q_grad_idx_s; }, [](Rank &r) -> auto & { return r.q_grad_idx_r; }, prev_cnt, 1);
  move_segments(w, [](Rank &r) -> auto & { return r.q_upd_s; }, [](Rank &r) -> auto & { return r.q_upd_r; }, prev_cnt, 1);
  move_segments(w, [](Rank &r) -> auto & { return r.q_val_s; }, [](Rank &r) -> auto & { return r.q_val_r; }, prev_cnt, W);
#ifdef HO_PARALLEL
#pragma omp parallel for if (w.n > 1) schedule(static, 1)
#endif
  for (int r = 0; r < w.n; r++) {
    try {
      handle_gradient(w, w.ranks[r]);
      handle_query(w, w.ranks[r]);
    } catch (std::exception &e) {
#ifdef HO_PARALLEL
#pragma omp critical
#endif
      w.err = e.what();
    }
  }
  if (!w.err.empty()) {
    std::string e = w.err;
    w.err.clear();
    throw std::runtime_error(e);
  }
  // all2allReturnOutdated (csrc/core/all2all.cu:89-101): flags travel back along the query
  // route, so the owner's per-source segment sizes are its exchanged counts *before*
  // handle_query overwrote shape[] — which move_segments reads from shape_exchanged.
  move_segments(w, [](Rank &r) -> auto & { return r.ret_outdated_s; }, [](Rank &r) -> auto & { return r.ret_outdated_r; },
                [](Rank &s, int d) { return s.cur.shape_exchanged[d]; }, 1);
  // all2allExchangeShape of the return counts (handle_query.cu:66), then all2allReturnValue
  // (all2all.cu:103-130): versions and rows of the flagged keys.
  exchange_shape(w, false);
  move_segments(w, [](Rank &r) -> auto & { return r.ret_ver_s; }, [](Rank &r) -> auto & { return r.ret_ver_r; }, cur_cnt, 1);
  move_segments(w, [](Rank &r) -> auto & { return r.ret_val_s; }, [](Rank &r) -> auto & { return r.ret_val_r; }, cur_cnt, W);
#ifdef HO_PARALLEL
#pragma omp parallel for if (w.n > 1) schedule(static, 1)
#endif
  for (int r = 0; r < w.n; r++) {
    w.ranks[r].received = w.ranks[r].ret_ver_r.size();
    write_back(w, w.ranks[r], dsts[r]);
  }
}

thread_local std::string g_err;

template <class F>
int guarded(F f) {
  try {
    f();
    return 0;
  } catch (std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

template <class T, class V>
size_t copy_out(const V &v, size_t n, T *out) {
  if (out)
    for (size_t i = 0; i < n; i++) out[i] = (T)v[i];
  return n;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// C interface for ctypes.  Every call returns 0 on success, -1 on error (see ho_last_error).
// ---------------------------------------------------------------------------------------------
extern "C" {

const char *ho_last_error() { return g_err.c_str(); }

int ho_num_threads() {
#ifdef HO_PARALLEL
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void *ho_world_create(int nrank, long long length, long long width, long long pull_bound,
                      long long push_bound, float learning_rate, const unsigned char *root_arr) {
  World *w = new World();
  w->n = nrank;
  w->length = (size_t)length;
  w->width = (size_t)width;
  w->pull_bound = pull_bound;
  w->push_bound = push_bound;
  w->lr = learning_rate;
  w->owner.assign(root_arr, root_arr + length);
  w->ranks = std::vector<Rank>(nrank);
  for (int r = 0; r < nrank; r++) w->ranks[r].rank = r;
  return w;
}

void ho_world_destroy(void *h) { delete (World *)h; }

int ho_set_storage(void *h, int rank, const long long *storage, long long n) {
  return guarded([&] { set_storage(*(World *)h, rank, storage, (size_t)n); });
}

// Initial row values are supplied by the caller in LOCAL ROW order (the reference's
// initialiser is a function of the local element index, csrc/core/table_initialize.cu:156).
int ho_set_embedding(void *h, int rank, const float *emb) {
  return guarded([&] {
    Rank &k = ((World *)h)->ranks[rank];
    std::copy(emb, emb + k.emb.size(), k.emb.p);
  });
}

int ho_preprocess(void *h, const long long *const *keys, const size_t *nkeys) {
  return guarded([&] { world_preprocess(*(World *)h, keys, nkeys); });
}

int ho_push_pull(void *h, const float *const *grads, float *const *dsts) {
  return guarded([&] { world_push_pull(*(World *)h, grads, dsts); });
}

// Introspection.  `what` selects an array of rank `rank`; the element count is returned and,
// when `out` is non-null, the array is written there as int64 (or float for value arrays).
long long ho_get_i64(void *h, int rank, const char *what, int prev, long long *out) {
  World &w = *(World *)h;
  Rank &k = w.ranks[rank];
  Batch &b = prev ? k.prev : k.cur;
  std::string s(what);
  if (s == "unique_idx") return copy_out(b.unique_idx, b.unique_size, out);
  if (s == "idx_map") return copy_out(b.idx_map, b.batch_size, out);
  if (s == "sorted_arg") return copy_out(b.sorted_arg, b.batch_size, out);
  if (s == "run_length") return copy_out(b.run_length, b.unique_size + 1, out);
  if (s == "root") return copy_out(b.root, b.unique_size, out);
  if (s == "offset") return copy_out(b.offset, b.unique_size, out);
  if (s == "shape") return copy_out(b.shape, (size_t)w.n, out);
  if (s == "shape_exchanged") return copy_out(b.shape_exchanged, (size_t)w.n, out);
  if (s == "need_update") return copy_out(k.need_update, k.need_update.size(), out);
  if (s == "version") return copy_out(k.ver, k.ver.size(), out);
  if (s == "updates") return copy_out(k.pend_cnt, k.pend_cnt.size(), out);
  if (s == "stored_keys") return copy_out(k.stored_keys, k.stored_keys.size(), out);
  if (s == "storage") { if (out) out[0] = (long long)k.storage; return 1; }
  if (s == "nonlocal") { if (out) out[0] = (long long)k.nonlocal; return 1; }
  if (s == "unique_size") { if (out) out[0] = (long long)b.unique_size; return 1; }
  if (s == "stats") {
    if (out) {
      out[0] = (long long)k.stat_push_rows;
      out[1] = (long long)k.stat_query_keys;
      out[2] = (long long)k.stat_return_rows;
      out[3] = (long long)k.stat_recv_rows;
      out[4] = (long long)k.grad_received;
    }
    return 5;
  }
  g_err = "unknown array: " + s;
  return -1;
}

long long ho_get_f32(void *h, int rank, const char *what, float *out) {
  Rank &k = ((World *)h)->ranks[rank];
  std::string s(what);
  if (s == "embedding") return copy_out(k.emb, k.emb.size(), out);
  if (s == "gradient") return copy_out(k.pend, k.pend.size(), out);
  g_err = "unknown array: " + s;
  return -1;
}

}  // extern "C"
