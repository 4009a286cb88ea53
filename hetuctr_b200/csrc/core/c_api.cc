// C-ABI of the table object (see hctr_table.h) on top of the C++ class.
#include <cstring>
#include <future>
#include <memory>
#include <string>

#include "core/hetu_table.h"
#include "hctr_table.h"
#include "utils/rendezvous.h"
#include "utils/thread_pool.h"

using hetuCTR::HetuTable;

struct hctr_table {
  std::unique_ptr<HetuTable> impl;
  std::unique_ptr<hetuCTR::ThreadPool> pool;  // created on the first asynchronous call
};

struct hctr_wait {
  std::future<void> fut;
};

namespace {
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
}  // namespace

extern "C" {

const char *hctr_last_error(void) { return g_err.c_str(); }

void hctr_seed(unsigned long seed) { hetuCTR::set_seed(seed); }

hctr_table *hctr_table_create(int rank, int nrank, int device_id, const char *ip, int port, size_t length,
                              size_t width, int64_t pull_bound, int64_t push_bound, const uint8_t *root_arr,
                              const int64_t *storage_arr, size_t storage_len, int init_type, float init_a,
                              float init_b, float learning_rate, int verbose) {
  hctr_table *t = nullptr;
  int rc = guarded([&] {
    hetuCTR::InitType it;
    switch (init_type) {
      case HCTR_INIT_ZERO: it = hetuCTR::InitType::kZero; break;
      case HCTR_INIT_NORMAL: it = hetuCTR::InitType::kNormal; break;
      case HCTR_INIT_UNIFORM: it = hetuCTR::InitType::kUniform; break;
      case HCTR_INIT_TRUNCATED_NORMAL: it = hetuCTR::InitType::kTruncatedNormal; break;
      default: throw std::runtime_error("Unknown initializer.");
    }
    hetuCTR::Initializer init(it, init_a, init_b);
    auto impl = std::make_unique<HetuTable>(rank, nrank, device_id, ip ? ip : "", port, length, width, pull_bound,
                                            push_bound, root_arr, length,
                                            reinterpret_cast<const hetuCTR::index_t *>(storage_arr), storage_len,
                                            init, learning_rate, verbose);
    t = new hctr_table();
    t->impl = std::move(impl);
  });
  return rc == 0 ? t : nullptr;
}

void hctr_table_destroy(hctr_table *t) {
  if (!t) return;
  t->pool.reset();  // drains queued asynchronous calls first
  delete t;
}

int hctr_table_preprocess(hctr_table *t, const int64_t *keys, size_t n_keys) {
  return guarded([&] {
    t->impl->preprocess(reinterpret_cast<hetuCTR::index_t *>(const_cast<int64_t *>(keys)), n_keys);
  });
}

int hctr_table_push_pull(hctr_table *t, const float *grad, float *dst) {
  return guarded([&] { t->impl->pushPull(const_cast<float *>(grad), dst); });
}

hctr_wait *hctr_table_preprocess_async(hctr_table *t, const int64_t *keys, size_t n_keys) {
  hctr_wait *w = nullptr;
  guarded([&] {
    if (!t->pool) t->pool = std::make_unique<hetuCTR::ThreadPool>(1);
    HetuTable *impl = t->impl.get();
    auto fut = t->pool->Enqueue([impl, keys, n_keys] {
      impl->preprocess(reinterpret_cast<hetuCTR::index_t *>(const_cast<int64_t *>(keys)), n_keys);
    });
    w = new hctr_wait{std::move(fut)};
  });
  return w;
}

hctr_wait *hctr_table_push_pull_async(hctr_table *t, const float *grad, float *dst) {
  hctr_wait *w = nullptr;
  guarded([&] {
    if (!t->pool) t->pool = std::make_unique<hetuCTR::ThreadPool>(1);
    HetuTable *impl = t->impl.get();
    auto fut = t->pool->Enqueue([impl, grad, dst] { impl->pushPull(const_cast<float *>(grad), dst); });
    w = new hctr_wait{std::move(fut)};
  });
  return w;
}

int hctr_wait_finish(hctr_wait *w) {
  if (!w) return -1;
  int rc = guarded([&] { w->fut.get(); });
  delete w;
  return rc;
}

int hctr_table_repr(hctr_table *t, int full, char *buf, size_t buf_len) {
  std::string s = full ? t->impl->debugStringFull() : t->impl->debugString();
  if (buf && buf_len) {
    std::strncpy(buf, s.c_str(), buf_len - 1);
    buf[buf_len - 1] = 0;
  }
  return (int)s.size();
}

long long hctr_table_dump(hctr_table *t, const char *what, int prev, void *out) {
  long long n = -1;
  guarded([&] { n = t->impl->dump(what, prev != 0, out); });
  return n;
}

int hctr_table_set_embedding(hctr_table *t, const float *rows) {
  return guarded([&] { t->impl->setEmbedding(rows); });
}

int hctr_table_export(hctr_table *t, const char *path) {
  return guarded([&] { t->impl->exportState(path); });
}

int hctr_table_import(hctr_table *t, const char *path) {
  return guarded([&] { t->impl->importState(path); });
}

int hctr_table_stats(hctr_table *t, long long out[13]) {
  const hetuCTR::StepStats &s = t->impl->stats();
  out[0] = (long long)s.batch;
  out[1] = (long long)s.unique;
  out[2] = (long long)s.prev_batch;
  out[3] = (long long)s.prev_unique;
  out[4] = (long long)s.pushed_rows;
  out[5] = (long long)s.received_push_rows;
  out[6] = (long long)s.queried_keys;
  out[7] = (long long)s.returned_rows;
  out[8] = (long long)s.received_rows;
  out[9] = (long long)t->impl->kStorageMax;
  out[10] = (long long)t->impl->kNonLocalStorageMax;
  out[11] = (long long)s.wait_queries_us;
  out[12] = (long long)s.wait_returns_us;
  return 0;
}

int hctr_table_profile(hctr_table *t, int enable) {
  t->impl->setProfile(enable);
  return 0;
}

int hctr_table_phase_times(hctr_table *t, double ms[HCTR_N_PHASES], long long calls[HCTR_N_PHASES], int reset) {
  static_assert(HCTR_N_PHASES == hetuCTR::kPhCount, "phase list out of sync");
  t->impl->phaseTimes(ms, calls, reset != 0);
  return 0;
}

int hctr_table_timeline(hctr_table *t, double *out, int max_spans) {
  return (int)t->impl->timeline(out, max_spans > 0 ? (size_t)max_spans : 0);
}

int hctr_rendezvous_broadcast(int rank, int nrank, const char *ip, int port, void *data, size_t len,
                              double timeout_s) {
  return guarded([&] {
    hetuCTR::TCPRendezvous tcp(rank, nrank, ip ? ip : "", port, timeout_s);
    tcp.broadcast(data, len);
  });
}

const char *hctr_table_exchange_name(hctr_table *t) { return t->impl->exchangeName(); }

void *hctr_table_stream(hctr_table *t) { return (void *)t->impl->stream(); }

}  // extern "C"
