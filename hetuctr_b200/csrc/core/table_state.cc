// Export / import of a table's learned state: stored keys (for identification), rows, versions and, for cached
// rows, the pending gradient and pending-update counts.  The reference has no checkpoint of any kind; the file
// layout is this library's own:
//   header (Header below) | keys i64[S] | version i64[S] | embedding f32[S*W] | updates i64[C] | gradient f32[C*W]
//   | u64 checksum (FNV-1a over everything before it)
// Data moves through one pinned staging buffer, so exporting a table far larger than host memory works.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>

#include <unistd.h>

#include "core/hetu_table.h"
#include "utils/errors.h"

namespace hetuCTR {

namespace {

struct Header {
  char magic[8];  // "HCTRTBL1"
  uint32_t width, rank, nrank, reserved;
  int64_t length, stored, cached, pull_bound, push_bound;
};

constexpr size_t kChunk = 32u << 20;

struct File {
  FILE *f = nullptr;
  uint64_t hash = 1469598103934665603ull;
  std::string path;
  File(const std::string &p, const char *mode) : f(std::fopen(p.c_str(), mode)), path(p) {
    if (!f) throw std::runtime_error("cannot open " + p);
  }
  ~File() {
    if (f) std::fclose(f);
  }
  void mix(const void *data, size_t n) {
    // FNV-1a over 8-byte words (the sections are all multiples of 4 bytes; a tail is mixed bytewise)
    const unsigned char *b = static_cast<const unsigned char *>(data);
    size_t i = 0;
    for (; i + 8 <= n; i += 8) {
      uint64_t w;
      std::memcpy(&w, b + i, 8);
      hash = (hash ^ w) * 1099511628211ull;
    }
    for (; i < n; i++) hash = (hash ^ b[i]) * 1099511628211ull;
  }
  void write(const void *data, size_t n) {
    if (n && std::fwrite(data, 1, n, f) != n) throw std::runtime_error("short write to " + path);
    mix(data, n);
  }
  void read(void *data, size_t n) {
    if (n && std::fread(data, 1, n, f) != n) throw std::runtime_error(path + " is truncated");
    mix(data, n);
  }
};

struct Pinned {
  void *p = nullptr;
  Pinned() { HCTR_CUDA(cudaMallocHost(&p, kChunk)); }
  ~Pinned() { cudaFreeHost(p); }
};

}  // namespace

void HetuTable::quiesce() {
  HCTR_CUDA(cudaSetDevice(device_id_));
  finalizePending();
  flushOrdering(cur_batch_);
  // whoever looks at a batch's position lists expects every run in ascending order
  for (BatchDesc *b : {&cur_batch_, &prev_batch_})
    if (b->batch_size > 0) orderLightRuns(*b, stream_side_);
  for (cudaStream_t s : {stream_main_, stream_side_, stream_reduce_, stream_reduce_side_})
    if (s) HCTR_CUDA(cudaStreamSynchronize(s));
}

void HetuTable::exportState(const std::string &path) {
  quiesce();
  const size_t S = kStorageMax, C = kNonLocalStorageMax, W = kEmbeddingWidth;
  Header h{};
  std::memcpy(h.magic, "HCTRTBL1", 8);
  h.width = (uint32_t)W;
  h.rank = (uint32_t)rank_;
  h.nrank = (uint32_t)nrank_;
  h.length = (int64_t)kEmbeddingIDMax;
  h.stored = (int64_t)S;
  h.cached = (int64_t)C;
  h.pull_bound = pull_bound_;
  h.push_bound = push_bound_;
  // Written beside the target and renamed over it at the end: a crash or a full disk half-way leaves the previous
  // file of that name intact instead of a truncated one.
  const std::string tmp = path + ".tmp";
  File out(tmp, "wb");
  out.write(&h, sizeof(h));
  Pinned stage;
  auto section = [&](const void *dev, size_t bytes) {
    for (size_t off = 0; off < bytes; off += kChunk) {
      const size_t n = std::min(kChunk, bytes - off);
      HCTR_CUDA(cudaMemcpyAsync(stage.p, static_cast<const char *>(dev) + off, n, cudaMemcpyDeviceToHost, stream_main_));
      HCTR_CUDA(cudaStreamSynchronize(stream_main_));
      out.write(stage.p, n);
    }
  };
  section(d_stored_keys_.p, S * sizeof(index_t));
  section(d_version_.p, S * sizeof(version_t));
  section(d_embedding_.p, S * W * sizeof(embed_t));
  section(d_updates_.p, C * sizeof(version_t));
  section(d_gradient_.p, C * W * sizeof(embed_t));
  const uint64_t sum = out.hash;
  if (std::fwrite(&sum, 1, sizeof(sum), out.f) != sizeof(sum) || std::fflush(out.f) != 0 || fsync(fileno(out.f)) != 0)
    throw std::runtime_error("short write to " + tmp);
  std::fclose(out.f);
  out.f = nullptr;
  if (std::rename(tmp.c_str(), path.c_str()) != 0) throw std::runtime_error("cannot rename " + tmp + " to " + path);
}

void HetuTable::importState(const std::string &path) {
  if (batch_open_)
    throw std::runtime_error("import: a batch is between preprocess and push_pull; finish the step first");
  quiesce();
  const size_t S = kStorageMax, C = kNonLocalStorageMax, W = kEmbeddingWidth;
  File in(path, "rb");
  Header h{};
  in.read(&h, sizeof(h));
  if (std::memcmp(h.magic, "HCTRTBL1", 8) != 0) throw std::runtime_error(path + " is not a table state file");
  if (h.width != W || h.length != (int64_t)kEmbeddingIDMax || h.stored != (int64_t)S || h.cached != (int64_t)C ||
      h.rank != (uint32_t)rank_ || h.nrank != (uint32_t)nrank_)
    throw std::runtime_error(path + " was exported from a table of another shape (rank, nrank, length, width, stored or cached rows differ)");
  Pinned stage;
  // pass 1: the whole file must be intact and list exactly this table's keys before any row is overwritten
  {
    std::unique_ptr<char[]> mine(new char[kChunk]);
    const size_t key_bytes = S * sizeof(index_t);
    for (size_t off = 0; off < key_bytes; off += kChunk) {
      const size_t n = std::min(kChunk, key_bytes - off);
      in.read(stage.p, n);
      HCTR_CUDA(cudaMemcpy(mine.get(), static_cast<const char *>(d_stored_keys_.p) + off, n, cudaMemcpyDeviceToHost));
      if (std::memcmp(mine.get(), stage.p, n) != 0)
        throw std::runtime_error(path + " holds other keys than this table stores (storage_arr differs)");
    }
    size_t rest = S * sizeof(version_t) + S * W * sizeof(embed_t) + C * sizeof(version_t) + C * W * sizeof(embed_t);
    for (; rest; rest -= std::min(kChunk, rest)) in.read(stage.p, std::min(kChunk, rest));
    uint64_t sum = 0;
    const uint64_t want = in.hash;
    if (std::fread(&sum, 1, sizeof(sum), in.f) != sizeof(sum)) throw std::runtime_error(path + " is truncated");
    if (sum != want) throw std::runtime_error(path + " is corrupt (checksum mismatch)");
  }
  // pass 2: load
  if (std::fseek(in.f, (long)(sizeof(Header) + S * sizeof(index_t)), SEEK_SET) != 0)
    throw std::runtime_error("cannot seek in " + path);
  auto section = [&](void *dev, size_t bytes) {
    for (size_t off = 0; off < bytes; off += kChunk) {
      const size_t n = std::min(kChunk, bytes - off);
      in.read(stage.p, n);
      HCTR_CUDA(cudaMemcpyAsync(static_cast<char *>(dev) + off, stage.p, n, cudaMemcpyHostToDevice, stream_main_));
      HCTR_CUDA(cudaStreamSynchronize(stream_main_));
    }
  };
  section(d_version_.p, S * sizeof(version_t));
  section(d_embedding_.p, S * W * sizeof(embed_t));
  section(d_updates_.p, C * sizeof(version_t));
  section(d_gradient_.p, C * W * sizeof(embed_t));
  // the batches preprocessed before the import belong to the old state: their gradients are not pushed
  for (BatchDesc *b : {&cur_batch_, &prev_batch_}) {
    b->batch_size = 0;
    b->unique_size = 0;
    b->n_heavy = 0;
    b->decided = false;
    std::fill(b->seg.begin(), b->seg.end(), 0);
    for (auto *v : {&b->query_send, &b->query_recv, &b->push_send, &b->push_recv, &b->ret_send, &b->ret_recv})
      std::fill(v->begin(), v->end(), 0);
  }
  prev_push_valid_ = false;
}

}  // namespace hetuCTR
