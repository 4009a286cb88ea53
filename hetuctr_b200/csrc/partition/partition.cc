#include "partition/partition.h"

#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace hetuCTR {

namespace {

// a^n by repeated squaring in single precision (same operation order as the reference's quickpow,
// csrc/partition/partition.cc:7-15, so the soft counts come out bit-identical)
float pow_by_squaring(float a, int n) {
  float ans = 1, t = a;
  while (n) {
    if (n & 1) ans *= t;
    n >>= 1;
    t *= t;
  }
  return ans;
}

int first_argmax(const std::vector<float> &v) {
  int best = 0;
  for (int i = 1; i < (int)v.size(); i++)
    if (v[i] > v[best]) best = i;
  return best;
}

// splitmix64: the assignment only needs to be uniform and reproducible
// i-th value (i = 1, 2, ...) of the splitmix64 stream started at `seed`: the stream's state is seed + i * gamma, so
// any element can be computed on its own
uint64_t splitmix_at(uint64_t seed, uint64_t i) {
  uint64_t z = seed + i * 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

}  // namespace

Partitioner::Partitioner(const int *data, int n_data, int n_slot, const float *comm, int n_part, int batch_size,
                         uint64_t seed)
    : n_part_(n_part), n_data_(n_data), n_slot_(n_slot), batch_size_(batch_size) {
  if (n_part < 1 || n_data < n_part || n_slot < 1 || batch_size < 1)
    throw std::runtime_error("partition: need n_part >= 1, n_data >= n_part, n_slot >= 1, batch_size >= 1");
  const size_t n_edge = (size_t)n_data * n_slot;
  int lowest = 0, highest = 0;
#pragma omp parallel for reduction(min : lowest) reduction(max : highest) schedule(static)
  for (long long i = 0; i < (long long)n_edge; i++) {
    lowest = std::min(lowest, data[i]);
    highest = std::max(highest, data[i]);
  }
  if (lowest < 0) throw std::runtime_error("partition: negative embedding id");
  n_embed_ = highest + 1;
  data_indices_.assign(data, data + n_edge);
  // occurrences of every embedding over all samples (the reference keeps a CSR of embedding -> samples,
  // csrc/partition/partition.cc:35-56; only its row lengths and per-part counts are ever needed, and the
  // latter are maintained incrementally in cnt_part_embed_)
  degree_.assign(n_embed_, 0);
  // (integer counts: the parallel loops below give the same result in any order)
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n_edge; i++) {
#pragma omp atomic
    degree_[data[i]]++;
  }

  // soft_cnt[k]: expected number of batches (scaled) in which a row with k occurrences among a part's
  // samples is needed: 1 - (1 - k/max)^batch, times max/batch; 1 beyond max (partition.cc:58-64)
  const int mx = n_data_ / n_part_;
  soft_cnt_.assign((size_t)n_data_ + 2, 1.0f);
  for (int i = 0; i < mx; i++) {
    float v = 1 - pow_by_squaring((float)(1.0 - (double)((float)i / (float)mx)), batch_size_);
    v *= (float)mx / (float)batch_size_;
    soft_cnt_[i] = v;
  }
  // balance weights (partition.cc:86-87)
  alpha_ = (float)(-100.0 / (n_data_ / n_part_));
  beta_ = (float)(-100.0 / std::max(n_embed_ / n_part_, 1));
  comm_.assign(comm, comm + (size_t)n_part * n_part);

  res_data_.resize(n_data_);
  res_embed_.resize(n_embed_);
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < n_data_; i++) res_data_[i] = (int)(splitmix_at(seed, (uint64_t)i + 1) % (uint64_t)n_part_);
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < n_embed_; i++)
    res_embed_[i] = (int)(splitmix_at(seed, (uint64_t)n_data_ + (uint64_t)i + 1) % (uint64_t)n_part_);
  rebuildCounts();
}

void Partitioner::rebuildCounts() {
  cnt_data_.assign(n_part_, 0);
  cnt_embed_.assign(n_part_, 0);
  cnt_part_embed_.assign((size_t)n_part_ * n_embed_, 0);
  for (int i = 0; i < n_data_; i++) cnt_data_[res_data_[i]]++;
  for (int e = 0; e < n_embed_; e++) cnt_embed_[res_embed_[e]]++;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < n_data_; i++) {
    const int p = res_data_[i];
    for (int j = 0; j < n_slot_; j++) {
#pragma omp atomic
      cnt_part_embed_[(size_t)data_indices_[(size_t)i * n_slot_ + j] * n_part_ + p]++;
    }
  }
}

void Partitioner::setResult(const int *data_part, const int *embed_part) {
  for (int i = 0; i < n_data_; i++)
    if (data_part[i] < 0 || data_part[i] >= n_part_) throw std::runtime_error("partition: part id out of range");
  for (int i = 0; i < n_embed_; i++)
    if (embed_part[i] < 0 || embed_part[i] >= n_part_) throw std::runtime_error("partition: part id out of range");
  res_data_.assign(data_part, data_part + n_data_);
  res_embed_.assign(embed_part, embed_part + n_embed_);
  rebuildCounts();
}

// csrc/partition/partition.cc:94-123.  score[k] = balance term - expected extra fetches if the sample joined
// part k: every row it uses costs (soft[c+1] - soft[c]) * comm[k][owner] where c is the row's occurrence
// count in part k without this sample.
void Partitioner::refineData() {
  constexpr int kAhead = 6;
  std::vector<float> score(n_part_);
  for (int i = 0; i < n_data_; i++) {
    const int old = res_data_[i];
    for (int j = 0; j < n_part_; j++) {
      const int c = old == j ? cnt_data_[j] - 1 : cnt_data_[j];
      score[j] = alpha_ * c;
    }
    const int *row = &data_indices_[(size_t)i * n_slot_];
    // the sweep is a chain of cache misses (two per slot); ask for the lines of a later sample now
    if (i + kAhead < n_data_) {
      const int *later = &data_indices_[(size_t)(i + kAhead) * n_slot_];
      for (int j = 0; j < n_slot_; j++) {
        __builtin_prefetch(&res_embed_[later[j]], 0, 1);
        __builtin_prefetch(&cnt_part_embed_[(size_t)later[j] * n_part_], 1, 1);
      }
    }
    for (int j = 0; j < n_slot_; j++) {
      const int e = row[j];
      const int owner = res_embed_[e];
      for (int k = 0; k < n_part_; k++) {
        int use = cnt_part_embed_[(size_t)e * n_part_ + k];
        if (k == old) use--;
        score[k] -= (soft_cnt_[use + 1] - soft_cnt_[use]) * comm_[(size_t)k * n_part_ + owner];
      }
    }
    const int s = first_argmax(score);
    if (s != old) {
      cnt_data_[old]--;
      cnt_data_[s]++;
      for (int j = 0; j < n_slot_; j++) {
        cnt_part_embed_[(size_t)row[j] * n_part_ + s]++;
        cnt_part_embed_[(size_t)row[j] * n_part_ + old]--;
      }
      res_data_[i] = s;
    }
  }
}

// csrc/partition/partition.cc:125-166.  score[k] = balance term - fetch cost of all requesters if the row
// lived on k - a small penalty on parts that already serve a lot of traffic.
void Partitioner::refineEmbed() {
  embed_weight_.assign(n_part_, 0.f);
  for (int i = 0; i < n_part_; i++)
    for (int j = 0; j < n_embed_; j++)
      if (res_embed_[j] != i) embed_weight_[res_embed_[j]] += soft_cnt_[cnt_part_embed_[(size_t)j * n_part_ + i]];
  const float scale = float(batch_size_ * n_part_) / n_data_;
  for (int i = 0; i < n_part_; i++) embed_weight_[i] *= scale;

  std::vector<float> score(n_part_), cnt(n_part_);
  for (int i = 0; i < n_embed_; i++) {
    const int old = res_embed_[i];
    // samples of every part that use row i (the reference recounts them from its CSR; the running counts
    // hold the same numbers because refine_embed moves no sample)
    for (int j = 0; j < n_part_; j++) cnt[j] = (float)cnt_part_embed_[(size_t)i * n_part_ + j];
    for (int j = 0; j < n_part_; j++) {
      const int c = old == j ? cnt_embed_[j] - 1 : cnt_embed_[j];
      score[j] = beta_ * c;
    }
    const int deg = degree_[i];
    for (int j = 0; j < n_part_; j++) {
      const float need = soft_cnt_[(size_t)cnt[j]];
      for (int k = 0; k < n_part_; k++) score[k] -= comm_[(size_t)j * n_part_ + k] * need;
      // evaluated in double precision, like the reference's literal 0.01
      score[j] = (float)((double)score[j] - 0.01 * (double)embed_weight_[j] * (double)soft_cnt_[deg]);
    }
    const int s = first_argmax(score);
    if (s != old) {
      cnt_embed_[old]--;
      cnt_embed_[s]++;
      res_embed_[i] = s;
      for (int j = 0; j < n_part_; j++) {
        const float w = soft_cnt_[cnt_part_embed_[(size_t)i * n_part_ + j]] * (batch_size_ * n_part_) / n_data_;
        if (j != s) embed_weight_[s] += w;
        if (j != old) embed_weight_[old] -= w;
      }
    }
  }
}

std::vector<float> Partitioner::communication() const {
  std::vector<float> cost((size_t)n_part_ * n_part_, 0.f);
  for (int i = 0; i < n_part_; i++)
    for (int j = 0; j < n_embed_; j++)
      cost[(size_t)i * n_part_ + res_embed_[j]] += soft_cnt_[cnt_part_embed_[(size_t)j * n_part_ + i]];
  const float scale = float(batch_size_ * n_part_) / n_data_;
  for (float &c : cost) c *= scale;
  return cost;
}

std::vector<float> Partitioner::priority() const {
  std::vector<float> pr((size_t)n_part_ * n_embed_, 0.f);
  for (int i = 0; i < n_part_; i++)
    for (int j = 0; j < n_embed_; j++) {
      const int c = cnt_part_embed_[(size_t)j * n_part_ + i];
      if (c == 0) continue;
      const double soft = soft_cnt_[c];
      const int deg = degree_[j];
      pr[(size_t)i * n_embed_ + j] =
          (float)(comm_[(size_t)i * n_part_ + res_embed_[j]] * (soft * soft) * ((1.0 / deg) + (1.0 / c)));
    }
  return pr;
}

}  // namespace hetuCTR
