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
uint64_t next_u64(uint64_t &s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
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
  n_embed_ = 0;
  for (size_t i = 0; i < n_edge; i++) {
    if (data[i] < 0) throw std::runtime_error("partition: negative embedding id");
    n_embed_ = std::max(n_embed_, data[i]);
  }
  n_embed_++;
  data_indices_.assign(data, data + n_edge);
  // CSR of embedding -> samples (sample ids ascending inside a row)
  embed_indptr_.assign(n_embed_ + 1, 0);
  for (size_t i = 0; i < n_edge; i++) embed_indptr_[data[i] + 1]++;
  for (int e = 0; e < n_embed_; e++) embed_indptr_[e + 1] += embed_indptr_[e];
  embed_indices_.resize(n_edge);
  std::vector<int> fill(embed_indptr_.begin(), embed_indptr_.end() - 1);
  for (size_t i = 0; i < n_edge; i++) embed_indices_[fill[data[i]]++] = (int)(i / n_slot);

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
  uint64_t s = seed;
  for (int i = 0; i < n_data_; i++) res_data_[i] = (int)(next_u64(s) % (uint64_t)n_part_);
  for (int i = 0; i < n_embed_; i++) res_embed_[i] = (int)(next_u64(s) % (uint64_t)n_part_);
  rebuildCounts();
}

void Partitioner::rebuildCounts() {
  cnt_data_.assign(n_part_, 0);
  cnt_embed_.assign(n_part_, 0);
  cnt_part_embed_.assign((size_t)n_part_ * n_embed_, 0);
  for (int i = 0; i < n_data_; i++) {
    const int p = res_data_[i];
    cnt_data_[p]++;
    for (int j = 0; j < n_slot_; j++) cnt_part_embed_[(size_t)p * n_embed_ + data_indices_[(size_t)i * n_slot_ + j]]++;
  }
  for (int e = 0; e < n_embed_; e++) cnt_embed_[res_embed_[e]]++;
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
  std::vector<float> score(n_part_);
  for (int i = 0; i < n_data_; i++) {
    const int old = res_data_[i];
    for (int j = 0; j < n_part_; j++) {
      const int c = old == j ? cnt_data_[j] - 1 : cnt_data_[j];
      score[j] = alpha_ * c;
    }
    const int *row = &data_indices_[(size_t)i * n_slot_];
    for (int j = 0; j < n_slot_; j++) {
      const int e = row[j];
      const int owner = res_embed_[e];
      for (int k = 0; k < n_part_; k++) {
        int use = cnt_part_embed_[(size_t)k * n_embed_ + e];
        if (k == old) use--;
        score[k] -= (soft_cnt_[use + 1] - soft_cnt_[use]) * comm_[(size_t)k * n_part_ + owner];
      }
    }
    const int s = first_argmax(score);
    if (s != old) {
      cnt_data_[old]--;
      cnt_data_[s]++;
      for (int j = 0; j < n_slot_; j++) {
        cnt_part_embed_[(size_t)s * n_embed_ + row[j]]++;
        cnt_part_embed_[(size_t)old * n_embed_ + row[j]]--;
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
      if (res_embed_[j] != i) embed_weight_[res_embed_[j]] += soft_cnt_[cnt_part_embed_[(size_t)i * n_embed_ + j]];
  const float scale = float(batch_size_ * n_part_) / n_data_;
  for (int i = 0; i < n_part_; i++) embed_weight_[i] *= scale;

  std::vector<float> score(n_part_), cnt(n_part_);
  for (int i = 0; i < n_embed_; i++) {
    const int old = res_embed_[i];
    std::fill(cnt.begin(), cnt.end(), 0.f);
    for (int j = embed_indptr_[i]; j < embed_indptr_[i + 1]; j++) cnt[res_data_[embed_indices_[j]]]++;
    for (int j = 0; j < n_part_; j++) {
      const int c = old == j ? cnt_embed_[j] - 1 : cnt_embed_[j];
      score[j] = beta_ * c;
    }
    const int deg = embed_indptr_[i + 1] - embed_indptr_[i];
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
        const float w = soft_cnt_[cnt_part_embed_[(size_t)j * n_embed_ + i]] * (batch_size_ * n_part_) / n_data_;
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
      cost[(size_t)i * n_part_ + res_embed_[j]] += soft_cnt_[cnt_part_embed_[(size_t)i * n_embed_ + j]];
  const float scale = float(batch_size_ * n_part_) / n_data_;
  for (float &c : cost) c *= scale;
  return cost;
}

std::vector<float> Partitioner::priority() const {
  std::vector<float> pr((size_t)n_part_ * n_embed_, 0.f);
  for (int i = 0; i < n_part_; i++)
    for (int j = 0; j < n_embed_; j++) {
      const int c = cnt_part_embed_[(size_t)i * n_embed_ + j];
      if (c == 0) continue;
      const double soft = soft_cnt_[c];
      const int deg = embed_indptr_[j + 1] - embed_indptr_[j];
      pr[(size_t)i * n_embed_ + j] =
          (float)(comm_[(size_t)i * n_part_ + res_embed_[j]] * (soft * soft) * ((1.0 / deg) + (1.0 / c)));
    }
  return pr;
}

}  // namespace hetuCTR
