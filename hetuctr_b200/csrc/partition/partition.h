// Offline sample/embedding co-partitioner (CPU): assigns every sample to a rank and every embedding
// row to an owner so that the expected per-batch communication is small, and scores which non-owned
// rows each rank should cache.  Same role, scoring formulas and Python interface as the reference's
// hetuCTR_partition module (csrc/partition/partition.{h,cc}); written from scratch, deterministic
// (explicit seed, sequential sweeps) where the reference uses unseeded rand() and racy OpenMP loops.
#pragma once
#include <cstdint>
#include <vector>

namespace hetuCTR {

class Partitioner {
 public:
  // data: [n_data, n_slot] embedding ids of every sample; comm: [n_part, n_part] relative cost of moving a
  // row from owner j to requester i; batch_size: global batch size the job will use.
  Partitioner(const int *data, int n_data, int n_slot, const float *comm, int n_part, int batch_size, uint64_t seed);

  // One sweep over all samples / all embeddings: each item moves to its best-scoring part, moves take
  // effect immediately (csrc/partition/partition.cc:94-166 evaluated sequentially).
  void refineData();
  void refineEmbed();

  // [n_part * n_part]: expected rows per batch that requester i fetches from owner j (partition.cc:168-180)
  std::vector<float> communication() const;
  // [n_part * n_embed]: caching priority of row j on rank i (partition.cc:182-193)
  std::vector<float> priority() const;

  // replace the current assignment (e.g. to continue from a saved partition); counts are rebuilt
  void setResult(const int *data_part, const int *embed_part);

  int nPart() const { return n_part_; }
  int nData() const { return n_data_; }
  int nEmbed() const { return n_embed_; }
  std::vector<int> res_data_, res_embed_;
  std::vector<int> cnt_data_, cnt_embed_;

 private:
  void rebuildCounts();
  int n_part_, n_data_, n_slot_, n_embed_, batch_size_;
  float alpha_, beta_;
  std::vector<int> data_indices_;                 // [n_data * n_slot]
  std::vector<int> degree_;                       // occurrences of every embedding over all samples
  std::vector<float> soft_cnt_;                   // expected distinct-batch hits for k occurrences
  std::vector<float> comm_;                       // [n_part * n_part]
  std::vector<int> cnt_part_embed_;               // [n_embed * n_part] occurrences of row j in part i's samples, part-minor
  std::vector<float> embed_weight_;
};

}  // namespace hetuCTR
