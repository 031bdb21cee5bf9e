// Host-side index builders for packed-token datasets (plain C ABI, no Python headers).
//
//  b200_build_sample_idx   where does training sample i start?  Documents are laid end to end in the order given
//                          by doc_idx; sample i covers tokens [i*seq_len, i*seq_len + seq_len] of that stream (one
//                          token of overlap for the shifted labels).  Output row i = (position in doc_idx, offset in
//                          that document).  Computed from a prefix sum of document lengths and a binary search per
//                          sample, split over threads - each sample is independent.
//  b200_build_blending_indices  interleave several datasets so that every prefix of the result follows the target
//                          weights as closely as possible (largest-deficit-first).
// Same results as the sequential builders of the reference's megatron data helpers
// (gpt-neox/megatron/data/helpers.cpp:34-171); used by aicomp_b200.utils.data_helpers.
#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

extern "C" long long b200_num_samples(int num_epochs, long long tokens_per_epoch, int seq_len) {
  if (seq_len <= 0) return -1;
  return (static_cast<long long>(num_epochs) * tokens_per_epoch - 1) / seq_len;
}

// sizes[n_docs], doc_idx[n_idx] (document ids, epochs already concatenated); out[(num_samples + 1) * 2] int64.
extern "C" int b200_build_sample_idx(const int32_t* sizes, long long n_docs, const int32_t* doc_idx, long long n_idx, int seq_len,
                                     long long num_samples, int64_t* out, int n_threads) {
  if (seq_len < 1 || n_idx <= 0 || num_samples < 0) return -1;
  std::vector<int64_t> start(static_cast<size_t>(n_idx) + 1, 0);  // start[j] = first stream position of doc_idx[j]
  for (long long j = 0; j < n_idx; ++j) {
    const int32_t d = doc_idx[j];
    if (d < 0 || d >= n_docs) return -2;
    start[j + 1] = start[j] + sizes[d];
  }
  const int64_t total = start[n_idx];
  if (num_samples * static_cast<int64_t>(seq_len) + 1 > total) return -3;  // the last sample would run off the stream
  if (n_threads < 1) n_threads = 1;
  auto work = [&](long long lo, long long hi) {
    for (long long i = lo; i < hi; ++i) {
      const int64_t pos = i * static_cast<int64_t>(seq_len);
      // last document whose first position is <= pos; empty documents are skipped by upper_bound
      const auto it = std::upper_bound(start.begin(), start.end() - 1, pos);
      const long long j = static_cast<long long>(it - start.begin()) - 1;
      out[2 * i] = j;
      out[2 * i + 1] = pos - start[j];
    }
  };
  const long long n = num_samples + 1;
  const long long per = (n + n_threads - 1) / n_threads;
  std::vector<std::thread> pool;
  for (int t = 0; t < n_threads; ++t) {
    const long long lo = t * per, hi = std::min(n, lo + per);
    if (lo < hi) pool.emplace_back(work, lo, hi);
  }
  for (auto& th : pool) th.join();
  return 0;
}

extern "C" int b200_build_blending_indices(uint8_t* dataset_index, int64_t* dataset_sample_index, const double* weights,
                                           int num_datasets, long long size) {
  if (num_datasets < 1 || num_datasets > 255) return -1;
  std::vector<int64_t> taken(num_datasets, 0);
  for (long long i = 0; i < size; ++i) {
    const double scale = i > 0 ? static_cast<double>(i) : 1.0;
    int pick = 0;
    double worst = weights[0] * scale - static_cast<double>(taken[0]);
    for (int d = 1; d < num_datasets; ++d) {
      const double deficit = weights[d] * scale - static_cast<double>(taken[d]);
      if (deficit > worst) { worst = deficit; pick = d; }
    }
    dataset_index[i] = static_cast<uint8_t>(pick);
    dataset_sample_index[i] = taken[pick]++;
  }
  return 0;
}
