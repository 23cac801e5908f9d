// Host-side index builders for the memory-mapped pretraining datasets, exported with C linkage for ctypes.
//
// These loops run once per dataset over up to billions of tokens, which is why the reference delegates them to a
// compiled helper (`fast_dataindex`, requirements.txt:12; used from paddleformers/data/causal_dataset.py:523-700).
//
//   pfb_build_sample_index   where every fixed-length training sample starts in the shuffled document stream
//   pfb_build_blend_index    deterministic weighted interleaving of several datasets (largest-deficit rule)
//   pfb_build_doc_bounds     per-token document end rows and restarting position ids of one packed sample
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// sizes[doc]: tokens of each document; doc_order[n_order]: the (shuffled, epoch-tiled) document stream.
// Writes (position in doc_order, token offset) for samples 0 .. n (n + 1 rows) and returns n, the number of complete
// samples of seq_length + 1 tokens with stride seq_length, capped by num_samples.
int64_t pfb_build_sample_index(const int32_t* sizes, const int64_t* doc_order, int64_t n_order, int64_t seq_length,
                               int64_t num_samples, int64_t* out /* [(num_samples + 1) * 2] */) {
  if (seq_length <= 0 || n_order <= 0) return 0;
  int64_t total = 0;
  for (int64_t i = 0; i < n_order; ++i) total += sizes[doc_order[i]];
  const int64_t max_samples = (total - 1) / seq_length;
  const int64_t n = num_samples < max_samples ? num_samples : max_samples;
  int64_t pos = 0;        // index into doc_order
  int64_t doc_start = 0;  // token offset of document `pos` in the stream
  for (int64_t k = 0; k <= n; ++k) {
    const int64_t start = k * seq_length;
    while (pos + 1 < n_order && doc_start + sizes[doc_order[pos]] <= start) {
      doc_start += sizes[doc_order[pos]];
      ++pos;
    }
    out[2 * k] = pos;
    out[2 * k + 1] = start - doc_start;
  }
  return n;
}

// Greedy largest-deficit interleaving: at step i pick the dataset d maximising weights[d] * (i + 1) - counts[d]
// (first maximum on ties), so that every prefix is as close to the target mixture as possible.
void pfb_build_blend_index(const double* weights, int32_t n_datasets, int64_t size, int32_t* dataset_index,
                           int64_t* sample_index) {
  std::vector<int64_t> counts(n_datasets, 0);
  for (int64_t i = 0; i < size; ++i) {
    int32_t best = 0;
    double best_deficit = weights[0] * static_cast<double>(i + 1) - static_cast<double>(counts[0]);
    for (int32_t d = 1; d < n_datasets; ++d) {
      const double deficit = weights[d] * static_cast<double>(i + 1) - static_cast<double>(counts[d]);
      if (deficit > best_deficit) { best_deficit = deficit; best = d; }
    }
    dataset_index[i] = best;
    sample_index[i] = counts[best]++;
  }
}

// ids[S]: tokens of one packed sample. A document ends after every eos token. Writes kend[j] = end row of the
// document that holds position j (the FlashMask start row of key column j) and pos[j] = position inside it.
void pfb_build_doc_bounds(const int64_t* ids, int64_t S, int64_t eos, int32_t* kend, int64_t* pos) {
  int64_t lo = 0;
  for (int64_t j = 0; j < S; ++j) {
    pos[j] = j - lo;
    if (ids[j] == eos || j == S - 1) {
      for (int64_t q = lo; q <= j; ++q) kend[q] = static_cast<int32_t>(j + 1);
      lo = j + 1;
    }
  }
}

}  // extern "C"
