// Dataset index builders (C ABI, loaded with ctypes).
//
// sample index  : packs documents (visited in `doc_idx` order) into samples of seq_length+1 tokens; consecutive
//                 samples share one token (the label of the last position is the first input of the next sample).
//                 Row i of the result is (position in doc_idx, token offset inside that document) where sample i
//                 starts; row num_samples closes the last sample.
// blending index: interleaves several datasets so that after every prefix the realised mixture is as close as
//                 possible to the requested weights (greedy largest-deficit choice).
// These match the index formats of the reference's pybind module (savanna/data/helpers.cpp:34-260), so index
// caches written by either side are interchangeable.
#include <algorithm>
#include <cstdint>
#include <cstring>

namespace {

template <typename IdxT>
int build_sample_idx_impl(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int32_t seq_length,
                          int64_t num_samples, IdxT* out /* [(num_samples+1) * 2] */) {
  int64_t pos = 0;        // position in doc_idx
  IdxT offset = 0;        // token offset inside the current document
  out[0] = 0;
  out[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int64_t need = static_cast<int64_t>(seq_length) + 1;
    while (need > 0) {
      if (pos >= doc_idx_len) return -1;                         // ran out of documents
      const int64_t avail = static_cast<int64_t>(sizes[doc_idx[pos]]) - offset;
      if (avail >= need) {
        // the sample ends inside this document; the next one starts on its last token
        offset += static_cast<IdxT>(need - 1);
        need = 0;
      } else {
        need -= avail;
        ++pos;
        offset = 0;
      }
    }
    out[2 * s] = static_cast<IdxT>(pos);
    out[2 * s + 1] = offset;
  }
  return 0;
}

}  // namespace

extern "C" {

int sbd_build_sample_idx_int32(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int32_t seq_length,
                               int64_t num_samples, int32_t* out) {
  return build_sample_idx_impl<int32_t>(sizes, doc_idx, doc_idx_len, seq_length, num_samples, out);
}

int sbd_build_sample_idx_int64(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int32_t seq_length,
                               int64_t num_samples, int64_t* out) {
  return build_sample_idx_impl<int64_t>(sizes, doc_idx, doc_idx_len, seq_length, num_samples, out);
}

// dataset_index[i] in [0, num_datasets), dataset_sample_index[i] = how many samples of that dataset precede i
int sbd_build_blending_indices(uint8_t* dataset_index, int64_t* dataset_sample_index, const double* weights,
                               int32_t num_datasets, int64_t size) {
  if (num_datasets <= 0 || num_datasets > 255) return -1;
  int64_t counts[256];
  std::memset(counts, 0, sizeof(counts));
  for (int64_t i = 0; i < size; ++i) {
    const double denom = static_cast<double>(i < 1 ? 1 : i);
    int32_t best = 0;
    double best_err = weights[0] * denom - static_cast<double>(counts[0]);
    for (int32_t d = 1; d < num_datasets; ++d) {
      const double err = weights[d] * denom - static_cast<double>(counts[d]);
      if (err > best_err) { best_err = err; best = d; }
    }
    dataset_index[i] = static_cast<uint8_t>(best);
    dataset_sample_index[i] = counts[best];
    ++counts[best];
  }
  return 0;
}

// Sentence-window map for masked-LM style datasets: for every document, consecutive sentences are grouped
// into samples of at most max_seq_length tokens (short samples with probability short_seq_prob, from a
// counter-based hash so the result is deterministic in `seed`).  Rows: (first sentence, one-past-last sentence,
// target length).  Two passes: count (maps == nullptr) then fill.
static inline uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull; x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull; x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

int64_t sbd_build_mapping(const int64_t* docs, int64_t num_docs_plus1, const int32_t* sizes, int32_t num_epochs,
                          int64_t max_num_samples, int32_t max_seq_length, double short_seq_prob, int32_t seed,
                          int32_t min_num_sent, int64_t* maps /* [n * 3] or nullptr */) {
  int64_t n = 0;
  uint64_t ctr = static_cast<uint64_t>(seed) << 32;
  for (int32_t epoch = 0; epoch < num_epochs && n < max_num_samples; ++epoch) {
    for (int64_t d = 0; d + 1 < num_docs_plus1 && n < max_num_samples; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      if (last - first < min_num_sent) continue;
      int64_t start = first;
      int32_t len = 0, nsent = 0;
      const uint64_t r0 = mix64(ctr++);
      int32_t target = max_seq_length;
      if ((r0 & 0xFFFFFF) < static_cast<uint64_t>(short_seq_prob * 0x1000000)) target = 2 + static_cast<int32_t>((r0 >> 24) % (max_seq_length - 1));
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++nsent;
        const bool last_sent = (s + 1 == last);
        if ((len >= target && nsent >= min_num_sent && last - s - 1 >= min_num_sent) || last_sent) {
          if (nsent >= min_num_sent) {
            if (maps) { maps[3 * n] = start; maps[3 * n + 1] = s + 1; maps[3 * n + 2] = target; }
            ++n;
            if (n >= max_num_samples) break;
          }
          start = s + 1; len = 0; nsent = 0;
          const uint64_t r = mix64(ctr++);
          target = max_seq_length;
          if ((r & 0xFFFFFF) < static_cast<uint64_t>(short_seq_prob * 0x1000000)) target = 2 + static_cast<int32_t>((r >> 24) % (max_seq_length - 1));
        }
      }
    }
  }
  return n;
}

// Block mapping for retrieval-style datasets (role of the reference's helpers.cpp build_blocks_mapping): every document
// (a run of sentences docs[d] .. docs[d+1]) is cut into blocks of whole sentences whose token count reaches
// max_seq_length minus the document's title length; a block is closed early enough that the rest of the document can
// still form a block of `min_num_sent` sentences.  Documents with fewer than `min_num_sent` sentences, and documents
// that hold a sentence longer than `long_sentence_len` tokens, are skipped.  Rows are (first sentence, one past the
// last sentence, document, block id), block ids counting up over the whole pass.  With `maps` the rows are written and
// then shuffled with a seeded Fisher-Yates pass; without it only the row count is returned.
int64_t sbd_build_blocks_mapping(const int64_t* docs, int64_t num_docs_plus1, const int32_t* sizes, const int32_t* title_sizes,
                                 int32_t num_epochs, int64_t max_num_samples, int32_t max_seq_length, int32_t seed,
                                 int32_t min_num_sent, int32_t long_sentence_len, int64_t* maps /* [n * 4] or nullptr */) {
  int64_t n = 0;
  for (int32_t epoch = 0; epoch < num_epochs && n < max_num_samples; ++epoch) {
    int64_t block_id = 0;
    for (int64_t d = 0; d + 1 < num_docs_plus1 && n < max_num_samples; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      if (last - first < min_num_sent) continue;
      bool too_long = false;
      for (int64_t s = first; s < last; ++s) too_long |= sizes[s] > long_sentence_len;
      if (too_long) continue;
      const int32_t target = max_seq_length - title_sizes[d];
      int64_t start = first;
      int32_t len = 0, nsent = 0;
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++nsent;
        const int64_t remain = last - s - 1;
        if ((len >= target && remain >= min_num_sent && nsent >= min_num_sent) || remain == 0) {
          if (maps) { maps[4 * n] = start; maps[4 * n + 1] = s + 1; maps[4 * n + 2] = d; maps[4 * n + 3] = block_id; }
          ++n; ++block_id;
          if (n >= max_num_samples) break;
          start = s + 1; len = 0; nsent = 0;
        }
      }
    }
  }
  if (maps) {
    uint64_t ctr = (static_cast<uint64_t>(seed) << 32) + 1;
    for (int64_t i = n - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(mix64(ctr++) % static_cast<uint64_t>(i + 1));
      for (int k = 0; k < 4; ++k) { const int64_t t = maps[4 * i + k]; maps[4 * i + k] = maps[4 * j + k]; maps[4 * j + k] = t; }
    }
  }
  return n;
}

}  // extern "C"
