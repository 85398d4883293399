// Native index builders for token datasets (CPU).
//
// build_location_idx: documents (token counts `sizes`, visited in the order `doc_idx`) are laid end
// to end into one token stream; sample i covers stream tokens [i*seq_length, (i+1)*seq_length] (one
// extra token so inputs and shifted labels both have seq_length entries).  For every sample boundary
// the function returns (index into doc_idx, offset inside that document) as int32 pairs, row 0 being
// (0, 0).  Same contract as the sample-index builder of the reference
// (llm/data/cores/helpers.cpp:36-122); the formulation here walks the boundaries with a running
// stream cursor instead of consuming a per-sample "remaining length", and is exported with a plain C
// ABI (ctypes + numpy buffers) so no Python headers are needed to build it.
//
// build_pack_index: greedy first-fit packing of variable-length samples into bins of `capacity`
// tokens (used by the packed variable-length synthetic / fine-tuning loaders).
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// Returns the number of samples written (num_samples + 1 rows), or -1 on inconsistent input.
// `out` must hold 2 * (num_samples + 1) int32 with num_samples = (num_epochs*tokens_per_epoch - 1) / seq_length.
int64_t ell_build_location_idx(const int32_t* sizes, int64_t n_sizes, const int32_t* doc_idx, int64_t n_docs,
                               int32_t seq_length, int32_t num_epochs, int64_t tokens_per_epoch, int32_t* out) {
  if (seq_length <= 1 || num_epochs <= 0 || tokens_per_epoch <= 1) return -1;
  const int64_t num_samples = (static_cast<int64_t>(num_epochs) * tokens_per_epoch - 1) / seq_length;
  int64_t doc_pos = 0;      // index into doc_idx of the document holding the cursor
  int64_t doc_begin = 0;    // stream position where that document starts
  out[0] = 0;
  out[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    // the boundary token of sample s is shared with sample s-1 (labels are inputs shifted by one)
    const int64_t cursor = s * static_cast<int64_t>(seq_length);
    while (true) {
      if (doc_pos >= n_docs) return -1;
      const int32_t id = doc_idx[doc_pos];
      if (id < 0 || id >= n_sizes) return -1;
      const int64_t len = sizes[id];
      if (cursor < doc_begin + len) break;
      doc_begin += len;
      ++doc_pos;
    }
    out[2 * s] = static_cast<int32_t>(doc_pos);
    out[2 * s + 1] = static_cast<int32_t>(cursor - doc_begin);
  }
  return num_samples + 1;
}

// First-fit-decreasing is left to the caller (pass lengths pre-sorted); this is first-fit in order.
// bin_of[i] receives the bin of sample i; returns the number of bins.
int64_t ell_build_pack_index(const int32_t* lengths, int64_t n, int32_t capacity, int32_t* bin_of) {
  std::vector<int32_t> room;
  for (int64_t i = 0; i < n; ++i) {
    int32_t len = lengths[i] > capacity ? capacity : lengths[i];
    int64_t b = -1;
    for (size_t j = 0; j < room.size(); ++j)
      if (room[j] >= len) { b = static_cast<int64_t>(j); break; }
    if (b < 0) { room.push_back(capacity); b = static_cast<int64_t>(room.size()) - 1; }
    room[b] -= len;
    bin_of[i] = static_cast<int32_t>(b);
  }
  return static_cast<int64_t>(room.size());
}

}  // extern "C"
