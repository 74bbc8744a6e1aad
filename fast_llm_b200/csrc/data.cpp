// Host-side helpers of the data pipeline (plain C ABI, loaded with ctypes).
//
//   flb_build_padded_token_cumsum  token count before every `rate`-th document when documents are packed into
//                                  fixed-size samples WITHOUT being split: a document that does not fit in the rest
//                                  of the current sample starts the next one (the gap is padding), and documents
//                                  longer than a sample are skipped.
//   flb_build_sample_idx           for a concatenated token stream, the (document, offset) at which each fixed-length
//                                  sample starts (Megatron-style index; consecutive samples overlap by one token).
//
// Counterparts of `fast_llm/csrc/data.cpp:43-212`; the Python restatements in `fast_llm_b200/data/sampled.py` are the
// test oracle.
#include <cstdint>

#define FLB_HOST_API extern "C" __attribute__((visibility("default")))

// sizes[num_documents]: document lengths in sampling order.  out[] must hold ceil(num_documents / rate) + 1 entries.
// `offset`: tokens already placed before the first document.  Returns the number of entries written; *total receives
// the padded token count after the last document.
FLB_HOST_API int64_t flb_build_padded_token_cumsum(const int32_t* sizes, int64_t num_documents, int32_t sample_size,
                                                   int32_t rate, int64_t offset, int64_t* out, int64_t* total) {
  int64_t cumsum = offset;
  int64_t written = 0;
  for (int64_t i = 0; i < num_documents; ++i) {
    if (i % rate == 0) out[written++] = cumsum;
    const int64_t size = sizes[i];
    if (size > sample_size) continue;  // cannot be placed whole: dropped
    const int64_t used = cumsum % sample_size;
    if (used + size > sample_size) cumsum += sample_size - used;  // pad to the next sample boundary
    cumsum += size;
  }
  if (num_documents % rate == 0) out[written++] = cumsum;
  if (total) *total = cumsum;
  return written;
}

// sizes[]: length of every document; doc_idx[num_doc_idx]: order in which documents are concatenated (with repeats
// over epochs).  sample_idx[(num_samples + 1) * 2] receives (position in doc_idx, offset in that document) of the first
// token of each sample and of the end of the last one.  Each sample covers seq_length + 1 tokens and the next sample
// starts on the last token of the previous one.  Returns 0 on success, -1 if doc_idx holds too few tokens, -2 if a
// document index is out of range.
FLB_HOST_API int32_t flb_build_sample_idx(const int32_t* sizes, int64_t num_documents, const int32_t* doc_idx,
                                          int64_t num_doc_idx, int32_t seq_length, int64_t num_samples,
                                          int32_t* sample_idx) {
  int64_t pos = 0;      // position in doc_idx
  int32_t doc_offset = 0;
  sample_idx[0] = 0;
  sample_idx[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int32_t remaining = seq_length + 1;
    while (remaining != 0) {
      if (pos >= num_doc_idx) return -1;
      const int32_t doc = doc_idx[pos];
      if (doc < 0 || doc >= num_documents) return -2;
      const int32_t doc_length = sizes[doc] - doc_offset;
      remaining -= doc_length;
      if (remaining <= 0) {
        // the sample ends inside this document; the next one re-reads its last token
        doc_offset += remaining + doc_length - 1;
        remaining = 0;
      } else {
        ++pos;
        doc_offset = 0;
      }
    }
    sample_idx[2 * s] = (int32_t)pos;
    sample_idx[2 * s + 1] = doc_offset;
  }
  return 0;
}
