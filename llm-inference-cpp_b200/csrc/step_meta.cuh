// How a step's ragged batch and the paged cache are described to the kernels.
//
// A step runs n_tokens tokens of n_seqs sequences, flattened in sequence order.
//   tok_seq[t]   index of the token's sequence within this step, or -1 for padding
//   tok_pos[t]   absolute position of the token in its sequence
//   seq_pages    [n_seqs, pages_stride]: the cache pages of each sequence, in position order
// Keys and values of one cache layer live in pages:
//   K[page][kv_head][page_size][head_dim]   (V alike)
// so that one (page, kv head) tile is contiguous: head-major inside the page, as the
// reference lays one sequence out (include/llmi/model/transformer.hpp:39-44).
#pragma once
#include <stdint.h>

namespace llmi {

struct PagedKV {
  const int32_t* seq_pages;  // [n_seqs, pages_stride]
  int pages_stride;
  int page_size;
  int n_kv_heads;
  int head_dim;
};

__device__ __forceinline__ size_t kv_row_offset(const PagedKV& c, int seq, int pos, int kv_head) {
  const int page = c.seq_pages[(size_t)seq * c.pages_stride + pos / c.page_size];
  return (((size_t)page * c.n_kv_heads + kv_head) * c.page_size + (pos % c.page_size)) * c.head_dim;
}

}  // namespace llmi
