// Causal chunked-prefill attention on tcgen05 / TMEM (interface; kernel in prefill_umma2.cu).
#pragma once

#include "common.cuh"

namespace qwb {

struct PrefillCall {
  const uint16_t *q;     // [n_seq][n_new][q_heads][256] bf16, un-rotated when do_rope
  const uint16_t *gate;  // same shape or null
  void *out;             // same shape, bf16 or fp32
  bool out_is_f32;
  float *lse;            // [n_seq][n_new][q_heads] or null
  const uint16_t *kc, *vc;
  int64_t cache_rows;
  const int64_t *cache_row;
  qwb::PageMap pages;   // block table, if the cache is paged
  const int *pos;
  const int *q_pos;     // null, or the absolute position of each sequence's first new row (RoPE angles)
  const int *mpos;
  int n_seq, n_new, q_heads, kv_heads;
  float scale;
  bool do_rope;
  int fast_p;            // 1: single bf16 P (faster, rel-L2 ~1.4e-3); 0: bf16 hi + lo pair
  int *status;
  RopeTable rope;
};

// True when the tcgen05 kernel takes a chunk of n_new rows (shorter chunks go to split-KV).
bool prefill_umma_supported(int n_new);
// Launches the CTA-pair kernel (tcgen05 cta_group::2; needs an even number of query heads);
// *n_launched receives how many kernels were launched.  Returns a QW_* code.
int launch_prefill_umma_pair(const PrefillCall &c, cudaStream_t st, int *n_launched);

}  // namespace qwb
