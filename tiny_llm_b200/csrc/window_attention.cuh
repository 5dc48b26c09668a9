// What the two window-attention kernels (CUDA cores: window_attention.cu; tensor cores: window_attention_mma.cu) are
// told about a step: the queries, the paged caches of tokens and of pooled blocks, and the design's constants.
#pragma once

namespace tllm {

struct WinArgs {
  const void* qkv;      // queries at the front of every row
  int row_stride;
  int nh, nkv, kd, vd;
  const void *k, *v;    // token pages
  const int* table; int max_blocks;
  long long k_page_stride, k_head_stride, v_page_stride, v_head_stride;
  const void *pk, *pv;  // block pages (or null)
  const int* ptable; int pmax_blocks;
  long long pk_page_stride, pk_head_stride, pv_page_stride, pv_head_stride;
  int page_size;
  const int* positions; const int* token_request;
  void* out;
  float scale, cap;     // cap <= 0: none
  const float* head_bias;
  int window, pool;     // window <= 0: every key; pool <= 0: no blocks
  const float* fv;      // frequencies of the value rotation, or null
  int n_tokens;
};

}  // namespace tllm
