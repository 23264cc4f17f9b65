// Argument block shared by the two prefill-attention kernels.
#pragma once

#include "common.cuh"

namespace dgpt {

struct FmhaArgs {
  const void* q;
  long long q_bs, q_rs;
  const int* kv_len;
  int kv_len_all;
  void* o;
  long long o_bs, o_rs;
  int o_f32;
  float* lse;
  int B, H, Tq, D, q_offset, causal, dtype;
  int* status;
  int max_ctas;  // two-CTAs-per-SM kernel only: at most this many CTAs, looping over the query tiles (0 = one CTA per tile)
  int two_cta;  // tensor-core path only: the 128-thread kernel with two CTAs per SM instead of the warp-specialised one
};

// warp-level kernel (fmha_simt.cu)
int fmha_simt(const FmhaArgs& a, const KvView& kv, cudaStream_t st);

// tcgen05 / TMEM kernel (fmha_tc.cu)
bool fmha_tc_supported(const FmhaArgs& a, const dgpt_kv_layout& kv);
int fmha_tc(const FmhaArgs& a, const dgpt_kv_layout& kv, cudaStream_t st);

}  // namespace dgpt
