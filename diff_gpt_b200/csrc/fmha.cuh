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
  int pingpong;  // tensor-core path only: the kernel with two query tiles per CTA
};

// What the tensor-core kernels need besides the three tensor maps.
struct TcParams {
  const int* kv_len;
  int kv_len_all;
  const int* page_table;
  int max_pages;
  int page_tokens;
  void* o;
  long long o_bs, o_rs;
  int o_f32;
  float* lse;
  int H, Tq, q_offset, causal;
  float scale_log2;
  int* status;
  int n_qt, n_work;  // query tiles per (batch, head) and work items in all (a capped grid loops over them)
  int d_head;        // head_dim of the tensors in global memory (32 rides on the 64-wide kernels: the TMA boxes are 64 wide
                     // and the columns past the tensor's extent arrive as zeros, so scores and outputs are unchanged)
  int BH, group_bh;  // two-query-tile kernel: (batch, head) pairs in all, and how many are worked on at a time
};

// warp-level kernel (fmha_simt.cu)
int fmha_simt(const FmhaArgs& a, const KvView& kv, cudaStream_t st);

// tcgen05 / TMEM kernel (fmha_tc.cu)
bool fmha_tc_supported(const FmhaArgs& a, const dgpt_kv_layout& kv);
int fmha_tc(const FmhaArgs& a, const dgpt_kv_layout& kv, cudaStream_t st);
// the same with two query tiles per CTA taking turns on the tensor cores (fmha_pp.cu); `tp` and the maps come from fmha_tc
struct TcMaps;
int fmha_tc_pp_launch(const FmhaArgs& a, const TcMaps& maps, TcParams p, long long kv_span, cudaStream_t st);
// the persistent warp-specialised kernel with one query tile per work item (fmha_ws.cu)
int fmha_tc_ws_launch(const FmhaArgs& a, const TcMaps& maps, TcParams p, long long kv_span, cudaStream_t st);

}  // namespace dgpt
