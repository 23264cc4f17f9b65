// The model's head as one call: tied-embedding logits (tcgen05 GEMM of gemm_tc.cu), logit soft-cap, and the draw of
// the next token with teacher forcing.
//
// Two forms.  With a top-p filter, or when the caller wants the logits, the GEMM writes bf16 logits and the
// sampling kernel of sample.cu reads them (the nucleus needs a row's whole distribution).  Otherwise nothing is
// written: every thread of the GEMM's epilogue soft-caps its logits, adds Gumbel noise keyed by (seed, trajectory,
// step, token) - the arg-max of z / T + G is a draw from softmax(z / T) - and raises its row's best (key, token)
// word with one atomicMax per tile; a small finishing kernel turns the winners into tokens, applies the forcing
// schedule and writes the history column.
#include "linear.cuh"

namespace dgpt {

__global__ void head_finish_kernel(const unsigned long long* __restrict__ best, int R, const int* __restrict__ step_ptr,
                                   const int* __restrict__ force, int force_rows, long long force_stride,
                                   int* __restrict__ out_tok, int* __restrict__ out_mask, int* __restrict__ hist_tok,
                                   int* __restrict__ hist_mask, long long hist_stride) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const int step = step_ptr ? *step_ptr : 0;
  const int forced = force ? force[(long long)(r / force_rows) * force_stride + step] : -1;
  const int token = forced >= 0 ? forced : (int)(~(uint32_t)(best[r] & 0xffffffffull));
  const int mask = forced >= 0 ? 0 : 1;
  out_tok[r] = token;
  if (out_mask) out_mask[r] = mask;
  if (hist_tok) hist_tok[(long long)r * hist_stride + step] = token;
  if (hist_mask) hist_mask[(long long)r * hist_stride + step] = mask;
}

}  // namespace dgpt

using namespace dgpt;

extern "C" size_t dgpt_lmhead_workspace_bytes(int32_t R) { return (size_t)(R > 0 ? R : 0) * sizeof(unsigned long long); }

extern "C" int dgpt_lmhead_sample(const void* xn, int64_t xn_row_stride, const void* emb, int64_t emb_row_stride, float cap,
                                  float temperature, float top_p, uint64_t seed, int64_t traj_id0,
                                  const int64_t* traj_ids, int32_t step_base, const int32_t* step_ptr,
                                  const int32_t* force_schedule, int32_t force_group_rows, int64_t force_group_stride,
                                  int32_t* out_tokens, int32_t* out_masks, int32_t* history_tokens,
                                  int32_t* history_masks, int64_t history_stride, void* logits_out,
                                  int64_t logits_row_stride, void* workspace, size_t workspace_bytes, int32_t R, int32_t C,
                                  int32_t V, int32_t dtype, int32_t* status, void* stream) {
  DGPT_REQUIRE(xn && emb && out_tokens, "lmhead_sample: NULL pointer");
  DGPT_REQUIRE(R >= 0 && C > 0 && V > 0, "lmhead_sample: bad sizes");
  DGPT_REQUIRE(temperature >= 0.f && cap >= 0.f, "lmhead_sample: temperature and cap must be non-negative");
  if (dtype != DGPT_BF16) {
    set_error("lmhead_sample: only bf16 is built (dtype %d)", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  if (R == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool nucleus = top_p < 1.f && temperature > 0.f;
  if (nucleus || logits_out) {
    DGPT_REQUIRE(logits_out, "lmhead_sample: a top-p filter needs the logits buffer (a row's whole distribution)");
    if (int e = linear_launch(xn, xn_row_stride, emb, emb_row_stride, logits_out, logits_row_stride, nullptr, 0, R, V, C, 0,
                              0.f, 0.f, dtype, status, nullptr, stream))
      return e;
    return dgpt_sample(logits_out, logits_row_stride, R, V, cap, temperature, top_p, seed, traj_id0, traj_ids, step_base,
                       step_ptr, force_schedule, force_group_rows, force_group_stride, out_tokens, out_masks,
                       history_tokens, history_masks, history_stride, dtype, stream);
  }
  const size_t need = dgpt_lmhead_workspace_bytes(R);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 7) != 0) {
    set_error("lmhead_sample: an 8-byte aligned workspace of %zu bytes is needed, %zu given", need, workspace_bytes);
    return DGPT_E_WORKSPACE;
  }
  if (cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess) {
    set_error("lmhead_sample: cudaMemsetAsync failed");
    return DGPT_E_CUDA;
  }
  HeadDraw d;
  d.cap = cap;
  d.inv_temperature = temperature > 0.f ? 1.f / temperature : 0.f;
  d.seed_lo = (uint32_t)seed;
  d.seed_hi = (uint32_t)(seed >> 32);
  d.traj_id0 = traj_id0;
  d.traj_ids = reinterpret_cast<const long long*>(traj_ids);
  d.step_base = step_base;
  d.step_ptr = step_ptr;
  d.best = static_cast<unsigned long long*>(workspace);
  if (int e = linear_launch(xn, xn_row_stride, emb, emb_row_stride, nullptr, 0, nullptr, 0, R, V, C, 3, 0.f, 0.f, dtype, status,
                            &d, stream))
    return e;
  const int fg = force_group_rows > 0 ? force_group_rows : 1;
  head_finish_kernel<<<(R + 255) / 256, 256, 0, st>>>(d.best, R, step_ptr, force_schedule, fg, force_group_stride, out_tokens,
                                                    out_masks, history_tokens, history_masks, history_stride);
  return launch_status("lmhead_finish");
}
