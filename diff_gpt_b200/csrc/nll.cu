// Negative log-likelihood of given tokens under rows of logits: one warp per row, one read of the row.
//   out[r] = log(sum_j exp(logits[r, j])) - logits[r, target[r]]
// This is the -log_softmax(...).gather(...) of the reference's anomaly score
// (src/diff_gpt/diff_gpt.py:352-356), without materialising the [R, V] log-probabilities.
#include "common.cuh"

namespace dgpt {

template <typename T>
__global__ void token_nll_kernel(const T* __restrict__ logits, long long stride, const int* __restrict__ targets,
                                 float* __restrict__ out, int R, int V, int* __restrict__ status) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= R) return;
  const int lane = threadIdx.x & 31;
  const T* row = logits + (long long)r * stride;
  const int tgt = targets[r];
  if (tgt < 0 || tgt >= V) {  // recorded, and the row is left as NaN rather than read out of bounds
    if (lane == 0) {
      out[r] = __int_as_float(0x7fc00000);
      if (status) atomicOr(status, 4);
    }
    return;
  }
  // online max / sum so that the row is read once
  float m = -INFINITY, s = 0.f;
  for (int i = lane; i < V; i += 32) {
    const float x = Io<T>::ld(row + i);
    if (x > m) {
      s *= __expf(m - x);  // m = -inf: s is 0 and stays 0
      m = x;
    }
    s += __expf(x - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
    m = mn;
  }
  if (lane == 0) {
    // the reference's log_softmax result has the storage type of the logits, so round once to it
    const float lp = Io<T>::round(Io<T>::ld(row + tgt) - (m + logf(s)));
    out[r] = -lp;
  }
}

}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_token_nll(const void* logits, int64_t logits_row_stride, const int32_t* targets, float* out,
                              int32_t R, int32_t V, int32_t dtype, int32_t* status, void* stream) {
  DGPT_REQUIRE(logits && targets && out, "token_nll: NULL pointer");
  DGPT_REQUIRE(R >= 0 && V > 0, "token_nll: bad sizes");
  if (R == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((R + 3) / 4);
  if (dtype == DGPT_F32) {
    token_nll_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float*>(logits), logits_row_stride, targets, out,
                                                  R, V, status);
  } else if (dtype == DGPT_BF16) {
    token_nll_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(logits),
                                                          logits_row_stride, targets, out, R, V, status);
  } else {
    set_error("token_nll: unknown dtype %d", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("token_nll");
}
