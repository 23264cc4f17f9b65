// Tokens of the generated horizon -> float64 values, for all trajectories at once.
//
// The reference decodes every sampled trajectory on the host (src/diff_gpt/diff_gpt.py:236-252 calling
// encoder_decoder.py:373-397 and :97-152): value = (token - V/2) / scale, then k cumulative sums seeded
// with the first values of the context.  A cumulative sum is a chain of float64 additions in time order,
// so it can be continued from the state it has at the end of the prompt: with
//     x_m(t) = level-m running sum after generated step t          (m = 1 .. k, x_0(t) = the step's value)
//     x_m(t) = x_m(t - 1) + x_{m-1}(t)
// every addition has the operands, and the order, of numpy's cumsum over the whole sequence, and the
// results are bit-identical.  The prompt is the same for all trajectories of a series, so its end state
// x_m(-1) is computed once on the host and passed in.  One thread per (trajectory, channel).
#include "common.cuh"

namespace dgpt {

constexpr int kMaxOrder = 8;

__global__ void integrate_tokens_kernel(const int* __restrict__ tokens, long long token_stride, int n_traj, int horizon,
                                        int n_chan, int half_vocab, const double* __restrict__ scale,
                                        const int* __restrict__ order, const double* __restrict__ state, int max_order,
                                        double* __restrict__ out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_traj * n_chan) return;
  const int n = (int)(idx / n_chan), c = (int)(idx - (long long)n * n_chan);
  const int k = order[c];
  const double sc = scale[c];
  double x[kMaxOrder];
#pragma unroll
  for (int m = 0; m < kMaxOrder; ++m) x[m] = (m < k) ? state[(long long)c * max_order + m] : 0.0;
  const int* row = tokens + (long long)n * token_stride;
  for (int t = 0; t < horizon; ++t) {
    double v = __ddiv_rn((double)(row[(long long)t * n_chan + c] - half_vocab), sc);
#pragma unroll
    for (int m = 0; m < kMaxOrder; ++m) {
      if (m < k) {
        x[m] = __dadd_rn(x[m], v);  // no contraction: one rounded addition, as numpy does
        v = x[m];
      }
    }
    out[((long long)n * horizon + t) * n_chan + c] = v;
  }
}

}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_integrate_tokens(const int32_t* tokens, int64_t token_row_stride, int32_t n_traj, int32_t horizon,
                                     int32_t n_chan, int32_t vocab_size, const double* scale, const int32_t* order,
                                     const double* state, int32_t max_order, double* out, void* stream) {
  DGPT_REQUIRE(tokens && scale && order && out, "integrate_tokens: NULL pointer");
  DGPT_REQUIRE(n_traj >= 0 && horizon >= 0 && n_chan > 0 && vocab_size >= 2, "integrate_tokens: bad sizes");
  DGPT_REQUIRE(max_order >= 0 && max_order <= kMaxOrder, "integrate_tokens: order of derivative above %d is not built",
               kMaxOrder);
  DGPT_REQUIRE(max_order == 0 || state, "integrate_tokens: state is NULL");
  if (n_traj == 0 || horizon == 0) return DGPT_OK;
  const long long n = (long long)n_traj * n_chan;
  integrate_tokens_kernel<<<(unsigned)((n + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      tokens, token_row_stride, n_traj, horizon, n_chan, vocab_size / 2, scale, order, state, max_order, out);
  return launch_status("integrate_tokens");
}
