// Values of many series -> prompt tokens, in one launch.
//
// The reference tokenises one series at a time on the host (src/diff_gpt/encoder_decoder.py:278-370):
// k-th finite differences per column (:36-94), a multiply by the column's scale, then one of three
// quantisers: plain rounding (order 0 among per-column orders), a first-order sigma-delta that carries the
// rounded running fraction (:229-275), or k cascaded first-order loops recombined through (1 - z^-1)^i
// (:155-226).  Every one of them is a short recurrence in time order over float64, so one thread per
// (series, column) walks the rows once and performs the additions, subtractions, the multiply and the
// roundings of numpy in numpy's order: the tokens and start rows are bit-identical to the host codec's.
//
// The same walk also integrates the de-quantised tokens, (token - V/2) / scale, back up through the k
// cumulative sums of the decoder (:97-152), which leaves the state `dgpt_integrate_tokens` continues
// from: a forecast is decoded without the prompt ever visiting the host.
#include "common.cuh"

namespace dgpt {

constexpr int kEncMaxOrder = 8;

struct EncodeParams {
  const double* values;   // [n_series][rows][n_chan]
  long long series_stride;
  int n_series, rows, n_chan, vocab, max_order, scalar_order;
  const int* order;       // [n_chan]
  const double* scale;    // [n_chan]
  int* tokens;            // [n_series][rows - max_order][n_chan]
  double* start;          // [n_series][max_order][n_chan]            (may be NULL)
  double* state;          // [n_series][n_chan][max(max_order, 1)]    (may be NULL)
};

__global__ void encode_series_kernel(EncodeParams p) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)p.n_series * p.n_chan) return;
  const int s = (int)(idx / p.n_chan), c = (int)(idx - (long long)s * p.n_chan);
  const int k = p.order[c], max_k = p.max_order, t0 = max_k - k;
  const int n_out = p.rows - max_k, half = p.vocab / 2;
  const double sc = p.scale[c];
  const bool mash = k >= 2 && p.vocab > (1 << k) + 2;
  const bool plain = k == 0 && !p.scalar_order;
  const double* x = p.values + (long long)s * p.series_stride + c;
  int* tok_out = p.tokens + ((long long)s * (n_out > 0 ? n_out : 0)) * p.n_chan + c;
  const int state_w = max_k > 1 ? max_k : 1;

  double prev[kEncMaxOrder], firsts[kEncMaxOrder], y[kEncMaxOrder], err[kEncMaxOrder];
  long long lag[kEncMaxOrder][kEncMaxOrder];  // lag[i][m]: previous output of the m-th difference of stage i
#pragma unroll
  for (int m = 0; m < kEncMaxOrder; ++m) {
    prev[m] = firsts[m] = y[m] = err[m] = 0.0;
#pragma unroll
    for (int j = 0; j < kEncMaxOrder; ++j) lag[m][j] = 0;
  }
  double frac_sum = 0.0, carried_prev = 0.0;
  bool first_frac = true;

  for (int t = 0; t < p.rows; ++t) {
    const double v = x[(long long)t * p.n_chan];
    // k-th difference: level m + 1 at t = level m at t minus level m at t - 1 (numpy.diff applied k times).
    double cur = v;
#pragma unroll
    for (int m = 0; m < kEncMaxOrder; ++m) {
      if (m < k) {
        if (t == t0 + m) firsts[m] = cur;
        const double nxt = __dsub_rn(cur, prev[m]);
        prev[m] = cur;
        cur = nxt;
      }
    }
    if (t < max_k) {
      if (p.start && !p.scalar_order) p.start[((long long)s * max_k + t) * p.n_chan + c] = v;
      if (t == max_k - 1) {
#pragma unroll
        for (int i = 0; i < kEncMaxOrder; ++i) {
          if (i < k) {
            y[i] = firsts[k - 1 - i];
            if (p.start && p.scalar_order) p.start[((long long)s * max_k + i) * p.n_chan + c] = firsts[i];
          }
        }
      }
      continue;
    }
    const double u = __dmul_rn(cur, sc);
    long long tok;
    if (mash) {
      long long total = 0;
      double feed = u;
#pragma unroll
      for (int i = 0; i < kEncMaxOrder; ++i) {
        if (i < k) {
          const double eff = __dsub_rn(feed, err[i]);
          const double q = rint(eff);
          err[i] = __dsub_rn(q, eff);
          feed = -err[i];
          // (1 - z^-1)^i on this stage's output: i first differences with zero history (integers: exact).
          long long d = (long long)q;
#pragma unroll
          for (int m = 0; m < kEncMaxOrder; ++m) {
            if (m < i) {
              const long long nd = d - lag[i][m];
              lag[i][m] = d;
              d = nd;
            }
          }
          total += d;
        }
      }
      tok = total + half;
    } else if (plain) {
      tok = (long long)rint(u) + half;
    } else {
      const double whole = trunc(u);
      const double f = __dsub_rn(u, whole);
      frac_sum = first_frac ? f : __dadd_rn(frac_sum, f);
      first_frac = false;
      const double carried = rint(frac_sum);
      const double step = __dsub_rn(carried, carried_prev);
      carried_prev = carried;
      double tv = __dadd_rn(__dadd_rn(whole, (double)half), step);
      tv = fmin(fmax(tv, 0.0), (double)(p.vocab - 1));
      tok = (long long)tv;
    }
    tok = tok < 0 ? 0 : (tok > p.vocab - 1 ? p.vocab - 1 : tok);
    tok_out[(long long)(t - max_k) * p.n_chan] = (int)tok;
    // decoder's cumulative sums over the de-quantised token, each level fed with the level below's value
    // of the previous position.
    const double dq = __ddiv_rn((double)(tok - half), sc);
#pragma unroll
    for (int i = kEncMaxOrder - 1; i >= 1; --i)
      if (i < k) y[i] = __dadd_rn(y[i], y[i - 1]);
    if (k > 0) y[0] = __dadd_rn(y[0], dq);
  }
  if (p.state) {
    // level i is one element longer than level i - 1: finish the trailing additions
    for (int e = 1; e < k; ++e) {
#pragma unroll
      for (int i = kEncMaxOrder - 1; i >= 1; --i)
        if (i < k && i >= e) y[i] = __dadd_rn(y[i], y[i - 1]);
    }
#pragma unroll
    for (int i = 0; i < kEncMaxOrder; ++i)
      if (i < state_w) p.state[((long long)s * p.n_chan + c) * state_w + i] = i < k ? y[i] : 0.0;
  }
}

}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_encode_series(const double* values, int64_t series_stride, int32_t n_series, int32_t rows,
                                  int32_t n_chan, int32_t vocab_size, const int32_t* order, int32_t max_order,
                                  int32_t scalar_order, const double* scale, int32_t* tokens, double* start,
                                  double* state, void* stream) {
  DGPT_REQUIRE(values && order && scale && (tokens || rows == max_order), "encode_series: NULL pointer");
  DGPT_REQUIRE(n_series >= 0 && rows >= 0 && n_chan > 0, "encode_series: bad sizes");
  DGPT_REQUIRE(vocab_size >= 4 && vocab_size % 2 == 0, "encode_series: vocab_size must be even and at least 4");
  DGPT_REQUIRE(max_order >= 0 && max_order <= kEncMaxOrder,
               "encode_series: order of derivative above %d is not built", kEncMaxOrder);
  DGPT_REQUIRE(max_order <= rows, "encode_series: max order %d above the %d rows of a series", max_order, rows);
  DGPT_REQUIRE(series_stride >= (int64_t)rows * n_chan, "encode_series: series overlap");
  if (n_series == 0) return DGPT_OK;
  EncodeParams p{values, series_stride, n_series, rows, n_chan, vocab_size, max_order, scalar_order,
                 order,  scale,         tokens,   start, state};
  const long long n = (long long)n_series * n_chan;
  encode_series_kernel<<<(unsigned)((n + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return launch_status("encode_series");
}
