// RoPE + QK RMSNorm + KV-cache append, one warp per (token, head).
//
// Each lane owns rotation pairs  p = lane, lane + 32, ...  (< D/2), i.e. elements
// (2p, 2p+1): a 4-byte (bf16) or 8-byte (fp32) access per lane, consecutive across
// the warp.  q is written to a dense [token, H*D] buffer, k and v go straight into
// their cache page, so the projection output is read once and the cache written once.
#include "common.cuh"

namespace dgpt {

template <typename T>
struct Pair;
template <>
struct Pair<float> {
  static __device__ __forceinline__ float2 ld(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void st(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
  }
};
template <>
struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 ld(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

constexpr int kMaxPairsPerLane = 4;  // head_dim <= 256

template <typename T>
__global__ void rope_qknorm_kvappend_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                            long long in_stride, T* __restrict__ q_out, long long q_out_stride,
                                            const T* __restrict__ cs, int table_len, KvView kv,
                                            const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot0,
                                            const int* __restrict__ step_ptr, int n_seq, int T_len, int H, int D,
                                            int* __restrict__ status) {
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)n_seq * T_len * H;
  if (wid >= total) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(wid % H);
  const long long tok = wid / H;
  const int s = (int)(tok / T_len), t = (int)(tok - (long long)s * T_len);
  const int step = step_ptr ? *step_ptr : 0;
  const int pos = seq_pos0[s] + step + t;
  const int slot = seq_slot0[s] + step + t;
  const int cap = kv.page_table ? kv.max_pages * kv.page_tokens : kv.page_tokens;
  if (pos < 0 || pos >= table_len || slot < 0 || slot >= cap) {
    if (lane == 0) atomicExch(status, 1);
    return;
  }
  const int half = D >> 1;
  const T* qs = q + tok * in_stride + (long long)h * D;
  const T* ks = k + tok * in_stride + (long long)h * D;
  const T* vs = v + tok * in_stride + (long long)h * D;
  const T* csr = cs + (long long)pos * D;  // (D/2, 2) per position

  float qa[kMaxPairsPerLane], qb[kMaxPairsPerLane], ka[kMaxPairsPerLane], kb[kMaxPairsPerLane];
  float qss = 0.f, kss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPairsPerLane; ++i) {
    const int p = lane + 32 * i;
    qa[i] = qb[i] = ka[i] = kb[i] = 0.f;
    if (p < half) {
      const float2 c = Pair<T>::ld(csr + 2 * p);  // (cos, sin), upcast from the storage type
      const float2 x = Pair<T>::ld(qs + 2 * p);
      const float2 y = Pair<T>::ld(ks + 2 * p);
      qa[i] = Io<T>::round(x.x * c.x - x.y * c.y);
      qb[i] = Io<T>::round(x.x * c.y + x.y * c.x);
      ka[i] = Io<T>::round(y.x * c.x - y.y * c.y);
      kb[i] = Io<T>::round(y.x * c.y + y.y * c.x);
      qss += qa[i] * qa[i] + qb[i] * qb[i];
      kss += ka[i] * ka[i] + kb[i] * kb[i];
    }
  }
  qss = warp_sum(qss);
  kss = warp_sum(kss);
  const float qinv = rsqrtf(qss / (float)D + kRmsEps);
  const float kinv = rsqrtf(kss / (float)D + kRmsEps);

  const long long off = kv_offset(kv, s, h, slot, D);
  T* kd = static_cast<T*>(kv.k) + off;
  T* vd = static_cast<T*>(kv.v) + off;
  T* qd = q_out + tok * q_out_stride + (long long)h * D;
#pragma unroll
  for (int i = 0; i < kMaxPairsPerLane; ++i) {
    const int p = lane + 32 * i;
    if (p < half) {
      Pair<T>::st(qd + 2 * p, qa[i] * qinv, qb[i] * qinv);
      Pair<T>::st(kd + 2 * p, ka[i] * kinv, kb[i] * kinv);
      const float2 vv = Pair<T>::ld(vs + 2 * p);
      Pair<T>::st(vd + 2 * p, vv.x, vv.y);
    }
  }
}

}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_rope_qknorm_kvappend(const void* q, const void* k, const void* v, int64_t in_row_stride,
                                         void* q_out, int64_t q_out_row_stride, const void* cs_table,
                                         int32_t table_len, const dgpt_kv_layout* kv, const int32_t* seq_pos0,
                                         const int32_t* seq_slot0, const int32_t* step_ptr, int32_t n_seq,
                                         int32_t T, int32_t H, int32_t D, int32_t dtype, int32_t* status,
                                         void* stream) {
  DGPT_REQUIRE(q && k && v && q_out && cs_table && seq_pos0 && seq_slot0 && status, "rope_qknorm_kvappend: NULL pointer");
  DGPT_REQUIRE(n_seq >= 0 && T >= 0 && H > 0, "rope_qknorm_kvappend: bad sizes");
  DGPT_REQUIRE(D > 0 && D % 2 == 0 && D <= 64 * kMaxPairsPerLane, "rope_qknorm_kvappend: head_dim must be even and <= 256");
  DGPT_REQUIRE(in_row_stride % 2 == 0 && q_out_row_stride % 2 == 0, "rope_qknorm_kvappend: row strides must be even");
  if (int e = validate_kv(kv, D)) return e;
  const long long total = (long long)n_seq * T * H;
  if (total == 0) return DGPT_OK;
  const int warps = 8;
  const unsigned grid = (unsigned)((total + warps - 1) / warps);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const KvView view = make_view(kv);
  if (dtype == DGPT_F32) {
    rope_qknorm_kvappend_kernel<float><<<grid, warps * 32, 0, st>>>(
        static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v), in_row_stride,
        static_cast<float*>(q_out), q_out_row_stride, static_cast<const float*>(cs_table), table_len, view, seq_pos0,
        seq_slot0, step_ptr, n_seq, T, H, D, status);
  } else if (dtype == DGPT_BF16) {
    using B = __nv_bfloat16;
    rope_qknorm_kvappend_kernel<B><<<grid, warps * 32, 0, st>>>(
        static_cast<const B*>(q), static_cast<const B*>(k), static_cast<const B*>(v), in_row_stride,
        static_cast<B*>(q_out), q_out_row_stride, static_cast<const B*>(cs_table), table_len, view, seq_pos0, seq_slot0,
        step_ptr, n_seq, T, H, D, status);
  } else {
    set_error("rope_qknorm_kvappend: unknown dtype %d", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("rope_qknorm_kvappend");
}
