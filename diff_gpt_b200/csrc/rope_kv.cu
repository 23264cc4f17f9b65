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

// Vector variant: LPH = D / VEC lanes own one (token, head), each lane one 16-byte vector (VEC / 2
// rotation pairs) of q, k, v and of the (cos, sin) row, so a warp covers 32 / LPH heads and every
// access is 16 bytes wide.  Same rounding points as the scalar kernel.
template <typename T, int D>
__global__ void rope_qknorm_kvappend_vec_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                const T* __restrict__ v, long long in_stride, T* __restrict__ q_out,
                                                long long q_out_stride, const T* __restrict__ cs, int table_len,
                                                KvView kv, const int* __restrict__ seq_pos0,
                                                const int* __restrict__ seq_slot0, const int* __restrict__ step_ptr,
                                                int n_seq, int T_len, int H, int* __restrict__ status) {
  constexpr int VEC = Io<T>::kVec16;
  constexpr int LPH = D / VEC;
  static_assert(LPH >= 1 && LPH <= 32 && (LPH & (LPH - 1)) == 0, "unsupported head_dim");
  dep_wait();
  const long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPH;  // (token, head)
  const int e = threadIdx.x % LPH;
  const long long total = (long long)n_seq * T_len * H;
  const bool live = unit < total;
  const long long u = live ? unit : total - 1;  // idle lanes shadow the last unit so that shuffles stay full
  const int h = (int)(u % H);
  const long long tok = u / H;
  const int s = (int)(tok / T_len), t = (int)(tok - (long long)s * T_len);
  const int step = step_ptr ? *step_ptr : 0;
  const int pos = seq_pos0[s] + step + t;
  const int slot = seq_slot0[s] + step + t;
  const int cap = kv.page_table ? kv.max_pages * kv.page_tokens : kv.page_tokens;
  const bool in_range = pos >= 0 && pos < table_len && slot >= 0 && slot < cap;
  if (live && !in_range && e == 0) atomicExch(status, 1);
  const int pos_c = in_range ? pos : 0;
  const long long src = tok * in_stride + (long long)h * D + e * VEC;
  float qf[VEC], kf[VEC], cf[VEC];
  ld16<T>(q + src, qf);
  ld16<T>(k + src, kf);
  ld16<T>(cs + (long long)pos_c * D + e * VEC, cf);  // (cos, sin) pairs of this lane's rotation pairs
  const uint4 vraw = *reinterpret_cast<const uint4*>(v + src);
  float qss = 0.f, kss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; i += 2) {
    const float c = cf[i], sn = cf[i + 1];
    const float qa = Io<T>::round(qf[i] * c - qf[i + 1] * sn), qb = Io<T>::round(qf[i] * sn + qf[i + 1] * c);
    const float ka = Io<T>::round(kf[i] * c - kf[i + 1] * sn), kb = Io<T>::round(kf[i] * sn + kf[i + 1] * c);
    qf[i] = qa; qf[i + 1] = qb; kf[i] = ka; kf[i + 1] = kb;
    qss += qa * qa + qb * qb;
    kss += ka * ka + kb * kb;
  }
#pragma unroll
  for (int o = LPH >> 1; o > 0; o >>= 1) {
    qss += __shfl_xor_sync(0xffffffffu, qss, o);
    kss += __shfl_xor_sync(0xffffffffu, kss, o);
  }
  if (!live || !in_range) return;
  const float qinv = rsqrtf(qss / (float)D + kRmsEps);
  const float kinv = rsqrtf(kss / (float)D + kRmsEps);
  const long long off = kv_offset(kv, s, h, slot, D) + e * VEC;
  st16<T>(q_out + tok * q_out_stride + (long long)h * D + e * VEC, qf, qinv);
  st16<T>(static_cast<T*>(kv.k) + off, kf, kinv);
  *reinterpret_cast<uint4*>(static_cast<T*>(kv.v) + off) = vraw;
}

template <typename T, int D>
static int rope_vec_launch(const void* q, const void* k, const void* v, long long in_stride, void* q_out,
                           long long q_out_stride, const void* cs, int table_len, const KvView& view,
                           const int* pos0, const int* slot0, const int* step_ptr, int n_seq, int T_len, int H,
                           int* status, cudaStream_t st) {
  constexpr int LPH = D / Io<T>::kVec16;
  const long long threads = (long long)n_seq * T_len * H * LPH;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  launch_dep(rope_qknorm_kvappend_vec_kernel<T, D>, dim3(grid), dim3(256), 0, st, static_cast<const T*>(q),
             static_cast<const T*>(k), static_cast<const T*>(v), in_stride, static_cast<T*>(q_out), q_out_stride,
             static_cast<const T*>(cs), table_len, view, pos0, slot0, step_ptr, n_seq, T_len, H, status);
  return launch_status("rope_qknorm_kvappend");
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
  {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec = dtype == DGPT_BF16 ? 8 : 4;
    const bool aligned = al(q) && al(k) && al(v) && al(q_out) && al(cs_table) && in_row_stride % vec == 0 &&
                         q_out_row_stride % vec == 0 && D % vec == 0;
#define DGPT_ROPE(TT, DD)                                                                                         \
  return rope_vec_launch<TT, DD>(q, k, v, in_row_stride, q_out, q_out_row_stride, cs_table, table_len, view,      \
                                 seq_pos0, seq_slot0, step_ptr, n_seq, T, H, status, st)
    if (aligned && dtype == DGPT_BF16) {
      switch (D) {
        case 8: DGPT_ROPE(__nv_bfloat16, 8);
        case 16: DGPT_ROPE(__nv_bfloat16, 16);
        case 32: DGPT_ROPE(__nv_bfloat16, 32);
        case 64: DGPT_ROPE(__nv_bfloat16, 64);
        case 128: DGPT_ROPE(__nv_bfloat16, 128);
      }
    } else if (aligned && dtype == DGPT_F32) {
      switch (D) {
        case 8: DGPT_ROPE(float, 8);
        case 16: DGPT_ROPE(float, 16);
        case 32: DGPT_ROPE(float, 32);
        case 64: DGPT_ROPE(float, 64);
        case 128: DGPT_ROPE(float, 128);
      }
    }
#undef DGPT_ROPE
  }
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
