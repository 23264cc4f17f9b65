// Prefill / chunk attention, warp-level online-softmax kernel (any dtype, any
// head_dim in {8, 16, 32, 64, 128}), plus the dgpt_fmha_prefill entry
// point that chooses between it and the tcgen05 kernel.
//
// A CTA of 128 threads owns a tile of queries of one (batch, head); K and V tiles
// of 32 keys are staged in shared memory as fp32 and read by every query thread
// as broadcasts.  A query is owned by SPLIT adjacent lanes, each holding D/SPLIT
// elements of q and of the output accumulator in registers.  Scores are produced
// eight keys at a time so that the accumulator is rescaled once per eight keys.
#include "common.cuh"
#include "fmha.cuh"

namespace dgpt {

constexpr int kSimtBN = 32;  // keys per shared-memory tile
constexpr int kSimtKB = 8;   // keys per softmax update

template <typename T, int D, int SPLIT>
__global__ void __launch_bounds__(128)
fmha_simt_kernel(const T* __restrict__ q, long long q_bs, long long q_rs, KvView kv, const int* __restrict__ kv_len,
                 int kv_len_all, void* __restrict__ o, long long o_bs, long long o_rs, int o_f32,
                 float* __restrict__ lse, int H, int Tq, int q_offset, int causal, float scale_log2) {
  constexpr int DP = D / SPLIT;       // elements per thread
  constexpr int BM = 128 / SPLIT;     // queries per CTA
  constexpr int VEC = Io<T>::kVec16;
  __shared__ __align__(16) float Ks[kSimtBN][D];
  __shared__ __align__(16) float Vs[kSimtBN][D];

  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = blockIdx.x * BM;
  const int tid = threadIdx.x;
  const int qi = q0 + tid / SPLIT;
  const int part = tid % SPLIT;
  const bool q_ok = qi < Tq;
  const int klen = kv_len ? kv_len[b] : kv_len_all;
  int kmax = klen;
  if (causal) kmax = min(klen, q_offset + min(q0 + BM, Tq));
  const int my_last = causal ? q_offset + qi : 0x7fffffff;  // last visible key of this query

  float qf[DP], acc[DP];
#pragma unroll
  for (int d = 0; d < DP; ++d) {
    acc[d] = 0.f;
    qf[d] = 0.f;
  }
  if (q_ok) {
    const T* qp = q + (long long)b * q_bs + (long long)qi * q_rs + (long long)h * D + part * DP;
#pragma unroll
    for (int d = 0; d < DP; d += VEC) {
      float t[VEC];
      ld16<T>(qp + d, t);
#pragma unroll
      for (int i = 0; i < VEC; ++i) qf[d + i] = t[i] * scale_log2;
    }
  }
  float m = -INFINITY, l = 0.f;
  const T* kbase = static_cast<const T*>(kv.k);
  const T* vbase = static_cast<const T*>(kv.v);

  for (int j0 = 0; j0 < kmax; j0 += kSimtBN) {
    __syncthreads();
    constexpr int VPR = D / VEC;  // 16-byte vectors per key row
    for (int idx = tid; idx < kSimtBN * VPR; idx += 128) {
      const int tk = idx / VPR, pv = idx - tk * VPR;
      const int slot = j0 + tk;
      float kf[VEC], vf[VEC];
      if (slot < klen) {
        const long long off = kv_offset(kv, b, h, slot, D) + pv * VEC;
        ld16<T>(kbase + off, kf);
        ld16<T>(vbase + off, vf);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) kf[i] = vf[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        *reinterpret_cast<float4*>(&Ks[tk][pv * VEC + i]) = make_float4(kf[i], kf[i + 1], kf[i + 2], kf[i + 3]);
        *reinterpret_cast<float4*>(&Vs[tk][pv * VEC + i]) = make_float4(vf[i], vf[i + 1], vf[i + 2], vf[i + 3]);
      }
    }
    __syncthreads();
    const int jn = min(kSimtBN, kmax - j0);
    for (int kb = 0; kb < jn; kb += kSimtKB) {
      float s[kSimtKB];
      float smax = -INFINITY;
#pragma unroll
      for (int kk = 0; kk < kSimtKB; ++kk) {
        const float* kr = &Ks[kb + kk][part * DP];
        float dot = 0.f;
#pragma unroll
        for (int d = 0; d < DP; d += 4) {
          const float4 kx = *reinterpret_cast<const float4*>(kr + d);
          dot += qf[d] * kx.x + qf[d + 1] * kx.y + qf[d + 2] * kx.z + qf[d + 3] * kx.w;
        }
#pragma unroll
        for (int x = 1; x < SPLIT; x <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
        const int j = j0 + kb + kk;
        s[kk] = (q_ok && j < klen && j <= my_last) ? dot : -INFINITY;
        smax = fmaxf(smax, s[kk]);
      }
      if (smax == -INFINITY) continue;  // nothing visible in this group (no shuffles below)
      const float mn = fmaxf(m, smax);
      const float resc = exp2f(m - mn);
      l *= resc;
#pragma unroll
      for (int d = 0; d < DP; ++d) acc[d] *= resc;
#pragma unroll
      for (int kk = 0; kk < kSimtKB; ++kk) {
        const float p = exp2f(s[kk] - mn);
        l += p;
        const float* vr = &Vs[kb + kk][part * DP];
#pragma unroll
        for (int d = 0; d < DP; d += 4) {
          const float4 vx = *reinterpret_cast<const float4*>(vr + d);
          acc[d] += p * vx.x;
          acc[d + 1] += p * vx.y;
          acc[d + 2] += p * vx.z;
          acc[d + 3] += p * vx.w;
        }
      }
      m = mn;
    }
  }
  if (!q_ok) return;
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const long long oo = (long long)b * o_bs + (long long)qi * o_rs + (long long)h * D + part * DP;
  if (o_f32) {
    float* op = static_cast<float*>(o) + oo;
#pragma unroll
    for (int d = 0; d < DP; ++d) op[d] = acc[d] * inv;
  } else {
    T* op = static_cast<T*>(o) + oo;
#pragma unroll
    for (int d = 0; d < DP; ++d) Io<T>::st(op + d, acc[d] * inv);
  }
  if (lse && part == 0) {
    const int Hn = H;
    lse[((long long)b * Tq + qi) * Hn + h] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
  }
}

template <typename T, int D>
static int fmha_simt_launch(const FmhaArgs& a, const KvView& kv, cudaStream_t st) {
  constexpr int SPLIT = D > 64 ? D / 64 : 1;
  constexpr int BM = 128 / SPLIT;
  dim3 grid((unsigned)((a.Tq + BM - 1) / BM), (unsigned)a.H, (unsigned)a.B);
  const float scale_log2 = kLog2e / sqrtf((float)D);
  fmha_simt_kernel<T, D, SPLIT><<<grid, 128, 0, st>>>(static_cast<const T*>(a.q), a.q_bs, a.q_rs, kv, a.kv_len,
                                                      a.kv_len_all, a.o, a.o_bs, a.o_rs, a.o_f32, a.lse, a.H, a.Tq,
                                                      a.q_offset, a.causal, scale_log2);
  return launch_status("fmha_simt");
}

int fmha_simt(const FmhaArgs& a, const KvView& kv, cudaStream_t st) {
#define DGPT_F(TT, DD) return fmha_simt_launch<TT, DD>(a, kv, st)
  if (a.dtype == DGPT_F32) {
    switch (a.D) {
      case 8: DGPT_F(float, 8);
      case 16: DGPT_F(float, 16);
      case 32: DGPT_F(float, 32);
      case 64: DGPT_F(float, 64);
      case 128: DGPT_F(float, 128);
    }
  } else if (a.dtype == DGPT_BF16) {
    switch (a.D) {
      case 8: DGPT_F(__nv_bfloat16, 8);
      case 16: DGPT_F(__nv_bfloat16, 16);
      case 32: DGPT_F(__nv_bfloat16, 32);
      case 64: DGPT_F(__nv_bfloat16, 64);
      case 128: DGPT_F(__nv_bfloat16, 128);
    }
  }
#undef DGPT_F
  set_error("fmha_prefill: dtype %d with head_dim %d is not built", a.dtype, a.D);
  return DGPT_E_UNSUPPORTED;
}

}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_fmha_prefill(const void* q, int64_t q_batch_stride, int64_t q_row_stride,
                                 const dgpt_kv_layout* kv, const int32_t* kv_len, int32_t kv_len_all, void* o,
                                 int64_t o_batch_stride, int64_t o_row_stride, int32_t o_f32, float* lse, int32_t B,
                                 int32_t H, int32_t Tq, int32_t D, int32_t q_offset, int32_t causal, int32_t dtype,
                                 int32_t impl, int32_t max_ctas, int32_t* status, void* stream) {
  DGPT_REQUIRE(q && o, "fmha_prefill: NULL pointer");
  DGPT_REQUIRE(B >= 0 && H > 0 && Tq >= 0 && B <= 65535 && H <= 65535, "fmha_prefill: bad sizes");
  DGPT_REQUIRE(kv_len || kv_len_all >= 0, "fmha_prefill: kv length missing");
  DGPT_REQUIRE(q_row_stride % 8 == 0 && q_batch_stride % 8 == 0 && o_row_stride % 8 == 0 && o_batch_stride % 8 == 0,
               "fmha_prefill: strides must be multiples of 8 elements");
  DGPT_REQUIRE(impl >= 0 && impl <= 4,
               "fmha_prefill: impl must be 0 (auto), 1 (warp-level), 2 (tensor-core, one query tile per CTA), 3 (tensor-core, "
               "two CTAs per SM) or 4 (tensor-core, two query tiles per CTA)");
  if (int e = validate_kv(kv, D)) return e;
  if (B == 0 || Tq == 0) return DGPT_OK;
  FmhaArgs a;
  a.q = q; a.q_bs = q_batch_stride; a.q_rs = q_row_stride;
  a.kv_len = kv_len; a.kv_len_all = kv_len_all;
  a.o = o; a.o_bs = o_batch_stride; a.o_rs = o_row_stride; a.o_f32 = o_f32; a.lse = lse;
  a.B = B; a.H = H; a.Tq = Tq; a.D = D; a.q_offset = q_offset; a.causal = causal; a.dtype = dtype;
  a.status = status;
  a.max_ctas = max_ctas;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const KvView view = make_view(kv);
  const bool tc_ok = fmha_tc_supported(a, *kv);
  // Which tensor-core kernel: the persistent warp-specialised one from 1024 keys on (measured against the small one on
  // one to 256 sequences of 1024 to 3584 keys, heads of 32, 64 and 128: 5 to 65 % ahead; level at 512 keys); below
  // that two smaller CTAs per SM, each done with its item after a few key tiles.
  const long long span = causal ? (long long)Tq + q_offset
                                : (kv_len ? (long long)kv->max_pages * kv->page_tokens : (long long)kv_len_all);
  a.two_cta = impl == 3 || (impl == 0 && span < 1024);
  a.pingpong = impl == 4;
  if (impl >= 2 && !tc_ok) {
    set_error("fmha_prefill: the tensor-core kernel does not cover dtype %d, head_dim %d with this layout", dtype, D);
    return DGPT_E_UNSUPPORTED;
  }
  if (tc_ok && impl != 1) return fmha_tc(a, *kv, st);
  return fmha_simt(a, view, st);
}
