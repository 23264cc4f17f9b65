// Decode attention (one query per row) over paged K/V, split along the keys.
//
// One warp per (row, head, split).  A K or V vector of D elements is read as
// D*sizeof(T)/16 sixteen-byte loads, one per lane, so a warp covers 32/LPT tokens
// per load instruction (LPT = lanes per token) and every byte of the cache is
// fetched with 128-bit coalesced accesses.  Each lane group keeps its own online
// softmax state; the groups are merged with shuffles at the end, so the inner
// loop has no cross-group dependency.  HBM-bound by design: the algorithmic
// traffic is 2 * D * sizeof(T) bytes per (row, head, key).
#include <atomic>

#include "common.cuh"

namespace dgpt {

template <typename T, int D>
struct DecodeCfg {
  static constexpr int VEC = Io<T>::kVec16;
  static constexpr int LPT = D / VEC;    // lanes per token
  static constexpr int TPW = 32 / LPT;   // tokens per warp-wide load
  static_assert(D % VEC == 0 && LPT >= 1 && LPT <= 32 && (LPT & (LPT - 1)) == 0, "unsupported head_dim");
};

struct MergeState {
  float m, l;
};

// merge (m,l,acc) with (m2,l2,acc2): log2-domain running max
template <int VEC>
__device__ __forceinline__ void merge_partial(float& m, float& l, float* acc, float m2, float l2, const float* acc2) {
  const float mn = fmaxf(m, m2);
  const float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
  const float b = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
  l = l * a + l2 * b;
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * a + acc2[i] * b;
  m = mn;
}

constexpr int kDecLoads = 8;    // 16-byte loads in flight per lane and per tensor
constexpr int kDecMinCtas = 4;  // minimum resident CTAs per SM asked of the compiler

// U = 16-byte loads in flight per lane and tensor, MINB = resident CTAs per SM asked of the compiler.  (8, 4) is the
// fastest form of the kernel by itself (99 % of the copy bandwidth); (4, 8) needs half the registers per CTA and is
// what the decode step uses while the shared-prompt kernel occupies part of every SM (1259 against 1272 ms per 255
// config-4 steps, although by itself it reaches 95 %).
template <typename T, int D, int U_, int MINB_>
__global__ void __launch_bounds__(128, MINB_)
decode_attn_kernel(const T* __restrict__ q, long long q_stride, KvView kv, const int* __restrict__ len0,
                   const int* __restrict__ start1, const int* __restrict__ len1, const int* __restrict__ step_ptr,
                   const float* __restrict__ prefix_o, const float* __restrict__ prefix_lse,
                   const T* __restrict__ gate, long long gate_stride, T* __restrict__ y, long long y_stride,
                   float* __restrict__ ws_ml, float* __restrict__ ws_o, float* __restrict__ part_o,
                   float* __restrict__ part_lse, int n_splits, int R, int H, float scale_log2) {
  using Cfg = DecodeCfg<T, D>;
  constexpr int VEC = Cfg::VEC, LPT = Cfg::LPT, TPW = Cfg::TPW;
  dep_wait();
  const long long rh = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rh >= (long long)R * H) return;
  const int r = (int)(rh / H), h = (int)(rh - (long long)r * H);
  const int lane = threadIdx.x & 31;
  const int g = lane / LPT, e = lane - g * LPT;
  const int split = blockIdx.y;
  const int step = step_ptr ? *step_ptr : 0;
  const bool have_prefix = prefix_lse != nullptr;
  // A range that would run past the sequence's slots is cut at the capacity (the append kernel reports such a
  // step through its status word); nothing outside the page table or the pool is ever read.
  const int cap = kv.page_table ? kv.max_pages * kv.page_tokens : kv.page_tokens;
  const int n0 = min(max((have_prefix || len0 == nullptr) ? 0 : len0[r], 0), cap);
  const int s1 = min(max(start1[r], 0), cap);
  const int n = n0 + min(max(len1[r] + step, 0), cap - s1);
  int chunk = (n + n_splits - 1) / n_splits;
  chunk = (chunk + 2 * TPW - 1) / (2 * TPW) * (2 * TPW);
  const int begin = split * chunk;
  const int end = min(n, begin + chunk);

  float qf[VEC];
  ld16<T>(q + (long long)r * q_stride + (long long)h * D + e * VEC, qf);
#pragma unroll
  for (int i = 0; i < VEC; ++i) qf[i] *= scale_log2;

  float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;

  const T* kbase = static_cast<const T*>(kv.k);
  const T* vbase = static_cast<const T*>(kv.v);
  constexpr int U = U_;
  // Walk the keys page by page: one page-table lookup per page, then a dense run of tokens.
  for (int i = begin; i < end;) {  // every quantity below is warp-uniform
    const bool in0 = i < n0;
    const int slot = in0 ? i : s1 + (i - n0);
    const int lp = slot / kv.page_tokens;
    const int in = slot - lp * kv.page_tokens;
    const int cnt = min((in0 ? min(n0, end) : end) - i, kv.page_tokens - in);
    long long pg = kv.page_table ? (long long)kv.page_table[(long long)r * kv.max_pages + lp] : (long long)r;
    if (kv.n_pages > 0 && (pg < 0 || pg >= kv.n_pages)) {  // a table entry outside the pool: skip its keys
      i += cnt;
      continue;
    }
    const long long base = pg * kv.page_stride + (long long)h * kv.head_stride + (long long)in * D + e * VEC;
    for (int t0 = 0; t0 < cnt; t0 += U * TPW) {
      uint4 kr[U], vr[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int t = t0 + u * TPW + g;
        ok[u] = t < cnt;
        kr[u] = vr[u] = make_uint4(0u, 0u, 0u, 0u);
        if (ok[u]) {
          kr[u] = *reinterpret_cast<const uint4*>(kbase + base + (long long)t * D);
          vr[u] = *reinterpret_cast<const uint4*>(vbase + base + (long long)t * D);
        }
      }
      float s[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float kf[VEC];
        unpack16<T>(kr[u], kf);
        float d = 0.f;
#pragma unroll
        for (int x = 0; x < VEC; ++x) d += qf[x] * kf[x];
        s[u] = d;  // 0 for a token past the end (its registers were cleared)
      }
#pragma unroll
      for (int o = LPT >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
      }
      if (ok[0]) {  // tokens of a lane group are valid in order, so ok[0] covers "any valid"
        float mb = s[0];
#pragma unroll
        for (int u = 1; u < U; ++u) mb = ok[u] ? fmaxf(mb, s[u]) : mb;
        const float mn = fmaxf(m, mb);
        const float resc = exp2f(m - mn);  // m = -inf -> 0
        l *= resc;
#pragma unroll
        for (int x = 0; x < VEC; ++x) acc[x] *= resc;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float pw = ok[u] ? exp2f(s[u] - mn) : 0.f;
          float vf[VEC];
          unpack16<T>(vr[u], vf);
          l += pw;
#pragma unroll
          for (int x = 0; x < VEC; ++x) acc[x] += pw * vf[x];
        }
        m = mn;
      }
    }
    i += cnt;
  }
  // merge the TPW lane groups (butterfly: every lane ends with the full state)
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
    float a2[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) a2[i] = __shfl_xor_sync(0xffffffffu, acc[i], o);
    merge_partial<VEC>(m, l, acc, m2, l2, a2);
  }
  if (g != 0) return;

  if (n_splits > 1) {  // ws_o comes first in the workspace, so every 16-byte store below is aligned
    const long long slot = (long long)split * R * H + rh;
    if (e == 0) {
      ws_ml[2 * slot] = m;
      ws_ml[2 * slot + 1] = l;
    }
    float* dst = ws_o + slot * D + e * VEC;
#pragma unroll
    for (int i = 0; i < VEC; i += 4)
      *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
    return;
  }
  if (part_lse) {  // normalised partial over this row's keys; the caller merges it with another partial later
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (e == 0) part_lse[rh] = l > 0.f ? (m + log2f(l)) * (1.f / kLog2e) : -INFINITY;
    float* dst = part_o + rh * D + e * VEC;
#pragma unroll
    for (int i = 0; i < VEC; i += 4)
      *reinterpret_cast<float4*>(dst + i) =
          make_float4(acc[i] * inv, acc[i + 1] * inv, acc[i + 2] * inv, acc[i + 3] * inv);
    return;
  }
  if (have_prefix) {
    const float mp = prefix_lse[rh] * kLog2e;  // normalised partial: l = 1
    float po[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(prefix_o + rh * D + e * VEC + i);
      po[i] = t.x; po[i + 1] = t.y; po[i + 2] = t.z; po[i + 3] = t.w;
    }
    merge_partial<VEC>(m, l, acc, mp, 1.f, po);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float out[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) out[i] = Io<T>::round(acc[i] * inv);
  if (gate) {
    float gf[VEC];
    ld16<T>(gate + (long long)r * gate_stride + (long long)h * D + e * VEC, gf);
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] *= Io<T>::round(1.f / (1.f + __expf(-gf[i])));
  }
  T* dst = y + (long long)r * y_stride + (long long)h * D + e * VEC;
#pragma unroll
  for (int i = 0; i < VEC; ++i) Io<T>::st(dst + i, out[i]);
}

// Second pass of the split path: one thread per (row, head, d).
template <typename T>
__global__ void decode_combine_kernel(const float* __restrict__ ws_ml, const float* __restrict__ ws_o, int n_splits,
                                      const float* __restrict__ prefix_o, const float* __restrict__ prefix_lse,
                                      const T* __restrict__ gate, long long gate_stride, T* __restrict__ y,
                                      long long y_stride, int R, int H, int D) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long RH = (long long)R * H;
  if (idx >= RH * D) return;
  const long long rh = idx / D;
  const int d = (int)(idx - rh * D);
  const int r = (int)(rh / H), h = (int)(rh - (long long)r * H);
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ws_ml[2 * (s * RH + rh)]);
  const float mp = prefix_lse ? prefix_lse[rh] * kLog2e : -INFINITY;
  m = fmaxf(m, mp);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = ws_ml[2 * (s * RH + rh)];
    const float w = ms == -INFINITY ? 0.f : exp2f(ms - m);
    l += ws_ml[2 * (s * RH + rh) + 1] * w;
    acc += ws_o[(s * RH + rh) * D + d] * w;
  }
  if (prefix_lse) {
    const float w = mp == -INFINITY ? 0.f : exp2f(mp - m);
    l += w;
    acc += prefix_o[rh * D + d] * w;
  }
  float out = Io<T>::round(l > 0.f ? acc / l : 0.f);
  if (gate) out *= Io<T>::round(1.f / (1.f + __expf(-Io<T>::ld(gate + (long long)r * gate_stride + (long long)h * D + d))));
  Io<T>::st(y + (long long)r * y_stride + (long long)h * D + d, out);
}

// Merge of two normalised partials (o, lse) per (row, head), then the sigmoid gate; one thread per 16 bytes of y.
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ oa, const float* __restrict__ lsea,
                                  const float* __restrict__ ob, const float* __restrict__ lseb,
                                  const T* __restrict__ gate, long long gate_stride, T* __restrict__ y,
                                  long long y_stride, int R, int H, int D) {
  constexpr int VEC = Io<T>::kVec16;
  dep_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long RH = (long long)R * H;
  const int DV = D / VEC;
  if (idx >= RH * DV) return;
  const long long rh = idx / DV;
  const int d = (int)(idx - rh * DV) * VEC;
  const int r = (int)(rh / H), h = (int)(rh - (long long)r * H);
  const float ma = lsea[rh], mb = lseb[rh];
  const float m = fmaxf(ma, mb);
  float wa = 0.f, wb = 0.f;
  if (m != -INFINITY) {
    wa = __expf(ma - m);  // exp(-inf) = 0 for an empty side
    wb = __expf(mb - m);
    const float inv = 1.f / (wa + wb);
    wa *= inv;
    wb *= inv;
  }
  float out[VEC];
#pragma unroll
  for (int i = 0; i < VEC; i += 4) {
    const float4 a = *reinterpret_cast<const float4*>(oa + rh * D + d + i);
    const float4 b = *reinterpret_cast<const float4*>(ob + rh * D + d + i);
    out[i] = a.x * wa + b.x * wb;
    out[i + 1] = a.y * wa + b.y * wb;
    out[i + 2] = a.z * wa + b.z * wb;
    out[i + 3] = a.w * wa + b.w * wb;
  }
  const long long col = (long long)h * D + d;
#pragma unroll
  for (int i = 0; i < VEC; ++i) out[i] = Io<T>::round(out[i]);
  if (gate) {
    float gf[VEC];
    ld16<T>(gate + (long long)r * gate_stride + col, gf);
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] *= Io<T>::round(1.f / (1.f + __expf(-gf[i])));
  }
  st16<T>(y + (long long)r * y_stride + col, out, 1.f);
}

template <typename T, int D>
static int decode_launch(const void* q, long long q_stride, const KvView& kv, const int* len0, const int* start1,
                         const int* len1, const int* step_ptr, const float* prefix_o, const float* prefix_lse,
                         const void* gate, long long gate_stride, void* y, long long y_stride, float* ws,
                         int n_splits, int R, int H, cudaStream_t st, float* part_o = nullptr,
                         float* part_lse = nullptr) {
  const long long RH = (long long)R * H;
  // Workspace = [n_splits][R*H][D] accumulators, then [n_splits][R*H][2] (max, sum).  The accumulators are written
  // with 16-byte stores and D is a multiple of 4 floats, so with the block first they are aligned for every R*H*n_splits.
  float* ws_o = ws;
  float* ws_ml = ws ? ws + RH * n_splits * D : nullptr;
  const float scale_log2 = kLog2e / sqrtf((float)D);
  dim3 grid((unsigned)((RH + 3) / 4), (unsigned)n_splits);
  if (part_lse)  // runs beside the shared-prompt kernel: the lighter form (the full form there: 1280 against 1255 ms)
    launch_dep(decode_attn_kernel<T, D, kDecLoads / 2, kDecMinCtas * 2>, grid, dim3(128), 0, st, static_cast<const T*>(q),
               q_stride, kv, len0, start1, len1, step_ptr, prefix_o, prefix_lse, static_cast<const T*>(gate), gate_stride,
               static_cast<T*>(y), y_stride, ws_ml, ws_o, part_o, part_lse, n_splits, R, H, scale_log2);
  else
    launch_dep(decode_attn_kernel<T, D, kDecLoads, kDecMinCtas>, grid, dim3(128), 0, st, static_cast<const T*>(q),
               q_stride, kv, len0, start1, len1, step_ptr, prefix_o, prefix_lse, static_cast<const T*>(gate), gate_stride,
               static_cast<T*>(y), y_stride, ws_ml, ws_o, part_o, part_lse, n_splits, R, H, scale_log2);
  if (int e = launch_status("decode_attn")) return e;
  if (n_splits > 1) {
    const long long n = RH * D;
    decode_combine_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        ws_ml, ws_o, n_splits, prefix_o, prefix_lse, static_cast<const T*>(gate), gate_stride, static_cast<T*>(y),
        y_stride, R, H, D);
    return launch_status("decode_combine");
  }
  return DGPT_OK;
}

}  // namespace dgpt

using namespace dgpt;

extern "C" size_t dgpt_decode_attn_workspace_bytes(int32_t R, int32_t H, int32_t D, int32_t n_splits) {
  if (n_splits <= 1) return 0;
  const size_t bytes = (size_t)R * H * n_splits * (size_t)(D + 2) * sizeof(float);
  return (bytes + 15) & ~(size_t)15;
}

extern "C" int dgpt_decode_attn(const void* q, int64_t q_row_stride, const dgpt_kv_layout* kv, const int32_t* len0,
                                const int32_t* start1, const int32_t* len1, const int32_t* step_ptr,
                                const float* prefix_o, const float* prefix_lse, const void* gate,
                                int64_t gate_row_stride, void* y, int64_t y_row_stride, void* workspace,
                                size_t workspace_bytes, int32_t n_splits, int32_t R, int32_t H, int32_t D,
                                int32_t dtype, void* stream) {
  DGPT_REQUIRE(q && y && len0 && start1 && len1, "decode_attn: NULL pointer");
  DGPT_REQUIRE(R >= 0 && H > 0 && n_splits >= 1 && n_splits <= 65535, "decode_attn: bad sizes");
  DGPT_REQUIRE((prefix_o == nullptr) == (prefix_lse == nullptr), "decode_attn: prefix_o and prefix_lse go together");
  DGPT_REQUIRE(q_row_stride % 8 == 0 && y_row_stride % 8 == 0 && gate_row_stride % 8 == 0,
               "decode_attn: row strides must be multiples of 8 elements");
  if (int e = validate_kv(kv, D)) return e;
  if (R == 0) return DGPT_OK;
  const size_t need = dgpt_decode_attn_workspace_bytes(R, H, D, n_splits);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
    set_error("decode_attn: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return DGPT_E_WORKSPACE;
  }
  DGPT_REQUIRE(need == 0 || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
               "decode_attn: the workspace must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const KvView view = make_view(kv);
  float* ws = static_cast<float*>(workspace);
#define DGPT_DEC(TT, DD)                                                                                         \
  return decode_launch<TT, DD>(q, q_row_stride, view, len0, start1, len1, step_ptr, prefix_o, prefix_lse, gate, \
                               gate_row_stride, y, y_row_stride, ws, n_splits, R, H, st)
  if (dtype == DGPT_F32) {
    switch (D) {
      case 8: DGPT_DEC(float, 8);
      case 16: DGPT_DEC(float, 16);
      case 32: DGPT_DEC(float, 32);
      case 64: DGPT_DEC(float, 64);
      case 128: DGPT_DEC(float, 128);
    }
  } else if (dtype == DGPT_BF16) {
    switch (D) {
      case 8: DGPT_DEC(__nv_bfloat16, 8);
      case 16: DGPT_DEC(__nv_bfloat16, 16);
      case 32: DGPT_DEC(__nv_bfloat16, 32);
      case 64: DGPT_DEC(__nv_bfloat16, 64);
      case 128: DGPT_DEC(__nv_bfloat16, 128);
      case 256: DGPT_DEC(__nv_bfloat16, 256);
    }
  }
#undef DGPT_DEC
  set_error("decode_attn: dtype %d with head_dim %d is not built", dtype, D);
  return DGPT_E_UNSUPPORTED;
}

// ---- the two halves of dgpt_decode_attn as separate launches ---------------------------------------
// The shared-prompt contraction and the per-row pass are independent until the merge, so a caller may
// run them on two streams; the merge waits for both.
extern "C" int dgpt_decode_attn_partial(const void* q, int64_t q_row_stride, const dgpt_kv_layout* kv,
                                        const int32_t* len0, const int32_t* start1, const int32_t* len1,
                                        const int32_t* step_ptr, float* part_o, float* part_lse, int32_t R,
                                        int32_t H, int32_t D, int32_t dtype, void* stream) {
  DGPT_REQUIRE(q && part_o && part_lse && start1 && len1, "decode_attn_partial: NULL pointer");
  DGPT_REQUIRE(R >= 0 && H > 0, "decode_attn_partial: bad sizes");
  DGPT_REQUIRE(q_row_stride % 8 == 0, "decode_attn_partial: row strides must be multiples of 8 elements");
  if (int e = validate_kv(kv, D)) return e;
  if (R == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const KvView view = make_view(kv);
#define DGPT_DEC(TT, DD)                                                                                           \
  return decode_launch<TT, DD>(q, q_row_stride, view, len0, start1, len1, step_ptr, nullptr, nullptr, nullptr, 0, \
                               nullptr, 0, nullptr, 1, R, H, st, part_o, part_lse)
  if (dtype == DGPT_F32) {
    switch (D) {
      case 8: DGPT_DEC(float, 8);
      case 16: DGPT_DEC(float, 16);
      case 32: DGPT_DEC(float, 32);
      case 64: DGPT_DEC(float, 64);
      case 128: DGPT_DEC(float, 128);
    }
  } else if (dtype == DGPT_BF16) {
    switch (D) {
      case 8: DGPT_DEC(__nv_bfloat16, 8);
      case 16: DGPT_DEC(__nv_bfloat16, 16);
      case 32: DGPT_DEC(__nv_bfloat16, 32);
      case 64: DGPT_DEC(__nv_bfloat16, 64);
      case 128: DGPT_DEC(__nv_bfloat16, 128);
      case 256: DGPT_DEC(__nv_bfloat16, 256);
    }
  }
#undef DGPT_DEC
  set_error("decode_attn_partial: dtype %d with head_dim %d is not built", dtype, D);
  return DGPT_E_UNSUPPORTED;
}

extern "C" int dgpt_attn_merge(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                               const void* gate, int64_t gate_row_stride, void* y, int64_t y_row_stride, int32_t R,
                               int32_t H, int32_t D, int32_t dtype, void* stream) {
  DGPT_REQUIRE(o_a && lse_a && o_b && lse_b && y, "attn_merge: NULL pointer");
  DGPT_REQUIRE(R >= 0 && H > 0 && D > 0 && D % 8 == 0, "attn_merge: head_dim must be a multiple of 8");
  DGPT_REQUIRE(y_row_stride % 8 == 0 && gate_row_stride % 8 == 0,
               "attn_merge: row strides must be multiples of 8 elements");
  if (R == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long n = (long long)R * H * (D / (dtype == DGPT_F32 ? 4 : 8));
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == DGPT_F32) {
    launch_dep(attn_merge_kernel<float>, dim3(blocks), dim3(256), 0, st, o_a, lse_a, o_b, lse_b,
               static_cast<const float*>(gate), gate_row_stride, static_cast<float*>(y), y_row_stride, R, H, D);
  } else if (dtype == DGPT_BF16) {
    launch_dep(attn_merge_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, o_a, lse_a, o_b, lse_b,
               static_cast<const __nv_bfloat16*>(gate), gate_row_stride, static_cast<__nv_bfloat16*>(y), y_row_stride,
               R, H, D);
  } else {
    set_error("attn_merge: dtype %d is not built", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("attn_merge");
}

// ---- split-K decode attention for callers that cannot allocate ------------------------------------
// The split-K partials normally live in a workspace the caller allocates.  Some callers have no
// allocator at hand at the point where they launch: code running under a framework that forbids
// cudaMalloc on its hot path, a plugin that is handed only its input and output buffers, or a
// latency-critical loop that must not touch the allocator.  For them the partials go into this
// fixed array, which every GPU that loads the library carries until the process exits.
namespace dgpt {
constexpr size_t kStaticScratchFloats = (size_t)4 << 20;  // 16 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
// Device address of the array, per device, filled on first use.  Host threads may race to fill an entry; they all
// store the same value.  The addresses belong to this process's contexts: after cudaDeviceReset they are stale.
static std::atomic<float*> g_scratch_addr[kMaxDevices];

// Host code sees `g_decode_scratch` only as a stand-in for the symbol; the address a kernel can use has
// to be asked for, with the device that will run the kernel current.
static int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("decode_attn_static: cannot identify the current device (%s)", cudaGetErrorString(e));
    return DGPT_E_CUDA;
  }
  float* known = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (known == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("decode_attn_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return DGPT_E_CUDA;
    }
    known = static_cast<float*>(p);
    g_scratch_addr[dev].store(known, std::memory_order_release);
  }
  *out = known;
  return DGPT_OK;
}
}  // namespace dgpt

extern "C" size_t dgpt_decode_attn_static_capacity_bytes(void) { return dgpt::kStaticScratchFloats * sizeof(float); }

extern "C" int dgpt_decode_attn_static(const void* q, int64_t q_row_stride, const dgpt_kv_layout* kv,
                                       const int32_t* len0, const int32_t* start1, const int32_t* len1,
                                       const int32_t* step_ptr, const float* prefix_o, const float* prefix_lse,
                                       const void* gate, int64_t gate_row_stride, void* y, int64_t y_row_stride,
                                       int32_t n_splits, int32_t R, int32_t H, int32_t D, int32_t dtype,
                                       void* stream) {
  DGPT_REQUIRE(q && y && len0 && start1 && len1, "decode_attn_static: NULL pointer");
  DGPT_REQUIRE(R >= 0 && H > 0 && n_splits >= 1 && n_splits <= 65535, "decode_attn_static: bad sizes");
  DGPT_REQUIRE((prefix_o == nullptr) == (prefix_lse == nullptr), "decode_attn_static: prefix_o and prefix_lse go together");
  DGPT_REQUIRE(q_row_stride % 8 == 0 && y_row_stride % 8 == 0 && gate_row_stride % 8 == 0,
               "decode_attn_static: row strides must be multiples of 8 elements");
  if (int e = validate_kv(kv, D)) return e;
  if (R == 0) return DGPT_OK;
  const size_t need = dgpt_decode_attn_workspace_bytes(R, H, D, n_splits);
  if (need > dgpt_decode_attn_static_capacity_bytes()) {
    set_error("decode_attn_static: R=%d H=%d D=%d n_splits=%d needs %zu bytes of partials, the built-in scratch holds %zu; "
              "use fewer splits or dgpt_decode_attn with a caller workspace",
              R, H, D, n_splits, need, dgpt_decode_attn_static_capacity_bytes());
    return DGPT_E_WORKSPACE;
  }
  float* ws = nullptr;
  if (int e = scratch_for_current_device(&ws)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const KvView view = make_view(kv);
#define DGPT_DECS(TT, DD)                                                                                        \
  return decode_launch<TT, DD>(q, q_row_stride, view, len0, start1, len1, step_ptr, prefix_o, prefix_lse, gate, \
                               gate_row_stride, y, y_row_stride, ws, n_splits, R, H, st)
  if (dtype == DGPT_F32) {
    switch (D) {
      case 8: DGPT_DECS(float, 8);
      case 16: DGPT_DECS(float, 16);
      case 32: DGPT_DECS(float, 32);
      case 64: DGPT_DECS(float, 64);
      case 128: DGPT_DECS(float, 128);
    }
  } else if (dtype == DGPT_BF16) {
    switch (D) {
      case 8: DGPT_DECS(__nv_bfloat16, 8);
      case 16: DGPT_DECS(__nv_bfloat16, 16);
      case 32: DGPT_DECS(__nv_bfloat16, 32);
      case 64: DGPT_DECS(__nv_bfloat16, 64);
      case 128: DGPT_DECS(__nv_bfloat16, 128);
      case 256: DGPT_DECS(__nv_bfloat16, 256);
    }
  }
#undef DGPT_DECS
  set_error("decode_attn_static: dtype %d with head_dim %d is not built", dtype, D);
  return DGPT_E_UNSUPPORTED;
}
