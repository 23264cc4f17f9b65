// Row-wise fused kernels: embedding gather + RMSNorm, Block-Attention-Residual
// depth mix + RMSNorm, SwiGLU, logit soft-cap, and the host-side error plumbing.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace dgpt {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return DGPT_E_CUDA;
  }
  return DGPT_OK;
}

// Dependent launches are off unless DGPT_DEP_LAUNCH=1 is in the environment (read at every launch, so both
// forms can be compared in one process).  Measured on the config-4 decode step: 1291 ms per 255 steps with
// them, 1272 ms without - blocks made resident early take room from the kernel that is still running.
bool dep_launch_enabled() {
  const char* e = getenv("DGPT_DEP_LAUNCH");
  return e && e[0] == '1';
}

// ---- embedding gather + RMSNorm ---------------------------------------------
// One warp per token.  The row is read twice (second read hits L1/L2).
template <typename T>
__global__ void embed_rmsnorm_kernel(const int* __restrict__ ids, const T* __restrict__ emb,
                                     T* __restrict__ out, long long n_tokens, int C, int V) {
  const long long tok = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n_tokens) return;
  const int lane = threadIdx.x & 31;
  int id = ids[tok];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const T* row = emb + (long long)id * C;
  float ss = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float x = Io<T>::ld(row + c);
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)C + kRmsEps);
  T* o = out + tok * C;
  for (int c = lane; c < C; c += 32) Io<T>::st(o + c, Io<T>::ld(row + c) * inv);
}

// ---- depth mix --------------------------------------------------------------
constexpr int kMaxCands = 64;
struct CandPtrs {
  const void* p[kMaxCands];
  unsigned char mult[kMaxCands];  // how many times the candidate occurs in the caller's list (read once, weighted)
  const float* inv[kMaxCands];    // rsqrt(mean(cand^2) + eps) per row from an earlier mix over the same data, or NULL
};

// One warp per row, one pass over the candidates with an online softmax across
// them: each candidate row is read exactly once and nothing is indexed
// dynamically in registers.  Lane l owns elements l + 32*i  (i < EPL).
template <typename T, int EPL>
__global__ void depthmix_kernel(CandPtrs cands, int n_cands, const T* __restrict__ w,
                                T* __restrict__ out_h, T* __restrict__ out_rn, long long rows, int C) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float acc[EPL], wv[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    acc[i] = 0.f;
    const int c = lane + 32 * i;
    wv[i] = (n_cands > 1 && c < C) ? Io<T>::ld(w + c) : 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int n = 0; n < n_cands; ++n) {
    const T* src = static_cast<const T*>(cands.p[n]) + row * C;
    float v[EPL];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int c = lane + 32 * i;
      v[i] = c < C ? Io<T>::ld(src + c) : 0.f;
      ss += v[i] * v[i];
    }
    if (n_cands == 1) {
#pragma unroll
      for (int i = 0; i < EPL; ++i) acc[i] = v[i];
      l = 1.f;
      break;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)C + kRmsEps);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) dot += Io<T>::round(v[i] * inv) * wv[i];
    dot = Io<T>::round(warp_sum(dot));
    const float m_new = fmaxf(m, dot);
    const float resc = __expf(m - m_new);
    const float p = __expf(dot - m_new) * (float)cands.mult[n];
    l = l * resc + p;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[i] = acc[i] * resc + p * v[i];
    m = m_new;
  }
  const float invl = 1.f / l;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    acc[i] = Io<T>::round(acc[i] * invl);
    ss += acc[i] * acc[i];
  }
  if (out_h) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int c = lane + 32 * i;
      if (c < C) Io<T>::st(out_h + row * C + c, acc[i]);
    }
  }
  if (out_rn) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)C + kRmsEps);
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int c = lane + 32 * i;
      if (c < C) Io<T>::st(out_rn + row * C + c, acc[i] * inv);
    }
  }
}

// Same algorithm with 16-byte accesses: lane l owns vectors l + 32*i (i < NV) of VEC elements each.
// Used when n_embd is a multiple of VEC and every pointer is 16-byte aligned.
template <typename T, int NV>
__global__ void __launch_bounds__(128, 4)
depthmix_vec_kernel(CandPtrs cands, int n_cands, const T* __restrict__ w, T* __restrict__ out_h,
                    T* __restrict__ out_rn, float* __restrict__ inv_out, int inv_out_index, long long rows, int C) {
  constexpr int VEC = Io<T>::kVec16;
  constexpr int E = NV * VEC;
  dep_wait();
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = C / VEC;
  float acc[E], wv[E];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = lane + 32 * i;
#pragma unroll
    for (int x = 0; x < VEC; ++x) acc[i * VEC + x] = wv[i * VEC + x] = 0.f;
    if (n_cands > 1 && j < nvec) ld16<T>(w + j * VEC, wv + i * VEC);
  }
  float m = -INFINITY, l = 0.f;
  // The candidates are reduced one after another (online softmax), so the rows of the next ones are
  // fetched (as raw 16-byte words) before the current one is reduced, to keep loads in flight.
#ifndef DGPT_MIX_AHEAD
#define DGPT_MIX_AHEAD 1  // candidates in flight beyond the current one (2 and 3 measured slower)
#endif
  constexpr int AHEAD = DGPT_MIX_AHEAD;
  uint4 nxt[AHEAD][NV];
  float inv_nxt = 0.f;  // the cached norm factor of the candidate in nxt[0], when it has one (AHEAD == 1)
  auto fetch = [&](int n, uint4* dst) {
    if (AHEAD == 1 && cands.inv[n]) inv_nxt = cands.inv[n][row];
    const T* src = static_cast<const T*>(cands.p[n]) + row * C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int j = lane + 32 * i;
      dst[i] = j < nvec ? *reinterpret_cast<const uint4*>(src + j * VEC) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
#pragma unroll
  for (int a = 0; a < AHEAD; ++a)
    if (a < n_cands) fetch(a, nxt[a]);
  for (int n = 0; n < n_cands; ++n) {
    float v[E];
    const bool cached = AHEAD == 1 && cands.inv[n] != nullptr;  // warp-uniform
    const float inv_cached = inv_nxt;
#pragma unroll
    for (int i = 0; i < NV; ++i) unpack16<T>(nxt[0][i], v + i * VEC);
#pragma unroll
    for (int a = 0; a + 1 < AHEAD; ++a) {
#pragma unroll
      for (int i = 0; i < NV; ++i) nxt[a][i] = nxt[a + 1][i];
    }
    if (n + AHEAD < n_cands) fetch(n + AHEAD, nxt[AHEAD - 1]);
    if (n_cands == 1) {
#pragma unroll
      for (int x = 0; x < E; ++x) acc[x] = v[x];
      l = 1.f;
      break;
    }
    // logit = rms_norm(v) . w = rsqrt(mean(v^2) + eps) * (v . w): both sums in one sweep and one
    // interleaved butterfly.  (The reference rounds rms_norm(v) to the storage type before the
    // product; for bf16 that changes the logit by ~1e-4 of its own rounding step.)
    // A committed candidate does not change between mixes, so its norm factor is computed by the first mix that
    // sees it and handed to the later ones: they skip the sum of squares and its half of the butterfly.  The
    // factor is the same number either way (same code computed it), so results do not depend on the cache.
    float s4[4] = {0.f, 0.f, 0.f, 0.f}, d4[4] = {0.f, 0.f, 0.f, 0.f};
    float inv;
    float dr;
    if (cached) {
#pragma unroll
      for (int x = 0; x < E; ++x) d4[x & 3] += v[x] * wv[x];
      dr = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dr += __shfl_xor_sync(0xffffffffu, dr, o);
      inv = inv_cached;
    } else {
#pragma unroll
      for (int x = 0; x < E; ++x) {
        s4[x & 3] += v[x] * v[x];
        d4[x & 3] += v[x] * wv[x];
      }
      float ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
      dr = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        dr += __shfl_xor_sync(0xffffffffu, dr, o);
      }
      inv = rsqrtf(ss / (float)C + kRmsEps);
      if (n == inv_out_index && lane == 0) inv_out[row] = inv;
    }
    const float dot = Io<T>::round(dr * inv);
    if (dot > m) {  // warp-uniform: the accumulator is rescaled only when the running maximum moves
      const float resc = __expf(m - dot);
      l *= resc;
#pragma unroll
      for (int x = 0; x < E; ++x) acc[x] *= resc;
      m = dot;
    }
    const float pw = __expf(dot - m) * (float)cands.mult[n];
    l += pw;
#pragma unroll
    for (int x = 0; x < E; ++x) acc[x] += pw * v[x];
  }
  const float invl = 1.f / l;
  float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int x = 0; x < E; ++x) {
    acc[x] = Io<T>::round(acc[x] * invl);
    s4[x & 3] += acc[x] * acc[x];
  }
  const float ss = warp_sum((s4[0] + s4[1]) + (s4[2] + s4[3]));
  const float inv = rsqrtf(ss / (float)C + kRmsEps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = lane + 32 * i;
    if (j >= nvec) continue;
    if (out_h) st16<T>(out_h + row * C + j * VEC, acc + i * VEC, 1.f);
    if (out_rn) st16<T>(out_rn + row * C + j * VEC, acc + i * VEC, inv);
  }
}

template <typename T>
static bool depthmix_vec_ok(const CandPtrs& cp, int n, const void* w, void* out_h, void* out_rn, int C) {
  constexpr int VEC = Io<T>::kVec16;
  if (C % VEC != 0 || C / VEC > 32 * 8) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  for (int i = 0; i < n; ++i)
    if (!al(cp.p[i])) return false;
  return al(w) && al(out_h) && al(out_rn);
}

template <typename T>
static int depthmix_launch(const CandPtrs& cp, int n, const void* w, void* out_h, void* out_rn, float* inv_out,
                           int inv_out_index, bool uses_cache, long long rows, int C, cudaStream_t st) {
  const int warps = 4;
  const unsigned grid = (unsigned)((rows + warps - 1) / warps);
  const bool vec = depthmix_vec_ok<T>(cp, n, w, out_h, out_rn, C);
  if (uses_cache && !vec) {
    set_error("depthmix: cached norm factors need 16-byte aligned rows of a multiple of %d elements", Io<T>::kVec16);
    return DGPT_E_UNSUPPORTED;
  }
  if (vec) {
    const int nv = (C / Io<T>::kVec16 + 31) / 32;
#define DGPT_MIXV(N)                                                                              \
  launch_dep(depthmix_vec_kernel<T, N>, dim3(grid), dim3(warps * 32), 0, st, cp, n, static_cast<const T*>(w), \
             static_cast<T*>(out_h), static_cast<T*>(out_rn), inv_out, inv_out_index, rows, C)
    if (nv <= 1) DGPT_MIXV(1);
    else if (nv <= 2) DGPT_MIXV(2);
    else if (nv <= 3) DGPT_MIXV(3);
    else if (nv <= 4) DGPT_MIXV(4);
    else DGPT_MIXV(8);
#undef DGPT_MIXV
    return launch_status("depthmix");
  }
  const int epl = (C + 31) / 32;
#define DGPT_MIX(E)                                                                        \
  depthmix_kernel<T, E><<<grid, warps * 32, 0, st>>>(cp, n, static_cast<const T*>(w),      \
                                                     static_cast<T*>(out_h), static_cast<T*>(out_rn), rows, C)
  if (epl <= 2) DGPT_MIX(2);
  else if (epl <= 4) DGPT_MIX(4);
  else if (epl <= 8) DGPT_MIX(8);
  else if (epl <= 16) DGPT_MIX(16);
  else if (epl <= 24) DGPT_MIX(24);
  else if (epl <= 32) DGPT_MIX(32);
  else if (epl <= 64) DGPT_MIX(64);
  else {
    set_error("depthmix: n_embd %d > 2048 is not built", C);
    return DGPT_E_UNSUPPORTED;
  }
#undef DGPT_MIX
  return launch_status("depthmix");
}

// ---- SwiGLU -----------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, long long n_pairs, float alpha,
                              float limit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  float g = Io<T>::ld(in + 2 * i), lin = Io<T>::ld(in + 2 * i + 1);
  g = fminf(g, limit);
  lin = fminf(fmaxf(lin, -limit), limit);
  // the reference materialises alpha*g, sigmoid(.), g*sig and lin+1 in the storage type
  const float sg = Io<T>::round(1.f / (1.f + __expf(-Io<T>::round(alpha * g))));
  const float a = Io<T>::round(g * sg);
  Io<T>::st(out + i, a * Io<T>::round(lin + 1.f));
}

template <>
__global__ void swiglu_kernel<__nv_bfloat16>(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                             long long n_pairs, float alpha, float limit) {
  // 4 pairs (16 bytes in, 8 bytes out) per thread
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= n_pairs) return;
  using B = Io<__nv_bfloat16>;
  if (i4 + 4 <= n_pairs) {
    float x[8];
    ld16<__nv_bfloat16>(in + 2 * i4, x);
    __nv_bfloat16 r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float g = fminf(x[2 * k], limit);
      const float lin = fminf(fmaxf(x[2 * k + 1], -limit), limit);
      const float sg = B::round(__fdividef(1.f, 1.f + __expf(-B::round(alpha * g))));
      r[k] = __float2bfloat16_rn(B::round(g * sg) * B::round(lin + 1.f));
    }
    *reinterpret_cast<uint2*>(out + i4) = *reinterpret_cast<uint2*>(r);
  } else {
    for (long long i = i4; i < n_pairs; ++i) {
      const float g = fminf(B::ld(in + 2 * i), limit);
      const float lin = fminf(fmaxf(B::ld(in + 2 * i + 1), -limit), limit);
      const float sg = B::round(__fdividef(1.f, 1.f + __expf(-B::round(alpha * g))));
      B::st(out + i, B::round(g * sg) * B::round(lin + 1.f));
    }
  }
}

// ---- soft cap ---------------------------------------------------------------
template <typename T>
__global__ void softcap_kernel(T* x, long long n, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Io<T>::st(x + i, cap * Io<T>::round(tanhf(Io<T>::round(Io<T>::ld(x + i) / cap))));
}

__global__ void step_advance_kernel(int* step, int delta) { *step += delta; }

// ---- y *= sigmoid(gate) -------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* y, long long y_stride, const T* __restrict__ gate, long long g_stride,
                                    long long rows, int n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * n) return;
  const long long r = i / n;
  const int c = (int)(i - r * n);
  const float sg = Io<T>::round(1.f / (1.f + __expf(-Io<T>::ld(gate + r * g_stride + c))));
  T* p = y + r * y_stride + c;
  Io<T>::st(p, Io<T>::ld(p) * sg);
}

}  // namespace dgpt

using namespace dgpt;

extern "C" {

int dgpt_last_error(char* buf, size_t n) {
  const size_t len = strlen(g_err);
  if (buf && n) {
    strncpy(buf, g_err, n - 1);
    buf[n - 1] = 0;
  }
  return (int)len;
}

int dgpt_version(void) { return 1; }

int dgpt_embed_rmsnorm(const int32_t* ids, const void* emb, void* out, int64_t n_tokens, int32_t C, int32_t V,
                       int32_t dtype, void* stream) {
  DGPT_REQUIRE(ids && emb && out, "embed_rmsnorm: NULL pointer");
  DGPT_REQUIRE(n_tokens >= 0 && C > 0 && V > 0, "embed_rmsnorm: bad sizes");
  if (n_tokens == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int warps = 4;
  const unsigned grid = (unsigned)((n_tokens + warps - 1) / warps);
  if (dtype == DGPT_F32)
    embed_rmsnorm_kernel<float><<<grid, warps * 32, 0, st>>>(ids, static_cast<const float*>(emb),
                                                            static_cast<float*>(out), n_tokens, C, V);
  else if (dtype == DGPT_BF16)
    embed_rmsnorm_kernel<__nv_bfloat16><<<grid, warps * 32, 0, st>>>(
        ids, static_cast<const __nv_bfloat16*>(emb), static_cast<__nv_bfloat16*>(out), n_tokens, C, V);
  else {
    set_error("embed_rmsnorm: unknown dtype %d", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("embed_rmsnorm");
}

int dgpt_depthmix_cached(const void* const* cands, const float* const* cand_inv, int32_t n_cands, const void* w,
                         void* out_h, void* out_rn, float* inv_out, int32_t inv_out_index, int64_t rows, int32_t C,
                         int32_t dtype, void* stream) {
  DGPT_REQUIRE(cands && n_cands >= 1 && n_cands <= kMaxCands, "depthmix: n_cands must be in [1, %d]", kMaxCands);
  DGPT_REQUIRE(n_cands == 1 || w, "depthmix: pseudo-query w is NULL");
  DGPT_REQUIRE(out_h || out_rn, "depthmix: no output requested");
  DGPT_REQUIRE(rows >= 0 && C > 0, "depthmix: bad sizes");
  DGPT_REQUIRE(inv_out == nullptr || (inv_out_index >= 0 && inv_out_index < n_cands),
               "depthmix: inv_out_index must name a candidate");
  DGPT_REQUIRE(inv_out == nullptr || cand_inv == nullptr || cand_inv[inv_out_index] == nullptr,
               "depthmix: the candidate whose norm factor is to be written must not have one passed in");
  if (rows == 0) return DGPT_OK;
  // A candidate listed several times (the reference commits the embedding twice) is read once and its
  // softmax weight multiplied: p v + p v = 2 p v exactly.
  CandPtrs cp;
  int n_unique = 0, out_index = -1;
  bool uses_cache = inv_out != nullptr;
  for (int i = 0; i < n_cands; ++i) {
    DGPT_REQUIRE(cands[i], "depthmix: candidate %d is NULL", i);
    int j = 0;
    while (j < n_unique && cp.p[j] != cands[i]) ++j;
    if (j == n_unique) {
      cp.p[n_unique] = cands[i];
      cp.inv[n_unique] = cand_inv ? cand_inv[i] : nullptr;
      uses_cache = uses_cache || cp.inv[n_unique] != nullptr;
      cp.mult[n_unique++] = 1;
    } else {
      ++cp.mult[j];
    }
    if (inv_out && i == inv_out_index) out_index = j;
  }
  n_cands = n_unique;
  if (n_cands == 1) out_index = -1;  // a single candidate is passed through: no norm factor is formed
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == DGPT_F32)
    return depthmix_launch<float>(cp, n_cands, w, out_h, out_rn, inv_out, out_index, uses_cache, rows, C, st);
  if (dtype == DGPT_BF16)
    return depthmix_launch<__nv_bfloat16>(cp, n_cands, w, out_h, out_rn, inv_out, out_index, uses_cache, rows, C, st);
  set_error("depthmix: unknown dtype %d", dtype);
  return DGPT_E_UNSUPPORTED;
}

int dgpt_depthmix(const void* const* cands, int32_t n_cands, const void* w, void* out_h, void* out_rn,
                  int64_t rows, int32_t C, int32_t dtype, void* stream) {
  return dgpt_depthmix_cached(cands, nullptr, n_cands, w, out_h, out_rn, nullptr, -1, rows, C, dtype, stream);
}

int dgpt_swiglu(const void* in, void* out, int64_t rows, int32_t n_out, float alpha, float limit, int32_t dtype,
                void* stream) {
  DGPT_REQUIRE(in && out, "swiglu: NULL pointer");
  DGPT_REQUIRE(rows >= 0 && n_out > 0, "swiglu: bad sizes");
  const long long n = (long long)rows * n_out;
  if (n == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == DGPT_F32) {
    swiglu_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<const float*>(in),
                                                                     static_cast<float*>(out), n, alpha, limit);
  } else if (dtype == DGPT_BF16) {
    DGPT_REQUIRE((reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0,
                 "swiglu: bf16 buffers must be 16-byte aligned");
    const long long nt = (n + 3) / 4;
    swiglu_kernel<__nv_bfloat16><<<(unsigned)((nt + 255) / 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), n, alpha, limit);
  } else {
    set_error("swiglu: unknown dtype %d", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("swiglu");
}

int dgpt_softcap(void* logits, int64_t n, float cap, int32_t dtype, void* stream) {
  DGPT_REQUIRE(logits && n >= 0 && cap >= 0.f, "softcap: bad arguments");
  if (n == 0 || cap == 0.f) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == DGPT_F32)
    softcap_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(logits), n, cap);
  else if (dtype == DGPT_BF16)
    softcap_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16*>(logits), n, cap);
  else {
    set_error("softcap: unknown dtype %d", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("softcap");
}

int dgpt_step_advance(int32_t* step_ptr, int32_t delta, void* stream) {
  DGPT_REQUIRE(step_ptr, "step_advance: NULL pointer");
  step_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(step_ptr, delta);
  return launch_status("step_advance");
}

}  // extern "C"

extern "C" int dgpt_sigmoid_gate(void* y, int64_t y_row_stride, const void* gate, int64_t gate_row_stride,
                                 int64_t rows, int32_t n_cols, int32_t dtype, void* stream) {
  DGPT_REQUIRE(y && gate && rows >= 0 && n_cols > 0, "sigmoid_gate: bad arguments");
  const long long n = (long long)rows * n_cols;
  if (n == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == DGPT_F32)
    sigmoid_gate_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(y), y_row_stride,
                                                     static_cast<const float*>(gate), gate_row_stride, rows, n_cols);
  else if (dtype == DGPT_BF16)
    sigmoid_gate_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16*>(y), y_row_stride,
                                                             static_cast<const __nv_bfloat16*>(gate), gate_row_stride,
                                                             rows, n_cols);
  else {
    set_error("sigmoid_gate: unknown dtype %d", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  return launch_status("sigmoid_gate");
}
