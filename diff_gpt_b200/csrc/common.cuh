// Shared helpers for the libdgpt_b200 kernels: storage-type traits, warp/block
// reductions, KV page addressing and host-side error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dgpt.h"

namespace dgpt {

// ---- host-side error text (thread local) ------------------------------------
void set_error(const char* fmt, ...);
int launch_status(const char* what);  // cudaGetLastError -> DGPT_OK / DGPT_E_CUDA

#define DGPT_REQUIRE(cond, ...)     \
  do {                              \
    if (!(cond)) {                  \
      dgpt::set_error(__VA_ARGS__); \
      return DGPT_E_ARG;            \
    }                               \
  } while (0)

// ---- programmatic dependent launch ----------------------------------------------
// A kernel launched through launch_dep may be made resident while the previous kernel on its stream is
// still draining (that hides most of the launch latency between two dependent kernels); it must call
// dep_wait() before it touches anything the previous kernel wrote.  dep_wait() is a no-op otherwise.
bool dep_launch_enabled();
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... P, typename... A>
inline void launch_dep(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dep_launch_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);  // errors surface through launch_status()
}

constexpr float kRmsEps = 1.1920928955078125e-07f;  // FLT_EPSILON: F.rms_norm's default eps
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---- storage types ----------------------------------------------------------
template <typename T>
struct Io;

template <>
struct Io<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
  static constexpr int kVec16 = 4;  // elements in 16 bytes
};

template <>
struct Io<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
  }
  static constexpr int kVec16 = 8;
};

// 16-byte vector load of VEC = 16/sizeof(T) consecutive elements, widened to fp32.
template <typename T>
__device__ __forceinline__ void ld16(const T* p, float* out);

template <>
__device__ __forceinline__ void ld16<float>(const float* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}

template <>
__device__ __forceinline__ void ld16<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// 16-byte vector store of VEC fp32 values scaled by `s` and rounded to the storage type.
template <typename T>
__device__ __forceinline__ void st16(T* p, const float* v, float s);

template <>
__device__ __forceinline__ void st16<float>(float* p, const float* v, float s) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0] * s, v[1] * s, v[2] * s, v[3] * s);
}

template <>
__device__ __forceinline__ void st16<__nv_bfloat16>(__nv_bfloat16* p, const float* v, float s) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i] * s, v[2 * i + 1] * s);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Widen the VEC elements held in one raw 16-byte register quad.
template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float* out);

template <>
__device__ __forceinline__ void unpack16<float>(const uint4& v, float* out) {
  out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y);
  out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
}

template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float* out) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// ---- reductions -------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum, result broadcast to every thread.  `scratch` holds >= 33 floats.
// The summation order is fixed (lane tree, then warp order), so results are reproducible.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---- KV page addressing -----------------------------------------------------
struct KvView {
  void* k;
  void* v;
  long long page_stride;
  long long head_stride;
  const int* page_table;
  int page_tokens;
  int max_pages;
  long long n_pages;  // pages addressable through the table (0 = not stated)
};

inline KvView make_view(const dgpt_kv_layout* l) {
  KvView w;
  w.k = l->k_base;
  w.v = l->v_base;
  w.page_stride = l->page_stride;
  w.head_stride = l->head_stride;
  w.page_table = l->page_table;
  w.page_tokens = l->page_tokens;
  w.max_pages = l->max_pages;
  w.n_pages = l->page_table ? l->n_pages : 0;
  return w;
}

// Element offset of (seq, head, slot, d = 0) inside the K or V storage of one layer.
__device__ __forceinline__ long long kv_offset(const KvView& kv, int seq, int head, int slot, int D) {
  const int lp = slot / kv.page_tokens;
  const int in = slot - lp * kv.page_tokens;
  const long long pg = kv.page_table ? (long long)kv.page_table[(long long)seq * kv.max_pages + lp]
                                     : (long long)seq;
  return pg * kv.page_stride + (long long)head * kv.head_stride + (long long)in * D;
}

inline int validate_kv(const dgpt_kv_layout* kv, int D) {
  DGPT_REQUIRE(kv != nullptr && kv->k_base && kv->v_base, "kv layout or its base pointers are NULL");
  DGPT_REQUIRE(kv->page_tokens > 0, "kv.page_tokens must be positive");
  DGPT_REQUIRE(kv->page_table == nullptr || kv->max_pages > 0, "kv.max_pages must be positive with a page table");
  DGPT_REQUIRE(kv->head_stride % 8 == 0 && kv->page_stride % 8 == 0, "kv strides must be multiples of 8 elements");
  DGPT_REQUIRE((reinterpret_cast<uintptr_t>(kv->k_base) & 15) == 0 && (reinterpret_cast<uintptr_t>(kv->v_base) & 15) == 0,
               "kv base pointers must be 16-byte aligned");
  (void)D;
  return DGPT_OK;
}

}  // namespace dgpt
