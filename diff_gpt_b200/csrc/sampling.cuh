// Pieces shared by the sampling kernel and the sampling epilogue of the head GEMM: the counter-based random
// stream and the logit soft-cap with the reference's rounding points.
#pragma once

#include "common.cuh"

namespace dgpt {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// Philox4x32-10 (Salmon et al., SC'11): counter (c0..c3), key (k0,k1) -> first output word.
__device__ __forceinline__ uint32_t philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                  uint32_t k1) {
  uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c[0];
}

// All four output words of the same generator.
__device__ __forceinline__ void philox4x32_10_words(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                    uint32_t k1, uint32_t (&out)[4]) {
  uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = c[i];
}

// cap * tanh(x / cap) with the reference's rounding points (each op materialised in the storage type).
template <typename T>
__device__ __forceinline__ float softcap_value(float x, float cap) {
  return Io<T>::round(cap * Io<T>::round(tanhf(Io<T>::round(x / cap))));
}
// bf16 keeps 8 bits of tanh, so the short form 1 - 2 / (e^{2|t|} + 1) (absolute error about 2e-7) gives
// the same rounded value except within 2e-7 of a rounding boundary.
template <>
__device__ __forceinline__ float softcap_value<__nv_bfloat16>(float x, float cap) {
  using B = Io<__nv_bfloat16>;
  const float t = B::round(__fdividef(x, cap));
  const float th = 1.f - __fdividef(2.f, __expf(2.f * fabsf(t)) + 1.f);  // e^{2|t|} = inf gives 1
  return B::round(cap * B::round(copysignf(th, t)));
}

}  // namespace dgpt
