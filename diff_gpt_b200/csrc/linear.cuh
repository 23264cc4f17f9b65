// The tcgen05 GEMM of gemm_tc.cu as seen by other translation units of the library.
#pragma once

#include "common.cuh"

namespace dgpt {

// Epilogue 3 of the GEMM: the tied-embedding head with the draw of the next token in its epilogue.
struct HeadDraw {
  float cap = 0.f;              // logit soft-cap (0 = none)
  float inv_temperature = 0.f;  // 0 = arg-max, else 1 / temperature
  uint32_t seed_lo = 0, seed_hi = 0;
  long long traj_id0 = 0;
  const long long* traj_ids = nullptr;  // per-row ids of the random stream (else traj_id0 + row)
  int step_base = 0;
  const int* step_ptr = nullptr;
  unsigned long long* best = nullptr;   // [M], zero before the launch
};

// dgpt_linear with the fourth epilogue reachable (draw != nullptr, epilogue == 3, out may be NULL).
int linear_launch(const void* a, int64_t a_row_stride, const void* w, int64_t w_row_stride, void* out,
                  int64_t out_row_stride, const void* resid, int64_t resid_row_stride, int32_t M, int32_t N, int32_t K,
                  int32_t epilogue, float alpha, float limit, int32_t dtype, int32_t* status, const HeadDraw* draw,
                  void* stream);

}  // namespace dgpt
