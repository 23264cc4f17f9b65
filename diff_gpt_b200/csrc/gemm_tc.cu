// tcgen05 / TMEM GEMM for the linear layers of the decode step (sm_100a), with the SwiGLU of the
// feed-forward block in its epilogue.
//
//   acc[m, n] = sum_k A[m, k] * W[n, k]        A: activations [M, K] bf16, W: nn.Linear weight [N, K] bf16
//   mode 0:  out[m, n]     = bf16(acc[m, n])
//   mode 1:  out[m, n / 2] = swiglu(bf16(acc[m, n]), bf16(acc[m, n + 1]))   for even n  (interleaved gate / linear)
//   mode 2:  out[m, n]     = bf16(resid[m, n] + acc[m, n])                    (the residual add of addmm, one rounding)
//   mode 3:  nothing is stored: row m keeps the best key of  key[m, n] = cap(bf16(acc[m, n])) / T + Gumbel noise(m, n)
//            (no noise and T = 1 for an arg-max) in best[m], a 64-bit word (order-preserving key bits, ~n) raised with
//            atomicMax - the tied-embedding head with the draw in its epilogue, so [M, N] logits never reach HBM
//
// Persistent, warp-specialised CTAs of 320 threads, one per SM, tiles of 128 x BN outputs (BN = 256, 192 or 128,
// whichever needs the fewest rounds of tiles over the SMs) taken round robin:
//   warp 9, lane 0  loader: TMA loads of the A (128 x 64) and W (BN x 64) blocks, 128-byte swizzle, ring of 4
//   warp 8, lane 0  issuer: four tcgen05.mma (M 128, N BN, K 16) per block into one of two TMEM accumulators
//   warps 0-7       epilogue: warp w owns the 32 output rows (TMEM lanes) 32 (w % 4) .. and the column half w / 4;
//                   it reads the finished accumulator 32 columns at a time, applies the epilogue and stores bf16
// so the epilogue of tile i runs while the tensor cores work on tile i + 1.  No cluster, no multicast.
// What bounds it: every CTA pulls its own A and W blocks through L2, about 220 MB for the 4096 x 3072 x 768 GEMM of
// the decode step, and the GPU delivers about 10 TB/s of that (cuBLAS's two-CTA tiles move less and take 18.5 us
// against 25 us here).  Tiles of 256 rows (two MMAs per W block) were measured: fewer bytes, but too few tiles to
// fill 148 SMs evenly and no overlapped epilogue - 30.7 us.
// Every mbarrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, is reported through
// the status word, and every role drains what it issued before TMEM is freed.
#include "linear.cuh"
#include "sampling.cuh"
#include "tcgen05.cuh"

namespace dgpt {
namespace tc {

constexpr int kGM = 128, kGK = 64, kGStages = 4;  // the tile is 128 x BN outputs, BN = 256, 192 or 128
constexpr uint32_t kGABytes = kGM * 128;
constexpr int kGThreads = 320;  // 8 epilogue warps, the MMA issuer's warp, the loader's warp
constexpr int kGEpiThreads = 256;
__host__ __device__ constexpr uint32_t gemm_idesc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kGM >> 4) << 24);
}

struct GemmParams {
  __nv_bfloat16* out;
  long long out_rs;
  const __nv_bfloat16* resid;  // mode 2: added to the accumulator before the one rounding (may alias out)
  long long resid_rs;
  int M, N, K, mode;
  float alpha, limit;
  int* status;
  HeadDraw draw;  // mode 3
};

// order-preserving map of a float onto unsigned integers
__device__ __forceinline__ uint32_t float_order_bits(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// DRAW selects the fourth epilogue at compile time, so that the three storing epilogues do not carry its registers
// and branches (with the mode tested at run time the feed-forward GEMM took 21.1 instead of 17.7 us on 2048 rows).
template <int BN, bool DRAW>
__global__ void __launch_bounds__(kGThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap ma, const __grid_constant__ CUtensorMap mw, const GemmParams p) {
  constexpr int kGN = BN;
  constexpr uint32_t kGBBytes = kGN * 128, kGStageBytes = kGABytes + kGBBytes;
  constexpr uint32_t kGIdesc = gemm_idesc(BN);
  constexpr int kAccStride = 256;  // TMEM columns between the two accumulators
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kGStages * kGStageBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t a0 = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kGStages, bar_accf = bar_empty + 8 * kGStages,
                 bar_acce = bar_accf + 16, bar_drain = bar_acce + 16;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_n = (p.N + kGN - 1) / kGN, tiles_m = (p.M + kGM - 1) / kGM;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (p.K + kGK - 1) / kGK;

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kGStages; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_accf + 8 * i, 1);
      mbar_init(bar_acce + 8 * i, kGEpiThreads);
    }
    mbar_init(bar_drain, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  dep_wait();  // everything above touched only this CTA's own shared memory and TMEM

  if (warp == 9) {
    // ================= loader =================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&ma)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mw)) : "memory");
      int last[kGStages];  // parity of the newest load per slot (for the drain on failure)
      for (int i = 0; i < kGStages; ++i) last[i] = -1;
      unsigned it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
        const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % kGStages;
          const uint32_t ph = (it / kGStages) & 1u;
          ok = wait_or_abort(bar_empty + 8 * s, ph ^ 1u, abort_flag, 32);  // a fresh barrier passes parity 1
          if (!ok) break;
          const uint32_t dst = a0 + s * kGStageBytes;
          mbar_expect_tx(bar_full + 8 * s, kGStageBytes);  // rows or columns outside the matrices are zero-filled and counted
          tma_load_2d(dst, &ma, bar_full + 8 * s, kb * kGK, tm * kGM);
          tma_load_2d(dst + kGABytes, &mw, bar_full + 8 * s, kb * kGK, tn * kGN);
          last[s] = (int)ph;
        }
      }
      if (!ok || *abort_flag) {
        if (p.status) atomicExch(p.status, *abort_flag ? *abort_flag : 32);
        for (int i = 0; i < kGStages; ++i)
          if (last[i] >= 0) mbar_wait(bar_full + 8 * i, (uint32_t)last[i]);  // bounded: let copies in flight land
      }
    }
  } else if (warp == 8) {
    // ================= MMA issuer =================
    if (lane == 0) {
      unsigned it = 0, t_local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++t_local) {
        const int a = t_local & 1;
        ok = wait_or_abort(bar_acce + 8 * a, ((t_local >> 1) & 1u) ^ 1u, abort_flag, 33);  // epilogue has emptied it
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % kGStages;
          ok = wait_or_abort(bar_full + 8 * s, (it / kGStages) & 1u, abort_flag, 34);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = a0 + s * kGStageBytes, sb = sa + kGABytes;
#pragma unroll
          for (int ks = 0; ks < kGK / 16; ++ks)
            umma_ss(tmem + a * kAccStride, smem_desc(sa + ks * 32, 16, 1024), smem_desc(sb + ks * 32, 16, 1024), kGIdesc,
                    (kb > 0 || ks > 0) ? 1u : 0u);
          umma_commit(bar_empty + 8 * s);  // the slot is free once these MMAs have read it
        }
        if (ok) umma_commit(bar_accf + 8 * a);
      }
      if (!ok || *abort_flag) {
        if (p.status) atomicExch(p.status, *abort_flag ? *abort_flag : 34);
        umma_commit(bar_drain);  // completes when everything issued so far has finished
        mbar_wait(bar_drain, 0);
      }
    }
  } else {
    // ================= epilogue =================
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // a warp reaches the TMEM lanes of its quarter only
    const int c_begin = (warp >> 2) * (kGN / 2);
    unsigned t_local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++t_local) {
      const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
      const int a = t_local & 1;
      ok = wait_or_abort(bar_accf + 8 * a, (t_local >> 1) & 1u, abort_flag, 35);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective: the warp leaves together
      if (!ok) break;
      tc_fence_after();
      const int row = tm * kGM + (warp & 3) * 32 + lane;
      const int col0 = tn * kGN;
      float best_v = -INFINITY;  // mode 3: this thread's best key over its columns of the tile, and where
      int best_n = 0x7fffffff;
      long long traj = 0;
      int step = 0;
      if (DRAW && row < p.M) {
        traj = p.draw.traj_ids ? p.draw.traj_ids[row] : p.draw.traj_id0 + row;
        step = p.draw.step_base + (p.draw.step_ptr ? *p.draw.step_ptr : 0);
      }
#pragma unroll 1
      for (int c = c_begin; c < c_begin + kGN / 2; c += 32) {
        float v[32];
        tmem_ld32(lane_addr + a * kAccStride + c, v);  // all lanes load; stores below are predicated
        if (row >= p.M) continue;
        if constexpr (DRAW) {
          using B = Io<__nv_bfloat16>;
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // four columns per random-number block
            const int n0 = col0 + c + 4 * q;
            if (n0 >= p.N) break;  // N is a multiple of 16
            uint32_t rnd[4] = {0u, 0u, 0u, 0u};
            if (p.draw.inv_temperature > 0.f)
              philox4x32_10_words((uint32_t)traj, (uint32_t)((unsigned long long)traj >> 32), (uint32_t)step,
                                  0x80000000u | (uint32_t)(n0 >> 2), p.draw.seed_lo, p.draw.seed_hi, rnd);
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              float z = B::round(v[4 * q + x]);  // the logit as a bf16 Linear would have written it
              if (p.draw.cap > 0.f) z = softcap_value<__nv_bfloat16>(z, p.draw.cap);
              float key = z;
              if (p.draw.inv_temperature > 0.f) {
                const float u = ((float)(rnd[x] >> 8) + 0.5f) * (1.f / 16777216.f);  // in (0, 1)
                key = z * p.draw.inv_temperature - __logf(-__logf(u));              // arg-max of these keys ~ softmax(z / T)
              }
              if (key > best_v) {  // columns are visited in increasing order: the lowest index wins ties
                best_v = key;
                best_n = n0 + x;
              }
            }
          }
          continue;
        }
        if (DRAW) continue;
        if (p.mode == 0 || p.mode == 2) {
          __nv_bfloat16* dst = p.out + (long long)row * p.out_rs + col0 + c;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (col0 + c + 8 * q >= p.N) break;  // N is a multiple of 8
            if (p.mode == 2) {
              float r8[8];
              ld16<__nv_bfloat16>(p.resid + (long long)row * p.resid_rs + col0 + c + 8 * q, r8);
#pragma unroll
              for (int x = 0; x < 8; ++x) v[8 * q + x] += r8[x];
            }
            st16<__nv_bfloat16>(dst + 8 * q, v + 8 * q, 1.f);
          }
        } else {
          using B = Io<__nv_bfloat16>;
          float r[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            // the reference's Linear writes bf16 before the activation reads it
            const float g = fminf(B::round(v[2 * k]), p.limit);
            const float lin = fminf(fmaxf(B::round(v[2 * k + 1]), -p.limit), p.limit);
            const float sg = B::round(__fdividef(1.f, 1.f + __expf(-B::round(p.alpha * g))));
            r[k] = B::round(g * sg) * B::round(lin + 1.f);
          }
          __nv_bfloat16* dst = p.out + (long long)row * p.out_rs + ((col0 + c) >> 1);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            if (col0 + c + 16 * q >= p.N) break;  // N is a multiple of 16
            st16<__nv_bfloat16>(dst + 8 * q, r + 8 * q, 1.f);
          }
        }
      }
      if (DRAW && row < p.M && best_n != 0x7fffffff)
        atomicMax(p.draw.best + row, ((unsigned long long)float_order_bits(best_v) << 32) | (uint32_t)(~(uint32_t)best_n));
      tc_fence_before();
      mbar_arrive(bar_acce + 8 * a);
    }
    if (!ok && p.status && tid == 0) atomicExch(p.status, *abort_flag ? *abort_flag : 35);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// The bounded wait by itself: two threads (of two warps) wait on a barrier that only one arrival could complete.  With
// `arrive` set the first thread arrives and both waits succeed; without it nothing ever arrives, the first
// wait gives up after `limit_cycles`, raises the flag, the second thread sees the flag and gives up too.
// out[0], out[1]: 1 where the wait succeeded; out[2]: the flag (the code of the wait that gave up);
// out[3]: clock cycles the first thread spent.
__global__ void bounded_wait_probe_kernel(int arrive, long long limit_cycles, int* out) {
  __shared__ uint64_t bar;
  __shared__ int flag;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    flag = 0;
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0 && arrive) mbar_arrive(b);
  if (threadIdx.x == 0 || threadIdx.x == 32) {  // two warps; the second has a limit it will not reach
    const int who = threadIdx.x >> 5;
    const long long t0 = clock64();
    const bool ok = wait_or_abort(b, 0, &flag, 40 + who, who == 0 ? limit_cycles : 16 * limit_cycles);
    out[who] = ok ? 1 : 0;
    if (who == 0) out[3] = (int)min(clock64() - t0, (long long)0x7fffffff);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[2] = flag;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with a [box_rows][64] box, 128-byte swizzle.
static bool encode_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long row_stride,
                      int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t ones[2] = {1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, ones,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("linear: cuTensorMapEncodeTiled failed with %d", (int)r);
    return false;
  }
  return true;
}

}  // namespace tc
}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_bounded_wait_probe(int32_t arrive, int64_t limit_cycles, int32_t* out, void* stream) {
  DGPT_REQUIRE(out, "bounded_wait_probe: NULL pointer");
  DGPT_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll, "bounded_wait_probe: limit must be in (0, 2e9] cycles");
  tc::bounded_wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(arrive, limit_cycles, out);
  return launch_status("bounded_wait_probe");
}

int dgpt::linear_launch(const void* a, int64_t a_row_stride, const void* w, int64_t w_row_stride, void* out,
                        int64_t out_row_stride, const void* resid, int64_t resid_row_stride, int32_t M, int32_t N,
                        int32_t K, int32_t epilogue, float alpha, float limit, int32_t dtype, int32_t* status,
                        const HeadDraw* draw, void* stream) {
  DGPT_REQUIRE(a && w && (out || epilogue == 3), "linear: NULL pointer");
  DGPT_REQUIRE(M >= 0 && N > 0 && K > 0, "linear: bad sizes");
  DGPT_REQUIRE(epilogue >= 0 && epilogue <= 3, "linear: epilogue must be 0 (store), 1 (SwiGLU of interleaved pairs), 2 (add) or 3 (draw)");
  DGPT_REQUIRE(epilogue != 2 || resid, "linear: epilogue 2 needs the matrix to add");
  DGPT_REQUIRE(epilogue != 3 || (draw && draw->best), "linear: epilogue 3 needs the draw parameters");
  if (dtype != DGPT_BF16) {
    set_error("linear: only bf16 is built (dtype %d)", dtype);
    return DGPT_E_UNSUPPORTED;
  }
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(a) || !al(w) || (out && !al(out)) || K % 8 != 0 || N % 16 != 0 || a_row_stride % 8 != 0 || w_row_stride % 8 != 0 ||
      out_row_stride % 8 != 0 || (epilogue == 2 && (!al(resid) || resid_row_stride % 8 != 0))) {
    set_error("linear: pointers must be 16-byte aligned, K and the row strides multiples of 8, N a multiple of 16");
    return DGPT_E_UNSUPPORTED;
  }
  if (M == 0) return DGPT_OK;
  if (!tc::device_is_sm100() || tc::encode_fn() == nullptr) {
    set_error("linear: needs an sm_100 device and cuTensorMapEncodeTiled");
    return DGPT_E_UNSUPPORTED;
  }
  // Tile width: the one that needs the fewest rounds of tiles over the SMs, then the widest (fewest bytes moved)
  static int n_sm[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("linear: cudaGetDevice failed");
    return DGPT_E_CUDA;
  }
  if (n_sm[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaSuccess;
    const int big = (int)((size_t)tc::kGStages * (tc::kGABytes + 256 * 128) + 256 + 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::gemm_tc_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::gemm_tc_kernel<192, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::gemm_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::gemm_tc_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::gemm_tc_kernel<192, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::gemm_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e != cudaSuccess || n <= 0) {
      set_error("linear: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return DGPT_E_CUDA;
    }
    n_sm[dev] = n;
  }
  const int tiles_m = (M + tc::kGM - 1) / tc::kGM;
  int bn = 256;
  double best = 1e30;
  for (int cand : {256, 192, 128}) {
    const int tiles = tiles_m * ((N + cand - 1) / cand);
    const double cost = (double)((tiles + n_sm[dev] - 1) / n_sm[dev]) * cand;  // rounds x time of one tile
    if (cost < best - 1e-9) {
      best = cost;
      bn = cand;
    }
  }
  CUtensorMap ma, mw;
  if (!tc::encode_2d(&ma, a, M, K, a_row_stride, tc::kGM) || !tc::encode_2d(&mw, w, N, K, w_row_stride, bn))
    return DGPT_E_CUDA;
  tc::GemmParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_rs = out_row_stride;
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.resid_rs = resid_row_stride;
  p.M = M; p.N = N; p.K = K; p.mode = epilogue;
  p.alpha = alpha; p.limit = limit;
  p.status = status;
  if (draw) p.draw = *draw;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)tc::kGStages * (tc::kGABytes + (size_t)bn * 128) + 256 + 1024;
  const int tiles = tiles_m * ((N + bn - 1) / bn);
  const int grid = tiles < n_sm[dev] ? tiles : n_sm[dev];
  if (epilogue == 3) {
    if (bn == 256) launch_dep(tc::gemm_tc_kernel<256, true>, dim3(grid), dim3(tc::kGThreads), smem, st, ma, mw, p);
    else if (bn == 192) launch_dep(tc::gemm_tc_kernel<192, true>, dim3(grid), dim3(tc::kGThreads), smem, st, ma, mw, p);
    else launch_dep(tc::gemm_tc_kernel<128, true>, dim3(grid), dim3(tc::kGThreads), smem, st, ma, mw, p);
  } else if (bn == 256) launch_dep(tc::gemm_tc_kernel<256, false>, dim3(grid), dim3(tc::kGThreads), smem, st, ma, mw, p);
  else if (bn == 192) launch_dep(tc::gemm_tc_kernel<192, false>, dim3(grid), dim3(tc::kGThreads), smem, st, ma, mw, p);
  else launch_dep(tc::gemm_tc_kernel<128, false>, dim3(grid), dim3(tc::kGThreads), smem, st, ma, mw, p);
  return launch_status("linear");
}

extern "C" int dgpt_linear(const void* a, int64_t a_row_stride, const void* w, int64_t w_row_stride, void* out,
                           int64_t out_row_stride, const void* resid, int64_t resid_row_stride, int32_t M, int32_t N,
                           int32_t K, int32_t epilogue, float alpha, float limit, int32_t dtype, int32_t* status,
                           void* stream) {
  DGPT_REQUIRE(epilogue >= 0 && epilogue <= 2, "linear: epilogue must be 0 (store), 1 (SwiGLU of interleaved pairs) or 2 (add)");
  return linear_launch(a, a_row_stride, w, w_row_stride, out, out_row_stride, resid, resid_row_stride, M, N, K, epilogue, alpha,
                       limit, dtype, status, nullptr, stream);
}
