// tcgen05 / TMEM attention for bf16, head_dim 64 or 128 (sm_100a): causal / chunk prefill, and the
// shared-prompt phase of the Monte-Carlo decode (all trajectories of a series against the prompt K/V).
//
// Three kernels share the tensor maps and parameters built here:
//   fmha_tc_ws_kernel (fmha_ws.cu, impl = 2 of dgpt_fmha_prefill, chosen from 1024 keys on): persistent, warp-specialised,
//                     one query tile per work item, scores double-buffered in TMEM
//   fmha_tc_pp_kernel (fmha_pp.cu, impl = 4): persistent, two query tiles per work item
//   fmha_tc_kernel    (below, impl = 3): the small one
//
// fmha_tc_kernel (impl = 3 of dgpt_fmha_prefill; the earlier, simpler form): 128 threads, no
// fixed roles, 256 TMEM columns and two CTAs per SM so that one CTA's softmax overlaps the other's MMAs.
//
// No cluster launch and no multicast.  Every wait on an mbarrier is bounded in clock cycles; if one runs
// out the CTA stores the code of the waiting site in a status word, raises a CTA-wide abort flag so the
// other roles stop waiting too, drains what it issued, frees its TMEM and returns.
#include "fmha.cuh"
#include "tcgen05.cuh"

namespace dgpt {
namespace tc {

constexpr int kTmemCols = 256;    // S/P: [0,128), O tile: [128, 128 + D)


template <int D>
__global__ void __launch_bounds__(128, 2)
fmha_tc_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
               const __grid_constant__ CUtensorMap mv, const TcParams p) {
  constexpr int kSub = D / 64;                  // 64-element (128-byte) column blocks per row
  constexpr uint32_t kSubBytes = kBN * 128;     // one [128 rows][64 bf16] swizzled block
  constexpr uint32_t kTileBytes = kSub * kSubBytes;
  constexpr uint32_t kIdescS = instr_desc(kBN, false);
  constexpr uint32_t kIdescPV = instr_desc(D, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes);  // q, k, v, s, o
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar_q = smem_u32(bars), bar_k = bar_q + 8, bar_v = bar_q + 16, bar_s = bar_q + 24, bar_o = bar_q + 32;
  const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int pt = p.page_tokens;
  auto init_barriers = [&]() {  // thread 0; every phase of the previous work item has completed
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  };
  if (tid == 0) {
    *abort_flag = 0;
    init_barriers();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  bool fail = false;
  int pend_k = -1, pend_v = -1, pend_s = -1, pend_o = -1;  // thread 0: parity of an outstanding phase, or -1

  // A CTA takes the work items blockIdx.x, blockIdx.x + gridDim.x, ...  (one each when the grid covers them all;
  // a smaller grid keeps the kernel on few SMs, which is how the decode step runs it beside the per-row kernel).
  for (int work = blockIdx.x; work < p.n_work; work += gridDim.x) {
  if (work != (int)blockIdx.x) {  // barriers start every work item in phase 0
    __syncthreads();
    if (tid == 0) {
      asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_q) : "memory");
      asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_k) : "memory");
      asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_v) : "memory");
      asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_s) : "memory");
      asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_o) : "memory");
      init_barriers();
    }
    __syncthreads();
  }
  const int qt_idx = work % p.n_qt, bh = work / p.n_qt;
  const int h = bh % p.H, b = bh / p.H;
  const int qt = p.causal ? p.n_qt - 1 - qt_idx : qt_idx;  // long tiles first
  const int q0 = qt * kBM;
  const int klen = p.kv_len ? p.kv_len[b] : p.kv_len_all;
  const int kmax = p.causal ? min(klen, p.q_offset + min(q0 + kBM, p.Tq)) : klen;
  const int n_tiles = kmax > 0 ? (kmax + kBN - 1) / kBN : 0;

  // Issue the TMA loads of key/value tile j (thread 0 only).  One box per page and per 64-wide half.
  auto load_kv = [&](const CUtensorMap* map, uint32_t dst, uint32_t bar, int j) {
    const int t0 = j * kBN;
    if (pt >= kBN) {
      const int lp = t0 / pt, in = t0 - lp * pt;
      const int pg = p.page_table ? p.page_table[(long long)b * p.max_pages + lp] : b;
      mbar_expect_tx(bar, kTileBytes);
#pragma unroll
      for (int s = 0; s < kSub; ++s) tma_load_4d(dst + s * kSubBytes, map, bar, s * 64, in, h, pg);
    } else {
      const int per = kBN / pt;
      int valid = 0;
      for (int q = 0; q < per; ++q) valid += (t0 + q * pt < klen) ? 1 : 0;
      mbar_expect_tx(bar, (uint32_t)valid * pt * 128u * kSub);
      for (int q = 0; q < valid; ++q) {
        const int lp = t0 / pt + q;
        const int pg = p.page_table ? p.page_table[(long long)b * p.max_pages + lp] : b;
#pragma unroll
        for (int s = 0; s < kSub; ++s) tma_load_4d(dst + s * kSubBytes + q * pt * 128, map, bar, s * 64, 0, h, pg);
      }
    }
  };

  float m = -INFINITY, l = 0.f;

  if (tid == 0 && n_tiles > 0) {
    mbar_expect_tx(bar_q, kTileBytes);
#pragma unroll
    for (int s = 0; s < kSub; ++s) tma_load_4d(aQ + s * kSubBytes, &mq, bar_q, s * 64, h, q0, b);
    load_kv(&mk, aK, bar_k, 0);
    load_kv(&mv, aV, bar_v, 0);
    pend_k = pend_v = 0;
  }

  for (int j = 0; j < n_tiles; ++j) {
    const uint32_t par = (uint32_t)(j & 1);
    const int t0 = j * kBN;
    // ---- S = Q K^T ----
    if (tid == 0) {
      bool ok = true;
      if (j == 0) ok = wait_or_abort(bar_q, 0, abort_flag);
      ok = ok && wait_or_abort(bar_k, par, abort_flag);
      if (ok) {
        pend_k = -1;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (uint32_t)(ks >> 2) * kSubBytes + (uint32_t)(ks & 3) * 32u;
          umma_ss(tmem, smem_desc(aQ + off, 16, 1024), smem_desc(aK + off, 16, 1024), kIdescS, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_s);
        pend_s = (int)par;
      } else {
        fail = true;
      }
    }
    if (!wait_or_abort(bar_s, par, abort_flag)) fail = true;
    if (!wait_or_abort(bar_v, par, abort_flag)) fail = true;
    tc_fence_after();
    if (tid == 0 && !fail) {
      pend_s = -1;
      pend_v = -1;
      if (j + 1 < n_tiles) {
        load_kv(&mk, aK, bar_k, j + 1);  // the K buffer is free once S has been produced
        pend_k = (int)(par ^ 1u);
      }
    }
    // value rows past the end of the sequence may hold anything: clear them so that 0 * x stays 0
    const int valid_rows = klen - t0;
    if (valid_rows < kBN && tid >= valid_rows) {
#pragma unroll
      for (int s = 0; s < kSub; ++s) {
        uint4* row = reinterpret_cast<uint4*>(sV + s * kSubBytes + tid * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) row[c] = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_async_smem();
    }
    // ---- softmax of this row ----
    const bool need_mask = (t0 + kBN > klen) || (p.causal && t0 + kBN - 1 > p.q_offset + q0);
    const int last_key = p.causal ? min(klen - 1, p.q_offset + q0 + tid) : klen - 1;
    float sv[kBN];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld32_nowait(lane_addr + c * 32, &sv[c * 32]);
    tc_wait_ld();
    float mx = -INFINITY;
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < kBN; ++i) {
        sv[i] = (t0 + i <= last_key) ? sv[i] : -INFINITY;
        mx = fmaxf(mx, sv[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kBN; ++i) mx = fmaxf(mx, sv[i]);
    }
    // Lazy rescale: the running maximum only moves when the new one exceeds it by 2^8, so the
    // output accumulator in TMEM is touched rarely.  Exponents then stay below 2^8.
    const float mx2 = mx * p.scale_log2;
    float alpha = 1.f;
    if (mx2 > m + 8.f || m == -INFINITY) {
      alpha = (m == -INFINITY) ? 0.f : ex2(m - mx2);
      m = mx2;
    }
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float v[32];
        tmem_ld32(lane_addr + 128 + c * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= alpha;
        tmem_st32(lane_addr + 128 + c * 32, v);
      }
    }
    const float m_use = (m == -INFINITY) ? 0.f : m;
    float rowsum = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float p0 = ex2(fmaf(sv[c * 32 + i], p.scale_log2, -m_use));      // -inf -> 0
        const float p1 = ex2(fmaf(sv[c * 32 + i + 1], p.scale_log2, -m_use));
        rowsum += p0 + p1;
        const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
      }
      tmem_st16(lane_addr + c * 16, packed);  // P overwrites S, which this row now holds in registers
    }
    l = l * alpha + rowsum;
    tc_wait_st();
    tc_fence_before();
    if (__syncthreads_or(fail ? 1 : 0)) {
      fail = true;
      break;
    }
    // ---- O += P V (accumulated in TMEM across tiles) ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kBN / 16; ++ks)
        umma_ts(tmem + 128, tmem + ks * 8, smem_desc(aV + ks * 2048, kSubBytes, 1024), kIdescPV,
                (j > 0 || ks > 0) ? 1u : 0u);
      umma_commit(bar_o);
      pend_o = (int)par;
    }
    if (!wait_or_abort(bar_o, par, abort_flag)) fail = true;
    tc_fence_after();
    if (tid == 0 && !fail) {
      pend_o = -1;
      if (j + 1 < n_tiles) {
        load_kv(&mv, aV, bar_v, j + 1);
        pend_v = (int)(par ^ 1u);
      }
    }
    tc_fence_before();
    if (__syncthreads_or(fail ? 1 : 0)) {
      fail = true;
      break;
    }
  }

  if (!fail) {
    // tcgen05.ld is warp-collective: every thread reads its row, only rows that exist are stored
    const int qi = q0 + tid;
    const bool row_ok = qi < p.Tq;
    const float inv = (l > 0.f && n_tiles > 0) ? 1.f / l : 0.f;
    const long long off = (long long)b * p.o_bs + (long long)qi * p.o_rs + (long long)h * p.d_head;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      float v[32];
      if (n_tiles > 0) {  // CTA-uniform
        tmem_ld32(lane_addr + 128 + c * 32, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      if (row_ok && c * 32 < p.d_head) {
        if (p.o_f32) {
          float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.o) + off + c * 32);
#pragma unroll
          for (int d = 0; d < 32; d += 4)
            dst[d >> 2] = make_float4(v[d] * inv, v[d + 1] * inv, v[d + 2] * inv, v[d + 3] * inv);
        } else {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.o) + off + c * 32;
#pragma unroll
          for (int d = 0; d < 32; d += 8) st16<__nv_bfloat16>(dst + d, v + d, inv);
        }
      }
    }
    if (row_ok && p.lse) p.lse[((long long)b * p.Tq + qi) * p.H + h] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
    tc_fence_before();  // the next work item's MMAs overwrite the TMEM columns just read
  } else {
    if (tid == 0) {
      // a wait ran out: record it, then give whatever is still in flight a bounded chance to land
      if (p.status) atomicExch(p.status, 2);
      if (pend_k >= 0) mbar_wait(bar_k, (uint32_t)pend_k);
      if (pend_v >= 0) mbar_wait(bar_v, (uint32_t)pend_v);
      if (pend_s >= 0) mbar_wait(bar_s, (uint32_t)pend_s);
      if (pend_o >= 0) mbar_wait(bar_o, (uint32_t)pend_o);
    }
    break;  // CTA-uniform: `fail` left the tile loop through __syncthreads_or
  }
  }  // work items
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace tc

bool fmha_tc_supported(const FmhaArgs& a, const dgpt_kv_layout& kv) {
  if (a.dtype != DGPT_BF16 || (a.D != 32 && a.D != 64 && a.D != 128)) return false;
  const int pt = kv.page_tokens;
  if (!((pt >= tc::kBN && pt % tc::kBN == 0) || (pt >= 8 && pt < tc::kBN && tc::kBN % pt == 0))) return false;
  if (kv.page_table == nullptr && pt < tc::kBN) return false;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(a.q) || !al16(a.o) || !al16(kv.k_base) || !al16(kv.v_base)) return false;
  if (a.q_rs % 8 || a.q_bs % 8 || a.o_rs % 8 || a.o_bs % 8 || kv.head_stride % 8 || kv.page_stride % 8) return false;
  if (a.q_rs <= 0 || kv.head_stride <= 0 || kv.page_stride <= 0) return false;
  return tc::device_is_sm100() && tc::encode_fn() != nullptr;
}

int fmha_tc(const FmhaArgs& a, const dgpt_kv_layout& kv, cudaStream_t st) {
  using namespace tc;
  // head_dim 32 runs on the 64-wide kernels: the boxes stay 64 elements wide, the tensor is 32 wide, and the TMA
  // engine fills what lies outside the tensor with zeros - Q K^T and P V see zero columns and are unchanged
  const int d_head = a.D;
  const int D = d_head == 32 ? 64 : d_head;
  TcMaps maps;
  CUtensorMap &mq = maps.q, &mk = maps.k, &mv = maps.v;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)d_head, (cuuint64_t)a.H, (cuuint64_t)a.Tq, (cuuint64_t)a.B};
    const cuuint64_t q_bs = a.q_bs > 0 ? (cuuint64_t)a.q_bs : (cuuint64_t)a.q_rs * a.Tq;
    const cuuint64_t strides[3] = {(cuuint64_t)d_head * 2, (cuuint64_t)a.q_rs * 2, q_bs * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kBM, 1};
    if (!encode_map(&mq, a.q, dims, strides, box)) return DGPT_E_CUDA;
  }
  {
    const int pt = kv.page_tokens;
    cuuint64_t n_pages = kv.page_table ? (kv.n_pages > 0 ? (cuuint64_t)kv.n_pages : (cuuint64_t)1 << 24) : (cuuint64_t)a.B;
    const cuuint64_t dims[4] = {(cuuint64_t)d_head, (cuuint64_t)pt, (cuuint64_t)a.H, n_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)d_head * 2, (cuuint64_t)kv.head_stride * 2, (cuuint64_t)kv.page_stride * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)(pt < kBN ? pt : kBN), 1, 1};
    if (!encode_map(&mk, kv.k_base, dims, strides, box)) return DGPT_E_CUDA;
    if (!encode_map(&mv, kv.v_base, dims, strides, box)) return DGPT_E_CUDA;
  }
  TcParams p;
  p.kv_len = a.kv_len;
  p.kv_len_all = a.kv_len_all;
  p.page_table = kv.page_table;
  p.max_pages = kv.max_pages;
  p.page_tokens = kv.page_tokens;
  p.o = a.o;
  p.o_bs = a.o_bs;
  p.o_rs = a.o_rs;
  p.o_f32 = a.o_f32;
  p.lse = a.lse;
  p.H = a.H;
  p.Tq = a.Tq;
  p.q_offset = a.q_offset;
  p.causal = a.causal;
  p.scale_log2 = kLog2e / sqrtf((float)d_head);
  p.d_head = d_head;
  p.status = a.status;
  p.n_qt = (a.Tq + kBM - 1) / kBM;
  p.n_work = p.n_qt * a.H * a.B;
  p.BH = a.B * a.H;
  p.group_bh = p.BH;
  if (a.pingpong) {
    const long long span = a.causal ? (long long)a.Tq + a.q_offset
                                    : (a.kv_len ? (long long)kv.max_pages * kv.page_tokens : (long long)a.kv_len_all);
    return fmha_tc_pp_launch(a, maps, p, span, st);
  }
  dim3 grid((unsigned)p.n_qt, (unsigned)a.H, (unsigned)a.B);
  // >= 80 KB per CTA keeps residency at two CTAs per SM, which is what the 2 x 256 TMEM columns allow
  size_t smem = (size_t)3 * (D / 64) * kBN * 128 + 64 + 1024;
  if (smem < 80 * 1024) smem = 80 * 1024;
  cudaError_t e;
  if (!a.two_cta) {
    const long long span = a.causal ? (long long)a.Tq + a.q_offset
                                    : (a.kv_len ? (long long)kv.max_pages * kv.page_tokens : (long long)a.kv_len_all);
    return fmha_tc_ws_launch(a, maps, p, span, st);
  }
  // one CTA per work item, or fewer CTAs that loop over the items when the caller wants the kernel on few SMs
  const unsigned n_cta = (a.max_ctas > 0 && a.max_ctas < p.n_work) ? (unsigned)a.max_ctas : (unsigned)p.n_work;
  if (D == 64) {
    e = cudaFuncSetAttribute(fmha_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) fmha_tc_kernel<64><<<n_cta, 128, smem, st>>>(mq, mk, mv, p);
  } else {
    e = cudaFuncSetAttribute(fmha_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) fmha_tc_kernel<128><<<n_cta, 128, smem, st>>>(mq, mk, mv, p);
  }
  if (e != cudaSuccess) {
    set_error("fmha_tc: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return DGPT_E_CUDA;
  }
  return launch_status("fmha_tc");
}

}  // namespace dgpt
