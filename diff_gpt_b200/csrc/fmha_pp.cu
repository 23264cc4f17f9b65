// tcgen05 / TMEM attention with TWO query tiles per CTA taking turns on the tensor cores (sm_100a, bf16,
// head_dim 64 or 128): causal / chunk prefill and the shared-prompt phase of the Monte-Carlo decode.
//
// One persistent CTA of 384 threads per SM works through (query-tile pair, head, batch) items.  A pair is
// 2 x 128 query rows of one (batch, head); both tiles meet the same K/V tiles, so every K/V tile brought into
// shared memory feeds four MMAs instead of two, and while the softmax threads of one tile turn its scores into
// probabilities the tensor cores work on the other tile.
//   warp 9, lane 0   loader: TMA loads of the two Q tiles of an item and of its K / V tiles (128-byte swizzle, one
//                    box per page and per 64-wide half of D) into rings of KS K slots and VS V slots; it runs
//                    ahead of the consumers across item boundaries, so the next item's Q, K0 and V0 arrive while
//                    the current item's last tiles are still being worked on
//   warp 8, lane 0   issuer, per key tile j:  O0 += P0_j V_j;  S0 = Q0 K_{j+1}^T;  O1 += P1_j V_j;  S1 = Q1 K_{j+1}^T
//                    (each product waits only for what it needs: P of its tile, the K or V slot).  The eight MMAs of a
//                    product are one asm statement with constant descriptor steps: this lane shares its scheduler
//                    with two busy softmax warps, and every instruction it does not execute is time the tensor pipe
//                    does not wait for.
//   warps 0-3 / 4-7  softmax of query tile 0 / 1, one thread per query row: tcgen05.ld of the row's 128 scores; from
//                    the second key tile on the probabilities are taken against the running maximum at once, the
//                    tile's own maximum is found in the same sweep, and only a score more than 2^8 above the running
//                    maximum sends the tile through the careful path (maximum first, O in TMEM rescaled); one pair
//                    of exponentials in four is computed on the FMA pipe (range reduction + cubic) to take load off
//                    the exp2 unit; packed bf16 P is written over the scores it came from (tcgen05.st), one mbarrier
//                    arrival per row; at the end of an item the row normalises its O and stores it
//   warps 10-11      idle: they make the helper warps a whole warpgroup, so that it can hand registers to the softmax
//                    warpgroups (setmaxnreg: 216 per softmax thread, 72 per helper thread)
// TMEM columns: S0 / P0 [0,128)   S1 / P1 [128,256)   O0 [256, 256 + D)   O1 [384, 384 + D).
// P_t overwrites S_t, so S_t of the next key tile is issued behind the P_t V product of this one; the tensor
// pipe runs the MMAs of one thread in issue order, which is what makes the overwrite safe.
//
// What bounds it (measured on a B200, config-5 shapes): each query tile is one chain S -> softmax -> P V -> next S;
// the chains of the two tiles interleave, but every change between a product with A in shared memory (Q K^T) and one
// with A in TMEM (P V) drains the tensor pipe for about 250 cycles, four times per key tile, and a row's 128
// exponentials keep its thread busy for about 1700 cycles while the exp2 unit is shared with the other tile's warp.
// The kernel reaches 795 / 880 / 900 TFLOP/s at S = 4096 / 8192 / 16384 against 904 / 1010 / 1014 for the kernel with one
// query tile per CTA and double-buffered scores (fmha_tc_ws_kernel), which therefore stays the default for prefill;
// this one is selected with impl = 4, and the decode step uses it for the shared-prompt phase, where it owns 64 SMs
// while the HBM-bound per-row kernel has the others.
//
// Every mbarrier completes once per use; each role keeps its own running use count, so phases carry across items
// and nothing is re-initialised between them.  Items are dealt to the CTAs in groups of a few (batch, head) pairs
// whose K/V fit the L2 together, longest first, in snake order, so that CTAs finish together and co-resident CTAs
// read the same K/V.  No cluster launch and no multicast.  Every wait is bounded in clock cycles; a wait that runs
// out stores its site in the status word, raises the CTA-wide abort flag so that the other roles stop waiting too,
// the loader drains the copies it issued, and the CTA frees its TMEM and returns.
#include "fmha.cuh"
#include "fmha_sched.cuh"
#include "tcgen05.cuh"

namespace dgpt {
namespace tc {

constexpr int kPpThreads = 384;  // three warpgroups: softmax of tile 0, softmax of tile 1, and (issuer, loader, two idle warps)
constexpr int kPpSoftmaxRegs = 216, kPpHelperRegs = 72;  // registers per thread after the warpgroups trade them

constexpr uint32_t kPpTmemCols = 512;

struct PpItem {
  int b, h, q0, klen;
  int n[2];  // key tiles of the two query tiles (0 = the tile does not exist or sees no key)
  int nmax;
};

__device__ __forceinline__ PpItem pp_item(const TcParams& p, int bh, int pair) {
  PpItem it;
  it.h = bh % p.H;
  it.b = bh / p.H;
  it.q0 = pair * 2 * kBM;
  it.klen = p.kv_len ? p.kv_len[it.b] : p.kv_len_all;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = it.q0 + t * kBM;
    int kmax = 0;
    if (q0t < p.Tq) kmax = p.causal ? min(it.klen, p.q_offset + min(q0t + kBM, p.Tq)) : it.klen;
    it.n[t] = kmax > 0 ? (kmax + kBN - 1) / kBN : 0;
  }
  it.nmax = max(it.n[0], it.n[1]);
  return it;
}

template <int D, int PARTS>
__global__ void __launch_bounds__(kPpThreads, 1)
fmha_tc_pp_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const TcParams p) {
  constexpr int kSub = D / 64;                // 64-element (128-byte) column blocks per row
  constexpr uint32_t kSubBytes = kBN * 128;   // one [128 rows][64 bf16] swizzled block
  constexpr uint32_t kTileBytes = kSub * kSubBytes;
  constexpr int KS = D == 128 ? 3 : 4;        // K ring
  constexpr int VS = D == 128 ? 2 : 4;        // V ring
  constexpr uint32_t kIdescS = instr_desc(kBN, false);
  constexpr uint32_t kIdescPV = instr_desc(D, true);
  constexpr uint32_t kOCol = 256;             // O_t at kOCol + 128 t; S_t / P_t at 128 t

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sV = smem + (2 + KS) * kTileBytes;  // Q0 Q1 | K ring | V ring | barriers
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + KS + VS) * kTileBytes);
  const uint32_t aQ = smem_u32(smem), aK = aQ + 2 * kTileBytes, aV = aQ + (2 + KS) * kTileBytes;
  const uint32_t bar0 = smem_u32(bars);
  // barrier indices
  // Q_t full / free; S_t^h ready (index 2 t + h); P_t^h written (128 arrivals); last product of an item into O_t done;
  // any product into O_t done; then the K and V rings (full, free)
  constexpr int iQ = 0, iQF = 2, iS = 4, iP = 8, iO = 12, iPV = 14, iK = 16, iKF = iK + KS, iV = iKF + KS, iVF = iV + VS,
                nBars = iVF + VS;
  constexpr int kHN = kBN / PARTS;  // keys per part of a tile (the softmax hands its probabilities over part by part)
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + nBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int pt = p.page_tokens;
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < nBars; ++i) mbar_init(bar(i), (i >= iP && i < iP + 4) ? kBM : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), kPpTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  ItemSched sched;
  sched.n_cta = (int)gridDim.x;
  sched.cta = (int)blockIdx.x;
  sched.n_units = (p.Tq + 2 * kBM - 1) / (2 * kBM);
  sched.BH = p.BH;
  sched.group_bh = p.group_bh;
  sched.causal = p.causal;
  int bh, pair;

  if (warp >= 10) {
    // idle warps: they exist so that the helper warps form a whole warpgroup that can hand its registers over
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kPpHelperRegs));
  } else if (warp == 9) {
    // ================= loader =================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kPpHelperRegs));
    if ((tid & 31) == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mq)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mk)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mv)) : "memory");
      unsigned qn[2] = {0u, 0u}, kn = 0u, vn = 0u;  // loads issued so far into Q_t, the K ring, the V ring
      bool ok = true;
      while (ok && sched.next(bh, pair)) {
        const PpItem it = pp_item(p, bh, pair);
        auto load_kv = [&](const CUtensorMap* map, uint32_t dst, uint32_t full, int j) {
          const int t0 = j * kBN;
          if (pt >= kBN) {
            const int lp = t0 / pt, in = t0 - lp * pt;
            const int pg = p.page_table ? p.page_table[(long long)it.b * p.max_pages + lp] : it.b;
            mbar_expect_tx(full, kTileBytes);
#pragma unroll
            for (int s = 0; s < kSub; ++s) tma_load_4d(dst + s * kSubBytes, map, full, s * 64, in, it.h, pg);
          } else {
            const int per = kBN / pt;
            int valid = 0;
            for (int q = 0; q < per; ++q) valid += (t0 + q * pt < it.klen) ? 1 : 0;
            mbar_expect_tx(full, (uint32_t)valid * pt * 128u * kSub);
            for (int q = 0; q < valid; ++q) {
              const int lp = t0 / pt + q;
              const int pg = p.page_table ? p.page_table[(long long)it.b * p.max_pages + lp] : it.b;
#pragma unroll
              for (int s = 0; s < kSub; ++s) tma_load_4d(dst + s * kSubBytes + q * pt * 128, map, full, s * 64, 0, it.h, pg);
            }
          }
        };
        for (int t = 0; t < 2 && ok; ++t) {
          if (it.n[t] == 0) continue;
          if (qn[t] > 0) ok = wait_or_abort(bar(iQF + t), (qn[t] - 1) & 1u, abort_flag, 40);  // the previous item's last S_t is done
          if (!ok) break;
          mbar_expect_tx(bar(iQ + t), kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(aQ + t * kTileBytes + s * kSubBytes, &mq, bar(iQ + t), s * 64, it.h, it.q0 + t * kBM, it.b);
          ++qn[t];
        }
        for (int j = 0; ok && j < it.nmax; ++j) {
          const unsigned ks = kn % KS, ku = kn / KS;
          if (ku > 0) ok = wait_or_abort(bar(iKF + ks), (ku - 1) & 1u, abort_flag, 41);
          if (!ok) break;
          load_kv(&mk, aK + ks * kTileBytes, bar(iK + ks), j);
          ++kn;
          const unsigned vs = vn % VS, vu = vn / VS;
          if (vu > 0) ok = wait_or_abort(bar(iVF + vs), (vu - 1) & 1u, abort_flag, 42);
          if (!ok) break;
          load_kv(&mv, aV + vs * kTileBytes, bar(iV + vs), j);
          ++vn;
        }
      }
      if (!ok || *abort_flag) {
        // something ran out of time: give the copies still in flight a bounded chance to land before the CTA leaves
        if (p.status) atomicExch(p.status, *abort_flag ? *abort_flag : 2);
        for (int t = 0; t < 2; ++t)
          if (qn[t] > 0) mbar_wait(bar(iQ + t), (qn[t] - 1) & 1u);
        for (unsigned i = 0; i < (unsigned)KS; ++i)
          if (kn > i) mbar_wait(bar(iK + (int)((kn - 1 - i) % KS)), ((kn - 1 - i) / KS) & 1u);
        for (unsigned i = 0; i < (unsigned)VS; ++i)
          if (vn > i) mbar_wait(bar(iV + (int)((vn - 1 - i) % VS)), ((vn - 1 - i) / VS) & 1u);
      }
    }
  } else if (warp == 8) {
    // ================= MMA issuer =================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kPpHelperRegs));
    if ((tid & 31) == 0) {
      unsigned qn[2] = {0u, 0u}, pn[4] = {0u, 0u, 0u, 0u}, kn = 0u, vn = 0u;  // uses so far: Q_t, P_t^h, K ring, V ring
      bool ok = true;
      while (ok && sched.next(bh, pair)) {
        const PpItem it = pp_item(p, bh, pair);
        if (it.nmax == 0) continue;
        // Descriptors differ only in their 14-bit address field (bytes >> 4), so each product's descriptors are one
        // 64-bit add away from a base built once per item; the issuing lane has no time for more.
        const uint64_t dQK = smem_desc(0, 16, 1024), dV = smem_desc(0, kSubBytes, 1024);
        auto issue_s = [&](int t, int j, unsigned kslot) {  // S_t = Q_t K_j^T
          tc_fence_after();
          umma_ss_chain<D / 16>(tmem + t * 128, dQK + ((aQ + t * kTileBytes) >> 4), dQK + ((aK + kslot * kTileBytes) >> 4),
                                kIdescS, kSubBytes >> 4);
          umma_commit(bar(iS + t));
          if (j == it.n[t] - 1) umma_commit(bar(iQF + t));  // Q_t may be overwritten by the next item's
        };
        auto issue_pv = [&](int t, int h, int j, unsigned vslot) {  // O_t (+)= P_t^h V_j[64 h .. 64 h + 64)
          tc_fence_after();
          umma_ts_chain<kHN / 16>(tmem + kOCol + t * 128, tmem + t * 128 + h * (kHN / 2),
                         dV + ((aV + vslot * kTileBytes + (uint32_t)h * (kHN / 16) * 2048u) >> 4), kIdescPV,
                         (j > 0 || h > 0) ? 1u : 0u);
          umma_commit(bar(iPV + t));
          if (h == PARTS - 1 && j == it.n[t] - 1) umma_commit(bar(iO + t));
        };
        // first key tile: the four score products
        {
          const unsigned ks = kn % KS;
          ok = wait_or_abort(bar(iK + ks), (kn / KS) & 1u, abort_flag, 43);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!ok || it.n[t] == 0) continue;
            ok = wait_or_abort(bar(iQ + t), qn[t] & 1u, abort_flag, 44);
            ++qn[t];
          }
          if (!ok) break;
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (it.n[t] > 0) issue_s(t, 0, ks);
          umma_commit(bar(iKF + ks));
          ++kn;
        }
        for (int j = 0; ok && j < it.nmax; ++j) {
          const unsigned vs = vn % VS;
          const bool more = j + 1 < it.nmax;
          const unsigned ks = kn % KS;
          ok = wait_or_abort(bar(iV + vs), (vn / VS) & 1u, abort_flag, 45);
          if (ok && more) ok = wait_or_abort(bar(iK + ks), (kn / KS) & 1u, abort_flag, 47);
#pragma unroll
          for (int h = 0; h < PARTS; ++h) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (ok && j < it.n[t]) {
                ok = wait_or_abort(bar(iP + 2 * t + h), pn[2 * t + h] & 1u, abort_flag, 46);
                ++pn[2 * t + h];
              }
              if (ok && j < it.n[t]) {
                issue_pv(t, h, j, vs);
              }
              if (ok && h == PARTS - 1 && j + 1 < it.n[t]) issue_s(t, j + 1, ks);
            }
          }
          if (!ok) break;
          umma_commit(bar(iVF + vs));
          ++vn;
          if (more) {
            umma_commit(bar(iKF + ks));
            ++kn;
          }
        }
      }
      if (!ok) {
        if (!*abort_flag) *abort_flag = 2;
        if (p.status) atomicExch(p.status, *abort_flag);
      }
    }
  } else {
    // ================= softmax: warps 0-3 own query tile 0, warps 4-7 query tile 1; one thread per row =================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kPpSoftmaxRegs));
    const int t = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + (tid & 31);
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + t * 128, o_addr = lane_addr + kOCol + t * 128;
    unsigned sn[2] = {0u, 0u}, on = 0u, vn = 0u, pvn = 0u;  // S_t^h consumed, items finished, V tiles so far, arrivals (= products into O_t)
    bool fail = false;
    const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2);
    while (!fail && sched.next(bh, pair)) {
      const PpItem it = pp_item(p, bh, pair);
      const int nt = it.n[t];
      const int q0 = it.q0 + t * kBM;
      const int qi = q0 + row;
      const bool row_ok = qi < p.Tq;
      const int last_key = p.causal ? min(it.klen - 1, p.q_offset + qi) : it.klen - 1;
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < nt && !fail; ++j) {
#pragma unroll
        for (int h = 0; h < PARTS; ++h) {
          const int t0 = j * kBN + h * kHN;
          // exits are taken by whole warps (the vote makes the decision uniform), never by single lanes
          if (h == 0) {
            if (!__all_sync(0xffffffffu, wait_or_abort(bar(iS + t), sn[0] & 1u, abort_flag, 49))) {
              fail = true;
              break;
            }
            ++sn[0];
            tc_fence_after();
          }
          if (h == 0 && it.klen - j * kBN < kBN) {
            // last, partial key tile: value rows past the end may hold anything; clear them so that 0 * x stays 0
            const unsigned vj = vn + (unsigned)j;
            if (!__all_sync(0xffffffffu, wait_or_abort(bar(iV + (int)(vj % VS)), (vj / VS) & 1u, abort_flag, 50))) {
              fail = true;
              break;
            }
            if (row >= it.klen - j * kBN) {
#pragma unroll
              for (int s = 0; s < kSub; ++s) {
                uint4* vrow = reinterpret_cast<uint4*>(sV + (vj % VS) * kTileBytes + s * kSubBytes + row * 128);
#pragma unroll
                for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
              }
              fence_async_smem();
            }
          }
          const bool need_mask = (t0 + kHN > it.klen) || (p.causal && t0 + kHN - 1 > p.q_offset + q0);
          float sv[kHN];
#pragma unroll
          for (int c = 0; c < kHN / 32; ++c) tmem_ld32_nowait(s_addr + h * kHN + c * 32, &sv[c * 32]);
          tc_wait_ld();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < kHN; ++i) sv[i] = (t0 + i <= last_key) ? sv[i] : -INFINITY;
          }
          // One sweep turns the scores into probabilities against a given reference maximum `ref` (log2 domain),
          // writes them as packed bf16 over the scores, and returns their sum and the largest exponent met.
          auto sweep = [&](float ref, float& sum, float& top) {
            const uint64_t negm2 = pack2(-ref, -ref);
            uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};  // four packed partial sums (bit pattern of 0.f, 0.f)
            float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < kHN / 32; ++c) {
              uint32_t packed[16];
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const uint64_t x2 = fma2(pack2(sv[c * 32 + i], sv[c * 32 + i + 1]), scale2, negm2);
                float x0, x1, p0, p1;
                unpack2(x2, x0, x1);
                tops[(i >> 1) & 3] = max3(tops[(i >> 1) & 3], x0, x1);
                if (((i >> 1) & 3) == kPolyPhase) {
                  exp2_pair_fma(x0, x1, p0, p1);  // one pair in four on the FMA pipe, to take load off the exp2 unit
                } else {
                  p0 = ex2(x0);  // -inf -> 0
                  p1 = ex2(x1);
                }
                rs2[(i >> 1) & 3] = add2(rs2[(i >> 1) & 3], pack2(p0, p1));
                const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
              }
              // part h goes to columns [32 h, 32 h + 32): over scores that are in registers by now, so the probabilities
              // of the whole tile are one contiguous A operand and a later part's scores stay untouched
              tmem_st16(s_addr + h * (kHN / 2) + c * 16, packed);
            }
            float ra, rb, rc, rd;
            unpack2(add2(rs2[0], rs2[1]), ra, rb);
            unpack2(add2(rs2[2], rs2[3]), rc, rd);
            sum = (ra + rb) + (rc + rd);
            top = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3]));
          };
          // From the second tile on the running maximum is almost always still good (it only has to be within 2^8 of
          // the true one), so the probabilities are taken against it at once and the tile's own maximum is found in the
          // same sweep; only if a score turned out more than 2^8 above it is the tile redone the careful way.
          bool settled = false;
          float alpha = 1.f;
          if (__all_sync(0xffffffffu, m != -INFINITY)) {
            float sum, top;
            sweep(m, sum, top);
            if (!__any_sync(0xffffffffu, top > 8.f)) {
              l += sum;
              settled = true;
            }
          }
          if (!settled) {
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < kHN; i += 8) {  // three-input maxima, four independent chains
#pragma unroll
              for (int c = 0; c < 4; ++c) mxs[c] = max3(mxs[c], sv[i + 2 * c], sv[i + 2 * c + 1]);
            }
            const float mx2 = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * p.scale_log2;
            if (mx2 > m + 8.f || m == -INFINITY) {  // lazy rescale: the running maximum only moves when exceeded by 2^8
              alpha = (m == -INFINITY) ? 0.f : ex2(m - mx2);
              m = mx2;
            }
            if ((j > 0 || h > 0) && __any_sync(0xffffffffu, alpha != 1.f)) {
              // O_t may only be touched when no product into it is in flight: the one this row last arrived for must be
              // done (the one before it is, or these scores could not have been produced)
              if (!__all_sync(0xffffffffu, wait_or_abort(bar(iPV + t), (pvn - 1) & 1u, abort_flag, 52))) {
                fail = true;
                break;
              }
              tc_fence_after();
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
                float v[32];
                tmem_ld32(o_addr + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= alpha;
                tmem_st32(o_addr + c * 32, v);
              }
            }
            float sum, top;
            sweep((m == -INFINITY) ? 0.f : m, sum, top);
            l = l * alpha + sum;
          }
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(iP + 2 * t + h));
          ++pvn;
        }
      }
      vn += (unsigned)it.nmax;
      if (fail) break;
      // ---- the item's output rows of this tile ----
      if (nt > 0) {
        if (!__all_sync(0xffffffffu, wait_or_abort(bar(iO + t), on & 1u, abort_flag, 51))) {
          fail = true;
          break;
        }
        ++on;
        tc_fence_after();
      }
      if (q0 < p.Tq) {  // warp-uniform; tcgen05.ld is warp-collective: every lane reads, only rows that exist are stored
        const float inv = (l > 0.f && nt > 0) ? 1.f / l : 0.f;
        const long long off = (long long)it.b * p.o_bs + (long long)qi * p.o_rs + (long long)it.h * p.d_head;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float v[32];
          if (nt > 0) {
            tmem_ld32(o_addr + c * 32, v);
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
        if (row_ok && p.lse)
          p.lse[((long long)it.b * p.Tq + qi) * p.H + it.h] = (l > 0.f && nt > 0) ? (m + log2f(l)) * kLn2 : -INFINITY;
        tc_fence_before();  // the next item's products overwrite the TMEM columns just read
      }
    }
    if (fail && p.status) atomicExch(p.status, *abort_flag ? *abort_flag : 2);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kPpTmemCols);
}

}  // namespace tc

int fmha_tc_pp_launch(const FmhaArgs& a, const TcMaps& maps, TcParams p, long long kv_span, cudaStream_t st) {
  using namespace tc;
  const int D = a.D == 32 ? 64 : a.D;  // head_dim 32 rides on the 64-wide kernel (zero-filled boxes)
  const int n_pairs = (a.Tq + 2 * kBM - 1) / (2 * kBM);
  p.BH = a.B * a.H;
  p.group_bh = sched_group_bh(kv_span, D, p.BH);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long n_work = (long long)n_pairs * p.BH;
  int n_cta = sms > 0 ? sms : 148;
  if (a.max_ctas > 0 && a.max_ctas < n_cta) n_cta = a.max_ctas;
  if (n_work < n_cta) n_cta = (int)n_work;
  const int KS = D == 128 ? 3 : 4, VS = D == 128 ? 2 : 4;
  const size_t smem = (size_t)(2 + KS + VS) * (D / 64) * kBN * 128 + 512 + 1024;  // tiles, barriers, alignment slack
  cudaError_t e;
  auto go = [&](auto kernel) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err == cudaSuccess) kernel<<<n_cta, kPpThreads, smem, st>>>(maps.q, maps.k, maps.v, p);
    return err;
  };
  // PARTS = 2 (probabilities handed over in halves of 64 keys so that the first half of P V starts early) measured
  // slower: 630 / 713 / 722 TFLOP/s on the shapes above - two more barrier round trips per key tile
  e = D == 64 ? go(fmha_tc_pp_kernel<64, 1>) : go(fmha_tc_pp_kernel<128, 1>);
  if (e != cudaSuccess) {
    set_error("fmha_tc: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return DGPT_E_CUDA;
  }
  return launch_status("fmha_tc_pp");
}

}  // namespace dgpt
