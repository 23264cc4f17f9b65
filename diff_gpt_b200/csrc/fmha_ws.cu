// tcgen05 / TMEM attention for bf16, head_dim 64 or 128 (32 rides on 64): the warp-specialised kernel with one query
// tile per work item, as a PERSISTENT kernel - one CTA of 320 threads per SM walks through (query tile, head, batch)
// items without ever re-initialising a barrier, so the loader brings in the next item's Q, K and V while the softmax
// warps still normalise and store the last item's output, and the first score products of the next item are issued
// behind the last P V of this one.
//   warp 9, lane 0  loader: TMA loads of Q and of the K / V tiles (128-byte swizzle, one box per page and per
//                   64-wide half of D) into a ring of 3 K slots and 2 V slots
//   warp 8, lane 0  issuer: S_g = Q K_g^T into one of two S buffers in TMEM and O += P_g V_g with P read from TMEM
//                   (A operand) and V MN-major; it issues P V for tile g, then S for tile g + 2, so the tensor cores
//                   work on one tile while the softmax warps work on the next.  Each product is one asm statement.
//   warps 0-7       softmax, two threads per query row: warp w owns the TMEM lanes of quarter w & 3 and the key
//                   columns of half w >> 2.  A thread reads its 64 scores with tcgen05.ld, turns them into
//                   probabilities against the running maximum in one sweep that also finds the tile's own maximum,
//                   writes P as packed bf16 into one of two P buffers (tcgen05.st), swaps that maximum with the row's
//                   other thread through an 8-byte shared-memory word (value + turn number, polled with the same
//                   clock limit as every wait), and only if the row's maximum has moved by more than 2^8 redoes the
//                   tile after rescaling its half of O in TMEM.  P V of a tile is issued BEFORE the scores of the
//                   tile after next, so that the arrival of those scores also says the P buffer has been read.
// TMEM columns: S0 [0,128)  S1 [128,256)  P0 [256,320)  P1 [320,384)  O [384, 384 + D).
// mbarriers: Q loaded / Q free; K slot full x3 / free x3; V slot full x2; S ready x2; P ready x2 (256 arrivals);
// P V done x2 (frees the P buffer and the V slot).  Every barrier completes once per use and each role derives the
// phase it waits for from a running count of key tiles (and of items) that it carries from item to item.
// Items are dealt to the CTAs longest first in snake order, a few (batch, head) pairs at a time so that co-resident
// CTAs read the same K/V through L2.  No cluster launch and no multicast.  Every wait is bounded in clock cycles; if
// one runs out the CTA stores the code of the waiting site in the status word, raises a CTA-wide abort flag so the
// other roles stop waiting too, drains the copies it issued, frees its TMEM and returns.
#include "fmha.cuh"
#include "fmha_sched.cuh"
#include "tcgen05.cuh"

namespace dgpt {
namespace tc {

constexpr int kWsThreads = 320;  // 8 softmax warps, the MMA issuer's warp, the loader's warp
constexpr uint32_t kWsTmemCols = 512;

struct WsItem {
  int b, h, q0, klen, n;  // n = key tiles
};

__device__ __forceinline__ WsItem ws_item(const TcParams& p, int bh, int qt) {
  WsItem it;
  it.h = bh % p.H;
  it.b = bh / p.H;
  it.q0 = qt * kBM;
  it.klen = p.kv_len ? p.kv_len[it.b] : p.kv_len_all;
  const int kmax = p.causal ? min(it.klen, p.q_offset + min(it.q0 + kBM, p.Tq)) : it.klen;
  it.n = kmax > 0 ? (kmax + kBN - 1) / kBN : 0;
  return it;
}

template <int D>
__global__ void __launch_bounds__(kWsThreads, 1)
fmha_tc_ws_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const TcParams p) {
  constexpr int kSub = D / 64;
  constexpr uint32_t kSubBytes = kBN * 128;
  constexpr uint32_t kTileBytes = kSub * kSubBytes;
  constexpr uint32_t kIdescS = instr_desc(kBN, false);
  constexpr uint32_t kIdescPV = instr_desc(D, true);
  constexpr uint32_t kPCol = 256;  // P buffer b: columns [256 + 64 b, +64)
  constexpr uint32_t kOCol = 384;
  constexpr int kStepsS = D / 16, kStepsPV = kBN / 16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sV = smem + 4 * kTileBytes;  // Q | K0 K1 K2 | V0 V1   (K is needed a tile earlier than V: deeper ring)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  constexpr int nBars = 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + nBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // [2 turns][2 halves][128 rows] words of (turn number + 1) << 32 | value: what the two threads of a row exchange
  volatile unsigned long long* xch = reinterpret_cast<volatile unsigned long long*>(bars + 32);
  const uint32_t aQ = smem_u32(smem), aK = aQ + kTileBytes, aV = aQ + 4 * kTileBytes;
  const uint32_t bar_q = smem_u32(bars), bar_qf = bar_q + 8, bar_k0 = bar_q + 16, bar_kf0 = bar_q + 40, bar_v0 = bar_q + 64,
                 bar_s0 = bar_q + 80, bar_p0 = bar_q + 96, bar_o0 = bar_q + 112;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int pt = p.page_tokens;
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < nBars; ++i) mbar_init(bar_q + 8 * i, (i == 12 || i == 13) ? 2 * kBM : 1);  // 12, 13: the P barriers
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (tid < 2 * kBM) {  // turn numbers of a previous CTA on this SM must not be mistaken for this one's
    xch[tid] = 0ull;
    xch[2 * kBM + tid] = 0ull;
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), kWsTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  ItemSched sched;
  sched.n_cta = (int)gridDim.x;
  sched.cta = (int)blockIdx.x;
  sched.n_units = p.n_qt;
  sched.BH = p.BH;
  sched.group_bh = p.group_bh;
  sched.causal = p.causal;
  int bh, qt;

  if (warp == 9) {
    // ================= loader: every TMA load (one lane) =================
    if ((tid & 31) == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mq)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mk)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mv)) : "memory");
      unsigned items = 0u, g = 0u;  // items with keys seen so far; key tiles of the items before this one
      unsigned kn = 0u, vn = 0u;    // K and V tiles whose loads have been issued (over all items)
      bool ok = true;
      while (ok && sched.next(bh, qt)) {
        const WsItem it = ws_item(p, bh, qt);
        if (it.n == 0) continue;
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
        if (items > 0) ok = wait_or_abort(bar_qf, (items - 1) & 1u, abort_flag, 16);  // the previous item's last S is done
        if (!ok) break;
        mbar_expect_tx(bar_q, kTileBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) tma_load_4d(aQ + s * kSubBytes, &mq, bar_q, s * 64, it.h, it.q0, it.b);
        ++items;
        // K tiles run one ahead of the V tiles (K0 K1 V0 K2 V1 ...): a K slot is free as soon as its score product is
        // done, long before the P V product that frees a V slot, and the loads should be in flight by then
        auto load_k = [&](int j) {
          const unsigned gk = g + (unsigned)j, ks = gk % 3u, ku = gk / 3u;
          if (ku > 0) ok = wait_or_abort(bar_kf0 + 8 * ks, (ku - 1) & 1u, abort_flag, 16);  // S of the slot's last tile is done
          if (ok) {
            load_kv(&mk, aK + ks * kTileBytes, bar_k0 + 8 * ks, j);
            ++kn;
          }
        };
        load_k(0);
        for (int j = 0; ok && j < it.n; ++j) {
          if (j + 1 < it.n) load_k(j + 1);
          if (!ok) break;
          const unsigned gv = g + (unsigned)j, vs = gv & 1u;
          if (gv >= 2) ok = wait_or_abort(bar_o0 + 8 * vs, ((gv - 2) >> 1) & 1u, abort_flag, 17);  // P V of the slot's last tile is done
          if (!ok) break;
          load_kv(&mv, aV + vs * kTileBytes, bar_v0 + 8 * vs, j);
          ++vn;
        }
        if (ok) g += (unsigned)it.n;
      }
      if (!ok || *abort_flag) {  // something ran out of time: give the copies still in flight a bounded chance to land
        if (p.status) atomicExch(p.status, *abort_flag ? *abort_flag : 2);
        if (items > 0) mbar_wait(bar_q, (items - 1) & 1u);
        for (unsigned i = 0; i < 3u && i < kn; ++i) mbar_wait(bar_k0 + 8 * ((kn - 1 - i) % 3u), ((kn - 1 - i) / 3u) & 1u);
        for (unsigned i = 0; i < 2u && i < vn; ++i) mbar_wait(bar_v0 + 8 * ((vn - 1 - i) & 1u), ((vn - 1 - i) >> 1) & 1u);
      }
    }
  } else if (warp == 8) {
    // ================= MMA issuer (one lane) =================
    if ((tid & 31) == 0) {
      // Each product is one asm statement with constant descriptor steps: this lane shares its scheduler with two
      // softmax warps, and every instruction it does not execute is time the tensor pipe does not wait for.
      const uint64_t dQK = smem_desc(0, 16, 1024), dV = smem_desc(0, kSubBytes, 1024);
      unsigned items = 0u, g0 = 0u;
      bool ok = true;
      while (ok && sched.next(bh, qt)) {
        const WsItem it = ws_item(p, bh, qt);
        const int n = it.n;
        if (n == 0) continue;
        auto issue_s = [&](unsigned g, bool last) {  // S(g & 1) = Q K(g % 3)^T
          const unsigned kslot = g % 3u, buf = g & 1u;
          tc_fence_after();
          umma_ss_chain<kStepsS>(tmem + buf * 128, dQK + (aQ >> 4), dQK + ((aK + kslot * kTileBytes) >> 4), kIdescS, kSubBytes >> 4);
          umma_commit(bar_s0 + 8 * buf);
          umma_commit(bar_kf0 + 8 * kslot);
          if (last) umma_commit(bar_qf);  // Q may be overwritten by the next item's
        };
        ok = wait_or_abort(bar_q, items & 1u, abort_flag, 18);
        ++items;
        for (int i = 0; ok && i < 2 && i < n; ++i) {
          const unsigned g = g0 + (unsigned)i;
          ok = wait_or_abort(bar_k0 + 8 * (g % 3u), (g / 3u) & 1u, abort_flag, 19);
          if (ok) issue_s(g, i == n - 1);
        }
        for (int j = 0; ok && j < n; ++j) {
          const unsigned g = g0 + (unsigned)j, buf = g & 1u, ph = (g >> 1) & 1u;
          // P_g is complete when every row has arrived; by then every row has also consumed S_g, so the same
          // buffer can take S_{g+2} at once (P lives in its own columns)
          ok = wait_or_abort(bar_p0 + 8 * buf, ph, abort_flag, 20);
          ok = ok && wait_or_abort(bar_v0 + 8 * buf, ph, abort_flag, 21);
          if (ok && j + 2 < n) ok = wait_or_abort(bar_k0 + 8 * ((g + 2) % 3u), ((g + 2) / 3u) & 1u, abort_flag, 22);
          if (!ok) break;
          tc_fence_after();
          umma_ts_chain<kStepsPV>(tmem + kOCol, tmem + kPCol + buf * 64, dV + ((aV + buf * kTileBytes) >> 4), kIdescPV, j > 0 ? 1u : 0u);
          umma_commit(bar_o0 + 8 * buf);
          // The scores of tile g + 2 go BEHIND this product: their completion (bar_s) then also says that P_g has been
          // read, which is what lets the softmax threads overwrite the P buffer without a wait of their own.
          if (j + 2 < n) issue_s(g + 2, j + 2 == n - 1);
        }
        g0 += (unsigned)n;
      }
      if (!ok) {
        if (!*abort_flag) *abort_flag = 2;
        if (p.status) atomicExch(p.status, *abort_flag);
      }
    }
  } else {
    // ================= softmax threads: two per query row, one for each half of the key tile =================
    constexpr int kHalf = kBN / 2;
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + (tid & 31);
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    unsigned g0 = 0u, turn = 0u;  // key tiles of the items before this one; hand-overs made so far
    bool fail = false;
    // Hand-over of one float between the two threads of a row: value and turn number travel in one 8-byte
    // shared-memory word (a single store, so no fence is needed), slots alternate with the turn's parity,
    // and the reader polls with a clock-cycle limit like every other wait of this kernel.
    const volatile unsigned long long* partner = nullptr;
    unsigned long long want = 0ull;
    auto publish = [&](float mine) {  // this thread's value for the current turn
      const unsigned xb = turn & 1u;
      want = (unsigned long long)(turn + 1u) << 32;
      xch[(xb * 2 + half) * kBM + row] = want | __float_as_uint(mine);
      partner = xch + (xb * 2 + (half ^ 1)) * kBM + row;
      ++turn;
    };
    auto collect = [&](bool& ok) -> float {  // the partner's value for the turn last published
      const long long t_begin = clock64();
      for (int spin = 0;; ++spin) {
        const unsigned long long got = *partner;  // one 8-byte load of what one 8-byte store wrote
        if ((got >> 32) == (want >> 32)) return __uint_as_float((uint32_t)got);
        if ((spin & 63) == 63 && (*abort_flag || clock64() - t_begin > kWaitLimitCycles)) {
          if (!*abort_flag) *abort_flag = 27;
          ok = false;
          return 0.f;
        }
      }
    };
    auto exchange = [&](float mine, bool& ok) -> float {
      publish(mine);
      return collect(ok);
    };
    while (!fail && sched.next(bh, qt)) {
      const WsItem it = ws_item(p, bh, qt);
      const int n_tiles = it.n, klen = it.klen, q0 = it.q0, b = it.b, h = it.h;
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < n_tiles; ++j) {
        const unsigned g = g0 + (unsigned)j, buf = g & 1u, ph = (g >> 1) & 1u;
        const int t0 = j * kBN;
        // exits are taken by whole warps (the vote makes the decision uniform), never by single lanes
        if (!__all_sync(0xffffffffu, wait_or_abort(bar_s0 + 8 * buf, ph, abort_flag, 23))) {
          fail = true;
          break;
        }
        tc_fence_after();
        const int valid_rows = klen - t0;
        if (valid_rows < kBN) {  // CTA-uniform: last, partial tile
          if (!__all_sync(0xffffffffu, wait_or_abort(bar_v0 + 8 * buf, ph, abort_flag, 24))) {
            fail = true;
            break;
          }
          if (half == 0 && row >= valid_rows) {  // value rows past the end may hold anything: clear them so that 0 * x stays 0
#pragma unroll
            for (int s = 0; s < kSub; ++s) {
              uint4* vrow = reinterpret_cast<uint4*>(sV + buf * kTileBytes + s * kSubBytes + row * 128);
#pragma unroll
              for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_async_smem();
          }
        }
        const bool need_mask = (t0 + kBN > klen) || (p.causal && t0 + kBN - 1 > p.q_offset + q0);
        const int last_key = p.causal ? min(klen - 1, p.q_offset + q0 + row) : klen - 1;
        const int c0 = t0 + half * kHalf;  // key index of this thread's first column
        float sv[kHalf];
#pragma unroll
        for (int c = 0; c < kHalf / 32; ++c) tmem_ld32_nowait(lane_addr + buf * 128 + half * kHalf + c * 32, &sv[c * 32]);
        tc_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < kHalf; ++i) sv[i] = (c0 + i <= last_key) ? sv[i] : -INFINITY;
        }
        // One sweep turns this thread's 64 scores into probabilities against a reference maximum `ref` (log2 domain),
        // writes them as packed bf16 into the P buffer and returns their sum.
        auto sweep = [&](float ref, float& top) -> float {
          const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negm2 = pack2(-ref, -ref);
          uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};  // four packed partial sums (bit pattern of 0.f, 0.f)
          float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // the largest exponent met, four chains
#pragma unroll
          for (int c = 0; c < kHalf / 32; ++c) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              unpack2(fma2(pack2(sv[c * 32 + i], sv[c * 32 + i + 1]), scale2, negm2), x0, x1);  // one issue slot for the pair
              tops[(i >> 1) & 3] = max3(tops[(i >> 1) & 3], x0, x1);
              const float p0 = ex2(x0), p1 = ex2(x1);  // -inf -> 0
              rs2[(i >> 1) & 3] = add2(rs2[(i >> 1) & 3], pack2(p0, p1));
              const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
              packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
            }
            tmem_st16(lane_addr + kPCol + buf * 64 + half * (kHalf / 2) + c * 16, packed);
          }
          float ra, rb, rc, rd;
          unpack2(add2(rs2[0], rs2[1]), ra, rb);
          unpack2(add2(rs2[2], rs2[3]), rc, rd);
          top = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3]));
          return (ra + rb) + (rc + rd);
        };
        // From an item's second tile on the running maximum is almost always still good (it only has to be within 2^8
        // of the true one), so the probabilities are taken against it at once and the tile's own maximum is found in
        // the same sweep, as the largest exponent met; the two threads of a row swap theirs afterwards and so hold the
        // same row maximum and take the same decision: only if it exceeds the running maximum by more than 2^8 is the
        // tile redone the careful way.  (m is the same in both threads, so the vote below is the same in both warps.)
        bool xok = true, settled = false;
        float mx2, sum = 0.f, top;
        const bool fast = __all_sync(0xffffffffu, m != -INFINITY);
        if (fast) {
          sum = sweep(m, top);
          const float theirs = exchange(top, xok);
          mx2 = fmaxf(top, theirs) + m;  // exponents were taken against m
        } else {  // first tile of an item: the maximum first
          float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < kHalf; i += 8) {  // three-input maxima, four independent chains
#pragma unroll
            for (int c = 0; c < 4; ++c) mxs[c] = max3(mxs[c], sv[i + 2 * c], sv[i + 2 * c + 1]);
          }
          const float mine = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
          const float theirs = exchange(mine, xok);
          mx2 = fmaxf(mine, theirs) * p.scale_log2;  // the same number in both threads of the row
        }
        if (!__all_sync(0xffffffffu, xok)) {
          fail = true;
          break;
        }
        if (fast && !__any_sync(0xffffffffu, mx2 > m + 8.f)) {
          l += sum;
          settled = true;
        }
        if (!settled) {
          float alpha = 1.f;  // lazy rescale: the running maximum only moves when exceeded by 2^8
          if (mx2 > m + 8.f || m == -INFINITY) {
            alpha = (m == -INFINITY) ? 0.f : ex2(m - mx2);
            m = mx2;
          }
          if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
            // O may only be touched when no P V product is in flight: tile g-1's must have finished
            // (tile g's cannot start before this row has arrived on bar_p below)
            const bool ok = wait_or_abort(bar_o0 + 8 * (buf ^ 1u), ((g - 1) >> 1) & 1u, abort_flag, 25);
            if (!__all_sync(0xffffffffu, ok)) {
              fail = true;
              break;
            }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {  // this thread's half of the row's O columns
              float v[32];
              tmem_ld32(lane_addr + kOCol + half * (D / 2) + c * 32, v);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= alpha;
              tmem_st32(lane_addr + kOCol + half * (D / 2) + c * 32, v);
            }
          }
          l = l * alpha + sweep((m == -INFINITY) ? 0.f : m, top);  // sum over this thread's columns only
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p0 + 8 * buf);
      }
      // every warp leaves the loop as a whole (waits are on CTA-wide events), so the collective loads below are safe
      if (!fail && n_tiles > 0) {
        const unsigned last = g0 + (unsigned)n_tiles - 1u;
        if (!wait_or_abort(bar_o0 + 8 * (last & 1u), (last >> 1) & 1u, abort_flag, 26)) fail = true;
        tc_fence_after();
      }
      if (!__any_sync(0xffffffffu, fail) && n_tiles > 0) {  // the row's sum is the sum of its two halves
        bool xok = true;
        const float theirs = exchange(l, xok);
        if (xok) l += theirs;
        else fail = true;
      }
      if (__any_sync(0xffffffffu, fail)) {
        fail = true;
        break;
      }
      const int qi = q0 + row;
      const bool row_ok = qi < p.Tq;
      const float inv = (l > 0.f && n_tiles > 0) ? 1.f / l : 0.f;
      const long long off = (long long)b * p.o_bs + (long long)qi * p.o_rs + (long long)h * p.d_head + half * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        float v[32];
        if (n_tiles > 0) {
          tmem_ld32(lane_addr + kOCol + half * (D / 2) + c * 32, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (row_ok && half * (D / 2) + c * 32 < p.d_head) {
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
      if (half == 0 && row_ok && p.lse)
        p.lse[((long long)b * p.Tq + qi) * p.H + h] = (l > 0.f && n_tiles > 0) ? (m + log2f(l)) * kLn2 : -INFINITY;
      tc_fence_before();  // the next item's first P V overwrites the O columns just read (it waits for this row's next arrival)
      g0 += (unsigned)n_tiles;
    }
    if (fail && p.status) atomicExch(p.status, *abort_flag ? *abort_flag : 2);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kWsTmemCols);
}

}  // namespace tc

int fmha_tc_ws_launch(const FmhaArgs& a, const TcMaps& maps, TcParams p, long long kv_span, cudaStream_t st) {
  using namespace tc;
  const int D = a.D == 32 ? 64 : a.D;  // head_dim 32 rides on the 64-wide kernel (zero-filled boxes)
  p.BH = a.B * a.H;
  p.group_bh = sched_group_bh(kv_span, D, p.BH);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int n_cta = sms > 0 ? sms : 148;
  if (a.max_ctas > 0 && a.max_ctas < n_cta) n_cta = a.max_ctas;
  if (p.n_work < n_cta) n_cta = p.n_work;
  // Q + three K + two V tiles, barriers and the hand-over words, alignment slack; padded so that one CTA owns an SM
  // (it allocates all 512 TMEM columns)
  size_t smem = (size_t)6 * (D / 64) * kBN * 128 + 8192 + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  cudaError_t e;
  if (D == 64) {
    e = cudaFuncSetAttribute(fmha_tc_ws_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) fmha_tc_ws_kernel<64><<<n_cta, kWsThreads, smem, st>>>(maps.q, maps.k, maps.v, p);
  } else {
    e = cudaFuncSetAttribute(fmha_tc_ws_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) fmha_tc_ws_kernel<128><<<n_cta, kWsThreads, smem, st>>>(maps.q, maps.k, maps.v, p);
  }
  if (e != cudaSuccess) {
    set_error("fmha_tc: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return DGPT_E_CUDA;
  }
  return launch_status("fmha_tc_ws");
}

}  // namespace dgpt
