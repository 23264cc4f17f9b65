// Soft-cap + top-p + temperature sampling, one CTA per row, everything on chip.
//
// The row of V logits is staged once in shared memory.  The nucleus is found
// without sorting: the boundary probability is located by bisection over the bit
// pattern of exp(z - max) (monotone for positive floats) with fixed-order block
// sums, so the result is reproducible; ties at the boundary are resolved by
// token id.  The draw is an inverse-CDF walk in token order driven by one
// Philox4x32-10 uniform keyed by (seed, trajectory id, step), which makes the
// stream independent of how rows are spread over GPUs.
#include "sampling.cuh"

namespace dgpt {

constexpr int kSampleThreads = 256;

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// inclusive block scan (fixed order); returns inclusive value, total in *total
__device__ __forceinline__ float block_scan_incl(float v, float* scratch, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = v;
  __syncthreads();
  float base = 0.f, tot = 0.f;
#pragma unroll
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    const float s = scratch[w];
    if (w < warp) base += s;
    tot += s;
  }
  *total = tot;
  return v + base;
}

enum { kModeSample = 0, kModeFilter = 1 };

template <typename T, int MODE>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, long long stride, int V, float cap, float temperature, float top_p,
              uint32_t seed_lo, uint32_t seed_hi, long long traj_id0, const long long* __restrict__ traj_ids,
              int step_base, const int* __restrict__ step_ptr, const int* __restrict__ force, int force_rows,
              long long force_stride, int* __restrict__ out_tok, int* __restrict__ out_mask, int* __restrict__ hist_tok,
              int* __restrict__ hist_mask, long long hist_stride, T* __restrict__ filtered, long long filt_stride) {
  extern __shared__ __align__(16) float smem[];
  float* z = smem;           // capped logits
  float* e = smem + V;       // exp(z - max)
  __shared__ float scratch[40];
  __shared__ ArgMax am[kSampleThreads / 32];
  __shared__ int sh_int[2];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int step = step_ptr ? *step_ptr : 0;

  if (MODE == kModeSample) {
    const int forced = force ? force[(long long)(r / force_rows) * force_stride + step] : -1;
    if (forced >= 0) {
      if (tid == 0) {
        out_tok[r] = forced;
        if (out_mask) out_mask[r] = 0;
        if (hist_tok) hist_tok[(long long)r * hist_stride + step] = forced;
        if (hist_mask) hist_mask[(long long)r * hist_stride + step] = 0;
      }
      return;
    }
  }
  // ---- stage the row, soft-cap, arg max ----
  ArgMax best{-INFINITY, 0x7fffffff};
  const T* row = logits + (long long)r * stride;
  for (int i = tid; i < V; i += kSampleThreads) {
    float x = Io<T>::ld(row + i);
    if (cap > 0.f) x = Io<T>::round(cap * Io<T>::round(tanhf(Io<T>::round(x / cap))));
    z[i] = x;
    if (x > best.v) best = ArgMax{x, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax t;
    t.v = __shfl_xor_sync(0xffffffffu, best.v, o);
    t.i = __shfl_xor_sync(0xffffffffu, best.i, o);
    best = better(best, t);
  }
  if (lane == 0) am[warp] = best;
  __syncthreads();
  best = am[0];
#pragma unroll
  for (int w = 1; w < kSampleThreads / 32; ++w) best = better(best, am[w]);
  const float zmax = best.v;

  int token = best.i;
  const bool greedy = (MODE == kModeSample) && temperature == 0.f;
  if (!greedy) {
    // ---- nucleus boundary ----
    uint32_t key_b = 0u;  // smallest kept key
    int i_cut = V;        // among keys == key_b, token ids <= i_cut are kept
    if (top_p < 1.f) {
      float part = 0.f;
      for (int i = tid; i < V; i += kSampleThreads) {
        const float ev = __expf(z[i] - zmax);
        e[i] = ev;
        part += ev;
      }
      const float Z = block_sum(part, scratch);
      const float target = fmaxf(top_p, 1e-30f) * Z;
      uint32_t lo = 0u, hi = 0x3f800000u;  // f(lo) >= target, f(hi) = 0 < target
      while (hi - lo > 1u) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        float s = 0.f;
        for (int i = tid; i < V; i += kSampleThreads) {
          const float ev = e[i];
          s += (__float_as_uint(ev) > mid) ? ev : 0.f;
        }
        s = block_sum(s, scratch);
        if (s < target) hi = mid; else lo = mid;
      }
      // smallest existing key >= hi, its multiplicity and the mass above it
      uint32_t kmin = 0xffffffffu;
      for (int i = tid; i < V; i += kSampleThreads) {
        const uint32_t k = __float_as_uint(e[i]);
        if (k >= hi) kmin = min(kmin, k);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
      __syncthreads();
      if (lane == 0) scratch[warp] = __uint_as_float(kmin);
      __syncthreads();
      kmin = 0xffffffffu;
#pragma unroll
      for (int w = 0; w < kSampleThreads / 32; ++w) kmin = min(kmin, __float_as_uint(scratch[w]));
      key_b = kmin;
      float above = 0.f, cnt = 0.f;
      for (int i = tid; i < V; i += kSampleThreads) {
        const float ev = e[i];
        const uint32_t k = __float_as_uint(ev);
        above += k > key_b ? ev : 0.f;
        cnt += k == key_b ? 1.f : 0.f;
      }
      above = block_sum(above, scratch);
      cnt = block_sum(cnt, scratch);
      const float eb = __uint_as_float(key_b);
      int keep = (int)ceilf((target - above) / eb);
      keep = max(1, min(keep, (int)cnt));
      if (keep < (int)cnt) {
        // id of the keep-th token (in id order) whose key equals key_b
        const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
        const int a = tid * chunk, bnd = min(V, a + chunk);
        float mine = 0.f;
        for (int i = a; i < bnd; ++i) mine += __float_as_uint(e[i]) == key_b ? 1.f : 0.f;
        float tot;
        if (tid == 0) sh_int[0] = V - 1;
        const float incl = block_scan_incl(mine, scratch, &tot);
        const int excl = (int)(incl - mine);
        if (excl < keep && keep <= (int)incl) {
          int seen = excl;
          for (int i = a; i < bnd; ++i)
            if (__float_as_uint(e[i]) == key_b && ++seen == keep) {
              sh_int[0] = i;
              break;
            }
        }
        __syncthreads();
        i_cut = sh_int[0];
      }
    }
    const bool filt = top_p < 1.f;
    if (MODE == kModeFilter) {
      T* dst = filtered + (long long)r * filt_stride;
      for (int i = tid; i < V; i += kSampleThreads) {
        bool kept = true;
        if (filt) {
          const uint32_t k = __float_as_uint(e[i]);
          kept = k > key_b || (k == key_b && i <= i_cut);
        }
        if (kept) dst[i] = row[i];
        else Io<T>::st(dst + i, -INFINITY);
      }
      return;
    }
    // ---- inverse-CDF draw in token order ----
    const float inv_t = 1.f / temperature;
    const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
    const int a = tid * chunk, bnd = min(V, a + chunk);
    float mine = 0.f;
    int last_kept = -1;
    for (int i = a; i < bnd; ++i) {
      bool kept = true;
      if (filt) {
        const uint32_t k = __float_as_uint(e[i]);
        kept = k > key_b || (k == key_b && i <= i_cut);
      }
      const float w = kept ? __expf((z[i] - zmax) * inv_t) : 0.f;
      z[i] = w;  // own chunk only: reuse the staging buffer for the weights
      mine += w;
      if (kept) last_kept = i;
    }
    float W;
    const float incl = block_scan_incl(mine, scratch, &W);
    const float excl = incl - mine;
    const long long traj = traj_ids ? traj_ids[r] : traj_id0 + r;
    const uint32_t bits = philox4x32_10((uint32_t)traj, (uint32_t)((unsigned long long)traj >> 32),
                                        (uint32_t)(step + step_base), 0u, seed_lo, seed_hi);
    const float u = (float)(bits >> 8) * (1.0f / 16777216.0f);
    const float target = u * W;
    if (tid == 0) sh_int[1] = -1;
    __syncthreads();
    if (mine > 0.f && excl <= target && target < incl) {
      const float local = target - excl;
      float c = 0.f;
      int pick = last_kept;
      for (int i = a; i < bnd; ++i) {
        c += z[i];
        if (z[i] > 0.f && c > local) {
          pick = i;
          break;
        }
      }
      sh_int[1] = pick;
    }
    __syncthreads();
    token = sh_int[1];
    if (token < 0) token = best.i;  // unreachable unless W is not finite
  }
  if (tid == 0) {
    out_tok[r] = token;
    if (out_mask) out_mask[r] = 1;
    if (hist_tok) hist_tok[(long long)r * hist_stride + step] = token;
    if (hist_mask) hist_mask[(long long)r * hist_stride + step] = 1;
  }
}

// ---- one warp per row -----------------------------------------------------------------------------
// Same rule and same draw as sample_kernel, but a row is handled by one warp with shuffles only (no
// block barriers), four rows per CTA.  exp(z - max) of the row lives in shared memory; token i sits at
// word i + (i >> log2(chunk)) so that both the strided sweeps and the per-lane contiguous chunks
// (needed where token order matters) are free of bank conflicts.  The bisection stops as soon as all
// keys left in the bracket are equal, which takes about log2(distinct keys) sweeps instead of 30.
constexpr int kWarpRows = 4;

template <typename T>
__global__ void __launch_bounds__(32 * kWarpRows)
sample_warp_kernel(const T* __restrict__ logits, long long stride, int R, int V, int log2c, float cap,
                   float temperature, float top_p, uint32_t seed_lo, uint32_t seed_hi, long long traj_id0,
                   const long long* __restrict__ traj_ids, int step_base, const int* __restrict__ step_ptr,
                   const int* __restrict__ force, int force_rows, long long force_stride, int* __restrict__ out_tok,
                   int* __restrict__ out_mask, int* __restrict__ hist_tok, int* __restrict__ hist_mask,
                   long long hist_stride) {
  extern __shared__ __align__(16) float smem[];
  dep_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x * kWarpRows + warp;
  if (r >= R) return;
  const int step = step_ptr ? *step_ptr : 0;
  const int forced = force ? force[(long long)(r / force_rows) * force_stride + step] : -1;
  int token, mask = 1;
  if (forced >= 0) {
    token = forced;
    mask = 0;
  } else {
    float* e = smem + (size_t)warp * (V + 33);
    auto at = [&](int i) -> float& { return e[i + (i >> log2c)]; };
    const T* row = logits + (long long)r * stride;
    ArgMax best{-INFINITY, 0x7fffffff};
    constexpr int VEC = Io<T>::kVec16;
    const bool vec_ok = V % VEC == 0 && stride % VEC == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    if (vec_ok) {
      // 16-byte loads, four in flight per lane; a lane visits its tokens in increasing order, so `>`
      // keeps the lowest index among equal values, and `better` does the same across lanes
      const int n_vec = V / VEC;
      for (int j0 = lane; j0 < n_vec; j0 += 128) {
        float x[4][VEC];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + 32 * u < n_vec) ld16<T>(row + (j0 + 32 * u) * VEC, x[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (j0 + 32 * u >= n_vec) continue;
          const int i0 = (j0 + 32 * u) * VEC;
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            float v = x[u][k];
            if (cap > 0.f) v = softcap_value<T>(v, cap);
            at(i0 + k) = v;
            if (v > best.v) best = ArgMax{v, i0 + k};
          }
        }
      }
    } else {
      for (int i = lane; i < V; i += 32) {
        float x = Io<T>::ld(row + i);
        if (cap > 0.f) x = softcap_value<T>(x, cap);
        at(i) = x;
        if (x > best.v) best = ArgMax{x, i};
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax t;
      t.v = __shfl_xor_sync(0xffffffffu, best.v, o);
      t.i = __shfl_xor_sync(0xffffffffu, best.i, o);
      best = better(best, t);
    }
    token = best.i;
    if (temperature != 0.f) {
      const float zmax = best.v;
      float p4[4] = {0.f, 0.f, 0.f, 0.f};  // four running sums: consecutive adds do not wait on one another
      int i = lane;
      for (; i + 96 < V; i += 128) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float ev = __expf(at(i + 32 * u) - zmax);
          at(i + 32 * u) = ev;
          p4[u] += ev;
        }
      }
      for (; i < V; i += 32) {
        const float ev = __expf(at(i) - zmax);
        at(i) = ev;
        p4[0] += ev;
      }
      const float Z = warp_sum((p4[0] + p4[1]) + (p4[2] + p4[3]));
      const bool filt = top_p < 1.f;
      uint32_t key_b = 0u;
      int i_cut = V;
      const int chunk = 1 << log2c;
      const int c0 = lane * chunk, c1 = min(V, c0 + chunk);  // this lane's tokens where order matters
      const long long traj = traj_ids ? traj_ids[r] : traj_id0 + r;
      // Fast path (rejection sampling): draw from softmax(z / T) over ALL tokens and accept the token if
      // it lies in the nucleus, i.e. if the mass ranked before it is below top_p.  Accepted draws follow
      // exactly the restricted distribution, and a draw costs two sweeps instead of a full boundary
      // search.  Attempt a uses Philox counter word 3 = a.  If kAttempts draws are rejected (a high
      // temperature over a tiny nucleus), the exact boundary is computed below.
      constexpr int kAttempts = 8;
      bool done = false;
      {
        __syncwarp();  // chunks below were written by other lanes
        const float inv_t = 1.f / temperature;
        const bool t1 = temperature == 1.f;
        float mine = 0.f;
        for (int i = c0; i < c1; ++i) {
          const float ev = at(i);
          mine += t1 ? ev : __expf(__logf(ev) * inv_t);
        }
        float incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const float W = __shfl_sync(0xffffffffu, incl, 31);
        const float excl = incl - mine;
        const float target = fmaxf(top_p, 1e-30f) * Z;
        for (int a = 0; a < kAttempts && !done; ++a) {
          const uint32_t bits = philox4x32_10((uint32_t)traj, (uint32_t)((unsigned long long)traj >> 32),
                                              (uint32_t)(step + step_base), (uint32_t)a, seed_lo, seed_hi);
          const float tgt = (float)(bits >> 8) * (1.0f / 16777216.0f) * W;
          const bool own = mine > 0.f && excl <= tgt && tgt < incl;
          int pick = best.i;
          if (own) {
            const float local = tgt - excl;
            float c = 0.f;
            for (int i = c0; i < c1; ++i) {
              const float ev = at(i);
              const float w = t1 ? ev : __expf(__logf(ev) * inv_t);
              c += w;
              if (w > 0.f) pick = i;
              if (w > 0.f && c > local) break;
            }
          }
          const unsigned who = __ballot_sync(0xffffffffu, own);
          pick = __shfl_sync(0xffffffffu, pick, who ? __ffs(who) - 1 : 0);
          if (!filt) {
            token = pick;
            done = true;
            break;
          }
          const float ek = at(pick);
          const uint32_t kk = __float_as_uint(ek);
          float a4[4] = {0.f, 0.f, 0.f, 0.f}, before = 0.f;
          int i = lane;
          for (; i + 96 < V; i += 128) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float ev = at(i + 32 * u);
              const uint32_t k = __float_as_uint(ev);
              a4[u] += k > kk ? ev : 0.f;
              before += (k == kk && i + 32 * u < pick) ? 1.f : 0.f;
            }
          }
          for (; i < V; i += 32) {
            const float ev = at(i);
            const uint32_t k = __float_as_uint(ev);
            a4[0] += k > kk ? ev : 0.f;
            before += (k == kk && i < pick) ? 1.f : 0.f;
          }
          float above = warp_sum((a4[0] + a4[1]) + (a4[2] + a4[3]));
          before = warp_sum(before);
          if (above + before * ek < target) {
            token = pick;
            done = true;
          }
        }
      }
      if (done) {
        // nothing left to do
      } else if (filt) {
        const float target = fmaxf(top_p, 1e-30f) * Z;
        uint32_t lo = 0u, hi = 0x3f800000u;  // mass above lo >= target, mass above hi = 0 < target
        while (hi - lo > 1u) {
          const uint32_t mid = lo + ((hi - lo) >> 1);
          float s = 0.f;
          uint32_t kmn = 0xffffffffu, kmx = 0u;
          for (int i = lane; i < V; i += 32) {
            const float ev = at(i);
            const uint32_t k = __float_as_uint(ev);
            if (k > lo && k <= hi) {
              kmn = min(kmn, k);
              kmx = max(kmx, k);
            }
            s += k > mid ? ev : 0.f;
          }
          s = warp_sum(s);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            kmn = min(kmn, __shfl_xor_sync(0xffffffffu, kmn, o));
            kmx = max(kmx, __shfl_xor_sync(0xffffffffu, kmx, o));
          }
          if (kmn == kmx) {  // a single key value is left in (lo, hi]: it is the boundary
            hi = kmn;
            break;
          }
          if (s < target) hi = mid; else lo = mid;
        }
        uint32_t kmin = 0xffffffffu;
        for (int i = lane; i < V; i += 32) {
          const uint32_t k = __float_as_uint(at(i));
          if (k >= hi) kmin = min(kmin, k);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
        key_b = kmin;
        float above = 0.f, cnt = 0.f;
        for (int i = lane; i < V; i += 32) {
          const float ev = at(i);
          const uint32_t k = __float_as_uint(ev);
          above += k > key_b ? ev : 0.f;
          cnt += k == key_b ? 1.f : 0.f;
        }
        above = warp_sum(above);
        cnt = warp_sum(cnt);
        int keep = (int)ceilf((target - above) / __uint_as_float(key_b));
        keep = max(1, min(keep, (int)cnt));
        if (keep < (int)cnt) {  // id of the keep-th token (in id order) whose key equals key_b
          __syncwarp();  // chunks below were written by other lanes
          int mine = 0;
          for (int i = c0; i < c1; ++i) mine += __float_as_uint(at(i)) == key_b ? 1 : 0;
          int incl = mine;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
          }
          const int excl = incl - mine;
          int found = V - 1;
          const bool own = excl < keep && keep <= incl;
          if (own) {
            int seen = excl;
            for (int i = c0; i < c1; ++i)
              if (__float_as_uint(at(i)) == key_b && ++seen == keep) {
                found = i;
                break;
              }
          }
          const unsigned who = __ballot_sync(0xffffffffu, own);
          i_cut = __shfl_sync(0xffffffffu, found, who ? __ffs(who) - 1 : 0);
        }
      }
      // exact path: inverse-CDF draw in token order over the kept tokens
      if (!done) {
      __syncwarp();  // chunks below were written by other lanes
      const float inv_t = 1.f / temperature;
      float mine = 0.f;
      int last_kept = -1;
      for (int i = c0; i < c1; ++i) {
        const float ev = at(i);
        bool kept = true;
        if (filt) {
          const uint32_t k = __float_as_uint(ev);
          kept = k > key_b || (k == key_b && i <= i_cut);
        }
        const float w = !kept ? 0.f : (temperature == 1.f ? ev : __expf(__logf(ev) * inv_t));
        at(i) = w;
        mine += w;
        if (kept) last_kept = i;
      }
      float incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const float W = __shfl_sync(0xffffffffu, incl, 31);
      const float excl = incl - mine;

      const uint32_t bits = philox4x32_10((uint32_t)traj, (uint32_t)((unsigned long long)traj >> 32),
                                          (uint32_t)(step + step_base), (uint32_t)kAttempts, seed_lo, seed_hi);
      const float u = (float)(bits >> 8) * (1.0f / 16777216.0f);
      const float tgt = u * W;
      const bool own = mine > 0.f && excl <= tgt && tgt < incl;
      int pick = last_kept;
      if (own) {
        const float local = tgt - excl;
        float c = 0.f;
        for (int i = c0; i < c1; ++i) {
          const float w = at(i);
          c += w;
          if (w > 0.f && c > local) {
            pick = i;
            break;
          }
        }
      }
      const unsigned who = __ballot_sync(0xffffffffu, own);
      if (who) token = __shfl_sync(0xffffffffu, pick, __ffs(who) - 1);
      }
    }
  }
  if (lane == 0) {
    out_tok[r] = token;
    if (out_mask) out_mask[r] = mask;
    if (hist_tok) hist_tok[(long long)r * hist_stride + step] = token;
    if (hist_mask) hist_mask[(long long)r * hist_stride + step] = mask;
  }
}

template <typename T, int MODE>
static int sample_launch(const void* logits, long long stride, int R, int V, float cap, float temperature, float top_p,
                         uint64_t seed, long long traj_id0, const long long* traj_ids, int step_base,
                         const int* step_ptr, const int* force, int force_rows, long long force_stride, int* out_tok,
                         int* out_mask, int* hist_tok, int* hist_mask, long long hist_stride, void* filtered, long long filt_stride,
                         cudaStream_t st) {
  if (MODE == kModeSample && V <= 12000) {  // warp-per-row kernel: four rows of exp() values per CTA
    const size_t wsmem = (size_t)kWarpRows * (V + 33) * sizeof(float);
    int chunk = 1, log2c = 0;
    while (chunk * 32 < V) {
      chunk <<= 1;
      ++log2c;
    }
    auto wk = sample_warp_kernel<T>;
    if (wsmem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(wk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem);
      if (e != cudaSuccess) {
        set_error("sample: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        return DGPT_E_CUDA;
      }
    }
    launch_dep(wk, dim3((R + kWarpRows - 1) / kWarpRows), dim3(32 * kWarpRows), wsmem, st, static_cast<const T*>(logits),
               stride, R, V, log2c, cap, temperature, top_p, (uint32_t)seed, (uint32_t)(seed >> 32), traj_id0, traj_ids,
               step_base, step_ptr, force, force_rows, force_stride, out_tok, out_mask, hist_tok, hist_mask, hist_stride);
    return launch_status("sample");
  }
  const size_t smem = (size_t)V * 2 * sizeof(float);
  auto kern = sample_kernel<T, MODE>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) {
      set_error("sample: vocab_size %d does not fit in shared memory (limit 25600)", V);
      return DGPT_E_UNSUPPORTED;
    }
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("sample: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return DGPT_E_CUDA;
    }
  }
  kern<<<R, kSampleThreads, smem, st>>>(static_cast<const T*>(logits), stride, V, cap, temperature, top_p,
                                        (uint32_t)seed, (uint32_t)(seed >> 32), traj_id0, traj_ids, step_base, step_ptr,
                                        force, force_rows, force_stride, out_tok, out_mask, hist_tok, hist_mask, hist_stride,
                                        static_cast<T*>(filtered), filt_stride);
  return launch_status("sample");
}

}  // namespace dgpt

using namespace dgpt;

extern "C" int dgpt_sample(const void* logits, int64_t logits_row_stride, int32_t R, int32_t V, float cap,
                           float temperature, float top_p, uint64_t seed, int64_t traj_id0, const int64_t* traj_ids,
                           int32_t step_base, const int32_t* step_ptr, const int32_t* force_schedule,
                           int32_t force_group_rows, int64_t force_group_stride, int32_t* out_tokens, int32_t* out_masks, int32_t* history_tokens, int32_t* history_masks,
                           int64_t history_stride, int32_t dtype, void* stream) {
  DGPT_REQUIRE(logits && out_tokens, "sample: NULL pointer");
  DGPT_REQUIRE(R >= 0 && V > 0, "sample: bad sizes");
  DGPT_REQUIRE(temperature >= 0.f && cap >= 0.f, "sample: temperature and cap must be non-negative");
  if (R == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long* tids = reinterpret_cast<const long long*>(traj_ids);
  const int fg = force_group_rows > 0 ? force_group_rows : 1;
  if (dtype == DGPT_F32)
    return sample_launch<float, kModeSample>(logits, logits_row_stride, R, V, cap, temperature, top_p, seed, traj_id0,
                                             tids, step_base, step_ptr, force_schedule, fg, force_group_stride, out_tokens, out_masks,
                                             history_tokens, history_masks, history_stride, nullptr, 0, st);
  if (dtype == DGPT_BF16)
    return sample_launch<__nv_bfloat16, kModeSample>(logits, logits_row_stride, R, V, cap, temperature, top_p, seed,
                                                     traj_id0, tids, step_base, step_ptr, force_schedule, fg, force_group_stride,
                                                     out_tokens, out_masks, history_tokens, history_masks, history_stride, nullptr,
                                                     0, st);
  set_error("sample: unknown dtype %d", dtype);
  return DGPT_E_UNSUPPORTED;
}

extern "C" int dgpt_nucleus_filter(const void* logits, int64_t logits_row_stride, void* filtered,
                                   int64_t filtered_row_stride, int32_t R, int32_t V, float top_p, int32_t dtype,
                                   void* stream) {
  DGPT_REQUIRE(logits && filtered, "nucleus_filter: NULL pointer");
  DGPT_REQUIRE(R >= 0 && V > 0, "nucleus_filter: bad sizes");
  if (R == 0) return DGPT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == DGPT_F32)
    return sample_launch<float, kModeFilter>(logits, logits_row_stride, R, V, 0.f, 1.f, top_p, 0, 0, nullptr, 0,
                                             nullptr, nullptr, 1, 0, nullptr, nullptr, nullptr, nullptr, 0, filtered,
                                             filtered_row_stride, st);
  if (dtype == DGPT_BF16)
    return sample_launch<__nv_bfloat16, kModeFilter>(logits, logits_row_stride, R, V, 0.f, 1.f, top_p, 0, 0, nullptr,
                                                     0, nullptr, nullptr, 1, 0, nullptr, nullptr, nullptr, nullptr, 0,
                                                     filtered, filtered_row_stride, st);
  set_error("nucleus_filter: unknown dtype %d", dtype);
  return DGPT_E_UNSUPPORTED;
}
