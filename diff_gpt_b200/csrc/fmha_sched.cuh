// Work distribution of the persistent attention kernels.
#pragma once

namespace dgpt {
namespace tc {

// Which item a persistent CTA works on next.  An item is (unit, batch, head), a unit being one query tile or a pair
// of them.  Groups of `group_bh` (batch, head) pairs whose K and V fit the L2 together; inside a group the items are
// ordered longest first and dealt to the CTAs round by round, every other round
// in reverse, so that each CTA gets about the same number of key tiles.
struct ItemSched {
  int n_cta, cta, n_units, BH, group_bh, causal;
  int group = 0, round = 0;
  __device__ bool next(int& bh, int& unit) {
    for (;;) {
      const int first = group * group_bh;
      if (first >= BH) return false;
      const int members = min(group_bh, BH - first);
      const int count = members * n_units;
      const int base = round * n_cta;
      if (base >= count) {
        ++group;
        round = 0;
        continue;
      }
      // every other round, and every other group, runs through the CTAs in reverse: a CTA that got a long item gets a
      // short one next, and the CTAs left without an item in a group's last, partial round change from group to group
      const int pos = base + (((round + group) & 1) ? (n_cta - 1 - cta) : cta);
      ++round;
      if (pos >= count) continue;
      const int rank = pos / members;
      bh = first + pos - rank * members;
      unit = causal ? n_units - 1 - rank : rank;
      return true;
    }
  }
};


// (batch, head) pairs worked on together: their K and V (2 x span x D bf16 each) should stay in L2 (32 MB of it)
inline int sched_group_bh(long long kv_span, int D, int BH) {
  const long long per_bh = 2ll * kv_span * D * 2;
  long long group = per_bh > 0 ? (32ll << 20) / per_bh : BH;  // measured: 16 / 32 / 48 / 96 MB give 874 / 920 / 920 / 899 TFLOP/s at S = 32768
  if (group < 1) group = 1;
  if (group > BH) group = BH;
  return (int)group;
}

}  // namespace tc
}  // namespace dgpt
