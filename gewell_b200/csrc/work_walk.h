// Which work a CTA of the persistent GEMM kernel takes, in which order.  Plain
// arithmetic, usable from host code as well (the host test walks every CTA of a
// launch and checks that the launch's work is covered exactly once).
//
// Normal mode: whole work items in chunks of `chunk` consecutive items; CTA b takes
// chunks b, b + grid, b + 2 * grid, ...  (consecutive items of a grouped launch share
// the token tile and the expert, so their descriptors stay hot).
// Split mode (decode shapes): the launch's (item, K-stage) units are cut into `grid`
// equal contiguous ranges, so a CTA may start and end in the middle of an item's K
// loop; every SM then streams the same number of weight bytes whatever the number of
// tiles.  An item is then finished by several CTAs: cta_of / range_begin tell the
// epilogue which CTAs hold its other parts.
#pragma once

#if defined(__CUDACC__)
#define GW_WALK_FN __host__ __device__
#else
#define GW_WALK_FN
#endif

namespace gw {

struct SegmentWalk {
  bool split;
  int w, step, total_work, k_stages, chunk, in_chunk;
  long long u, u_begin, u_end, total_units;
  GW_WALK_FN SegmentWalk(int cta, int grid, bool split_, int total_work_, int k_stages_, int chunk_ = 1)
      : split(split_), w(0), step(grid), total_work(total_work_), k_stages(k_stages_),
        chunk(chunk_ > 1 ? chunk_ : 1), in_chunk(0) {
    w = cta * chunk;
    total_units = (long long)total_work * k_stages;
    u_begin = u = total_units * cta / grid;
    u_end = total_units * (cta + 1) / grid;
  }
  // next segment: work item `tile`, K stages [ks0, ks1)
  GW_WALK_FN bool next(int& tile, int& ks0, int& ks1, bool& at_range_start) {
    if (!split) {
      if (w >= total_work) return false;
      tile = w; ks0 = 0; ks1 = k_stages; at_range_start = false;
      // `chunk` consecutive items, then on to this CTA's next chunk
      if (++in_chunk == chunk) { in_chunk = 0; w += (step - 1) * chunk + 1; } else { ++w; }
      return true;
    }
    if (u >= u_end) return false;
    tile = int(u / k_stages);
    ks0 = int(u % k_stages);
    const long long left = u_end - u;
    ks1 = left < (long long)(k_stages - ks0) ? ks0 + int(left) : k_stages;
    at_range_start = u == u_begin;
    u += ks1 - ks0;
    return true;
  }
  // CTA whose range holds unit x
  GW_WALK_FN int cta_of(long long x) const { return int(((x + 1) * step + total_units - 1) / total_units) - 1; }
  GW_WALK_FN long long range_begin(int cta) const { return total_units * cta / step; }
};

}  // namespace gw
