// Host test of the persistent kernels' work distribution (gewell_b200/csrc/work_walk.h): walks every
// CTA of a launch and checks that the launch's work is covered exactly once, in both modes.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "work_walk.h"

static int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      if (failures < 20) { std::printf("FAIL %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); } \
      ++failures;                                          \
    }                                                      \
  } while (0)

static void whole_items(int total_work, int k_stages, int grid, int chunk) {
  std::vector<int> seen(total_work, 0);
  const int c = chunk > 1 ? chunk : 1;
  for (int cta = 0; cta < grid; ++cta) {
    gw::SegmentWalk walk(cta, grid, false, total_work, k_stages, chunk);
    int tile, ks0, ks1, last = -1, taken = 0;
    bool start;
    while (walk.next(tile, ks0, ks1, start)) {
      CHECK(tile >= 0 && tile < total_work, "tile %d of %d", tile, total_work);
      if (tile < 0 || tile >= total_work) return;
      CHECK(ks0 == 0 && ks1 == k_stages && !start, "whole K loop expected");
      CHECK(tile > last, "ascending order");
      // inside a chunk the items are consecutive; a chunk starts at a multiple of the chunk size
      if (taken % c == 0) CHECK(tile % c == 0 && (tile / c) % grid == cta, "chunk %d does not belong to CTA %d", tile / c, cta);
      else CHECK(tile == last + 1, "items of a chunk are consecutive");
      last = tile;
      ++taken;
      ++seen[tile];
    }
  }
  for (int t = 0; t < total_work; ++t) CHECK(seen[t] == 1, "item %d taken %d times (work %d grid %d chunk %d)", t, seen[t], total_work, grid, chunk);
}

static void split_units(int total_work, int k_stages, int grid) {
  const long long total_units = (long long)total_work * k_stages;
  std::vector<int> covered(total_units, 0);
  for (int cta = 0; cta < grid; ++cta) {
    gw::SegmentWalk walk(cta, grid, true, total_work, k_stages);
    int tile, ks0, ks1, segments = 0, partial = 0;
    long long units = 0, expect = walk.range_begin(cta);
    bool start;
    while (walk.next(tile, ks0, ks1, start)) {
      CHECK(tile >= 0 && tile < total_work && 0 <= ks0 && ks0 < ks1 && ks1 <= k_stages, "segment out of range");
      if (!(tile >= 0 && tile < total_work && 0 <= ks0 && ks0 < ks1 && ks1 <= k_stages)) return;
      CHECK(start == (segments == 0), "only the first segment starts the range");
      CHECK((long long)tile * k_stages + ks0 == expect, "segments are contiguous");
      for (int ks = ks0; ks < ks1; ++ks) {
        const long long unit = (long long)tile * k_stages + ks;
        ++covered[unit];
        CHECK(walk.cta_of(unit) == cta, "cta_of(%lld) = %d, walked by %d", unit, walk.cta_of(unit), cta);
      }
      if (ks1 - ks0 != k_stages) ++partial;
      units += ks1 - ks0;
      expect += ks1 - ks0;
      ++segments;
    }
    CHECK(partial <= 2, "a CTA holds parts of at most two items (has %d)", partial);   // two partial slots per CTA
    const long long lo = total_units / grid, hi = (total_units + grid - 1) / grid;
    CHECK(units >= lo && units <= hi, "CTA %d walks %lld units, expected %lld..%lld", cta, units, lo, hi);
    CHECK(expect == (cta + 1 < grid ? walk.range_begin(cta + 1) : total_units), "range ends where the next begins");
  }
  for (long long x = 0; x < total_units; ++x) CHECK(covered[x] == 1, "unit %lld covered %d times", x, covered[x]);
}

int main() {
  const int works[] = {1, 2, 3, 21, 147, 148, 149, 336, 672, 1375, 12672};
  const int grids[] = {1, 2, 74, 148};
  const int chunks[] = {0, 1, 2, 3, 4, 22};
  for (int work : works)
    for (int grid : grids) {
      for (int chunk : chunks) whole_items(work, 11, grid < work ? grid : work, chunk);
      if (work <= 1375)
        for (int k_stages : {1, 3, 11, 42, 84}) {
          const long long units = (long long)work * k_stages;
          split_units(work, k_stages, units < grid ? int(units) : grid);
        }
    }
  if (failures) { std::printf("%d checks failed\n", failures); return 1; }
  std::printf("PASS\n");
  return 0;
}
