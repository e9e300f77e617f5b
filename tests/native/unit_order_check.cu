// Host-side check of the tile / unit enumerations of the persistent GEMM kernels: every output tile of a
// problem is produced exactly once, inside the matrix, and (symmetric products) in the lower triangle.
// Compiled by tests/test_unit_order.py with nvcc as plain host code; prints "ok" or the first violation.
#include <cstdio>
#include <set>
#include <utility>
#include "gemm_wholek_wide.cuh"

using namespace i8m;

static int check(int tiles_m, int tiles_n, int sym, int group, int batch) {
  GemmGeom g{};
  g.tiles_m = tiles_m; g.tiles_n = tiles_n; g.sym = sym; g.group = group; g.batch = batch;
  g.tiles_per_batch = sym ? tiles_m * (tiles_m + 1) / 2 : tiles_m * tiles_n;
  const size_t want = size_t(g.tiles_per_batch);
  // 128 x 256 units of the wide kernel
  const int upb = wide_units_per_batch(tiles_m, tiles_n, sym);
  for (int bb = 0; bb < batch; ++bb) {
    std::set<std::pair<int, int>> seen;
    for (int u = 0; u < upb; ++u) {
      int b, tm, tn, width;
      decode_unit(g, upb, bb * upb + u, b, tm, tn, width);
      if (b != bb || width < 1 || width > 2) return std::printf("unit: bad batch/width m%d n%d sym%d g%d u%d\n", tiles_m, tiles_n, sym, group, u);
      for (int s = 0; s < width; ++s) {
        const int c = tn + s;
        if (tm < 0 || tm >= tiles_m || c < 0 || c >= tiles_n || (sym && c > tm) || !seen.insert({tm, c}).second)
          return std::printf("unit: bad tile m%d n%d sym%d g%d u%d -> (%d,%d)\n", tiles_m, tiles_n, sym, group, u, tm, c);
      }
    }
    if (seen.size() != want) return std::printf("unit: %zu of %zu tiles m%d n%d sym%d g%d\n", seen.size(), want, tiles_m, tiles_n, sym, group);
  }
  // 128 x 128 tiles of the other persistent kernels
  std::set<std::pair<int, int>> seen;
  for (int t = 0; t < g.tiles_per_batch; ++t) {
    int b, tm, tn;
    decode_tile(g, (batch - 1) * g.tiles_per_batch + t, b, tm, tn);
    if (b != batch - 1 || tm < 0 || tm >= tiles_m || tn < 0 || tn >= tiles_n || (sym && tn > tm) || !seen.insert({tm, tn}).second)
      return std::printf("tile: bad tile m%d n%d sym%d g%d t%d -> (%d,%d)\n", tiles_m, tiles_n, sym, group, t, tm, tn);
  }
  if (seen.size() != want) return std::printf("tile: %zu of %zu tiles m%d n%d sym%d g%d\n", seen.size(), want, tiles_m, tiles_n, sym, group);
  return 0;
}

int main() {
  const int groups[] = {8, 10, 16, 32, 64};
  for (int group : groups)
    for (int sym = 0; sym < 2; ++sym)
      for (int m = 1; m <= 120; ++m)
        for (int n = sym ? m : 1; n <= (sym ? m : 36); ++n)
          if (check(m, n, sym, group, m <= 3 ? 3 : 1)) return 1;
  std::puts("ok");
  return 0;
}
