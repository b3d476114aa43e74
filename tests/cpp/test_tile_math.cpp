// Host-side checks of the tile schedulers' index arithmetic (csrc/tile_math.h), built with
// -fsanitize=address,undefined by tests/test_tile_math_host.py.  Every table the kernels index is allocated at its
// exact size here, so an out-of-range read of the arithmetic shows up as a sanitizer report.
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <random>
#include <vector>

#include "tile_math.h"

using namespace kf::tilemath;

static int failures = 0;
#define CHECK(cond)                                                            \
  do {                                                                         \
    if (!(cond)) {                                                             \
      std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                                              \
    }                                                                          \
  } while (0)

// the rasterisation visits every tile of the grid exactly once, and a group's tiles are contiguous in t
static void test_raster() {
  for (int mb = 1; mb <= 37; ++mb)
    for (int nb = 1; nb <= 19; ++nb)
      for (int gm : {1, 3, 8, 64}) {
        std::vector<int> seen(size_t(mb) * nb, 0);
        int prev_group = 0;
        for (int t = 0; t < mb * nb; ++t) {
          int m = -1, n = -1;
          raster(t, mb, nb, gm, m, n);
          CHECK(m >= 0 && m < mb && n >= 0 && n < nb);
          if (m < 0 || m >= mb || n < 0 || n >= nb) return;
          seen[size_t(m) * nb + n] += 1;
          const int group = m / gm;
          CHECK(group >= prev_group);  // groups are walked in order: column tiles of a group stay hot in L2
          prev_group = group;
        }
        for (int v : seen) CHECK(v == 1);
      }
}

static void check_grouped(const std::vector<int>& counts, int n_blocks, int bm) {
  const int E = int(counts.size());
  std::vector<int> offsets(E + 1, 0);
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  std::vector<int> tile_start(E + 1, -1);
  const int row_tiles = grouped_tile_starts(offsets.data(), E, bm, tile_start.data());
  int want_tiles = 0;
  for (int c : counts) want_tiles += ceil_div(c, bm);
  CHECK(row_tiles == want_tiles && tile_start[E] == want_tiles && tile_start[0] == 0);
  // every row of every expert is covered exactly once per column block, by a tile of its own expert
  const size_t cells = static_cast<size_t>(offsets[E]) * static_cast<size_t>(n_blocks);
  std::vector<int> cover(cells, 0);
  for (int t = 0; t < row_tiles * n_blocks; ++t) {
    const GroupedTile g = grouped_decode(t, n_blocks, tile_start.data(), offsets.data(), E, bm);
    CHECK(g.e >= 0 && g.e < E && g.nb >= 0 && g.nb < n_blocks);
    CHECK(g.valid >= 1 && g.valid <= bm);
    CHECK(g.row0 >= offsets[g.e] && g.row0 + g.valid <= offsets[g.e + 1]);
    CHECK((g.row0 - offsets[g.e]) % bm == 0);
    if (g.e < 0 || g.e >= E || g.row0 < 0 || g.row0 + g.valid > offsets[E]) return;
    for (int r = 0; r < g.valid; ++r) cover[size_t(g.row0 + r) * n_blocks + g.nb] += 1;
  }
  for (int v : cover) CHECK(v == 1);
}

static void test_grouped() {
  check_grouped({128, 128, 128, 128}, 2, 128);
  check_grouped({5, 0, 300, 77, 130, 1}, 3, 128);
  check_grouped({0, 0, 513}, 1, 128);
  check_grouped({0}, 4, 128);
  check_grouped({1}, 1, 128);
  check_grouped({0, 0, 0, 7, 0, 0}, 2, 128);
  std::mt19937 rng(7);
  for (int trial = 0; trial < 200; ++trial) {
    const int E = 1 + int(rng() % 64);
    std::vector<int> counts(E);
    for (int& c : counts) c = (rng() % 4 == 0) ? 0 : int(rng() % 700);
    check_grouped(counts, 1 + int(rng() % 5), 128);
  }
}

static void test_wgrad() {
  const std::vector<int> offsets = {0, 5, 5, 305, 382, 512, 513};
  const int E = int(offsets.size()) - 1, bm = 128, bn = 256;
  for (int M : {8, 128, 200, 2048})
    for (int N : {8, 256, 328, 5632}) {
      const int mb = ceil_div(M, bm), nb = ceil_div(N, bn);
      std::vector<int> seen(size_t(E) * mb * nb, 0);
      for (int t = 0; t < E * mb * nb; ++t) {
        const WgradTile w = wgrad_decode(t, mb, nb, bm, bn, offsets.data());
        CHECK(w.e >= 0 && w.e < E && w.m0 % bm == 0 && w.n0 % bn == 0 && w.m0 < M && w.n0 < N);
        CHECK(w.row0 == offsets[w.e] && w.rows == offsets[w.e + 1] - offsets[w.e] && w.rows >= 0);
        if (w.e < 0 || w.e >= E) return;
        seen[(size_t(w.e) * mb + w.m0 / bm) * nb + w.n0 / bn] += 1;
      }
      for (int v : seen) CHECK(v == 1);
    }
}

// the chunks cleared at the ragged end of a reduction range are exactly the rows valid..bk-1 of every block
static void test_tail_chunks() {
  const int bk = 64, blocks = 6, block_bytes = 64 * bk * 2;
  for (int valid = 0; valid < bk; ++valid) {
    std::vector<unsigned char> stage(size_t(blocks) * block_bytes, 1);
    const int n = tail_chunks(valid, bk, blocks);
    CHECK(n == (bk - valid) * 8 * blocks);
    for (int i = 0; i < n; ++i) {
      const int off = tail_chunk_offset(i, valid, bk, block_bytes);
      CHECK(off >= 0 && off % 16 == 0 && off + 16 <= int(stage.size()));
      if (off < 0 || off + 16 > int(stage.size())) return;
      for (int b = 0; b < 16; ++b) {
        CHECK(stage[off + b] == 1);  // no chunk is written twice
        stage[off + b] = 0;
      }
    }
    for (int blk = 0; blk < blocks; ++blk)
      for (int row = 0; row < bk; ++row)
        for (int b = 0; b < 128; ++b)
          CHECK(stage[size_t(blk) * block_bytes + row * 128 + b] == (row < valid ? 1 : 0));
  }
}

int main() {
  test_raster();
  test_grouped();
  test_wgrad();
  test_tail_chunks();
  if (failures) {
    std::fprintf(stderr, "%d check(s) failed\n", failures);
    return 1;
  }
  std::puts("tile_math: all checks passed");
  return 0;
}
