// Index arithmetic of the persistent tile schedulers, shared by the kernels and by a host-side unit test
// (tests/cpp/test_tile_math.cpp, built with -fsanitize=address,undefined): which tile a linear index names,
// which rows of a ragged expert range a tile covers, and how many tiles a problem has.  Plain integer code that
// compiles for the host and for the device.
#pragma once

#if defined(__CUDACC__)
#define KF_TM_HD __host__ __device__ __forceinline__
#else
#define KF_TM_HD inline
#endif

namespace kf {
namespace tilemath {

KF_TM_HD int imin(int a, int b) { return a < b ? a : b; }
KF_TM_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Grouped rasterisation of an m_blocks x n_blocks tile grid: `group_m` consecutive row blocks share each sweep
// over the column blocks (so the column operand's tiles stay in L2).  Linear index t -> (m, n); a bijection
// onto the grid for 0 <= t < m_blocks * n_blocks, the last group may have fewer rows.
KF_TM_HD void raster(int t, int m_blocks, int n_blocks, int group_m, int& m, int& n) {
  const int per_group = group_m * n_blocks;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int rows = imin(group_m, m_blocks - first_m);
  const int r = t - g * per_group;
  m = first_m + r % rows;
  n = r / rows;
}

// Ragged grouped GEMM.  tile_start[e] = number of row tiles (of `bm` rows) of experts 0..e-1, tile_start[E] the
// total; offsets[e] .. offsets[e+1] are expert e's rows.  Fills tile_start and returns the total.
KF_TM_HD int grouped_tile_starts(const int* offsets, int E, int bm, int* tile_start) {
  int acc = 0;
  for (int e = 0; e < E; ++e) {
    tile_start[e] = acc;
    acc += ceil_div(offsets[e + 1] - offsets[e], bm);
  }
  tile_start[E] = acc;
  return acc;
}

struct GroupedTile {
  int e;      // expert
  int row0;   // first row of the tile in the sorted activation matrix
  int valid;  // rows of the tile that belong to the expert (1 .. bm)
  int nb;     // column block
};

// Linear tile index t (column block fastest) -> the tile; experts without rows own no tile.
KF_TM_HD GroupedTile grouped_decode(int t, int n_blocks, const int* tile_start, const int* offsets, int E, int bm) {
  const int nb = t % n_blocks;
  const int tmi = t / n_blocks;
  int lo = 0, hi = E;  // largest e with tile_start[e] <= tmi (among equal starts the last one owns the tile)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_start[mid] <= tmi) lo = mid; else hi = mid;
  }
  GroupedTile x;
  x.e = lo;
  const int mb = tmi - tile_start[lo];
  x.row0 = offsets[lo] + mb * bm;
  x.valid = imin(bm, offsets[lo + 1] - x.row0);
  x.nb = nb;
  return x;
}

struct WgradTile {
  int e, m0, n0;  // expert, first output row / column of the tile
  int row0, rows; // the expert's range of the reduction dimension
};

// Grouped weight gradient: every expert owns m_blocks x n_blocks output tiles, whatever its row count.
KF_TM_HD WgradTile wgrad_decode(int t, int m_blocks, int n_blocks, int bm, int bn, const int* offsets) {
  WgradTile x;
  const int per_e = m_blocks * n_blocks;
  x.e = t / per_e;
  const int r = t - x.e * per_e;
  x.m0 = (r / n_blocks) * bm;
  x.n0 = (r % n_blocks) * bn;
  x.row0 = offsets[x.e];
  x.rows = offsets[x.e + 1] - x.row0;
  return x;
}

// Number of zeroed 16-byte chunks, and the address of chunk i, when the rows `valid .. bk-1` of every
// {64 columns x bk rows} block of a stage (128 bytes per row, `blocks` blocks of `block_bytes`) are cleared.
KF_TM_HD int tail_chunks(int valid, int bk, int blocks) { return (bk - valid) * 8 * blocks; }
KF_TM_HD int tail_chunk_offset(int i, int valid, int bk, int block_bytes) {
  const int per_block = (bk - valid) * 8;
  const int blk = i / per_block, j = i - blk * per_block;
  return blk * block_bytes + valid * 128 + j * 16;
}

}  // namespace tilemath
}  // namespace kf
