// Tile scheduler shared by the grouped expert GEMMs: work item g of a persistent CTA -> (row group,
// first slab row, valid rows, weight-row tile), decoded from the device-side offsets of the row groups
// with no host synchronisation and no count-dependent launch.
#pragma once
#include "msl_common.cuh"

namespace msl {

struct TileInfo {
  int expert, row0, rows, nt;   // row group, first slab row, valid rows in the tile, n tile
};

// mt_prefix[e] = number of row tiles of the groups before e (mt_prefix[experts] = all of them), formed by
// one warp from the offsets.
__device__ __forceinline__ void row_tile_prefix(const int* __restrict__ offsets, int experts, int tile_m,
                                                int* mt_prefix, int lane) {
  int carry = 0;
  for (int b0 = 0; b0 < experts; b0 += 32) {
    const int i = b0 + lane;
    const int c = i < experts ? (offsets[i + 1] - offsets[i] + tile_m - 1) / tile_m : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int nb = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += nb;
    }
    if (i < experts) mt_prefix[i] = carry + inc - c;
    carry += __shfl_sync(0xffffffffu, inc, 31);
  }
  if (lane == 0) mt_prefix[experts] = carry;
}

// Tiles of one (group, n tile) are adjacent so the weight tile they share stays in L2.
__device__ __forceinline__ TileInfo decode_tile(int g, const int* mt_prefix, const int* offsets, int experts,
                                                int n_tiles, int tile_m) {
  int lo = 0, hi = experts - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (mt_prefix[mid] * n_tiles <= g) lo = mid; else hi = mid - 1;
  }
  const int e = lo;
  const int mte = mt_prefix[e + 1] - mt_prefix[e];
  const int r = g - mt_prefix[e] * n_tiles;
  const int nt = r / mte, mt = r - nt * mte;
  const int start = offsets[e], cnt = offsets[e + 1] - start;
  TileInfo ti;
  ti.expert = e;
  ti.row0 = start + mt * tile_m;
  ti.rows = min(tile_m, cnt - mt * tile_m);
  ti.nt = nt;
  return ti;
}

}  // namespace msl
