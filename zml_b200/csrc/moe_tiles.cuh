// Tile enumeration of the grouped (per-expert) GEMMs: the number of tiles of an expert depends on its
// token count, which lives on the device, so every CTA builds the table "first tile of expert e" once,
// in shared memory, and every role finds the expert of a tile by bisection.  (Walking the experts with
// global loads at every tile change cost about 1.5 us per tile on 128 experts.)
#pragma once
#include "common.cuh"

constexpr int kZbMaxExperts = 1024;

struct ZbTilePos {
  int e;       // expert
  int wt;      // weight tile within the expert
  int tt;      // token tile within the expert
};

// prefix[e] = tiles of experts 0..e-1, prefix[e_local] = all tiles.  Tiles of an expert: w_tiles weight
// tiles x ceil(tokens / rows_per_token_tile) token tiles.  Called by all threads of the CTA (after the
// offsets are visible); ends with a __syncthreads.
ZB_DEVICE void zb_tile_prefix_build(int32_t* prefix, const int32_t* offsets, int e_local, int w_tiles, int rows_per_token_tile) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (e_local + 31) / 32;
  if (warp == 0) {
    const int e0 = lane * per, e1 = min(e_local, e0 + per);
    int s = 0;
    for (int e = e0; e < e1; ++e) s += w_tiles * ((offsets[e + 1] - offsets[e] + rows_per_token_tile - 1) / rows_per_token_tile);
    int incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - s;
    for (int e = e0; e < e1; ++e) {
      prefix[e] = run;
      run += w_tiles * ((offsets[e + 1] - offsets[e] + rows_per_token_tile - 1) / rows_per_token_tile);
    }
    if (lane == 31) prefix[e_local] = incl;
  }
  __syncthreads();
}

// Tile g -> (expert, weight tile, token tile); token tile varies slowest so that CTAs running together share
// the expert's tokens.  `hint` is the expert of this role's previous tile (tiles are visited in increasing order).
ZB_DEVICE bool zb_tile_locate(const int32_t* prefix, int e_local, int w_tiles, int g, int& hint, ZbTilePos& pos) {
  if (g >= prefix[e_local]) return false;
  int lo = hint, hi = e_local;            // prefix[lo] <= g < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= g) lo = mid;
    else hi = mid;
  }
  hint = lo;
  const int local = g - prefix[lo];
  pos.e = lo;
  pos.tt = local / w_tiles;
  pos.wt = local - pos.tt * w_tiles;
  return true;
}
