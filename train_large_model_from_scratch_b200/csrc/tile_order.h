// Block order of the causal attention grids, written once for the device and for a host test
// (tests/tile_order_host_test.cpp).
#pragma once

#ifdef __CUDACC__
#define TLM_TILE_HD __host__ __device__ __forceinline__
#else
#define TLM_TILE_HD inline
#endif

namespace tlm {

// Heavy-first order for causal attention grids. Tiles of one (batch, head) differ in work by the causal mask (rank 0
// heaviest); blocks start in linear order, so the order decides the tail: with all tiles of one head adjacent, the last
// head's heaviest tiles start when the grid is almost drained and run alone. Here the heads are taken in groups of
// `group` (few enough that the group's tensors stay in L2), and inside a group all heads' rank-0 tiles come first, then
// all rank-1 tiles, ...: every group, the last one included, ends on its lightest tiles.
//   linear block id in [0, n_tiles * n_heads) -> (rank of the tile within its head, head); a bijection.
TLM_TILE_HD void heavy_first_decode(int linear, int n_tiles, int n_heads, int group, int& tile_rank, int& head) {
  const int per_group = n_tiles * group;
  const int g = linear / per_group, r = linear - g * per_group;
  const int left = n_heads - g * group;
  const int g_heads = group < left ? group : left;            // the last group may be smaller
  tile_rank = r / g_heads;
  head = g * group + (r - tile_rank * g_heads);
}

}  // namespace tlm
