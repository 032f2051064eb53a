// Host test of the attention kernels' block order (csrc/tile_order.h): for a range of grid shapes the decode must be a
// bijection onto (tile rank, head), keep every group's heads together, and never start a lighter tile of a group
// before a heavier one.
#include <cstdio>
#include <vector>

#include "tile_order.h"

int main() {
  const int shapes[][3] = {{32, 128, 24}, {32, 64, 16}, {32, 64, 1}, {32, 64, 64}, {7, 5, 3}, {1, 9, 4}, {13, 1, 8}, {256, 2, 1}, {32, 10, 4}};
  for (const auto& sh : shapes) {
    const int n_tiles = sh[0], n_heads = sh[1], group = sh[2] > n_heads ? n_heads : sh[2];
    std::vector<int> seen(n_tiles * n_heads, 0);
    int prev_group = 0, prev_rank = 0;
    for (int c = 0; c < n_tiles * n_heads; ++c) {
      int rank = -1, head = -1;
      tlm::heavy_first_decode(c, n_tiles, n_heads, group, rank, head);
      if (rank < 0 || rank >= n_tiles || head < 0 || head >= n_heads) { std::printf("out of range at %d\n", c); return 1; }
      if (seen[head * n_tiles + rank]++) { std::printf("duplicate at %d\n", c); return 1; }
      const int g = head / group;
      if (g < prev_group) { std::printf("group order at %d\n", c); return 1; }
      if (g == prev_group && rank < prev_rank) { std::printf("a heavier tile after a lighter one at %d\n", c); return 1; }
      prev_group = g; prev_rank = rank;
    }
  }
  std::printf("ok\n");
  return 0;
}
