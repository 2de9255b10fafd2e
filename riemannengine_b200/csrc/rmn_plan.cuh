// Layout of a convolution plan in device memory (see rmn_plan.cu):
//   [ PlanHeader (256 B) | perm int32[n_pos] | tile_mask uint32[n_tiles] | nbr_p int32[K][n_pos] ]
// n_pos = n_dst rounded up to 512 rows (the largest super-tile of the convolution kernels), so a
// tile never straddles the end of the table; every section starts on a 256-byte boundary.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace rmn {

constexpr int kPlanMaxK = 32;       // kernel volumes up to 32 offsets (one mask word per tile)
constexpr uint32_t kPlanMagic = 0x524d4e50u;  // "RMNP"
constexpr uint32_t kPlanRowPad = 512;

struct PlanHeader {
  uint32_t magic, n_dst, K, n_pos, n_tiles, words;
  uint32_t pad[58];
};
static_assert(sizeof(PlanHeader) == 256, "plan header must be 256 bytes");

struct PlanLayout {
  uint32_t n_pos, n_tiles;
  size_t perm, tile_mask, nbr_p, total;
};

inline PlanLayout plan_layout(uint32_t n_dst, int K) {
  PlanLayout L;
  L.n_pos = (n_dst + kPlanRowPad - 1) / kPlanRowPad * kPlanRowPad;
  L.n_tiles = L.n_pos / 128;
  const size_t words = (size_t)((K + 31) >> 5);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  L.perm = sizeof(PlanHeader);
  L.tile_mask = L.perm + up((size_t)L.n_pos * 4);
  L.nbr_p = L.tile_mask + up((size_t)L.n_tiles * words * 4);
  L.total = L.nbr_p + up((size_t)K * L.n_pos * 4);
  return L;
}

}  // namespace rmn
