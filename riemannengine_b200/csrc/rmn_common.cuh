// Shared device/host definitions of the rmn_b200 library (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "rmn_b200.h"

namespace rmn {

// ---------------------------------------------------------------------------
// Hash-table layout in device memory:
//   [ TableHeader (256 B) | Slot[capacity] ]
// A coordinate row is packed into one 63-bit key: column c contributes
// (value - mn[c]) << shift[c] using bits[c] bits, where mn/mx are the column
// extrema of the rows the table was built from. A query row outside the
// bounding box cannot be in the table and is rejected before probing.
// ---------------------------------------------------------------------------
struct __align__(16) Slot {
  unsigned long long key;  // kEmptyKey when free
  uint32_t first_row;      // smallest input row holding this key
  uint32_t uid;            // row in the unique (first-occurrence) numbering; bit 31: kPassedBit
};
static_assert(sizeof(Slot) == 16, "slot must be 16 bytes");

constexpr unsigned long long kEmptyKey = ~0ull;
// Bit 31 of Slot::uid (row counts stay below 2^31): some other key was displaced past this occupied slot
// during the build. A lookup that meets a different key in a slot WITHOUT the bit stops there - nothing it
// could be looking for lies beyond - instead of walking on to the first free slot. More than half of a kernel
// map's probes are misses; at load 1/3 such a walk costs a miss 0.5 further buckets (cache lines) on average,
// with the bit about 0.05.
constexpr uint32_t kPassedBit = 0x80000000u;
constexpr uint32_t kTableMagic = 0x524d4e54u;  // "RMNT"

struct __align__(16) TableHeader {
  uint32_t magic;
  uint32_t W;
  uint32_t n_rows;
  uint32_t n_unique;
  uint32_t status;
  uint32_t capacity;   // number of slots (a multiple of 32, about 3 x n_rows)
  uint32_t total_bits;
  uint32_t n_dups;     // rows that found their key already present (0: unique rows == input rows)
  int32_t mn[RMN_MAX_W];
  int32_t mx[RMN_MAX_W];
  uint32_t bits[RMN_MAX_W];
  uint32_t shift[RMN_MAX_W];
  uint32_t range_blocks_done;  // ticket counter of the fill + range kernel (its last block plans the packing)
  uint32_t count_blocks_done;  // ticket counter of the first-occurrence count (its last block scans the counts)
  // Column bounds while they are being reduced, encoded so that an all-zero header means "no row yet" and
  // both are running maxima: mx_enc = max(v ^ 0x80000000), mn_enc = max(~(v ^ 0x80000000)).
  uint32_t mn_enc[RMN_MAX_W];
  uint32_t mx_enc[RMN_MAX_W];
  // Bits of the first spatial column that are the same in every row (the rows of a map at tensor
  // stride 2^s sit on a 2^s grid): x_or is the OR over the rows of (x - x of row 0), pos_shift its
  // number of trailing zeros. The position inside a bucket is taken from the bits above them.
  uint32_t x_or;
  uint32_t pos_shift;
  uint32_t pad[4];
};
static_assert(sizeof(TableHeader) == 256, "header must be 256 bytes");

// Packing parameters held in registers by the kernels.
template <int W>
struct Packer {
  int32_t mn[W];
  uint32_t span[W];  // mx - mn
  uint32_t shift[W];

  __device__ __forceinline__ void load(const TableHeader* h) {
#pragma unroll
    for (int c = 0; c < W; ++c) {
      mn[c] = h->mn[c];
      span[c] = (uint32_t)(h->mx[c] - h->mn[c]);
      shift[c] = h->shift[c];
    }
  }
  // false when the row lies outside the bounding box of the table's rows
  __device__ __forceinline__ bool pack(const int32_t (&c)[W], unsigned long long& key) const {
    unsigned long long k = 0;
    bool ok = true;
#pragma unroll
    for (int i = 0; i < W; ++i) {
      uint32_t d = (uint32_t)c[i] - (uint32_t)mn[i];
      ok = ok && (d <= span[i]);
      k |= (unsigned long long)d << shift[i];
    }
    key = k;
    return ok;
  }
};

// Slot of a key: three bits of the first spatial column (packed first, so they are key bits
// [pos_shift, pos_shift + 3)) select the position inside an 8-slot (128-byte) bucket; the bits
// above them are mixed to 32 bits and range-reduced (multiply-shift) onto the bucket index.
// pos_shift skips the low bits that are equal in all rows of the table (a map at tensor stride 4
// only has x = 0 mod 4: taking the raw low three bits would leave six of the eight positions of
// every bucket unused). Eight voxels that are consecutive along the first spatial axis (in units
// of the map's grid) therefore share one 128-byte line, so the x-1 / x / x+1 probes of a kernel
// map hit the line the thread has just pulled into L1. Collisions step to the same position of
// the next bucket. A query key whose low pos_shift bits are not zero matches no stored key.
__device__ __forceinline__ uint32_t hash_key(unsigned long long k, uint32_t capacity, uint32_t pos_shift) {
  const unsigned long long b = k >> (3u + pos_shift);
  uint32_t h = (uint32_t)b ^ ((uint32_t)(b >> 32) * 0x9E3779B1u);
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return __umulhi(h, capacity >> 3) * 8u + ((uint32_t)(k >> pos_shift) & 7u);
}
__device__ __forceinline__ uint32_t next_slot(uint32_t s, uint32_t capacity) {
  s += 8u;
  return s >= capacity ? s - capacity : s;
}

__device__ __forceinline__ ulonglong2 load_slot(const Slot* s) {
  return __ldg(reinterpret_cast<const ulonglong2*>(s));
}

// Lookup; returns uid or 0xFFFFFFFF. Probing is bounded by the bucket count.
__device__ __forceinline__ uint32_t table_find(const Slot* slots, uint32_t capacity, uint32_t pos_shift,
                                               unsigned long long key) {
  uint32_t s = hash_key(key, capacity, pos_shift);
  for (uint32_t probe = 0; probe < (capacity >> 3); ++probe) {
    ulonglong2 v = load_slot(slots + s);
    const uint32_t uid = (uint32_t)(v.y >> 32);
    if (v.x == key) return uid & ~kPassedBit;
    if (v.x == kEmptyKey || !(uid & kPassedBit)) return 0xFFFFFFFFu;
    s = next_slot(s, capacity);
  }
  return 0xFFFFFFFFu;
}

template <int W>
__device__ __forceinline__ void load_row(const int32_t* __restrict__ coords, uint32_t row,
                                         int32_t (&c)[W]) {
  if constexpr (W == 4) {
    int4 v = __ldg(reinterpret_cast<const int4*>(coords) + row);
    c[0] = v.x; c[1] = v.y; c[2] = v.z; c[3] = v.w;
  } else if constexpr (W == 2) {
    int2 v = __ldg(reinterpret_cast<const int2*>(coords) + row);
    c[0] = v.x; c[1] = v.y;
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) c[i] = __ldg(coords + (size_t)row * W + i);
  }
}

// Slot count for n_rows inserted rows: load factor <= 1/4 (<= 1/3 for large tables, below), a multiple of 32,
// at least 64. (Measured on
// 1.2 M voxels, insert + self-map probe / general 27-offset probe: 2 n slots 0.312 / 0.435 ms, 3 n
// 0.228 / 0.238, 4 n 0.216 / 0.198, 6 n 0.216 / 0.173, 8 n 0.225 / 0.165: displaced keys cost a further
// cache line per lookup, the slot fill grows with the table.)
// A table that no longer fits the 126 MB L2 gets 3 n slots: its misses then go to DRAM whatever its
// size, and the smaller table keeps more of its lines cached (4.8 M rows of a 4-D map, 81 offsets:
// 5.29 ms per step with 3 n, 5.57 ms with 4 n).
inline uint32_t table_capacity(uint32_t n_rows) {
  const unsigned long long per_row = (4ull * n_rows + 64ull) * 16ull <= (120ull << 20) ? 4ull : 3ull;
  const unsigned long long want = per_row * n_rows + 64ull;
  return (uint32_t)((want + 31ull) / 32ull * 32ull);
}

// load_row uses 16-byte (W == 4) / 8-byte (W == 2) vector loads
inline bool coords_aligned(const void* p, int W) {
  const uintptr_t a = (uintptr_t)p;
  return W == 4 ? (a & 15) == 0 : W == 2 ? (a & 7) == 0 : (a & 3) == 0;
}

void count_launch();

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? RMN_OK : RMN_ERR_CUDA; }

#define RMN_CUDA_TRY(expr)                        \
  do {                                            \
    cudaError_t _e = (expr);                      \
    if (_e != cudaSuccess) return RMN_ERR_CUDA;   \
  } while (0)

// Every kernel launch of the library is followed by exactly one RMN_LAUNCH_CHECK, which also
// feeds the launch counter read by rmn_launch_count().
#define RMN_LAUNCH_CHECK()                 \
  do {                                     \
    ::rmn::count_launch();                 \
    RMN_CUDA_TRY(cudaGetLastError());      \
  } while (0)

// Dispatch a functor templated on the coordinate width.
#define RMN_DISPATCH_W(W_, ...)                   \
  switch (W_) {                                   \
    case 2: { constexpr int kW = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int kW = 3; __VA_ARGS__; } break; \
    case 4: { constexpr int kW = 4; __VA_ARGS__; } break; \
    case 5: { constexpr int kW = 5; __VA_ARGS__; } break; \
    case 6: { constexpr int kW = 6; __VA_ARGS__; } break; \
    case 7: { constexpr int kW = 7; __VA_ARGS__; } break; \
    case 8: { constexpr int kW = 8; __VA_ARGS__; } break; \
    default: return RMN_ERR_BAD_ARG;              \
  }

}  // namespace rmn
