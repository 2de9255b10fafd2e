// Convolution plan: an internal row order for the output-stationary convolution kernels in
// which (128-row tile, kernel offset) pairs are either mostly full or completely empty, so
// that empty pairs are skipped (no gather, no zero fill, no MMA).
//
// Output rows of a sparse tensor arrive in arbitrary order, so a tile of 128 consecutive rows
// has at least one neighbour at every offset and nothing can be skipped, although more than
// half of all (row, offset) entries are empty. Rows of one geometric situation share the empty
// offsets: a voxel on the bottom layer of a floor has no neighbour at any offset with dz = -1.
// The plan therefore sorts the rows by a small class key - one bit per (axis, sign): "has a
// neighbour at some offset on that side" - with a stable counting sort inside chunks of 32 768
// consecutive public rows (rows never leave their chunk: a batch is a concatenation of samples, and
// the CTAs that run at one time then gather from, and store to, the same few samples as they do in
// public order, so the rows they share stay in L2), and stores
//   perm[p]            public output row at internal position p (-1 in the padding),
//   tile_mask[t][w]    bit k of word k / 32: some row of tile t has a neighbour at offset k,
//   nbr_p[k][p]        the neighbour table in internal order (nbr[k][perm[p]]),
// which the planned convolution entry points consume. The public row numbering (first
// occurrence, the reference's contract: engine/grid/lattice_cpu.hpp:419-444) is untouched:
// the kernels store output row perm[p]. Results are bit-identical to the unplanned kernels'
// (every output row still accumulates its offsets in ascending order; a skipped offset
// contributed exact zeros).
//
// Build = three launches: row masks + class histogram, scan, scatter (permutation, tile
// masks, permuted table). It is paid once per kernel map and serves every convolution
// (forward, input gradient) that uses the map. The reference has no counterpart: its
// convolution is a per-offset torch loop over pair lists (engine/nn/conv.cpp:47-64).
#include "rmn_common.cuh"
#include "rmn_plan.cuh"

namespace rmn {

constexpr int kPlanBlock = 1024;          // rows per block of the histogram and scatter kernels
constexpr int kPlanBlocksPerChunk = 32;   // a chunk = 32 768 rows, sorted by class on its own

struct GroupBits {
  uint8_t g[kPlanMaxK];  // class bits an offset contributes when it has a neighbour
};

// Row masks, class keys and per-(chunk, class, block) counts. A block of 256 threads covers 1024 rows,
// four consecutive rows per thread: when the row count is a multiple of four every table read is one
// 16-byte load (kVec), else four 4-byte loads.
template <bool kVec>
__global__ void __launch_bounds__(256) k_plan_masks(const int32_t* __restrict__ nbr, uint32_t n, int K, GroupBits gb,
                                                    uint32_t* __restrict__ rowmask, uint8_t* __restrict__ cls,
                                                    uint32_t* __restrict__ hist, int n_bins) {
  __shared__ uint32_t s_hist[256];
  __shared__ uint8_t s_g[kPlanMaxK];
  s_hist[threadIdx.x] = 0;
  if (threadIdx.x < kPlanMaxK) s_g[threadIdx.x] = gb.g[threadIdx.x];
  __syncthreads();
  const uint32_t row0 = blockIdx.x * kPlanBlock + threadIdx.x * 4;
  uint32_t m[4] = {0, 0, 0, 0};  // bit k: a neighbour at offset k (plans cover up to 32 offsets)
  uint32_t c[4] = {0, 0, 0, 0};
  if (row0 < n) {
    for (int k0 = 0; k0 < K; k0 += 4) {  // four offsets x four rows in flight per thread
      int32_t v[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int32_t* src = nbr + (size_t)min(k0 + u, K - 1) * n + row0;
        if constexpr (kVec) {
          const int4 q = __ldg(reinterpret_cast<const int4*>(src));
          v[u][0] = q.x; v[u][1] = q.y; v[u][2] = q.z; v[u][3] = q.w;
        } else {
#pragma unroll
          for (int r = 0; r < 4; ++r) v[u][r] = row0 + r < n ? __ldg(src + r) : -1;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u;
        if (k < K) {
          const uint32_t g = s_g[k];
#pragma unroll
          for (int r = 0; r < 4; ++r)
            if (v[u][r] >= 0) {
              m[r] |= 1u << k;
              c[r] |= g;
            }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
      if (row0 + r < n) {
        rowmask[row0 + r] = m[r];
        cls[row0 + r] = (uint8_t)c[r];
      }
  }
  // one shared-memory atomic per class present in the warp (a block holds few classes: per-row atomics
  // would serialise on a handful of addresses)
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const bool live = row0 + r < n;
    const uint32_t peers = __match_any_sync(0xFFFFFFFFu, live ? c[r] : 0x1000u);
    if (live && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&s_hist[c[r]], (uint32_t)__popc(peers));
  }
  __syncthreads();
  // counts of (chunk, class) over the chunk's 32 blocks are contiguous
  const uint32_t chunk = blockIdx.x / kPlanBlocksPerChunk, in_chunk = blockIdx.x % kPlanBlocksPerChunk;
  if ((int)threadIdx.x < n_bins)
    hist[((size_t)chunk * n_bins + threadIdx.x) * kPlanBlocksPerChunk + in_chunk] = s_hist[threadIdx.x];
}

// One warp per (chunk, class): exclusive scan of its 32 per-block counts in place, totals[chunk][class] = rows
// of the class in the chunk. (Blocks past the end of the table were never written: n_blocks bounds the reads.)
// The first thread also writes the plan's header (handed over as a kernel argument: a host-to-device copy of
// it would wait behind whatever large upload - the next batch of an input pipeline - is on the copy engine).
__global__ void __launch_bounds__(256) k_plan_scan(uint32_t* __restrict__ hist, uint32_t n_blocks, int n_bins,
                                                   uint32_t n_chunks, uint32_t* __restrict__ totals,
                                                   const PlanHeader hdr, PlanHeader* __restrict__ hdr_out) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *hdr_out = hdr;
  const uint32_t pair = blockIdx.x * 8 + (threadIdx.x >> 5);  // chunk * n_bins + class
  const int lane = threadIdx.x & 31;
  if (pair >= n_chunks * (uint32_t)n_bins) return;
  const uint32_t chunk = pair / (uint32_t)n_bins;
  const bool present = chunk * kPlanBlocksPerChunk + lane < n_blocks;
  uint32_t* p = hist + (size_t)pair * kPlanBlocksPerChunk + lane;
  const uint32_t v = present ? *p : 0u;
  uint32_t incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if (lane >= d) incl += t;
  }
  if (present) *p = incl - v;
  if (lane == 31) totals[pair] = incl;
}

// Stable scatter of the rows into class order inside their chunk: position = chunk start + (rows of smaller
// classes in the chunk) + (rows of the same class in earlier blocks of the chunk) + (rank inside the block). Writes the permutation, ORs the row masks into the
// tile masks and copies the neighbour table into internal order through shared memory, so that the rows
// of one class in a block (consecutive positions) leave as coalesced runs.
__global__ void __launch_bounds__(kPlanBlock) k_plan_scatter(
    const int32_t* __restrict__ nbr, uint32_t n, int K, const uint32_t* __restrict__ rowmask,
    const uint8_t* __restrict__ cls, const uint32_t* __restrict__ hist, const uint32_t* __restrict__ totals,
    uint32_t n_blocks, int n_bins, uint32_t n_pos, int32_t* __restrict__ perm, uint32_t* __restrict__ tile_mask,
    int32_t* __restrict__ nbr_p) {
  __shared__ uint32_t s_base[256];        // first position of (class, this block)
  __shared__ uint32_t s_local[256];       // first block-local slot of the class
  __shared__ uint16_t s_warp[32][256];    // rows of the class in the warp -> exclusive prefix over the warps
  __shared__ uint32_t s_dest[kPlanBlock];
  __shared__ int32_t s_buf[2][kPlanBlock];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int words = (K + 31) >> 5;
  const uint32_t chunk = blockIdx.x / kPlanBlocksPerChunk, in_chunk = blockIdx.x % kPlanBlocksPerChunk;

  for (int i = tid; i < 32 * 256; i += kPlanBlock) (&s_warp[0][0])[i] = 0;
  if (warp == 0) {
    // exclusive scan of the class totals: eight classes per lane
    uint32_t t[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int b = lane * 8 + i;
      t[i] = b < n_bins ? totals[(size_t)chunk * n_bins + b] : 0u;
      sum += t[i];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += o;
    }
    uint32_t run = chunk * (uint32_t)(kPlanBlocksPerChunk * kPlanBlock) + incl - sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int b = lane * 8 + i;
      s_base[b] = run + (b < n_bins ? hist[((size_t)chunk * n_bins + b) * kPlanBlocksPerChunk + in_chunk] : 0u);
      run += t[i];
    }
  }
  __syncthreads();

  const uint32_t row = blockIdx.x * kPlanBlock + tid;
  const bool active = row < n;
  const uint32_t c = active ? (uint32_t)cls[row] : 0u;
  const uint32_t peers = __match_any_sync(0xFFFFFFFFu, active ? c : 0x1000u);
  const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
  if (active && rank == 0) s_warp[warp][c] = (uint16_t)__popc(peers);
  __syncthreads();
  if (tid < 256) {
    uint32_t run = 0;
    for (int w = 0; w < 32; ++w) {
      const uint32_t v = s_warp[w][tid];
      s_warp[w][tid] = (uint16_t)run;
      run += v;
    }
    s_local[tid] = run;  // rows of the class in this block, scanned below
  }
  __syncthreads();
  if (warp == 0) {
    uint32_t t[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      t[i] = s_local[lane * 8 + i];
      sum += t[i];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += o;
    }
    uint32_t run = incl - sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s_local[lane * 8 + i] = run;
      run += t[i];
    }
  }
  __syncthreads();

  uint32_t pos = 0xFFFFFFFFu, slot = 0;
  if (active) {
    const uint32_t in_block = (uint32_t)s_warp[warp][c] + rank;
    pos = s_base[c] + in_block;
    slot = s_local[c] + in_block;
    s_dest[slot] = pos;
    perm[pos] = (int32_t)row;
  }
  // tile masks: the lanes of a warp that land in one tile OR their masks first, one atomic per group
  const uint32_t tpeers = __match_any_sync(0xFFFFFFFFu, active ? (pos >> 7) : 0xFFFFFFFFu);
  for (int w = 0; w < words; ++w) {
    const uint32_t m = active ? rowmask[(size_t)w * n + row] : 0u;
    const uint32_t all = __reduce_or_sync(tpeers, m);
    if (active && lane == __ffs(tpeers) - 1 && all) atomicOr(&tile_mask[(size_t)(pos >> 7) * words + w], all);
  }
  __syncthreads();

  const uint32_t block_rows = min((uint32_t)kPlanBlock, n - blockIdx.x * kPlanBlock);
  const uint32_t my_dest = (uint32_t)tid < block_rows ? s_dest[tid] : 0u;
  for (int k0 = 0; k0 < K; k0 += 9) {  // nine table reads in flight per thread, then one exchange per offset
    int32_t v[9];
#pragma unroll
    for (int u = 0; u < 9; ++u) v[u] = (active && k0 + u < K) ? __ldg(nbr + (size_t)(k0 + u) * n + row) : -1;
#pragma unroll
    for (int u = 0; u < 9; ++u) {
      if (k0 + u < K) {  // uniform across the block
        if (active) s_buf[(k0 + u) & 1][slot] = v[u];  // buffers alternate across the groups too
        __syncthreads();
        if ((uint32_t)tid < block_rows) __stcs(nbr_p + (size_t)(k0 + u) * n_pos + my_dest, s_buf[(k0 + u) & 1][tid]);
      }
    }
  }
  // padding positions [n, n_pos): no row, no neighbour
  if (blockIdx.x == gridDim.x - 1) {
    const uint32_t pad = n_pos - n;
    for (uint32_t i = tid; i < pad * (uint32_t)(K + 1); i += kPlanBlock) {
      const uint32_t k = i / pad, p = n + i % pad;
      if (k == (uint32_t)K) perm[p] = -1;
      else nbr_p[(size_t)k * n_pos + p] = -1;
    }
  }
}

}  // namespace rmn

using namespace rmn;

extern "C" size_t rmn_conv_plan_bytes(uint32_t n_dst, int K) {
  if (K < 1 || K > kPlanMaxK) return 0;
  return plan_layout(n_dst, K).total;
}

extern "C" size_t rmn_conv_plan_workspace_bytes(uint32_t n_dst, int K) {
  if (K < 1 || K > kPlanMaxK) return 0;
  const size_t nb = (n_dst + kPlanBlock - 1) / kPlanBlock;
  const size_t chunks = (nb + kPlanBlocksPerChunk - 1) / kPlanBlocksPerChunk;
  const size_t words = (K + 31) >> 5;
  // row masks | class keys | per-(chunk, class, block) counts | per-(chunk, class) totals
  return (size_t)n_dst * 4 * words + (((size_t)n_dst + 255) & ~(size_t)255) +
         chunks * 256 * kPlanBlocksPerChunk * 4 + chunks * 256 * 4 + 256;
}

extern "C" int rmn_conv_plan_build(const int32_t* d_nbr, uint32_t n_dst, int K, const int32_t* offsets, int D,
                                   void* d_plan, size_t plan_bytes, void* d_workspace, size_t workspace_bytes,
                                   void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (K < 1 || D < 1 || D >= RMN_MAX_W || !offsets || !d_plan) return RMN_ERR_BAD_ARG;
  if (K > kPlanMaxK) return RMN_ERR_UNSUPPORTED;
  if (n_dst == 0 || n_dst >= 0x7FFFFE00u) return RMN_ERR_BAD_ARG;
  if (!d_nbr || !d_workspace || ((uintptr_t)d_plan & 255)) return RMN_ERR_BAD_ARG;
  const PlanLayout L = plan_layout(n_dst, K);
  if (plan_bytes < L.total || workspace_bytes < rmn_conv_plan_workspace_bytes(n_dst, K)) return RMN_ERR_ALLOC;

  // class bits: one per (axis, sign) of the first four axes; an offset sets the bits of the sides it lies on
  GroupBits gb;
  const int axes = D < 4 ? D : 4;
  for (int k = 0; k < kPlanMaxK; ++k) gb.g[k] = 0;
  for (int k = 0; k < K; ++k)
    for (int a = 0; a < axes; ++a) {
      const int32_t o = offsets[(size_t)k * D + a];
      if (o < 0) gb.g[k] |= (uint8_t)(1u << (2 * a));
      if (o > 0) gb.g[k] |= (uint8_t)(1u << (2 * a + 1));
    }
  const int n_bins = 1 << (2 * axes);

  const uint32_t nb = (n_dst + kPlanBlock - 1) / kPlanBlock;
  const int words = (K + 31) >> 5;
  char* ws = static_cast<char*>(d_workspace);
  uint32_t* rowmask = reinterpret_cast<uint32_t*>(ws);
  uint8_t* cls = reinterpret_cast<uint8_t*>(ws + (size_t)n_dst * 4 * words);
  uint32_t* hist = reinterpret_cast<uint32_t*>(ws + (size_t)n_dst * 4 * words + (((size_t)n_dst + 255) & ~(size_t)255));
  const uint32_t chunks = (nb + kPlanBlocksPerChunk - 1) / kPlanBlocksPerChunk;
  uint32_t* totals = hist + (size_t)chunks * 256 * kPlanBlocksPerChunk;

  char* plan = static_cast<char*>(d_plan);
  PlanHeader hdr = {};
  hdr.magic = kPlanMagic;
  hdr.n_dst = n_dst;
  hdr.K = (uint32_t)K;
  hdr.n_pos = L.n_pos;
  hdr.n_tiles = L.n_tiles;
  hdr.words = (uint32_t)words;
  RMN_CUDA_TRY(cudaMemsetAsync(plan + L.tile_mask, 0, (size_t)L.n_tiles * words * 4, stream));
  if ((n_dst & 3u) == 0 && ((uintptr_t)d_nbr & 15) == 0)
    k_plan_masks<true><<<nb, 256, 0, stream>>>(d_nbr, n_dst, K, gb, rowmask, cls, hist, n_bins);
  else
    k_plan_masks<false><<<nb, 256, 0, stream>>>(d_nbr, n_dst, K, gb, rowmask, cls, hist, n_bins);
  RMN_LAUNCH_CHECK();
  k_plan_scan<<<(chunks * (uint32_t)n_bins + 7) / 8, 256, 0, stream>>>(hist, nb, n_bins, chunks, totals, hdr,
                                                                       reinterpret_cast<PlanHeader*>(plan));
  RMN_LAUNCH_CHECK();
  k_plan_scatter<<<nb, kPlanBlock, 0, stream>>>(d_nbr, n_dst, K, rowmask, cls, hist, totals, nb, n_bins, L.n_pos,
                                                reinterpret_cast<int32_t*>(plan + L.perm),
                                                reinterpret_cast<uint32_t*>(plan + L.tile_mask),
                                                reinterpret_cast<int32_t*>(plan + L.nbr_p));
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}
