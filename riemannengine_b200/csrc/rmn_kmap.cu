// Kernel-map generation: for every query row and kernel offset, probe the
// coordinate table; results land in an offset-major neighbour table
// nbr[K][n_query] (what the convolution kernels consume) and, on request, in
// CSR-over-offsets pair lists (the reference's per-offset in/out vectors,
// engine/grid/maps.hpp:19-79).
//
// Pass 1 (k_kmap_probe): one thread per query row keeps the row in registers
// (one vectorised 16-byte load for W = 4), loops over the K offsets held in
// shared memory, probes, writes nbr[k][q] (coalesced: consecutive lanes are
// consecutive rows) and counts hits per offset with warp ballots.
// Pass 2 (k_kmap_scan): exclusive scan of the per-(offset, block) hit counts
// and of the per-offset totals -> offset_ptr[K+1].
// Pass 3 (k_kmap_pairs, optional): ballot compaction of nbr into (a, q) pair
// lists at deterministic positions (pairs of one offset sorted by query row),
// with no sort and no atomics. The reference instead sorts all triplets by
// offset (engine/grid/lattice_gpu.cuh:440-488).
#include "rmn_common.cuh"

#include <mutex>

namespace rmn {

constexpr int kKmapBlock = 256;

// The packed key is linear in the coordinates: key(c + off) = key(c) + sum_i (off_i << shift_i)
// in 64-bit modular arithmetic, so each probe costs one 64-bit add on top of the range test
// (a neighbour outside the table's bounding box is a miss without touching memory).
template <int W>
__global__ void __launch_bounds__(kKmapBlock) k_kmap_probe(
    const TableHeader* __restrict__ h, const Slot* __restrict__ slots,
    const int32_t* __restrict__ query, uint32_t n_query, const int32_t* __restrict__ offsets,
    int K, int32_t* __restrict__ nbr, uint32_t* __restrict__ block_counts, uint32_t n_blocks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int D = W - 1;
  long long* s_delta = reinterpret_cast<long long*>(smem_raw);           // [K]
  int32_t* s_off = reinterpret_cast<int32_t*>(s_delta + K);              // [K][D]
  uint32_t* s_cnt = reinterpret_cast<uint32_t*>(s_off + K * D);          // [K]
  for (int i = threadIdx.x; i < K * D; i += kKmapBlock) s_off[i] = offsets[i];
  for (int k = threadIdx.x; k < K; k += kKmapBlock) {
    long long d = 0;
#pragma unroll
    for (int a = 0; a < D; ++a) d += (long long)offsets[k * D + a] << h->shift[a + 1];
    s_delta[k] = d;
    s_cnt[k] = 0;
  }
  __syncthreads();

  const uint32_t capacity = h->capacity, pos_shift = h->pos_shift;
  const uint32_t q = blockIdx.x * kKmapBlock + threadIdx.x;
  const bool active = q < n_query;
  int32_t c[W];
  if (active) {
    load_row<W>(query, q, c);
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) c[i] = 0;
  }
  // distance from the box minimum per column, the packed centre key, and the box spans
  uint32_t dist[W], span[W];
  long long ckey = 0;
#pragma unroll
  for (int i = 0; i < W; ++i) {
    const int32_t mn = h->mn[i];
    dist[i] = (uint32_t)c[i] - (uint32_t)mn;
    span[i] = (uint32_t)(h->mx[i] - mn);
    ckey += (long long)((long long)c[i] - (long long)mn) << h->shift[i];
  }
  const bool batch_ok = active && dist[0] <= span[0];
  const int lane = threadIdx.x & 31;
  // Offsets are handled kUnroll at a time: the first-probe loads of a batch are issued before any
  // is examined, so a thread keeps several table reads in flight. With the region's first axis
  // varying fastest, a batch of three is the x-1 / x / x+1 triple that shares one table line.
  // Only the HOME slot is read here. One lookup in eight has to walk on (a foreign key with the
  // passed-over bit), but in almost every warp some lane does, so walking inside this loop made
  // every warp pay a second and third dependent table read per offset; those lookups are noted in
  // a bit mask instead (64 offsets per chunk) and finished, thread by thread, after the chunk.
  constexpr int kUnroll = 3;
  for (int chunk0 = 0; chunk0 < K; chunk0 += 64) {
    const int chunk_end = min(K, chunk0 + 64);
    unsigned long long pending = 0ull;
    for (int k0 = chunk0; k0 < chunk_end; k0 += kUnroll) {
      unsigned long long key[kUnroll];
      ulonglong2 first[kUnroll];
      bool valid[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = min(k0 + u, chunk_end - 1);
        bool in_box = batch_ok && (k0 + u < chunk_end);
#pragma unroll
        for (int a = 0; a < D; ++a) in_box = in_box && (dist[a + 1] + (uint32_t)s_off[k * D + a] <= span[a + 1]);
        valid[u] = in_box;
        key[u] = (unsigned long long)(ckey + s_delta[k]);
        first[u] = make_ulonglong2(kEmptyKey, 0ull);
        if (in_box) first[u] = load_slot(slots + hash_key(key[u], capacity, pos_shift));
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = k0 + u;
        if (k < chunk_end) {  // uniform across the block
          const uint32_t found = (uint32_t)(first[u].y >> 32);
          uint32_t uid = 0xFFFFFFFFu;
          if (valid[u]) {
            if (first[u].x == key[u]) uid = found & ~kPassedBit;
            else if (first[u].x != kEmptyKey && (found & kPassedBit)) pending |= 1ull << (k - chunk0);
          }
          if (active) __stcs(nbr + (size_t)k * n_query + q, (int32_t)uid);
          const uint32_t hits = __ballot_sync(0xFFFFFFFFu, uid != 0xFFFFFFFFu);
          if (lane == 0) atomicAdd(&s_cnt[k], (uint32_t)__popc(hits));
        }
      }
    }
    while (pending) {  // the lookups that walk on: from the slot behind the home slot
      const int k = chunk0 + __ffsll((long long)pending) - 1;
      pending &= pending - 1ull;
      const unsigned long long key = (unsigned long long)(ckey + s_delta[k]);
      uint32_t s = next_slot(hash_key(key, capacity, pos_shift), capacity);
      for (uint32_t probe = 1; probe < (capacity >> 3); ++probe) {
        const ulonglong2 v = load_slot(slots + s);
        const uint32_t found = (uint32_t)(v.y >> 32);
        if (v.x == key) {
          __stcs(nbr + (size_t)k * n_query + q, (int32_t)(found & ~kPassedBit));
          atomicAdd(&s_cnt[k], 1u);
          break;
        }
        if (v.x == kEmptyKey || !(found & kPassedBit)) break;
        s = next_slot(s, capacity);
      }
    }
  }
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += kKmapBlock)
    block_counts[(size_t)k * n_blocks + blockIdx.x] = s_cnt[k];
}

// Self map with a point-symmetric region (stride-1 convolution: the query rows ARE the table's
// rows, offsets[K-1-k] == -offsets[k], offsets[K/2] == 0). A pair (q -> a) at offset k implies
// (a -> q) at offset K-1-k, so only the first K/2 offsets are probed; every hit also fills its
// mirror entry (one scattered 4-byte store instead of a second probe) and the centre offset is
// the identity. The mirrored half of nbr must hold -1 before the launch.
template <int W>
__global__ void __launch_bounds__(kKmapBlock) k_kmap_probe_self(
    const TableHeader* __restrict__ h, const Slot* __restrict__ slots,
    const int32_t* __restrict__ coords, uint32_t n, const int32_t* __restrict__ offsets, int K,
    int32_t* __restrict__ nbr, uint32_t* __restrict__ block_counts, uint32_t n_blocks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int D = W - 1;
  const int half = K / 2;
  long long* s_delta = reinterpret_cast<long long*>(smem_raw);   // [half]
  int32_t* s_off = reinterpret_cast<int32_t*>(s_delta + (half > 0 ? half : 1));  // [half][D]
  uint32_t* s_cnt = reinterpret_cast<uint32_t*>(s_off + (half > 0 ? half : 1) * D);  // [half]
  for (int i = threadIdx.x; i < half * D; i += kKmapBlock) s_off[i] = offsets[i];
  for (int k = threadIdx.x; k < half; k += kKmapBlock) {
    long long d = 0;
#pragma unroll
    for (int a = 0; a < D; ++a) d += (long long)offsets[k * D + a] << h->shift[a + 1];
    s_delta[k] = d;
    s_cnt[k] = 0;
  }
  __syncthreads();

  const uint32_t capacity = h->capacity, pos_shift = h->pos_shift;
  const uint32_t q = blockIdx.x * kKmapBlock + threadIdx.x;
  const bool active = q < n;
  int32_t c[W];
  if (active) {
    load_row<W>(coords, q, c);
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) c[i] = 0;
  }
  uint32_t dist[W], span[W];
  long long ckey = 0;
#pragma unroll
  for (int i = 0; i < W; ++i) {
    const int32_t mn = h->mn[i];
    dist[i] = (uint32_t)c[i] - (uint32_t)mn;
    span[i] = (uint32_t)(h->mx[i] - mn);
    ckey += (long long)((long long)c[i] - (long long)mn) << h->shift[i];
  }
  const int lane = threadIdx.x & 31;
  if (active) __stcs(nbr + (size_t)half * n + q, (int32_t)q);  // centre offset: identity
  // (Deferring the few lookups that walk past their home slot to a second loop, as the general builder does,
  // made this kernel slower: 0.153 against 0.144 ms.)
  for (int k = 0; k < half; ++k) {
    bool in_box = active;
#pragma unroll
    for (int a = 0; a < D; ++a) in_box = in_box && (dist[a + 1] + (uint32_t)s_off[k * D + a] <= span[a + 1]);
    uint32_t uid = 0xFFFFFFFFu;
    if (in_box) uid = table_find(slots, capacity, pos_shift, (unsigned long long)(ckey + s_delta[k]));
    if (active) {
      __stcs(nbr + (size_t)k * n + q, (int32_t)uid);
      if (uid != 0xFFFFFFFFu) nbr[(size_t)(K - 1 - k) * n + uid] = (int32_t)q;  // mirror entry
    }
    const uint32_t hits = __ballot_sync(0xFFFFFFFFu, uid != 0xFFFFFFFFu);
    if (lane == 0) atomicAdd(&s_cnt[k], (uint32_t)__popc(hits));
  }
  __syncthreads();
  for (int k = threadIdx.x; k < half; k += kKmapBlock)
    block_counts[(size_t)k * n_blocks + blockIdx.x] = s_cnt[k];
  if (threadIdx.x == 0) {
    const uint32_t row0 = blockIdx.x * kKmapBlock;
    block_counts[(size_t)half * n_blocks + blockIdx.x] = row0 < n ? min((uint32_t)kKmapBlock, n - row0) : 0u;
  }
}

// grid = K blocks of 1024 threads: exclusive scan of block_counts[k][0..n_blocks) in place,
// totals[k] = number of pairs of offset k.
__global__ void __launch_bounds__(1024) k_kmap_scan_blocks(uint32_t* __restrict__ block_counts,
                                                           uint32_t n_blocks,
                                                           uint32_t* __restrict__ totals) {
  __shared__ uint32_t warp_sums[32];
  uint32_t* counts = block_counts + (size_t)blockIdx.x * n_blocks;
  const uint32_t per = (n_blocks + 1023u) / 1024u;
  const uint32_t begin = min(n_blocks, threadIdx.x * per), end = min(n_blocks, begin + per);
  uint32_t sum = 0;
  for (uint32_t i = begin; i < end; ++i) sum += counts[i];
  uint32_t incl = sum;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_sums[lane], wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xFFFFFFFFu, wi, d);
      if (lane >= d) wi += t;
    }
    warp_sums[lane] = wi - w;
    if (lane == 31) totals[blockIdx.x] = wi;
  }
  __syncthreads();
  uint32_t run = warp_sums[warp] + incl - sum;
  for (uint32_t i = begin; i < end; ++i) {
    uint32_t v = counts[i];
    counts[i] = run;
    run += v;
  }
}

// one thread: offset_ptr[0..K] = exclusive scan of totals (K is small)
// mirror_half > 0 (self map): offsets K-1-k and k hold the same number of pairs, so the totals of
// the mirrored half are copied from the probed half, and *mirror_flag records the half: the pair
// lists of the mirrored offsets are then the exchanged lists of their mirror offsets (written by
// k_kmap_pairs together with the originals) and need no per-block counts.
__global__ void k_kmap_offset_ptr(uint32_t* __restrict__ totals, int K, int64_t* __restrict__ offset_ptr,
                                  int mirror_half, uint32_t* mirror_flag) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  for (int k = K - mirror_half; k < K; ++k) totals[k] = totals[K - 1 - k];
  *mirror_flag = (uint32_t)mirror_half;
  totals[K] = 0;  // "pair lists did not fit" flag of rmn_kmap_pairs (read by rmn_kmap_pairs_status)
  int64_t run = 0;
  for (int k = 0; k < K; ++k) {
    offset_ptr[k] = run;
    run += totals[k];
  }
  offset_ptr[K] = run;
}

// Block b covers query rows [b*256, b*256+256). Warp w handles offsets
// k = w, w+8, ...; for each it walks the 8 row groups of the block keeping a
// running prefix, so no block-level synchronisation is needed.
__device__ __forceinline__ void kmap_pairs_body(
    const int32_t* __restrict__ nbr, uint32_t n_query, int K,
    const int64_t* __restrict__ offset_ptr, const uint32_t* __restrict__ block_prefix,
    uint32_t n_blocks, int32_t* __restrict__ a_idx, int32_t* __restrict__ q_idx,
    unsigned long long capacity, uint32_t* __restrict__ overflow) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row0 = blockIdx.x * kKmapBlock;
  // Self map (flag word after the overflow word = K / 2): only the offsets up to the centre are walked;
  // a pair (a, q) of offset k < K / 2 is also stored, exchanged, at the same rank of offset K-1-k, whose
  // list therefore comes out sorted by table row.
  const int mirror_half = (int)overflow[1];
  const int K_full = K;
  K -= mirror_half;
  for (int k = warp; k < K; k += (int)(blockDim.x >> 5)) {
    const unsigned long long base = (unsigned long long)offset_ptr[k];
    unsigned long long pos = base + block_prefix[(size_t)k * n_blocks + blockIdx.x];
    const bool mirror = k < mirror_half;
    const unsigned long long mbase = mirror ? (unsigned long long)offset_ptr[K_full - 1 - k] : 0ull;
    // all eight row groups are loaded before the first ballot (eight independent 128-byte reads in flight)
    int32_t av[kKmapBlock / 32];
#pragma unroll
    for (int g = 0; g < kKmapBlock / 32; ++g) {
      const uint32_t q = row0 + g * 32 + lane;
      av[g] = q < n_query ? __ldcs(nbr + (size_t)k * n_query + q) : -1;
    }
#pragma unroll
    for (int g = 0; g < kKmapBlock / 32; ++g) {
      const uint32_t q = row0 + g * 32 + lane;
      const int32_t a = av[g];
      const uint32_t hits = __ballot_sync(0xFFFFFFFFu, a >= 0);
      if (a >= 0) {
        const unsigned long long p = pos + __popc(hits & ((1u << lane) - 1u));
        if (p < capacity) {
          __stcs(a_idx + p, a);
          __stcs(q_idx + p, (int32_t)q);
        } else {
          *overflow = 1;
        }
        if (mirror) {
          const unsigned long long d = mbase + (p - base);
          if (d < capacity) {
            __stcs(a_idx + d, (int32_t)q);
            __stcs(q_idx + d, a);
          } else {
            *overflow = 1;
          }
        }
      }
      pos += __popc(hits);
    }
  }
}

__global__ void __launch_bounds__(kKmapBlock) k_kmap_pairs(
    const int32_t* __restrict__ nbr, uint32_t n_query, int K, const int64_t* __restrict__ offset_ptr,
    const uint32_t* __restrict__ block_prefix, uint32_t n_blocks, int32_t* __restrict__ a_idx,
    int32_t* __restrict__ q_idx, unsigned long long capacity, uint32_t* __restrict__ overflow) {
  kmap_pairs_body(nbr, n_query, K, offset_ptr, block_prefix, n_blocks, a_idx, q_idx, capacity, overflow);
}

// The same compaction built to become resident BESIDE a convolution CTA: 128 threads of at most 32
// registers. A convolution CTA (672 threads x 80 registers, allocated in groups of four warps) leaves
// 4096 registers of an SM free, and one shared-memory / L1 split serves all CTAs of an SM, so this kernel
// is launched with the convolution's split. It runs at a fraction of the stand-alone speed (4 KB of loads
// in flight per SM) but inside the convolution's shadow.
__global__ void __maxnreg__(32) k_kmap_pairs_background(
    const int32_t* __restrict__ nbr, uint32_t n_query, int K, const int64_t* __restrict__ offset_ptr,
    const uint32_t* __restrict__ block_prefix, uint32_t n_blocks, int32_t* __restrict__ a_idx,
    int32_t* __restrict__ q_idx, unsigned long long capacity, uint32_t* __restrict__ overflow) {
  kmap_pairs_body(nbr, n_query, K, offset_ptr, block_prefix, n_blocks, a_idx, q_idx, capacity, overflow);
}

__global__ void __launch_bounds__(256) k_kmap_transpose(const int32_t* __restrict__ nbr,
                                                        uint32_t n_query, int K, uint32_t n_a,
                                                        int32_t* __restrict__ nbr_t) {
  const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= (uint64_t)K * n_query) return;
  const int32_t a = __ldg(nbr + i);
  if (a < 0 || (uint32_t)a >= n_a) return;
  const uint64_t k = i / n_query;
  const uint32_t q = (uint32_t)(i - k * n_query);
  nbr_t[k * n_a + (uint32_t)a] = (int32_t)q;
}

inline uint32_t kmap_blocks(uint32_t n_query) { return (n_query + kKmapBlock - 1) / kKmapBlock; }

}  // namespace rmn

using namespace rmn;

extern "C" int rmn_region_volume(int region_type, int D, const int32_t* kernel_size, int n_custom) {
  if (D < 1 || D >= RMN_MAX_W) return -RMN_ERR_BAD_ARG;
  if (region_type == RMN_CUSTOM) return n_custom;
  if (!kernel_size) return -RMN_ERR_BAD_ARG;
  long long v = 1;
  if (region_type == RMN_HYPER_CUBE) {
    for (int a = 0; a < D; ++a) v *= kernel_size[a];
  } else if (region_type == RMN_HYPER_CROSS) {
    for (int a = 0; a < D; ++a) v += kernel_size[a] - 1;
  } else {
    return -RMN_ERR_BAD_ARG;
  }
  return v > 0 && v < (1 << 20) ? (int)v : -RMN_ERR_BAD_ARG;
}

extern "C" int rmn_region_offsets(int region_type, int D, const int32_t* kernel_size,
                                  const int32_t* dilation, const int32_t* tensor_stride,
                                  const int32_t* custom_offsets, int n_custom, int32_t* offsets) {
  const int K = rmn_region_volume(region_type, D, kernel_size, n_custom);
  if (K < 0) return K;
  if (!dilation || !tensor_stride || !offsets) return -RMN_ERR_BAD_ARG;
  if (region_type == RMN_CUSTOM && n_custom > 0 && !custom_offsets) return -RMN_ERR_BAD_ARG;
  for (int k = 0; k < K; ++k) {
    int32_t* o = offsets + (size_t)k * D;
    for (int a = 0; a < D; ++a) o[a] = 0;
    if (region_type == RMN_HYPER_CUBE) {
      int idx = k;
      for (int a = 0; a < D; ++a) {
        const int ks = kernel_size[a];
        const int cur = idx % ks;
        const int step = dilation[a] * tensor_stride[a];
        o[a] = (ks % 2 == 0) ? cur * step : (cur - ks / 2) * step;
        idx /= ks;
      }
    } else if (region_type == RMN_HYPER_CROSS) {
      if (k == 0) continue;
      int ind = k - 1, axis = 0;
      while (axis < D && ind >= kernel_size[axis] - 1) {
        ind -= kernel_size[axis] - 1;
        ++axis;
      }
      const int r = (kernel_size[axis] - 1) / 2;
      const int co = ind < r ? ind + 1 : ind - 2 * r;
      o[axis] = co * dilation[axis] * tensor_stride[axis];
    } else {
      for (int a = 0; a < D; ++a)
        o[a] = (int32_t)((long long)custom_offsets[(size_t)k * D + a] * tensor_stride[a] *
                         dilation[a]);
    }
  }
  return K;
}

extern "C" size_t rmn_kmap_workspace_bytes(uint32_t n_query, int K) {
  if (K < 1) K = 1;
  return ((size_t)K * kmap_blocks(n_query) + (size_t)K + 64) * sizeof(uint32_t);
}

extern "C" int rmn_kmap_build(const void* d_table, const int32_t* d_query, uint32_t n_query, int W,
                              const int32_t* d_offsets, int K, int32_t* d_nbr,
                              int64_t* d_offset_ptr, void* d_workspace, size_t workspace_bytes,
                              void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_table || W < 2 || W > RMN_MAX_W || K < 1 || K > 4096 || !d_offsets || !d_offset_ptr ||
      !d_workspace)
    return RMN_ERR_BAD_ARG;
  if (workspace_bytes < rmn_kmap_workspace_bytes(n_query, K)) return RMN_ERR_ALLOC;
  const uint32_t nb = kmap_blocks(n_query);
  uint32_t* block_counts = reinterpret_cast<uint32_t*>(d_workspace);
  uint32_t* totals = block_counts + (size_t)K * nb;
  if (n_query == 0) {
    RMN_CUDA_TRY(cudaMemsetAsync(d_offset_ptr, 0, sizeof(int64_t) * (K + 1), stream));
    return RMN_OK;
  }
  if (!d_query || !d_nbr || !coords_aligned(d_query, W)) return RMN_ERR_BAD_ARG;
  auto* h = reinterpret_cast<const TableHeader*>(d_table);
  auto* slots =
      reinterpret_cast<const Slot*>(reinterpret_cast<const char*>(d_table) + sizeof(TableHeader));
  const size_t smem = (size_t)K * 8 + (size_t)K * (W - 1) * 4 + (size_t)K * 4;
  RMN_DISPATCH_W(W, k_kmap_probe<kW><<<nb, kKmapBlock, smem, stream>>>(
                        h, slots, d_query, n_query, d_offsets, K, d_nbr, block_counts, nb));
  RMN_LAUNCH_CHECK();
  k_kmap_scan_blocks<<<K, 1024, 0, stream>>>(block_counts, nb, totals);
  RMN_LAUNCH_CHECK();
  k_kmap_offset_ptr<<<1, 32, 0, stream>>>(totals, K, d_offset_ptr, 0, totals + K + 1);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_kmap_build_self(const void* d_table, const int32_t* d_coords, uint32_t n_rows, int W,
                                   const int32_t* d_offsets, int K, int32_t* d_nbr, int64_t* d_offset_ptr,
                                   void* d_workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_table || W < 2 || W > RMN_MAX_W || K < 1 || K > 4096 || (K & 1) == 0 || !d_offsets || !d_offset_ptr ||
      !d_workspace)
    return RMN_ERR_BAD_ARG;
  if (workspace_bytes < rmn_kmap_workspace_bytes(n_rows, K)) return RMN_ERR_ALLOC;
  const uint32_t nb = kmap_blocks(n_rows);
  uint32_t* block_counts = reinterpret_cast<uint32_t*>(d_workspace);
  uint32_t* totals = block_counts + (size_t)K * nb;
  if (n_rows == 0) {
    RMN_CUDA_TRY(cudaMemsetAsync(d_offset_ptr, 0, sizeof(int64_t) * (K + 1), stream));
    return RMN_OK;
  }
  if (!d_coords || !d_nbr || !coords_aligned(d_coords, W)) return RMN_ERR_BAD_ARG;
  auto* h = reinterpret_cast<const TableHeader*>(d_table);
  auto* slots =
      reinterpret_cast<const Slot*>(reinterpret_cast<const char*>(d_table) + sizeof(TableHeader));
  const int half = K / 2;
  if (half > 0)  // the mirrored half starts as "no neighbour"
    RMN_CUDA_TRY(cudaMemsetAsync(d_nbr + (size_t)(half + 1) * n_rows, 0xFF, (size_t)half * n_rows * sizeof(int32_t),
                                 stream));
  const int hs = half > 0 ? half : 1;
  const size_t smem = (size_t)hs * 8 + (size_t)hs * (W - 1) * 4 + (size_t)hs * 4;
  RMN_DISPATCH_W(W, k_kmap_probe_self<kW><<<nb, kKmapBlock, smem, stream>>>(
                        h, slots, d_coords, n_rows, d_offsets, K, d_nbr, block_counts, nb));
  RMN_LAUNCH_CHECK();
  // only the probed half (and the centre) is scanned here; see k_kmap_offset_ptr
  k_kmap_scan_blocks<<<half + 1, 1024, 0, stream>>>(block_counts, nb, totals);
  RMN_LAUNCH_CHECK();
  k_kmap_offset_ptr<<<1, 32, 0, stream>>>(totals, K, d_offset_ptr, half, totals + K + 1);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

static int kmap_pairs_launch(const int32_t* d_nbr, uint32_t n_query, int K, const int64_t* d_offset_ptr,
                             const void* d_workspace, int32_t* d_a_idx, int32_t* d_q_idx, uint64_t capacity,
                             cudaStream_t stream, bool background) {
  if (K < 1 || !d_offset_ptr || !d_workspace) return RMN_ERR_BAD_ARG;
  if (n_query == 0 || capacity == 0) return RMN_OK;
  if (!d_nbr || !d_a_idx || !d_q_idx) return RMN_ERR_BAD_ARG;
  const uint32_t nb = kmap_blocks(n_query);
  const uint32_t* block_prefix = reinterpret_cast<const uint32_t*>(d_workspace);
  // the word after the totals flags a capacity overflow (zeroed by the build, read by rmn_kmap_pairs_status)
  uint32_t* overflow = const_cast<uint32_t*>(block_prefix) + (size_t)K * nb + K;
  if (!background) {
    k_kmap_pairs<<<nb, kKmapBlock, 0, stream>>>(d_nbr, n_query, K, d_offset_ptr, block_prefix, nb, d_a_idx,
                                                d_q_idx, capacity, overflow);
  } else {
    static std::once_flag once[64];
    int dev = 0;
    RMN_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64)
      std::call_once(once[dev], [] {
        cudaFuncSetAttribute(k_kmap_pairs_background, cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
      });
    k_kmap_pairs_background<<<nb, 128, 0, stream>>>(d_nbr, n_query, K, d_offset_ptr, block_prefix, nb, d_a_idx,
                                                    d_q_idx, capacity, overflow);
  }
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_kmap_pairs_status(const void* d_workspace, uint32_t n_query, int K, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (K < 1 || !d_workspace) return RMN_ERR_BAD_ARG;
  if (n_query == 0) return RMN_OK;
  const uint32_t* flag = reinterpret_cast<const uint32_t*>(d_workspace) + (size_t)K * kmap_blocks(n_query) + K;
  uint32_t v = 0;
  RMN_CUDA_TRY(cudaMemcpyAsync(&v, flag, sizeof(v), cudaMemcpyDeviceToHost, stream));
  RMN_CUDA_TRY(cudaStreamSynchronize(stream));
  return v ? RMN_ERR_ALLOC : RMN_OK;
}

extern "C" int rmn_kmap_pairs(const int32_t* d_nbr, uint32_t n_query, int K,
                              const int64_t* d_offset_ptr, const void* d_workspace,
                              int32_t* d_a_idx, int32_t* d_q_idx, uint64_t capacity,
                              void* stream_) {
  return kmap_pairs_launch(d_nbr, n_query, K, d_offset_ptr, d_workspace, d_a_idx, d_q_idx, capacity,
                           (cudaStream_t)stream_, false);
}

extern "C" int rmn_kmap_pairs_background(const int32_t* d_nbr, uint32_t n_query, int K,
                                         const int64_t* d_offset_ptr, const void* d_workspace,
                                         int32_t* d_a_idx, int32_t* d_q_idx, uint64_t capacity,
                                         void* stream_) {
  return kmap_pairs_launch(d_nbr, n_query, K, d_offset_ptr, d_workspace, d_a_idx, d_q_idx, capacity,
                           (cudaStream_t)stream_, true);
}

extern "C" int rmn_kmap_transpose(const int32_t* d_nbr, uint32_t n_query, int K, uint32_t n_a,
                                  int32_t* d_nbr_t, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (K < 1) return RMN_ERR_BAD_ARG;
  if (n_a == 0) return RMN_OK;
  if (!d_nbr_t) return RMN_ERR_BAD_ARG;
  RMN_CUDA_TRY(cudaMemsetAsync(d_nbr_t, 0xFF, (size_t)K * n_a * sizeof(int32_t), stream));
  if (n_query == 0) return RMN_OK;
  if (!d_nbr) return RMN_ERR_BAD_ARG;
  const uint64_t total = (uint64_t)K * n_query;
  k_kmap_transpose<<<(uint32_t)((total + 255) / 256), 256, 0, stream>>>(d_nbr, n_query, K, n_a,
                                                                       d_nbr_t);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}
