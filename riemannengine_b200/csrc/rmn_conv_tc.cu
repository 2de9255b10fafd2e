// Tensor-core sparse convolution for sm_100a: gathered feature tiles in shared
// memory feed tcgen05.mma (bf16 x bf16 -> fp32 in TMEM); the output tile is
// stationary across all kernel offsets, so the scatter-accumulate of the
// reference (index_add_, engine/nn/conv.cpp:62-63) becomes one store per row.
//
//   forward         out[j] = sum_k F[nbr[k][j]]    . W[k]      B = W[k]   read MN-major
//   backward input  dF[i]  = sum_k dY[nbr_t[k][i]] . W[k]^T    B = W[k]   read K-major
//
// One persistent CTA per SM loops over super-tiles of T x 128 destination rows
// (T = 4 for up to 64 output channels, 2 up to 128) so that one copy of W[k] in shared memory serves
// T row tiles. Warp roles (4T producer warps + 1 + 4):
//   first 4T    producers: for every offset k (and 64-channel block of the
//               reduction) gather the source rows named by nbr[k][super-tile]
//               (16-byte cp.async, zero-fill for -1) and copy the W[k] slice
//               into a ring of shared-memory stages;
//   warp  8     issues tcgen05.mma for each stage (one lane), commits the stage
//               back to the producers and the finished accumulators to the
//               epilogue;
//   warps 9-12  epilogue: tcgen05.ld the fp32 accumulators (double-buffered in
//               TMEM, so it overlaps the next super-tile's MMAs), convert to
//               bf16, store.
//
// Shared-memory operand images are the swizzled canonical layouts: a line of
// 128 bytes (64 bf16; 64 bytes when only 32 channels) per matrix row, 16-byte
// chunk c of row r stored at chunk position c ^ (r % 8) (64-byte lines:
// c ^ ((r / 2) % 4)). Eight consecutive lanes copy the eight chunks of ONE
// source row: the global read is a whole 128-byte line and the shared-memory
// write is conflict-free.
//
// Every mbarrier wait is bounded: after ~2 s without progress a role records
// RMN_ERR_TIMEOUT in a device status word and leaves; all roles then meet at
// the final barrier and the TMEM allocation is released.
#include "rmn_common.cuh"
#include "rmn_plan.cuh"
#include "rmn_tc.cuh"

#include <cuda_bf16.h>

#include <atomic>
#include <mutex>

namespace rmn {

// Launches of the tcgen05 kernels of this file (forward, input gradient, weight gradient) in this process:
// lets a host or a test tell that a convolution ran on the tensor cores rather than on the SIMT kernels.
static std::atomic<unsigned long long> g_tc_launches{0};
unsigned long long tc_launch_count() { return g_tc_launches.load(std::memory_order_relaxed); }
static inline void count_tc_launch() { g_tc_launches.fetch_add(1, std::memory_order_relaxed); }

// Sticky status word of the tensor-core kernels, one per device (not per stream): a kernel whose
// bounded wait ran out stores RMN_ERR_TIMEOUT here and returns early. Hosts read it (and clear it)
// through rmn_device_status, and rmn_table_info reports it at the read-back every table build makes.
__device__ uint32_t g_tc_status = 0;

namespace tc {

constexpr int kTileM = 128;

// chunk position of 16-byte chunk c in row r of a swizzled image with SW-byte lines
template <int SW>
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) {
  if constexpr (SW == 128) return c ^ (r & 7u);
  else return c ^ ((r >> 1) & 3u);
}

template <int CR, int CC>
struct Cfg {
  static constexpr int KB = CR < 64 ? CR : 64;  // reduction channels per pipeline stage
  static constexpr int NKB = CR / KB;
  // row tiles sharing one W[k] stage: as many as the 512 TMEM columns allow with two accumulator sets
  static constexpr int T = CC <= 64 ? 4 : (CC <= 128 ? 2 : 1);
  static constexpr int PRODUCER_WARPS = T < 2 ? 8 : 4 * T;  // one warp per 32 gathered rows (>= 8 for the weights)
  static constexpr int PRODUCERS = PRODUCER_WARPS * 32;
  static constexpr int THREADS = PRODUCERS + 32 + 128;
  static constexpr int SWA = KB * 2;            // bytes per A line
  static constexpr uint32_t A_TILE = kTileM * SWA;
  static constexpr uint32_t A_BYTES = T * A_TILE;
  static constexpr uint32_t B_BYTES = KB * CC * 2;
  static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = STAGE * 5 <= 216 * 1024 ? 5 : (STAGE * 4 <= 216 * 1024 ? 4 : 3);
  static constexpr uint32_t BAR_OFFSET = STAGES * STAGE;
  static constexpr uint32_t EP_OFFSET = BAR_OFFSET + 256;  // 2 * 256 floats of epilogue scale / shift
  static constexpr uint32_t STATS_BYTES = 4 * 2 * CC * 4;  // per-warp channel statistics of the kStats epilogue
  static constexpr uint32_t SMEM = EP_OFFSET + 2 * 256 * 4 + STATS_BYTES;
  static constexpr uint32_t TMEM_COLS = pow2_at_least(2 * T * CC);
};

// Sum over the 32 lanes of v[c] for c = 0..31, delivered to lane c (a transposing butterfly:
// 31 shuffles instead of 32 five-step reductions). v is destroyed.
__device__ __forceinline__ float warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    const bool upper = (lane & d) != 0;
#pragma unroll
    for (int i = 0; i < d; ++i) {
      const float keep = upper ? v[i + d] : v[i];
      const float send = upper ? v[i] : v[i + d];
      v[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, d);
    }
  }
  return v[0];
}

// CR: reduction channels per offset; CC: output channels; kWT: weights are read transposed
// (backward input). Weight tensor is [K][CIN_w][COUT_w] with (CIN_w, COUT_w) = kWT ? (CC, CR) : (CR, CC).
// kStats: the epilogue also accumulates, per output channel, the sum and the sum of squares of the
// values it stores (the batch statistics of a following batch normalisation) and writes them to
// stats_partial[blockIdx.x][2][CC]; a second kernel adds the per-CTA partials in a fixed order.
//
// kPlan: the rows are processed in the internal order of a convolution plan (rmn_plan.cu): `nbr` is the
// plan's permuted table [K][n_dst] (n_dst = the padded position count), `perm` maps a position to the
// output row it is stored to (-1: padding) and `tile_mask` holds, per 128-row tile, the offsets at which
// any row of the tile has a neighbour. An offset at which none of the T tiles of a super-tile has a
// neighbour takes no pipeline stage: no gather, no zero fill, no copy of W[k], no MMA.
template <int CR, int CC, bool kWT, bool kStats = false, bool kPlan = false>
__global__ void __launch_bounds__(Cfg<CR, CC>::THREADS, 1) k_conv_tc(const __nv_bfloat16* __restrict__ src,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const int32_t* __restrict__ nbr,
                                                            uint32_t n_dst, int K,
                                                            __nv_bfloat16* __restrict__ out,
                                                            uint32_t n_super,
                                                            const float* __restrict__ ep_scale,
                                                            const float* __restrict__ ep_shift, int ep_relu,
                                                            float* __restrict__ stats_partial = nullptr,
                                                            const int32_t* __restrict__ perm = nullptr,
                                                            const uint32_t* __restrict__ tile_mask = nullptr) {
  using C = Cfg<CR, CC>;
  constexpr int STAGES = C::STAGES, KB = C::KB, NKB = C::NKB, T = C::T, SWA = C::SWA;
  constexpr int kFwdProducerWarps = C::PRODUCER_WARPS, kFwdProducers = C::PRODUCERS;
  constexpr int CIN_W = kWT ? CC : CR, COUT_W = kWT ? CR : CC;
  // Weight image of one stage: lines of SWB bytes.
  //   forward (MN-major): one line per reduction row ci (KB lines) and 64-column atom;
  //   backward input (K-major): one line per output row ci (CC lines) holding the KB reduction channels.
  constexpr int SWB = kWT ? KB * 2 : (CC < 64 ? CC : 64) * 2;
  constexpr int B_LINES = kWT ? CC : KB;
  constexpr int B_ATOMS = kWT ? 1 : (CC * 2) / SWB;
  constexpr int B_CPL = SWB / 16;                   // chunks per line
  constexpr uint32_t B_ATOM_BYTES = B_LINES * SWB;  // forward: distance between 64-column atoms
  constexpr int A_CPL = SWA / 16;
  constexpr uint32_t LT_A = SWA == 128 ? 2u : 4u, LT_B = SWB == 128 ? 2u : 4u;
  static_assert(CR % 32 == 0 && CC % 32 == 0 && CC <= 256 && CR % KB == 0, "channel counts");

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  // fused epilogue out = act(acc * scale + shift): per-channel scale | shift, staged once per CTA
  float* s_ep = reinterpret_cast<float*>(smem + C::EP_OFFSET);
  const bool has_ep = ep_scale != nullptr || ep_shift != nullptr || ep_relu != 0;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (has_ep && tid < CC) {
    s_ep[tid] = ep_scale ? __ldg(ep_scale + tid) : 1.f;
    s_ep[CC + tid] = ep_shift ? __ldg(ep_shift + tid) : 0.f;
  }

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], kFwdProducers);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == kFwdProducerWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t smem_base = smem_u32(smem);
  bool timed_out = false;

  if (warp < kFwdProducerWarps) {
    // ------------------------------ producers ------------------------------------------
    // warp w owns rows [32w, 32w + 32) of the (T * 128)-row super-tile; warps beyond T * 4 only copy weights
    const bool has_rows = warp < T * 4;
    const uint32_t a_tile_off = (uint32_t)(warp >> 2) * C::A_TILE;
    const uint32_t row_in_tile0 = (uint32_t)(warp & 3) * 32;
    constexpr int ROWS_PER_INSTR = 32 / A_CPL;
    const uint32_t a_chunk = lane % A_CPL, a_row_sub = lane / A_CPL;
    uint32_t it = 0;

    // kPlan: OR of the tile masks of a super-tile (the offsets at which some row has a neighbour; a plan covers
    // at most 32 offsets), requested one super-tile ahead
    uint32_t pf_mask = 0;
    auto load_mask = [&](uint32_t st_next) {
      pf_mask = 0;
      if (st_next < n_super) {
#pragma unroll
        for (int t = 0; t < T; ++t) pf_mask |= __ldg(tile_mask + (size_t)st_next * T + t);
      }
    };
    if constexpr (kPlan) load_mask(blockIdx.x);
    for (uint32_t st = blockIdx.x; st < n_super && !timed_out; st += gridDim.x) {
      const uint32_t row = st * (kTileM * T) + warp * 32 + lane;
      const bool row_ok = has_rows && row < n_dst;
      // kPlan: the offsets of this super-tile that still have to run; only offsets at which some row has a
      // neighbour take a stage. Everything the per-stage path needs stays in registers: a producer's stage
      // must not wait for a round trip through the load/store pipe (a shared-memory list of the offsets, or
      // a spilled register, costs a quarter of a stage: the pipe's queue is full of the gathers).
      uint32_t todo = 0;
      if constexpr (kPlan) {
        todo = pf_mask;
        load_mask(st + gridDim.x);
      }
      // Neighbour indices are fetched four stages ahead of their use (an L2 round trip is about
      // one stage long). The window rotates through named registers: no dynamic indexing.
      auto load_idx = [&](int kk) -> int32_t {
        return (row_ok && kk < K) ? __ldg(nbr + (size_t)kk * n_dst + row) : -1;
      };
      // One offset of the super-tile: fill the next ring stage(s) with the rows `idx` names and W[k].
      auto do_offset = [&](int k, const int32_t idx) {
        const __nv_bfloat16* wk = w + (size_t)k * CIN_W * COUT_W;
#pragma unroll 1
        for (int kb = 0; kb < NKB; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) { timed_out = true; break; }
          const uint32_t a_s = smem_base + s * C::STAGE, b_s = a_s + C::A_BYTES;

          if (has_rows) {
            // A: a quarter-warp copies the whole line of one gathered row
#pragma unroll
            for (int g = 0; g < 32 / ROWS_PER_INSTR; ++g) {
              const uint32_t r_local = g * ROWS_PER_INSTR + a_row_sub;
              const int32_t sidx = __shfl_sync(0xFFFFFFFFu, idx, r_local);
              const uint32_t r = row_in_tile0 + r_local;
              cp_async16(a_s + a_tile_off + r * SWA + (swz<SWA>(r, a_chunk) << 4),
                         src + (size_t)(sidx < 0 ? 0 : sidx) * CR + kb * KB + a_chunk * 8, sidx < 0 ? 0u : 16u);
            }
          } else {
            __syncwarp();
          }

          // B: this stage's slice of W[k], one line (and atom) per B_CPL consecutive threads
#pragma unroll
          for (int q = tid; q < B_LINES * B_ATOMS * B_CPL; q += kFwdProducers) {
            const uint32_t c = q % B_CPL, unit = q / B_CPL;
            const uint32_t line = unit % B_LINES, atom = unit / B_LINES;
            const __nv_bfloat16* g = kWT ? wk + (size_t)line * COUT_W + kb * KB + c * 8
                                         : wk + (size_t)(kb * KB + line) * COUT_W + atom * (SWB / 2) + c * 8;
            cp_async16(b_s + atom * B_ATOM_BYTES + line * SWB + (swz<SWB>(line, c) << 4), g, 16u);
          }
          // The stage's "full" barrier fires by itself once this thread's copies have landed
          // (cp.async.mbarrier.arrive.noinc), so producers never wait for data: they run ahead
          // until the ring is full and every stage of shared memory can be in flight.
          cp_async_arrive_noinc(&full[s]);
        }
      };
      // The four-deep window is unrolled by hand, each slot a register of its own that is reloaded right
      // after it is read: a rotating window (w0 = w1; w1 = w2; ...) would copy registers whose loads
      // are still in flight, and a copy waits for its source like any other use.
      if constexpr (!kPlan) {
        // The four-deep window is unrolled by hand, each slot a register of its own that is reloaded right
        // after it is read: a rotating window (w0 = w1; w1 = w2; ...) would copy registers whose loads
        // are still in flight, and a copy waits for its source like any other use.
        int32_t idx_w0 = load_idx(0), idx_w1 = load_idx(1), idx_w2 = load_idx(2), idx_w3 = load_idx(3);
        for (int k = 0; k < K && !timed_out; k += 4) {
          {
            const int32_t idx = idx_w0;
            idx_w0 = load_idx(k + 4);
            do_offset(k, idx);
          }
          if (k + 1 < K && !timed_out) {
            const int32_t idx = idx_w1;
            idx_w1 = load_idx(k + 5);
            do_offset(k + 1, idx);
          }
          if (k + 2 < K && !timed_out) {
            const int32_t idx = idx_w2;
            idx_w2 = load_idx(k + 6);
            do_offset(k + 2, idx);
          }
          if (k + 3 < K && !timed_out) {
            const int32_t idx = idx_w3;
            idx_w3 = load_idx(k + 7);
            do_offset(k + 3, idx);
          }
        }
      } else {
        // Planned: a two-deep window over the set bits of `todo` in ascending order (two registers fewer than
        // the plain window, which pays for the mask: the CTA is at its register limit). The offset to
        // prefetch is the third lowest bit still set.
        auto bit_at = [&](uint32_t m) -> int { return m ? __ffs(m) - 1 : K; };
        int32_t idx_w0 = load_idx(bit_at(todo)), idx_w1 = load_idx(bit_at(todo & (todo - 1u)));
        while (todo && !timed_out) {
          {
            const int k = __ffs(todo) - 1;
            todo &= todo - 1u;
            const int32_t idx = idx_w0;
            idx_w0 = load_idx(bit_at(todo & (todo - 1u)));
            do_offset(k, idx);
          }
          if (!todo || timed_out) break;
          {
            const int k = __ffs(todo) - 1;
            todo &= todo - 1u;
            const int32_t idx = idx_w1;
            idx_w1 = load_idx(bit_at(todo & (todo - 1u)));
            do_offset(k, idx);
          }
        }
      }
    }
    cp_async_wait<0>();  // nothing may still be writing shared memory when the CTA exits
  } else if (warp == kFwdProducerWarps) {
    // ------------------------------ MMA issuer -----------------------------------------
    constexpr uint32_t IDESC = instr_desc(kTileM, CC, !kWT);
    // descriptors with a zero start address
    constexpr uint64_t A_DESC0 = smem_desc_sw_const(16, 8 * SWA, LT_A);
    constexpr uint64_t B_DESC0 = kWT ? smem_desc_sw_const(16, 8 * SWB, LT_B) : smem_desc_sw_const(B_ATOM_BYTES, 8 * SWB, LT_B);
    constexpr uint32_t A_DESC_HI = (uint32_t)(A_DESC0 >> 32), B_DESC_HI = (uint32_t)(B_DESC0 >> 32);
    uint32_t it = 0, tile_iter = 0;
    for (uint32_t st = blockIdx.x; st < n_super && !timed_out; st += gridDim.x, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u)) { timed_out = true; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * (T * CC);
      // kPlan: this warp only needs the NUMBER of stages of the super-tile (the offsets at which some row has
      // a neighbour; which ones they are only matters to the producers). The count goes through a warp vote:
      // a vote's result is warp-uniform by construction, so the loop below stays on the uniform datapath with
      // its descriptors in uniform registers, like the fixed-count loop of the plain kernel. (Per-tile
      // predicates on the MMAs were tried: derived from loaded data they are per-thread values, every MMA then
      // moves its operands across, and the issue thread becomes the limit at 3x the plain kernel's cost.)
      uint32_t n_stage = (uint32_t)K * NKB;
      if constexpr (kPlan) {
        uint32_t m = 0;
#pragma unroll
        for (int t = 0; t < T; ++t) m |= __ldg(tile_mask + (size_t)st * T + t);
        const uint32_t cnt = (uint32_t)__popc(__ballot_sync(0xFFFFFFFFu, (m >> lane) & 1u));
        n_stage = cnt * NKB;
      }
      for (uint32_t sg = 0; sg < n_stage; ++sg, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        if (!mbar_wait(&full[s], ph)) { timed_out = true; break; }
        // the copies were generic-proxy writes; the tensor core reads through the async proxy
        fence_proxy_async();
        tc_fence_after();
        {
          // Warp-uniform code, one elected lane issues. Descriptors differ from stage to stage (and
          // from MMA to MMA) only in the 14-bit start address field: everything else is folded
          // into constants, one add per operand.
          const uint32_t a_s = smem_base + s * C::STAGE;
          const uint32_t a_lo = (a_s >> 4) + (uint32_t)(A_DESC0 & 0xFFFFFFFFu);
          const uint32_t b_lo = ((a_s + C::A_BYTES) >> 4) + (uint32_t)(B_DESC0 & 0xFFFFFFFFu);
          static_for<T * (KB / 16)>([&](auto tj) {
            constexpr int t = decltype(tj)::value / (KB / 16), j = decltype(tj)::value % (KB / 16);
            {
              // A, K-major swizzled: 8-row groups 8 * SWA apart (SBO); a K step of 16 channels is 32 bytes.
              // B forward, MN-major: 8-row K groups 8 * SWB apart (SBO), 64-column atoms B_ATOM_BYTES apart
              // (LBO), a K step is 16 lines; B backward input, K-major: a K step is 32 bytes.
              const uint64_t a_desc = ((uint64_t)A_DESC_HI << 32) | (a_lo + (uint32_t)((t * C::A_TILE + j * 32) >> 4));
              const uint64_t b_desc = ((uint64_t)B_DESC_HI << 32) | (b_lo + (uint32_t)((kWT ? j * 32 : j * 16 * SWB) >> 4));
              const uint32_t accumulate = (sg | (uint32_t)j) != 0 ? 1u : 0u;
              // Row tile 0 reads the K slice j of W[k] from shared memory into collector buffer j;
              // the other row tiles of the stage reuse it (shared-memory bandwidth, which the
              // gathers and the operand fetches compete for, bounds this kernel).
              if constexpr (T > 1 && (CC == 64 || CC == 128) && KB / 16 <= 4)  // .ws takes N = 64, 128, 256
                tc_mma_bf16_ws_elect<j, t == 0 ? 0 : (t == T - 1 ? 2 : 1)>(d_tmem + t * CC, a_desc, b_desc, IDESC, accumulate);
              else
                tc_mma_bf16_elect(d_tmem + t * CC, a_desc, b_desc, IDESC, accumulate);
            }
          });
          tc_commit_elect(&empty[s]);
        }
      }
      if (timed_out) break;
      tc_commit_elect(&tmem_full[acc]);
    }
  } else {
    // ------------------------------ epilogue -------------------------------------------
    const uint32_t quad = warp & 3;  // TMEM lanes [32*quad, 32*quad + 32)
    uint32_t tile_iter = 0;
    // kStats: lane l of this warp accumulates channel c0 + l of every 32-channel chunk
    float st_sum[kStats ? CC / 32 : 1], st_sq[kStats ? CC / 32 : 1];
#pragma unroll
    for (int i = 0; i < (kStats ? CC / 32 : 1); ++i) st_sum[i] = st_sq[i] = 0.f;
    for (uint32_t st = blockIdx.x; st < n_super && !timed_out; st += gridDim.x, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_ph)) { timed_out = true; break; }
      tc_fence_after();
#pragma unroll
      for (int t = 0; t < T; ++t) {
        uint32_t row = st * (kTileM * T) + t * kTileM + quad * 32 + lane;
        bool tile_any = true;  // false: no MMA wrote this tile's accumulator (no neighbour at any offset)
        if constexpr (kPlan) {
          const int32_t orow = __ldg(perm + row);
          row = orow < 0 ? 0xFFFFFFFFu : (uint32_t)orow;   // padding positions store nothing
          // the accumulators of a super-tile were written iff one of its tiles has a neighbour at some offset
          uint32_t m = 0;
#pragma unroll
          for (int tt = 0; tt < T; ++tt) m |= __ldg(tile_mask + (size_t)st * T + tt);
          tile_any = __any_sync(0xFFFFFFFFu, m != 0);  // (warp-uniform: the TMEM load below is warp-collective)
        }
#pragma unroll
        for (int c0 = 0; c0 < CC; c0 += 32) {
          uint32_t r[32];
          if (tile_any) {
            tc_ld32(tmem_base + ((quad * 32u) << 16) + acc * (T * CC) + t * CC + c0, r);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int v = 0; v < 32; ++v) r[v] = 0u;
          }
          if (has_ep) {
#pragma unroll
            for (int v = 0; v < 32; ++v) {
              float f = fmaf(__uint_as_float(r[v]), s_ep[c0 + v], s_ep[CC + c0 + v]);
              if (ep_relu) f = fmaxf(f, 0.f);
              r[v] = __float_as_uint(f);
            }
          }
          if (row < n_dst) {
            uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * CC + c0);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              o.x = *reinterpret_cast<uint32_t*>(&p0);
              o.y = *reinterpret_cast<uint32_t*>(&p1);
              o.z = *reinterpret_cast<uint32_t*>(&p2);
              o.w = *reinterpret_cast<uint32_t*>(&p3);
              dst[v] = o;
            }
          }
          if constexpr (kStats) {
            // statistics of the values as stored (rounded to bf16); rows past the end count as zero
            float val[32], sq[32];
#pragma unroll
            for (int v = 0; v < 32; ++v) {
              const float f = row < n_dst ? __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[v]))) : 0.f;
              val[v] = f;
              sq[v] = f * f;
            }
            st_sq[c0 / 32] += warp_column_sums(sq, lane);
            st_sum[c0 / 32] += warp_column_sums(val, lane);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
    }
    if constexpr (kStats) {
      // the four epilogue warps add their partials in warp order through shared memory
      float* s_st = s_ep + 2 * 256;  // [4 warps][2][CC]
#pragma unroll
      for (int i = 0; i < CC / 32; ++i) {
        s_st[(quad * 2 + 0) * CC + i * 32 + lane] = st_sum[i];
        s_st[(quad * 2 + 1) * CC + i * 32 + lane] = st_sq[i];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
      for (int c = (int)(quad * 32) + lane; c < 2 * CC; c += 128) {
        float t = 0.f;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) t += s_st[q4 * 2 * CC + c];
        stats_partial[(size_t)blockIdx.x * 2 * CC + c] = t;
      }
    }
  }

  if (timed_out) atomicExch(&g_tc_status, (uint32_t)RMN_ERR_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == kFwdProducerWarps) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS)
                 : "memory");
  }
}

// stats_partial != nullptr selects the kStats instantiation (forward only); *grid_out receives the
// number of CTAs, i.e. of [2][CC] partials written.
// plan != nullptr: run in the internal order of that convolution plan (built for n_dst rows, K offsets).
template <int CR, int CC, bool kWT, bool kStats = false, bool kPlan = false>
int launch(const void* src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, void* out,
           const float* ep_scale, const float* ep_shift, int ep_relu, cudaStream_t stream,
           float* stats_partial = nullptr, uint32_t* grid_out = nullptr, const void* plan = nullptr) {
  using C = Cfg<CR, CC>;
  auto kern = k_conv_tc<CR, CC, kWT, kStats, kPlan>;
  const int32_t* perm = nullptr;
  const uint32_t* tile_mask = nullptr;
  if constexpr (kPlan) {
    const PlanLayout L = plan_layout(n_dst, K);
    const char* base = static_cast<const char*>(plan);
    perm = reinterpret_cast<const int32_t*>(base + L.perm);
    tile_mask = reinterpret_cast<const uint32_t*>(base + L.tile_mask);
    nbr = reinterpret_cast<const int32_t*>(base + L.nbr_p);
    n_dst = L.n_pos;  // positions, a multiple of every super-tile size
  }
  // once per device and instantiation, safe when several host threads make the first call together
  static std::once_flag configured[64];
  int dev = 0;
  RMN_CUDA_TRY(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  if (dev >= 0 && dev < 64)
    std::call_once(configured[dev], [&] {
      attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    });
  else
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
  RMN_CUDA_TRY(attr_err);
  int sms = 148;
  RMN_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const uint32_t rows_per_super = kTileM * C::T;
  const uint32_t n_super = (n_dst + rows_per_super - 1) / rows_per_super;
  // one CTA per SM unless two fit (shared memory and TMEM columns)
  const uint32_t per_sm = (C::SMEM <= 110 * 1024 && C::TMEM_COLS <= 256) ? 2u : 1u;
  uint32_t grid = (uint32_t)sms * per_sm;
  if (grid > n_super) grid = n_super;
  kern<<<grid, C::THREADS, C::SMEM, stream>>>((const __nv_bfloat16*)src, (const __nv_bfloat16*)w, nbr, n_dst, K,
                                               (__nv_bfloat16*)out, n_super, ep_scale, ep_shift, ep_relu,
                                               stats_partial, perm, tile_mask);
  RMN_LAUNCH_CHECK();
  count_tc_launch();
  if (grid_out) *grid_out = grid;
  return RMN_OK;
}

}  // namespace tc

}  // namespace rmn

#include "rmn_conv_tc_tma.cuh"
#include "rmn_conv_tc_wgrad.cuh"

#include <cstdlib>

namespace rmn {

// RMN_B200_CONV_TMA=1 selects the TMA gather4 producers. They are correct but, measured on the
// 1.2 M-voxel 64 -> 64 workload, 2.4x slower than the cp.async producers (1.13 ms vs 0.47 ms):
// the TMA engine retires one four-row gather (512 B) every ~38 cycles per SM, well below what the
// load/store unit sustains for the same rows. Read on every call so that tests can toggle it.
static bool use_tma() {
  const char* e = std::getenv("RMN_B200_CONV_TMA");
  return e && e[0] == '1';
}

template <int CR, int CC, bool kWT>
static int launch_best(const void* src, uint32_t n_src, const void* w, const int32_t* nbr, uint32_t n_dst, int K,
                       void* out, const float* ep_scale, const float* ep_shift, int ep_relu, cudaStream_t stream,
                       const void* plan) {
  if (plan)
    return tc::launch<CR, CC, kWT, false, true>(src, w, nbr, n_dst, K, out, ep_scale, ep_shift, ep_relu, stream,
                                                nullptr, nullptr, plan);
  if (use_tma() && !ep_scale && !ep_shift && !ep_relu) {
    const int st = tc::launch_tma<CR, CC, kWT>(src, n_src, w, nbr, n_dst, K, out, stream);
    if (st != RMN_ERR_UNSUPPORTED) return st;
  }
  return tc::launch<CR, CC, kWT>(src, w, nbr, n_dst, K, out, ep_scale, ep_shift, ep_relu, stream);
}

// Returns RMN_ERR_UNSUPPORTED when no tensor-core instantiation covers the shape.
// plan: a convolution plan built for (nbr, n_dst, K), or nullptr (K above the plan limit is run unplanned).
int tc_conv(const void* src, uint32_t n_src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, int c_red,
            int c_col, bool transposed_weights, void* out, const float* ep_scale, const float* ep_shift, int ep_relu,
            cudaStream_t stream, const void* plan) {
  if (K > kPlanMaxK) plan = nullptr;
#define RMN_TC_CASE(R, Cc)                                                                            \
  if (c_red == R && c_col == Cc)                                                                      \
    return transposed_weights                                                                         \
               ? launch_best<R, Cc, true>(src, n_src, w, nbr, n_dst, K, out, ep_scale, ep_shift, ep_relu, stream, plan)  \
               : launch_best<R, Cc, false>(src, n_src, w, nbr, n_dst, K, out, ep_scale, ep_shift, ep_relu, stream, plan);
  RMN_TC_CASE(32, 32)
  RMN_TC_CASE(32, 64)
  RMN_TC_CASE(64, 32)
  RMN_TC_CASE(64, 64)
  RMN_TC_CASE(64, 128)
  RMN_TC_CASE(128, 64)
  RMN_TC_CASE(128, 128)
  RMN_TC_CASE(128, 256)
  RMN_TC_CASE(256, 128)
  RMN_TC_CASE(256, 256)
#undef RMN_TC_CASE
  return RMN_ERR_UNSUPPORTED;
}

// Forward pass that also leaves per-CTA channel statistics ([*n_partials][2][c_col] floats: sums,
// sums of squares of the stored values) in stats_partial (room for 2 * SM count partials).
int tc_conv_stats(const void* src, uint32_t n_src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, int c_red,
                  int c_col, void* out, const float* ep_scale, const float* ep_shift, int ep_relu,
                  float* stats_partial, uint32_t* n_partials, cudaStream_t stream, const void* plan) {
  (void)n_src;
  if (K > kPlanMaxK) plan = nullptr;
#define RMN_TC_CASE(R, Cc)            \
  if (c_red == R && c_col == Cc)      \
    return plan ? tc::launch<R, Cc, false, true, true>(src, w, nbr, n_dst, K, out, ep_scale, ep_shift, ep_relu,   \
                                                       stream, stats_partial, n_partials, plan)                 \
                : tc::launch<R, Cc, false, true>(src, w, nbr, n_dst, K, out, ep_scale, ep_shift, ep_relu, stream, \
                                                 stats_partial, n_partials);
  RMN_TC_CASE(32, 32)
  RMN_TC_CASE(32, 64)
  RMN_TC_CASE(64, 32)
  RMN_TC_CASE(64, 64)
  RMN_TC_CASE(64, 128)
  RMN_TC_CASE(128, 64)
  RMN_TC_CASE(128, 128)
  RMN_TC_CASE(128, 256)
  RMN_TC_CASE(256, 128)
  RMN_TC_CASE(256, 256)
#undef RMN_TC_CASE
  return RMN_ERR_UNSUPPORTED;
}

// Synchronises `stream`, returns the status word and resets it when it was set, so that one
// time-out is reported once and later queries start clean.
int tc_read_status(cudaStream_t stream, uint32_t* status) {
  RMN_CUDA_TRY(cudaStreamSynchronize(stream));
  RMN_CUDA_TRY(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(uint32_t)));
  if (*status != 0) {
    const uint32_t zero = 0;
    RMN_CUDA_TRY(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(uint32_t)));
  }
  return RMN_OK;
}

// Queues a copy of the status word into page-locked host memory on `stream` (no synchronisation):
// for hosts that already wait on that stream for something else.
int tc_copy_status_async(uint32_t* host_dst, cudaStream_t stream) {
  RMN_CUDA_TRY(cudaMemcpyFromSymbolAsync(host_dst, g_tc_status, sizeof(uint32_t), 0, cudaMemcpyDeviceToHost, stream));
  return RMN_OK;
}

// Device address of the status word on the current device (looked up once per device), for kernels of other
// translation units that read it; NULL when the lookup fails.
const uint32_t* tc_status_device_address() {
  constexpr int kMaxDevices = 64;
  static std::atomic<const uint32_t*> address[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return nullptr;
  }
  const uint32_t* p = address[dev].load(std::memory_order_acquire);
  if (!p) {
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, g_tc_status) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    p = static_cast<const uint32_t*>(q);
    address[dev].store(p, std::memory_order_release);
  }
  return p;
}

int tc_clear_status() {
  const uint32_t zero = 0;
  RMN_CUDA_TRY(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(uint32_t)));
  return RMN_OK;
}

}  // namespace rmn
