// Tensor-core sparse convolution for sm_100a: gathered feature tiles in shared
// memory feed tcgen05.mma (bf16 x bf16 -> fp32 in TMEM); the output tile is
// stationary across all kernel offsets, so the scatter-accumulate of the
// reference (index_add_, engine/nn/conv.cpp:62-63) becomes one store per row.
//
//   forward         out[j] = sum_k F[nbr[k][j]]    . W[k]      B = W[k]   read MN-major
//   backward input  dF[i]  = sum_k dY[nbr_t[k][i]] . W[k]^T    B = W[k]   read K-major
//
// One persistent CTA per SM slot loops over tiles of 128 destination rows.
// Warp roles (288 threads):
//   warps 0-3  producers: for every offset k gather the 128 source rows named
//              by nbr[k][tile] (16-byte cp.async, zero-fill for -1) and copy
//              W[k] into a ring of shared-memory stages;
//   warp  4    issues tcgen05.mma for each stage (one elected lane), commits
//              the stage back to the producers and the finished accumulator to
//              the epilogue;
//   warps 5-8  epilogue: tcgen05.ld the fp32 accumulator (double-buffered in
//              TMEM so it overlaps the next tile's MMAs), convert to bf16,
//              store.
//
// Shared-memory operand image (no swizzle, "core matrices" of 8 x 16 bytes):
//   A  [chunk c = channel/8][row r]      : c * 2048 + r * 16            (K-major)
//   B  [ci / 8][c8 = co/8][ci % 8]       : (ci/8) * (C8*128) + c8*128 + (ci%8)*16
// The same B image is read MN-major (reduction over ci, forward) or K-major
// (reduction over co, backward input) by choosing the descriptor strides.
//
// Every mbarrier wait is bounded: after ~2 s without progress a role records
// RMN_ERR_TIMEOUT in a device status word and leaves; all roles then meet at
// the final barrier and the TMEM allocation is released.
#include "rmn_common.cuh"
#include "rmn_tc.cuh"

#include <cuda_bf16.h>

namespace rmn {

__device__ uint32_t g_tc_status = 0;

namespace tc {

constexpr int kTileM = 128;
constexpr int kThreads = 288;

template <int CR, int CC>
struct Cfg {
  static constexpr int KB = CR < 64 ? CR : 64;  // reduction channels per pipeline stage
  static constexpr int NKB = CR / KB;
  static constexpr uint32_t A_BYTES = kTileM * KB * 2;
  static constexpr uint32_t B_BYTES = KB * CC * 2;
  static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = 4;
  static constexpr uint32_t BAR_OFFSET = STAGES * STAGE;
  static constexpr uint32_t SMEM = BAR_OFFSET + 256;
  static constexpr uint32_t TMEM_COLS = pow2_at_least(2 * CC);
};

// CR: reduction channels per offset; CC: output channels; kWT: weights are read transposed
// (backward input). Weight tensor is [K][CIN_w][COUT_w] with (CIN_w, COUT_w) = kWT ? (CC, CR) : (CR, CC).
template <int CR, int CC, bool kWT>
__global__ void __launch_bounds__(kThreads, 1) k_conv_tc(const __nv_bfloat16* __restrict__ src,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         const int32_t* __restrict__ nbr,
                                                         uint32_t n_dst, int K,
                                                         __nv_bfloat16* __restrict__ out,
                                                         uint32_t n_tiles) {
  using C = Cfg<CR, CC>;
  constexpr int STAGES = C::STAGES, KB = C::KB, NKB = C::NKB;
  constexpr int CIN_W = kWT ? CC : CR, COUT_W = kWT ? CR : CC;
  // weight image of one stage: B_ROWS rows of B_C8 16-byte chunks
  constexpr int B_ROWS = kWT ? CC : KB, B_C8 = (kWT ? KB : CC) / 8;
  constexpr uint32_t W_ROWGROUP = B_C8 * 128;  // bytes of 8 weight rows in the image
  static_assert(CR % 32 == 0 && CC % 32 == 0 && CC <= 256 && CR % KB == 0, "channel counts");

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], kProducerThreads);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == 4) {
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

  if (warp < 4) {
    // ------------------------------ producers ------------------------------------------
    uint32_t it = 0;
    for (uint32_t tile = blockIdx.x; tile < n_tiles && !timed_out; tile += gridDim.x) {
      const uint32_t row = tile * kTileM + warp * 32 + lane;
      int32_t idx_next = row < n_dst ? __ldg(nbr + row) : -1;
      for (int k = 0; k < K && !timed_out; ++k) {
        const int32_t idx = idx_next;
        if (k + 1 < K) idx_next = row < n_dst ? __ldg(nbr + (size_t)(k + 1) * n_dst + row) : -1;
        const __nv_bfloat16* wk = w + (size_t)k * CIN_W * COUT_W;
#pragma unroll 1
        for (int kb = 0; kb < NKB; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) { timed_out = true; break; }
          const uint32_t a_s = smem_base + s * C::STAGE, b_s = a_s + C::A_BYTES;
          // A: 8 rows x 4 chunks per warp instruction (64 contiguous bytes per source row;
          // each quarter-warp writes 8 distinct rows of one chunk -> conflict-free)
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int r_local = g * 8 + (lane & 7);
            const int32_t sidx = __shfl_sync(0xFFFFFFFFu, idx, r_local);
            const __nv_bfloat16* base = src + (size_t)(sidx < 0 ? 0 : sidx) * CR + kb * KB;
            const uint32_t bytes = sidx < 0 ? 0u : 16u;
#pragma unroll
            for (int cq = 0; cq < KB / 32; ++cq) {
              const int chunk = cq * 4 + (lane >> 3);
              cp_async16(a_s + chunk * (kTileM * 16) + (warp * 32 + r_local) * 16, base + chunk * 8, bytes);
            }
          }
          // B: this stage's slice of W[k]
#pragma unroll
          for (int i = 0; i < (B_ROWS * B_C8) / kProducerThreads; ++i) {
            const int u = i * 4 + warp;  // one (8-row group, 4-chunk group) per warp instruction
            const int c8 = (u % (B_C8 / 4)) * 4 + (lane >> 3);
            const int r = (u / (B_C8 / 4)) * 8 + (lane & 7);
            const __nv_bfloat16* g = kWT ? wk + (size_t)r * COUT_W + kb * KB + c8 * 8
                                         : wk + (size_t)(kb * KB + r) * COUT_W + c8 * 8;
            cp_async16(b_s + (r >> 3) * W_ROWGROUP + c8 * 128 + (r & 7) * 16, g, 16u);
          }
          cp_async_commit();
          if (it >= (uint32_t)kLag) {
            cp_async_wait<kLag>();
            fence_proxy_async();
            mbar_arrive(&full[(it - kLag) % STAGES]);
          }
        }
      }
    }
    // drain the stages still in flight
    cp_async_wait<0>();
    fence_proxy_async();
    if (!timed_out) {
      const uint32_t pending = it < (uint32_t)kLag ? it : (uint32_t)kLag;
      for (uint32_t j = it - pending; j < it; ++j) mbar_arrive(&full[j % STAGES]);
    }
  } else if (warp == 4) {
    // ------------------------------ MMA issuer -----------------------------------------
    constexpr uint32_t IDESC = instr_desc(kTileM, CC, !kWT);
    uint32_t it = 0, tile_iter = 0;
    for (uint32_t tile = blockIdx.x; tile < n_tiles && !timed_out; tile += gridDim.x, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u)) { timed_out = true; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * CC;
      const uint32_t n_stage = (uint32_t)K * NKB;
      for (uint32_t st = 0; st < n_stage; ++st, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        if (!mbar_wait(&full[s], ph)) { timed_out = true; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_s = smem_base + s * C::STAGE, b_s = a_s + C::A_BYTES;
#pragma unroll
          for (int j = 0; j < KB / 16; ++j) {
            // A, K-major: row groups 128 B apart (SBO), the two 8-channel chunks 2048 B apart (LBO)
            const uint64_t a_desc = smem_desc(a_s + j * 2 * (kTileM * 16), kTileM * 16, 128);
            uint64_t b_desc;
            if constexpr (!kWT)  // MN-major: column groups 128 B apart (SBO), 8-row groups W_ROWGROUP apart (LBO)
              b_desc = smem_desc(b_s + j * 2 * W_ROWGROUP, W_ROWGROUP, 128);
            else                 // K-major: N groups (weight rows) W_ROWGROUP apart (SBO), K chunks 128 B apart (LBO)
              b_desc = smem_desc(b_s + j * 2 * 128, 128, W_ROWGROUP);
            tc_mma_bf16(d_tmem, a_desc, b_desc, IDESC, (st | (uint32_t)j) != 0 ? 1u : 0u);
          }
          tc_commit(&empty[s]);
        }
        __syncwarp();
      }
      if (timed_out) break;
      if (lane == 0) tc_commit(&tmem_full[acc]);
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue -------------------------------------------
    const uint32_t quad = warp & 3;  // TMEM lanes [32*quad, 32*quad + 32)
    uint32_t tile_iter = 0;
    for (uint32_t tile = blockIdx.x; tile < n_tiles && !timed_out; tile += gridDim.x, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_ph)) { timed_out = true; break; }
      tc_fence_after();
      const uint32_t row = tile * kTileM + quad * 32 + lane;
#pragma unroll
      for (int c0 = 0; c0 < CC; c0 += 32) {
        uint32_t r[32];
        tc_ld32(tmem_base + ((quad * 32u) << 16) + acc * CC + c0, r);
        tc_wait_ld();
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
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
    }
  }

  if (timed_out) atomicExch(&g_tc_status, (uint32_t)RMN_ERR_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS)
                 : "memory");
  }
}

template <int CR, int CC, bool kWT>
int launch(const void* src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, void* out,
           cudaStream_t stream) {
  using C = Cfg<CR, CC>;
  auto kern = k_conv_tc<CR, CC, kWT>;
  static bool configured[64] = {};
  int dev = 0;
  RMN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    RMN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    configured[dev] = true;
  }
  int sms = 148;
  RMN_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const uint32_t n_tiles = (n_dst + kTileM - 1) / kTileM;
  const uint32_t per_sm = (C::SMEM <= 110 * 1024 && C::TMEM_COLS <= 256) ? 2u : 1u;
  uint32_t grid = (uint32_t)sms * per_sm;
  if (grid > n_tiles) grid = n_tiles;
  kern<<<grid, kThreads, C::SMEM, stream>>>((const __nv_bfloat16*)src, (const __nv_bfloat16*)w, nbr, n_dst, K,
                                            (__nv_bfloat16*)out, n_tiles);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

}  // namespace tc

}  // namespace rmn

#include "rmn_conv_tc_wgrad.cuh"

namespace rmn {

// Returns RMN_ERR_UNSUPPORTED when no tensor-core instantiation covers the shape.
int tc_conv(const void* src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, int c_red,
            int c_col, bool transposed_weights, void* out, cudaStream_t stream) {
#define RMN_TC_CASE(R, Cc)                                                                      \
  if (c_red == R && c_col == Cc)                                                                \
    return transposed_weights ? tc::launch<R, Cc, true>(src, w, nbr, n_dst, K, out, stream)     \
                              : tc::launch<R, Cc, false>(src, w, nbr, n_dst, K, out, stream);
  RMN_TC_CASE(32, 32)
  RMN_TC_CASE(32, 64)
  RMN_TC_CASE(64, 32)
  RMN_TC_CASE(64, 64)
  RMN_TC_CASE(64, 128)
  RMN_TC_CASE(128, 64)
  RMN_TC_CASE(128, 128)
  RMN_TC_CASE(128, 256)
  RMN_TC_CASE(256, 128)
#undef RMN_TC_CASE
  return RMN_ERR_UNSUPPORTED;
}

int tc_read_status(cudaStream_t stream, uint32_t* status) {
  RMN_CUDA_TRY(cudaStreamSynchronize(stream));
  RMN_CUDA_TRY(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(uint32_t)));
  return RMN_OK;
}

}  // namespace rmn
