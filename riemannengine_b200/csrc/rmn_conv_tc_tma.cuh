// TMA-fed variant of the tensor-core convolution (forward and backward input).
//
// Same tiling, operand images, MMA issue and epilogue as k_conv_tc, but nothing goes through
// the load/store unit: every group of four gathered feature rows is one
// cp.async.bulk.tensor ... tile::gather4 (the TMA engine fetches the four rows named by the
// neighbour table, applies the 128-byte swizzle and zero-fills rows whose index lies outside
// the tensor), and the W[k] slice is one or two ordinary tiled TMA loads. Completion is
// tracked by the stage's mbarrier transaction count, so the four producer warps only read
// indices and issue one instruction per lane and stage, and every stage of shared memory can
// be in flight. Every load is CTA-local (one destination CTA) and addresses this GPU's memory only.
//
// Included by rmn_conv_tc.cu (needs Cfg<>, swz<> and the helpers of rmn_tc.cuh).
#pragma once

#include <cuda.h>

namespace rmn {
namespace tc {

constexpr int kTmaThreads = 288;  // 4 producer warps, 1 MMA warp, 4 epilogue warps

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int32_t col,
                                            int32_t r0, int32_t r1, int32_t r2, int32_t r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(col), "r"(r0), "r"(r1), "r"(r2),
      "r"(r3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int32_t x,
                                            int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

template <int CR, int CC, bool kWT>
__global__ void __launch_bounds__(kTmaThreads, 1) k_conv_tma(const __grid_constant__ CUtensorMap map_src,
                                                            const __grid_constant__ CUtensorMap map_w,
                                                            const int32_t* __restrict__ nbr, uint32_t n_src,
                                                            uint32_t n_dst, int K, __nv_bfloat16* __restrict__ out,
                                                            uint32_t n_super) {
  using C = Cfg<CR, CC>;
  constexpr int STAGES = C::STAGES, KB = C::KB, NKB = C::NKB, T = C::T, SWA = C::SWA;
  constexpr int CIN_W = kWT ? CC : CR;
  constexpr int SWB = kWT ? KB * 2 : (CC < 64 ? CC : 64) * 2;
  constexpr int B_LINES = kWT ? CC : KB;
  constexpr int B_ATOMS = kWT ? 1 : (CC * 2) / SWB;
  constexpr uint32_t B_ATOM_BYTES = B_LINES * SWB;
  constexpr uint32_t LT_A = SWA == 128 ? 2u : 4u, LT_B = SWB == 128 ? 2u : 4u;
  static_assert(T <= 4, "one producer warp per row tile");

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);   // one arrive.expect_tx per stage; the data arrives as transaction bytes
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
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
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
    // warp t feeds row tile t: lane l owns rows 4l .. 4l+3 of the tile (one gather4 per stage)
    const bool has_tile = warp < T;
    const int32_t oob = (int32_t)n_src;  // a row index outside the tensor reads as zeros
    uint32_t it = 0;
    for (uint32_t st = blockIdx.x; st < n_super && !timed_out; st += gridDim.x) {
      const uint32_t row0 = st * (kTileM * T) + warp * kTileM + lane * 4;
      int32_t nxt[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) nxt[j] = (has_tile && row0 + j < n_dst) ? __ldg(nbr + row0 + j) : -1;
      for (int k = 0; k < K && !timed_out; ++k) {
        int32_t idx[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) idx[j] = nxt[j] < 0 ? oob : nxt[j];
        if (k + 1 < K) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            nxt[j] = (has_tile && row0 + j < n_dst) ? __ldg(nbr + (size_t)(k + 1) * n_dst + row0 + j) : -1;
        }
#pragma unroll 1
        for (int kb = 0; kb < NKB; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) { timed_out = true; break; }
          const uint32_t a_s = smem_base + s * C::STAGE, b_s = a_s + C::A_BYTES;
          if (warp == 0 && lane == 0) {
            mbar_arrive_expect_tx(&full[s], C::STAGE);
            if constexpr (!kWT) {
#pragma unroll
              for (int atom = 0; atom < B_ATOMS; ++atom)
                tma_load_2d(b_s + atom * B_ATOM_BYTES, &map_w, &full[s], atom * (SWB / 2), k * CIN_W + kb * KB);
            } else {
              tma_load_2d(b_s, &map_w, &full[s], kb * KB, k * CIN_W);
            }
          }
          if (has_tile)
            tma_gather4(a_s + warp * C::A_TILE + (uint32_t)lane * 4u * SWA, &map_src, &full[s], kb * KB, idx[0],
                        idx[1], idx[2], idx[3]);
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------ MMA issuer -----------------------------------------
    constexpr uint32_t IDESC = instr_desc(kTileM, CC, !kWT);
    uint32_t it = 0, tile_iter = 0;
    for (uint32_t st = blockIdx.x; st < n_super && !timed_out; st += gridDim.x, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u)) { timed_out = true; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * (T * CC);
      const uint32_t n_stage = (uint32_t)K * NKB;
      for (uint32_t sg = 0; sg < n_stage; ++sg, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        if (!mbar_wait(&full[s], ph)) { timed_out = true; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_s = smem_base + s * C::STAGE, b_s = a_s + C::A_BYTES;
#pragma unroll
          for (int t = 0; t < T; ++t) {
#pragma unroll
            for (int j = 0; j < KB / 16; ++j) {
              const uint64_t a_desc = smem_desc_sw(a_s + t * C::A_TILE + j * 32, 16, 8 * SWA, LT_A);
              uint64_t b_desc;
              if constexpr (!kWT)
                b_desc = smem_desc_sw(b_s + j * 16 * SWB, B_ATOM_BYTES, 8 * SWB, LT_B);
              else
                b_desc = smem_desc_sw(b_s + j * 32, 16, 8 * SWB, LT_B);
              tc_mma_bf16(d_tmem + t * CC, a_desc, b_desc, IDESC, (sg | (uint32_t)j) != 0 ? 1u : 0u);
            }
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
    const uint32_t quad = warp & 3;
    uint32_t tile_iter = 0;
    for (uint32_t st = blockIdx.x; st < n_super && !timed_out; st += gridDim.x, ++tile_iter) {
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_ph)) { timed_out = true; break; }
      tc_fence_after();
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const uint32_t row = st * (kTileM * T) + t * kTileM + quad * 32 + lane;
#pragma unroll
        for (int c0 = 0; c0 < CC; c0 += 32) {
          uint32_t r[32];
          tc_ld32(tmem_base + ((quad * 32u) << 16) + acc * (T * CC) + t * CC + c0, r);
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

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 row-major [rows, cols] tensor, box = [box_rows, box_cols], swizzle span = box_cols * 2 bytes
inline bool make_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                          uint32_t box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || ((uintptr_t)base & 15) || (cols * 2) % 16 != 0) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = box_cols * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// RMN_ERR_UNSUPPORTED when the tensor maps cannot be built (the caller then uses k_conv_tc).
template <int CR, int CC, bool kWT>
int launch_tma(const void* src, uint32_t n_src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, void* out,
               cudaStream_t stream) {
  using C = Cfg<CR, CC>;
  constexpr int KB = C::KB;
  constexpr int CIN_W = kWT ? CC : CR, COUT_W = kWT ? CR : CC;
  CUtensorMap map_src, map_w;
  if (!make_map_bf16(&map_src, src, n_src, CR, 1, KB)) return RMN_ERR_UNSUPPORTED;
  const bool ok_w = kWT ? make_map_bf16(&map_w, w, (uint64_t)K * CIN_W, COUT_W, CC, KB)
                        : make_map_bf16(&map_w, w, (uint64_t)K * CIN_W, COUT_W, KB, CC < 64 ? CC : 64);
  if (!ok_w) return RMN_ERR_UNSUPPORTED;
  auto kern = k_conv_tma<CR, CC, kWT>;
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
  const uint32_t per_sm = (C::SMEM <= 110 * 1024 && C::TMEM_COLS <= 256) ? 2u : 1u;
  uint32_t grid = (uint32_t)sms * per_sm;
  if (grid > n_super) grid = n_super;
  kern<<<grid, kTmaThreads, C::SMEM, stream>>>(map_src, map_w, nbr, n_src, n_dst, K, (__nv_bfloat16*)out, n_super);
  RMN_LAUNCH_CHECK();
  count_tc_launch();
  return RMN_OK;
}

}  // namespace tc
}  // namespace rmn
