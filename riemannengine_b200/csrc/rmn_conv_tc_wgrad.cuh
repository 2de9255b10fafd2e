// Tensor-core weight gradient for sm_100a (bf16 features, fp32 accumulation):
//   dW[k][ci][co] = sum_j F[nbr[k][j]][ci] * dY[j][co]
// As a GEMM the reduction runs over destination rows j, so both operands are
// "MN-major" (channels contiguous for a fixed row): A' = gathered feature rows,
// B' = dY rows. G = 128 / C_in kernel offsets are stacked along M so that every
// tcgen05.mma uses the full M = 128 (TMEM lane = offset-in-group * C_in + ci)
// while sharing the same dY tile.
//
// Grid = (row slices, offset sets). A CTA keeps the accumulators of its offset
// set resident in TMEM (groups * C_out <= 512 columns) while it walks its row
// slice in blocks of 64 rows. Slice c is the row blocks c, c + slices, c + 2 slices, ...: all CTAs
// sweep the rows together, so the feature rows being gathered at any moment are the neighbours of one
// narrow band of rows (one sample of the batch) and stay in L2; contiguous chunks would spread the
// gathers of the CTAs over the whole feature array at once. One pipeline stage = (row block, GP offset groups):
// GP x 64 x G gathered rows (GP x 16 KB) + the 64 dY rows, which the GP groups
// share (copied once, and read from shared memory once per K slice: the other
// groups' MMAs reuse the collector buffer). At the end the four producer
// warps read the accumulators back and write an fp32 partial
// [chunk][K][C_in][C_out]; a second kernel adds the chunks in a fixed order, so
// the result is bit-reproducible (no atomics).
//
// Waits are bounded like in the forward kernel (status word g_tc_status).
//
// Included at the end of rmn_conv_tc.cu (one translation unit, one status word).
#pragma once

namespace rmn {
namespace tc {

constexpr int kRowsPerStage = 64;
constexpr int kWgProducerWarps = 16;  // gather warps (the first four also run the epilogue)
constexpr int kWgProducers = kWgProducerWarps * 32;
constexpr int kWgLinesPerGroup = kRowsPerStage * 2 * 8 / kWgProducers;  // A' lines per thread, stage and group
constexpr int kWgradThreads = kWgProducers + 32;

constexpr uint32_t instr_desc_mn(int m, int n) {
  // D fp32, A/B bf16, both operands MN-major
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

template <int CIN, int COUT>
struct WgradCfg {
  static constexpr int G = 128 / CIN;                     // offsets stacked along M
  static constexpr int MAX_GROUPS = 512 / COUT;           // accumulators resident in TMEM
  static constexpr uint32_t A_GROUP = kRowsPerStage * 128 * 2;   // gathered rows of one offset group
  static constexpr uint32_t B_BYTES = kRowsPerStage * COUT * 2;
  // Offset groups per stage (they share the stage's dY rows): four where two such stages fit in shared
  // memory, else two where three such stages fit, else one. Fewer, larger stages carry the per-stage work of a warp (index load, shuffles, barrier
  // wait) over more copies.
  static constexpr int GP = (MAX_GROUPS >= 4 && (4 * A_GROUP + B_BYTES) * 2 <= 227 * 1024 - 256)
                                ? 4
                                : ((MAX_GROUPS >= 2 && (2 * A_GROUP + B_BYTES) * 3 <= 200 * 1024) ? 2 : 1);
  static constexpr uint32_t A_BYTES = GP * A_GROUP;
  static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
  static constexpr int IDX_PER_THREAD = GP * kWgLinesPerGroup;
  // as many stages (up to six) as 227 KB of shared memory hold beside the barriers;
  // more than 114 KB in total also keeps one CTA (one TMEM owner) per SM
  static constexpr uint32_t STAGE_BUDGET = 227 * 1024 - 256;
  static constexpr int STAGES = STAGE * 6 <= STAGE_BUDGET ? 6 : (STAGE * 5 <= STAGE_BUDGET ? 5 : (STAGE * 4 <= STAGE_BUDGET ? 4 : (STAGE * 3 <= STAGE_BUDGET ? 3 : 2)));
  static_assert(STAGE * STAGES <= STAGE_BUDGET, "stages do not fit in shared memory");
  static constexpr uint32_t BAR_OFFSET = STAGES * STAGE;
  static constexpr uint32_t SMEM = BAR_OFFSET + 256;
};

template <int CIN, int COUT>
__global__ void __launch_bounds__(kWgradThreads, 1) k_conv_tc_wgrad(
    const __nv_bfloat16* __restrict__ feats, const __nv_bfloat16* __restrict__ grad_out,
    const int32_t* __restrict__ nbr, uint32_t n_dst, int K, int groups_per_set,
    uint32_t tmem_cols, float* __restrict__ partial, uint32_t feat_stride) {
  using C = WgradCfg<CIN, COUT>;
  constexpr int STAGES = C::STAGES, G = C::G, GP = C::GP, kWgIdxPerThread = C::IDX_PER_THREAD;
  constexpr int SWB = (COUT < 64 ? COUT : 64) * 2;     // bytes per dY line
  constexpr int B_CPL = SWB / 16;                      // chunks per dY line
  constexpr uint32_t A_ATOM = kRowsPerStage * 128;     // bytes of one 64-channel atom of A' (all stage rows)
  constexpr uint32_t B_ATOM = kRowsPerStage * SWB;
  constexpr uint32_t LT_B = SWB == 128 ? 2u : 4u;
  static_assert(128 % CIN == 0 && CIN >= 32 && COUT % 32 == 0 && COUT <= 256, "channel counts");

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* done = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_groups_total = (K + G - 1) / G;
  const int group0 = blockIdx.y * groups_per_set;
  const int n_groups = min(groups_per_set, n_groups_total - group0);  // offset groups of this CTA
  const int n_sg = (n_groups + GP - 1) / GP;                          // stages per row block
  // row block b of this CTA covers rows [(blockIdx.x + b * gridDim.x) * 64, +64)
  const uint32_t total_blocks = (n_dst + kRowsPerStage - 1) / kRowsPerStage;
  const uint32_t j_end = n_dst;
  const uint32_t n_blocks = blockIdx.x < total_blocks ? (total_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t n_stage = n_blocks * (uint32_t)n_sg;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], kWgProducers);
      mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == kWgProducerWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t smem_base = smem_u32(smem);
  bool timed_out = false;

  if (warp < kWgProducerWarps) {
    // ------------------------------ producers ------------------------------------------
    // A' image: one 128-byte swizzled line per (stage row, 64-channel atom of the stacked M axis);
    // eight consecutive lanes copy one line, i.e. one (CIN >= 64) or two (CIN = 32) gathered rows.
    // Neighbour indices: warp w copies rows [4w, 4w + 4) of every stage, for all G * GP offsets of the
    // stage, i.e. 4 * G * GP <= 64 table entries: lane l loads entry l = (offset l / 4, row l % 4) (and entry
    // l + 32 where there are more than 32) with one coalesced load per warp, stage and 32 entries, six stages
    // before use (the table is streamed from DRAM; a rotating window of named registers); the lanes of a line
    // fetch theirs with a shuffle when the stage is issued.
    uint32_t it = 0;
    constexpr int NIDX = 4 * G * GP;
    uint32_t pf_blk = 0;
    int pf_sg = 0;
    // a warp's 4 * G * GP table entries of a stage: entry e = (offset e / 4, row e % 4), lane l holds
    // entries l and (for more than 32 entries) l + 32
    constexpr int NREG = (NIDX + 31) / 32;
    struct Entries {
      int32_t v[NREG];
    };
    auto load_indices = [&]() -> Entries {
      Entries out;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        int32_t v = -1;
        const int e = r * 32 + lane;
        if (e < NIDX) {
          const int combo = e >> 2, gp = combo / G, gg = combo % G;
          const uint32_t j = (blockIdx.x + pf_blk * gridDim.x) * kRowsPerStage + warp * 4 + (lane & 3);
          const int k = (group0 + pf_sg * GP + gp) * G + gg;
          if (pf_blk < n_blocks && j < j_end && k < K && pf_sg * GP + gp < n_groups) v = __ldg(nbr + (size_t)k * n_dst + j);
        }
        out.v[r] = v;
      }
      if (++pf_sg == n_sg) { pf_sg = 0; ++pf_blk; }
      return out;
    };
    Entries idx_w0 = load_indices(), idx_w1 = load_indices(), idx_w2 = load_indices(), idx_w3 = load_indices(),
            idx_w4 = load_indices(), idx_w5 = load_indices();
    for (uint32_t blk = 0; blk < n_blocks && !timed_out; ++blk) {
      const uint32_t j0 = (blockIdx.x + blk * gridDim.x) * kRowsPerStage;
#pragma unroll 1
      for (int sg = 0; sg < n_sg; ++sg, ++it) {
        const Entries mine = idx_w0;
        idx_w0 = idx_w1; idx_w1 = idx_w2; idx_w2 = idx_w3; idx_w3 = idx_w4; idx_w4 = idx_w5;
        idx_w5 = load_indices();
        int32_t idx[kWgIdxPerThread];
#pragma unroll
        for (int i = 0; i < kWgIdxPerThread; ++i) {
          const int gp = i / kWgLinesPerGroup, atom = i % kWgLinesPerGroup;
          const int gg = (atom * 8 + (lane & 7)) / (CIN / 8);
          const int e = (gp * G + gg) * 4 + (lane >> 3);  // < 32 * NREG; which register is uniform per warp only
          // when gg is, so both are read and the right one kept
          int32_t got = __shfl_sync(0xFFFFFFFFu, mine.v[0], e & 31);
          if constexpr (NREG > 1) {
            const int32_t hi = __shfl_sync(0xFFFFFFFFu, mine.v[1], e & 31);
            got = e >= 32 ? hi : got;
          }
          idx[i] = got;
        }
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        if (!mbar_wait(&empty[s], ph ^ 1u)) { timed_out = true; break; }
        const uint32_t a_s = smem_base + s * C::STAGE, b_s = a_s + C::A_BYTES;
#pragma unroll
        for (int i = 0; i < kWgIdxPerThread; ++i) {
          const int gp = i / kWgLinesPerGroup;
          const int unit = ((i % kWgLinesPerGroup) * kWgProducerWarps + warp) * 4 + (lane >> 3);
          const uint32_t r = unit & (kRowsPerStage - 1), atom = unit / kRowsPerStage, c = lane & 7;
          const int cch = (atom * 8 + c) % (CIN / 8);
          cp_async16(a_s + gp * C::A_GROUP + atom * A_ATOM + r * 128 + (swz<128>(r, c) << 4),
                     feats + (size_t)(idx[i] < 0 ? 0 : idx[i]) * feat_stride + cch * 8, idx[i] < 0 ? 0u : 16u);
        }
        // B': the 64 dY rows of this block, one swizzled line per (row, 64-column atom)
#pragma unroll
        for (int q = tid; q < kRowsPerStage * (COUT / 8); q += kWgProducers) {
          const uint32_t c = q % B_CPL, unit = q / B_CPL;
          const uint32_t r = unit & (kRowsPerStage - 1), atom = unit / kRowsPerStage;
          const uint32_t j = j0 + r;
          const bool ok = j < j_end;
          cp_async16(b_s + atom * B_ATOM + r * SWB + (swz<SWB>(r, c) << 4),
                     grad_out + (size_t)(ok ? j : 0) * COUT + atom * (SWB / 2) + c * 8, ok ? 16u : 0u);
        }
        cp_async_arrive_noinc(&full[s]);  // fires when this thread's copies have landed
      }
    }
    cp_async_wait<0>();
    // ------------------------------ epilogue (first four producer warps) ----------------
    if (warp < 4) {
    if (!timed_out && n_stage > 0 && !mbar_wait(done, 0)) timed_out = true;
    timed_out = __any_sync(0xFFFFFFFFu, timed_out);  // the TMEM loads below are warp-collective
    tc_fence_after();
    const int m = warp * 32 + lane;  // TMEM lane
    const int gg = m / CIN, ci = m % CIN;
    for (int g = 0; g < n_groups; ++g) {
      const int k = (group0 + g) * G + gg;
#pragma unroll
      for (int c0 = 0; c0 < COUT; c0 += 32) {
        uint32_t r[32];
        if (n_stage > 0 && !timed_out) {
          tc_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + g * COUT + c0, r);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int v = 0; v < 32; ++v) r[v] = 0u;
        }
        if (k < K) {
          float4* dst = reinterpret_cast<float4*>(partial + (((size_t)blockIdx.x * K + k) * CIN + ci) * COUT + c0);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            dst[v] = make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                                 __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
        }
      }
    }
    }
  } else {
    // ------------------------------ MMA issuer -----------------------------------------
    constexpr uint32_t IDESC = instr_desc_mn(128, COUT);
    constexpr uint64_t A_DESC0 = smem_desc_sw_const(A_ATOM, 8 * 128, 2u);
    constexpr uint64_t B_DESC0 = smem_desc_sw_const(B_ATOM, 8 * SWB, LT_B);
    constexpr uint32_t A_DESC_HI = (uint32_t)(A_DESC0 >> 32), B_DESC_HI = (uint32_t)(B_DESC0 >> 32);
    uint32_t it = 0;
    for (uint32_t blk = 0; blk < n_blocks && !timed_out; ++blk) {
      for (int sg = 0; sg < n_sg; ++sg, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
        if (!mbar_wait(&full[s], ph)) { timed_out = true; break; }
        fence_proxy_async();  // cp.async wrote through the generic proxy; the MMA reads through the async proxy
        tc_fence_after();
        {
          // warp-uniform code, one elected lane issues; descriptors are a constant plus the
          // operand's start address field
          const uint32_t a_s = smem_base + s * C::STAGE;
          const uint32_t a_lo = (a_s >> 4) + (uint32_t)(A_DESC0 & 0xFFFFFFFFu);
          const uint32_t b_lo = ((a_s + C::A_BYTES) >> 4) + (uint32_t)(B_DESC0 & 0xFFFFFFFFu);
          const uint32_t d0 = tmem_base + (uint32_t)(sg * GP) * COUT;
          static_for<kRowsPerStage / 16>([&](auto jc) {
            constexpr int jj = decltype(jc)::value;
            // MN-major swizzled operands: 8-row K groups 8 lines apart (SBO), 64-channel atoms one ATOM apart (LBO)
            const uint64_t a_desc = ((uint64_t)A_DESC_HI << 32) | (a_lo + (uint32_t)((jj * 16 * 128) >> 4));
            const uint64_t b_desc = ((uint64_t)B_DESC_HI << 32) | (b_lo + (uint32_t)((jj * 16 * SWB) >> 4));
            const uint32_t accumulate = (blk | (uint32_t)jj) != 0 ? 1u : 0u;
            if constexpr (GP >= 2) {
              // the GP groups of the stage multiply the same dY slice: the first MMA reads it from shared
              // memory into collector buffer jj, the others reuse it (.ws shapes only)
              static_for<GP>([&](auto gc) {
                constexpr int g = decltype(gc)::value;
                const uint64_t ag_desc = a_desc + (uint64_t)((g * C::A_GROUP) >> 4);
                if constexpr (COUT == 64 || COUT == 128 || COUT == 256)
                  tc_mma_bf16_ws_elect<jj & 3, g == 0 ? 0 : (g == GP - 1 ? 2 : 1)>(d0 + g * COUT, ag_desc, b_desc, IDESC,
                                                                                  accumulate);
                else
                  tc_mma_bf16_elect(d0 + g * COUT, ag_desc, b_desc, IDESC, accumulate);
              });
            } else {
              tc_mma_bf16_elect(d0, a_desc, b_desc, IDESC, accumulate);
            }
          });
          tc_commit_elect(&empty[s]);
        }
      }
    }
    if (!timed_out) tc_commit_elect(done);
  }

  if (timed_out) atomicExch(&g_tc_status, (uint32_t)RMN_ERR_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == kWgProducerWarps) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols)
                 : "memory");
  }
}

// out[k][col0 + ci][co] = sum over the chunks of partial[chunk][k][ci][co] (ci < cin of the launch; the output
// has cin_total input channels: a 256-channel gradient is produced as two 128-channel halves)
__global__ void __launch_bounds__(256) k_reduce_chunks(const float* __restrict__ partial, uint32_t n_chunks,
                                                       size_t elems, float* __restrict__ out, uint32_t cin,
                                                       uint32_t cout, uint32_t cin_total, uint32_t col0) {
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= elems) return;
  float s = 0.f;
  for (uint32_t c = 0; c < n_chunks; ++c) s += partial[(size_t)c * elems + e];
  const size_t k = e / ((size_t)cin * cout), r = e % ((size_t)cin * cout);
  out[(k * cin_total + col0) * cout + r] = s;
}

struct WgradPlan {
  uint32_t chunks;  // row slices = CTAs per offset set
  int sets, groups_per_set;
  uint32_t tmem_cols;
};

template <int CIN, int COUT>
WgradPlan plan(uint32_t n_dst, int K, int sms) {
  using C = WgradCfg<CIN, COUT>;
  WgradPlan p;
  const int groups = (K + C::G - 1) / C::G;
  p.sets = (groups + C::MAX_GROUPS - 1) / C::MAX_GROUPS;
  p.groups_per_set = (groups + p.sets - 1) / p.sets;
  // (a stage always carries GP groups: an odd set is padded with an all-zero group)
  p.tmem_cols = pow2_at_least((uint32_t)((p.groups_per_set + C::GP - 1) / C::GP * C::GP) * COUT);
  uint32_t want = (uint32_t)(sms / p.sets);
  if (want < 1) want = 1;
  // at least 32 row blocks (2048 rows) per slice: fewer, and the fp32 partials cost more than they spread
  const uint32_t total_blocks = (n_dst + kRowsPerStage - 1) / kRowsPerStage;
  uint32_t slices = total_blocks / 32;
  if (slices < 1) slices = 1;
  p.chunks = slices < want ? slices : want;
  return p;
}

// feats: [*, cin_total] rows of which this launch takes the CIN channels from column col0 on
template <int CIN, int COUT>
int launch_wgrad(const void* feats, const void* grad_out, const int32_t* nbr, uint32_t n_dst, int K, float* dw,
                 void* workspace, size_t workspace_bytes, size_t* need, cudaStream_t stream, int cin_total = CIN,
                 int col0 = 0) {
  using C = WgradCfg<CIN, COUT>;
  int dev = 0, sms = 148;
  RMN_CUDA_TRY(cudaGetDevice(&dev));
  RMN_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const WgradPlan p = plan<CIN, COUT>(n_dst, K, sms);
  const size_t elems = (size_t)K * CIN * COUT;
  *need = (size_t)p.chunks * elems * sizeof(float);
  if (!feats) return RMN_OK;  // size query
  if (workspace_bytes < *need) return RMN_ERR_ALLOC;
  auto kern = k_conv_tc_wgrad<CIN, COUT>;
  static std::once_flag configured[64];
  cudaError_t attr_err = cudaSuccess;
  if (dev >= 0 && dev < 64)
    std::call_once(configured[dev], [&] {
      attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    });
  else
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
  RMN_CUDA_TRY(attr_err);
  dim3 grid(p.chunks, p.sets);
  kern<<<grid, kWgradThreads, C::SMEM, stream>>>((const __nv_bfloat16*)feats + col0, (const __nv_bfloat16*)grad_out,
                                                 nbr, n_dst, K, p.groups_per_set, p.tmem_cols, (float*)workspace,
                                                 (uint32_t)cin_total);
  RMN_LAUNCH_CHECK();
  count_tc_launch();
  k_reduce_chunks<<<(uint32_t)((elems + 255) / 256), 256, 0, stream>>>((const float*)workspace, p.chunks, elems, dw,
                                                                        (uint32_t)CIN, (uint32_t)COUT,
                                                                        (uint32_t)cin_total, (uint32_t)col0);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

}  // namespace tc

// feats == nullptr: only report the workspace bytes in *need. RMN_ERR_UNSUPPORTED when no
// tensor-core instantiation covers the shape.
int tc_conv_wgrad(const void* feats, const void* grad_out, const int32_t* nbr, uint32_t n_dst, int K, int c_in,
                  int c_out, float* dw, void* workspace, size_t workspace_bytes, size_t* need,
                  cudaStream_t stream) {
#define RMN_WG_CASE(I, O) \
  if (c_in == I && c_out == O) \
    return tc::launch_wgrad<I, O>(feats, grad_out, nbr, n_dst, K, dw, workspace, workspace_bytes, need, stream);
  RMN_WG_CASE(32, 32)
  RMN_WG_CASE(32, 64)
  RMN_WG_CASE(64, 32)
  RMN_WG_CASE(64, 64)
  RMN_WG_CASE(64, 128)
  RMN_WG_CASE(128, 64)
  RMN_WG_CASE(128, 128)
  RMN_WG_CASE(128, 256)
#undef RMN_WG_CASE
  // 256 input channels: the kernel stacks 128 / C_in offsets along M, so the two 128-channel halves of the
  // feature rows are run one after the other (same workspace: the launches are ordered on the stream)
#define RMN_WG_SPLIT(O)                                                                                          \
  if (c_in == 256 && c_out == O) {                                                                               \
    int st = tc::launch_wgrad<128, O>(feats, grad_out, nbr, n_dst, K, dw, workspace, workspace_bytes, need, stream, 256, 0); \
    if (st != RMN_OK || !feats) return st;                                                                       \
    return tc::launch_wgrad<128, O>(feats, grad_out, nbr, n_dst, K, dw, workspace, workspace_bytes, need, stream, 256, 128); \
  }
  RMN_WG_SPLIT(128)
  RMN_WG_SPLIT(256)
  RMN_WG_SPLIT(64)
#undef RMN_WG_SPLIT
  return RMN_ERR_UNSUPPORTED;
}

}  // namespace rmn
