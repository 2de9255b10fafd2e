// Batch-normalisation pieces that sit next to the convolution: per-channel batch statistics
// (sum, sum of squares) of a feature matrix, and the per-channel affine + ReLU that applies a
// normalisation. The reference runs torch::nn::BatchNorm1d on the feature matrix after every
// convolution (engine/nn/normalization.hpp:11-34, engine/nn/residual.cpp:44-52): one pass for the
// statistics, one to normalise, one for the ReLU. Here the statistics come out of the convolution's
// epilogue (rmn_conv_forward_stats: no extra pass) and normalise + ReLU are one pass.
#include "rmn_common.cuh"

#include <cuda_bf16.h>


namespace rmn {

// defined in rmn_conv_tc.cu
int tc_conv_stats(const void* src, uint32_t n_src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, int c_red,
                  int c_col, void* out, const float* ep_scale, const float* ep_shift, int ep_relu,
                  float* stats_partial, uint32_t* n_partials, cudaStream_t stream, const void* plan);

constexpr uint32_t kMaxStatPartials = 1024;

__device__ __forceinline__ float ld_f32(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ld_f32(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Partial channel sums of x[n][C]: block b adds rows b, b + gridDim.x, ... ; thread (row slot, channel).
// partial[b][0][c] = sum, partial[b][1][c] = sum of squares.
template <typename T>
__global__ void __launch_bounds__(256) k_channel_stats_partial(const T* __restrict__ x, uint32_t n, int C,
                                                               float* __restrict__ partial) {
  extern __shared__ float s_red[];  // [2][256]
  const int cpr = C < 256 ? C : 256;          // channels handled per pass
  const int slots = 256 / cpr;                // rows in flight per block
  const int slot = threadIdx.x / cpr, cl = threadIdx.x % cpr;
  for (int c0 = 0; c0 < C; c0 += cpr) {
    const int c = c0 + cl;
    float sum = 0.f, sq = 0.f;
    if (slot < slots && c < C) {
      for (uint32_t r = blockIdx.x * slots + slot; r < n; r += gridDim.x * slots) {
        const float v = ld_f32(x + (size_t)r * C + c);
        sum += v;
        sq += v * v;
      }
    }
    s_red[threadIdx.x] = sum;
    s_red[256 + threadIdx.x] = sq;
    __syncthreads();
    if (slot == 0 && c < C) {
      for (int s2 = 1; s2 < slots; ++s2) {
        sum += s_red[s2 * cpr + cl];
        sq += s_red[256 + s2 * cpr + cl];
      }
      partial[(size_t)blockIdx.x * 2 * C + c] = sum;
      partial[(size_t)blockIdx.x * 2 * C + C + c] = sq;
    }
    __syncthreads();
  }
}

// stats[2][C] (double) = sum over the partials, in partial order (deterministic).
__global__ void k_stats_reduce(const float* __restrict__ partial, uint32_t n_partials, int C,
                               double* __restrict__ stats) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * C) return;
  double t = 0.0;
  for (uint32_t p = 0; p < n_partials; ++p) t += (double)partial[(size_t)p * 2 * C + i];
  stats[i] = t;
}

template <typename T>
__global__ void __launch_bounds__(256) k_affine_act(const T* __restrict__ x, size_t total, int C,
                                                    const float* __restrict__ scale, const float* __restrict__ shift,
                                                    int relu, T* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    float v = ld_f32(x + i) * (scale ? __ldg(scale + c) : 1.f) + (shift ? __ldg(shift + c) : 0.f);
    if (relu) v = fmaxf(v, 0.f);
    if constexpr (sizeof(T) == 4) out[i] = v;
    else out[i] = __float2bfloat16_rn(v);
  }
}

// eight bf16 per thread; C % 8 == 0 and 16-byte aligned pointers
__global__ void __launch_bounds__(256) k_affine_act_bf16x8(const uint4* __restrict__ x, size_t total_vec, int C,
                                                           const float* __restrict__ scale,
                                                           const float* __restrict__ shift, int relu,
                                                           uint4* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (size_t)gridDim.x * blockDim.x) {
    const int c0 = (int)((i * 8) % C);
    const uint4 v = __ldg(x + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
      const int c = c0 + 2 * j;
      f.x = f.x * (scale ? __ldg(scale + c) : 1.f) + (shift ? __ldg(shift + c) : 0.f);
      f.y = f.y * (scale ? __ldg(scale + c + 1) : 1.f) + (shift ? __ldg(shift + c + 1) : 0.f);
      if (relu) { f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f); }
      const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
      o[j] = *reinterpret_cast<const uint32_t*>(&b);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

static int channel_stats(const void* x, uint32_t n, int C, int dtype, double* stats, float* partial,
                         cudaStream_t stream) {
  uint32_t blocks = n < 148u * 4u ? (n ? n : 1u) : 148u * 4u;
  if (blocks > kMaxStatPartials) blocks = kMaxStatPartials;
  if (dtype == RMN_F32)
    k_channel_stats_partial<float><<<blocks, 256, 2 * 256 * sizeof(float), stream>>>((const float*)x, n, C, partial);
  else
    k_channel_stats_partial<__nv_bfloat16><<<blocks, 256, 2 * 256 * sizeof(float), stream>>>((const __nv_bfloat16*)x,
                                                                                              n, C, partial);
  RMN_LAUNCH_CHECK();
  k_stats_reduce<<<(2 * C + 127) / 128, 128, 0, stream>>>(partial, blocks, C, stats);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

}  // namespace rmn

using namespace rmn;

extern "C" size_t rmn_channel_stats_workspace_bytes(int channels) {
  return channels < 1 ? 0 : (size_t)kMaxStatPartials * 2 * (size_t)channels * sizeof(float);
}

extern "C" int rmn_channel_stats(const void* d_x, uint32_t n_rows, int channels, int dtype, double* d_stats,
                                 void* d_workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_stats || channels < 1 || (dtype != RMN_F32 && dtype != RMN_BF16)) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) {
    RMN_CUDA_TRY(cudaMemsetAsync(d_stats, 0, 2 * (size_t)channels * sizeof(double), stream));
    return RMN_OK;
  }
  if (!d_x || !d_workspace) return RMN_ERR_BAD_ARG;
  if (workspace_bytes < rmn_channel_stats_workspace_bytes(channels)) return RMN_ERR_ALLOC;
  return channel_stats(d_x, n_rows, channels, dtype, d_stats, (float*)d_workspace, stream);
}

extern "C" int rmn_conv_forward_stats(const void* d_feats, uint32_t n_src, int c_in, const void* d_weights, int K,
                                      int c_out, const int32_t* d_nbr, uint32_t n_dst, void* d_out, int dtype,
                                      const float* d_scale, const float* d_shift, int relu, double* d_stats,
                                      void* d_workspace, size_t workspace_bytes, void* stream_) {
  return rmn_conv_forward_stats_planned(d_feats, n_src, c_in, d_weights, K, c_out, d_nbr, nullptr, n_dst, d_out, dtype,
                                        d_scale, d_shift, relu, d_stats, d_workspace, workspace_bytes, stream_);
}

extern "C" int rmn_conv_forward_stats_planned(const void* d_feats, uint32_t n_src, int c_in, const void* d_weights,
                                              int K, int c_out, const int32_t* d_nbr, const void* d_plan,
                                              uint32_t n_dst, void* d_out, int dtype, const float* d_scale,
                                              const float* d_shift, int relu, double* d_stats, void* d_workspace,
                                              size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_stats || c_out < 1) return RMN_ERR_BAD_ARG;
  if (n_dst == 0) {
    RMN_CUDA_TRY(cudaMemsetAsync(d_stats, 0, 2 * (size_t)c_out * sizeof(double), stream));
    return RMN_OK;
  }
  if (!d_workspace) return RMN_ERR_BAD_ARG;
  if (workspace_bytes < rmn_channel_stats_workspace_bytes(c_out)) return RMN_ERR_ALLOC;
  if (dtype == RMN_BF16 && n_src > 0 && d_feats && d_weights && d_nbr && d_out && K >= 1) {
    uint32_t n_partials = 0;
    const int st = tc_conv_stats(d_feats, n_src, d_weights, d_nbr, n_dst, K, c_in, c_out, d_out, d_scale, d_shift,
                                 relu, (float*)d_workspace, &n_partials, stream, d_plan);
    if (st == RMN_OK) {
      k_stats_reduce<<<(2 * c_out + 127) / 128, 128, 0, stream>>>((const float*)d_workspace, n_partials, c_out,
                                                                  d_stats);
      RMN_LAUNCH_CHECK();
      return RMN_OK;
    }
    if (st != RMN_ERR_UNSUPPORTED) return st;
  }
  // shapes or dtypes without a tensor-core kernel: convolution, then a statistics pass over its output
  const int st = rmn_conv_forward_fused(d_feats, n_src, c_in, d_weights, K, c_out, d_nbr, n_dst, d_out, dtype, d_scale,
                                        d_shift, relu, stream_);
  if (st != RMN_OK) return st;
  return channel_stats(d_out, n_dst, c_out, dtype, d_stats, (float*)d_workspace, stream);
}

extern "C" int rmn_affine_act(const void* d_x, uint32_t n_rows, int channels, const float* d_scale,
                              const float* d_shift, int relu, void* d_out, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (channels < 1 || (dtype != RMN_F32 && dtype != RMN_BF16)) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_x || !d_out) return RMN_ERR_BAD_ARG;
  const size_t total = (size_t)n_rows * channels;
  if (dtype == RMN_BF16 && channels % 8 == 0 && !((uintptr_t)d_x & 15) && !((uintptr_t)d_out & 15)) {
    const size_t vec = total / 8;
    const size_t blocks = (vec + 255) / 256;
    k_affine_act_bf16x8<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, stream>>>(
        (const uint4*)d_x, vec, channels, d_scale, d_shift, relu, (uint4*)d_out);
  } else {
    const size_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    if (dtype == RMN_F32)
      k_affine_act<float><<<grid, 256, 0, stream>>>((const float*)d_x, total, channels, d_scale, d_shift, relu,
                                                    (float*)d_out);
    else
      k_affine_act<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)d_x, total, channels, d_scale,
                                                            d_shift, relu, (__nv_bfloat16*)d_out);
  }
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}
