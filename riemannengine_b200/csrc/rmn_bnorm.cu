// Training-mode batch normalisation of a feature matrix [N, C] as streaming passes at memory speed:
//   forward : per-channel sums (one read), coefficients (one tiny kernel), y = x * scale + shift (one read + write)
//   backward: per-channel sums of dy and dy * x (one read of both), coefficients, dx = a * dy + b * x + c
// The reference normalises with torch::nn::BatchNorm1d on the feature matrix after every convolution
// (engine/nn/normalization.hpp:11-34); in an encoder/decoder that is as many passes over [N, C] as the
// convolutions make, and torch's channels-last kernels run them at a fraction of memory speed for the narrow
// matrices of sparse networks (32 - 256 channels, millions of rows).
#include "rmn_common.cuh"

#include <cuda_bf16.h>

namespace rmn {

constexpr uint32_t kDotPartials = 148 * 4;  // blocks of the reduction = per-channel partial sums

template <typename T>
struct Vec16;  // sixteen bytes of T as floats
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// partial[block][0][c] = sum over the block's rows of a[r][c], partial[block][1][c] = sum of a[r][c] * b[r][c].
// A row is C / VEC lanes of 16 bytes; LPR = lanes per row divides 32, a warp reads 32 / LPR rows per step
// (whole 128-byte lines), every lane keeps its VEC channels in registers, and the lanes, warps and blocks are
// combined in a fixed order (deterministic).
template <typename T>
__global__ void __launch_bounds__(256) k_channel_dot_partial(const T* __restrict__ a, const T* __restrict__ b,
                                                             uint32_t n, int C, float* __restrict__ partial) {
  constexpr int VEC = Vec16<T>::N;
  extern __shared__ float s_part[];  // [8 warps][2][C]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lpr = C / VEC, rows_per_step = 32 / lpr;
  const int g = lane % lpr, sub = lane / lpr;
  float sa[VEC], sab[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) sa[i] = sab[i] = 0.f;
  const uint32_t warps = gridDim.x * 8u;
  for (uint32_t r = (blockIdx.x * 8u + warp) * rows_per_step + sub; r < n; r += warps * rows_per_step) {
    float va[VEC], vb[VEC];
    Vec16<T>::load(a + (size_t)r * C + g * VEC, va);
    Vec16<T>::load(b + (size_t)r * C + g * VEC, vb);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      sa[i] += va[i];
      sab[i] = fmaf(va[i], vb[i], sab[i]);
    }
  }
  // lanes that hold the same channels (same g): xor offsets lpr, 2 lpr, ... < 32
  for (int d = lpr; d < 32; d <<= 1) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      sa[i] += __shfl_xor_sync(0xFFFFFFFFu, sa[i], d);
      sab[i] += __shfl_xor_sync(0xFFFFFFFFu, sab[i], d);
    }
  }
  if (sub == 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      s_part[(warp * 2 + 0) * C + g * VEC + i] = sa[i];
      s_part[(warp * 2 + 1) * C + g * VEC + i] = sab[i];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * C; c += 256) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += s_part[w * 2 * C + c];
    partial[(size_t)blockIdx.x * 2 * C + c] = t;
  }
}

// stats[2][C] (double) = sum over the partials: one warp per output, lanes stride over the partials and are
// combined by a fixed butterfly (deterministic; a serial loop of ~600 dependent loads per output cost more than
// the statistics pass itself)
__global__ void __launch_bounds__(256) k_dot_reduce(const float* __restrict__ partial, uint32_t n_partials, int C,
                                                    double* __restrict__ stats) {
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= 2 * C) return;
  double t = 0.0;
  for (uint32_t p = lane; p < n_partials; p += 32) t += (double)partial[(size_t)p * 2 * C + i];
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, d);
  if (lane == 0) stats[i] = t;
}

__device__ __forceinline__ float ld_param(const void* p, int i, int dtype) {
  return dtype == RMN_F32 ? reinterpret_cast<const float*>(p)[i]
                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_param(void* p, int i, int dtype, float v) {
  if (dtype == RMN_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// From the sums of a batch (stats[0] = sum x, stats[1] = sum x^2 over `count` rows): mean, 1 / sqrt(var + eps),
// the affine y = x * scale + shift that normalises and applies gamma / beta, and the running statistics
// (momentum m: new = (1 - m) * old + m * batch, the variance unbiased) - torch.nn.BatchNorm1d's rules.
__global__ void k_bn_forward_coeffs(const double* __restrict__ stats, double count, const void* gamma, const void* beta,
                                    void* running_mean, void* running_var, int param_dtype, float momentum, float eps,
                                    int C, float* __restrict__ scale, float* __restrict__ shift,
                                    float* __restrict__ mean_out, float* __restrict__ inv_out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const double n = count > 0.0 ? count : 1.0;
  const double mean = stats[c] / n;
  double var = stats[C + c] / n - mean * mean;
  if (var < 0.0) var = 0.0;
  const float inv = (float)(1.0 / sqrt(var + (double)eps));
  const float g = gamma ? ld_param(gamma, c, param_dtype) : 1.f;
  const float b = beta ? ld_param(beta, c, param_dtype) : 0.f;
  scale[c] = g * inv;
  shift[c] = b - (float)mean * g * inv;
  mean_out[c] = (float)mean;
  inv_out[c] = inv;
  if (running_mean) st_param(running_mean, c, param_dtype, (1.f - momentum) * ld_param(running_mean, c, param_dtype) + momentum * (float)mean);
  if (running_var) {
    const double unbiased = n > 1.0 ? var * n / (n - 1.0) : var;
    st_param(running_var, c, param_dtype, (1.f - momentum) * ld_param(running_var, c, param_dtype) + momentum * (float)unbiased);
  }
}

// From dots[0] = sum dy, dots[1] = sum dy * x: the gradients of gamma and beta and the coefficients of
//   dx = c_dy * dy + c_x * x + c_0      (x_hat = (x - mean) * inv;  dx = gamma * inv * (dy - mean(dy) - x_hat * mean(dy * x_hat)))
__global__ void k_bn_backward_coeffs(const double* __restrict__ dots, const float* __restrict__ mean,
                                     const float* __restrict__ inv, const void* gamma, int param_dtype, double count,
                                     int C, float* __restrict__ c_dy, float* __restrict__ c_x, float* __restrict__ c_0,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const double n = count > 0.0 ? count : 1.0;
  const double m = mean[c], iv = inv[c];
  const double s_dy = dots[c];
  const double s_dyxh = (dots[C + c] - m * s_dy) * iv;  // sum dy * x_hat
  const double g = gamma ? (double)ld_param(gamma, c, param_dtype) : 1.0;
  dgamma[c] = (float)s_dyxh;
  dbeta[c] = (float)s_dy;
  const double k = g * iv;
  const double kx = -k * iv * s_dyxh / n;   // multiplies (x - mean)
  c_dy[c] = (float)k;
  c_x[c] = (float)kx;
  c_0[c] = (float)(-k * s_dy / n - kx * m);
}

// out = c_a[c] * a + c_b[c] * b + c_0[c], sixteen bytes per thread
template <typename T>
__global__ void __launch_bounds__(256) k_affine2(const T* __restrict__ a, const T* __restrict__ b, size_t total_vec, int C,
                                                 const float* __restrict__ c_a, const float* __restrict__ c_b,
                                                 const float* __restrict__ c_0, T* __restrict__ out) {
  constexpr int VEC = Vec16<T>::N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (size_t)gridDim.x * blockDim.x) {
    const int c0 = (int)((i * VEC) % (size_t)C);
    float va[VEC], vb[VEC], o[VEC];
    Vec16<T>::load(a + i * VEC, va);
    Vec16<T>::load(b + i * VEC, vb);
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      o[j] = fmaf(__ldg(c_a + c0 + j), va[j], fmaf(__ldg(c_b + c0 + j), vb[j], __ldg(c_0 + c0 + j)));
    Vec16<T>::store(out + i * VEC, o);
  }
}

template <typename T>
static bool dot_fast_shape(int C) {
  constexpr int VEC = Vec16<T>::N;
  if (C % VEC) return false;
  const int lpr = C / VEC;
  return lpr >= 1 && lpr <= 32 && (32 % lpr) == 0;
}

}  // namespace rmn

using namespace rmn;

extern "C" size_t rmn_channel_dot_stats_workspace_bytes(int channels) {
  return channels < 1 ? 0 : (size_t)kDotPartials * 2 * (size_t)channels * sizeof(float);
}

extern "C" int rmn_channel_dot_stats(const void* d_a, const void* d_b, uint32_t n_rows, int channels, int dtype,
                                     double* d_stats, void* d_workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_stats || channels < 1 || (dtype != RMN_F32 && dtype != RMN_BF16)) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) {
    RMN_CUDA_TRY(cudaMemsetAsync(d_stats, 0, 2 * (size_t)channels * sizeof(double), stream));
    return RMN_OK;
  }
  if (!d_a || !d_b || !d_workspace) return RMN_ERR_BAD_ARG;
  if (workspace_bytes < rmn_channel_dot_stats_workspace_bytes(channels)) return RMN_ERR_ALLOC;
  if (((uintptr_t)d_a & 15) || ((uintptr_t)d_b & 15)) return RMN_ERR_UNSUPPORTED;
  const bool ok = dtype == RMN_F32 ? dot_fast_shape<float>(channels) : dot_fast_shape<__nv_bfloat16>(channels);
  if (!ok) return RMN_ERR_UNSUPPORTED;
  float* partial = static_cast<float*>(d_workspace);
  const int vec = dtype == RMN_F32 ? 4 : 8;
  const uint32_t rows_per_block = 8u * (uint32_t)(32 / (channels / vec));
  uint32_t blocks = (n_rows + rows_per_block - 1) / rows_per_block;
  if (blocks > kDotPartials) blocks = kDotPartials;
  const size_t smem = (size_t)8 * 2 * channels * sizeof(float);
  if (dtype == RMN_F32)
    k_channel_dot_partial<float><<<blocks, 256, smem, stream>>>((const float*)d_a, (const float*)d_b, n_rows, channels,
                                                                partial);
  else
    k_channel_dot_partial<__nv_bfloat16><<<blocks, 256, smem, stream>>>((const __nv_bfloat16*)d_a,
                                                                        (const __nv_bfloat16*)d_b, n_rows, channels,
                                                                        partial);
  RMN_LAUNCH_CHECK();
  k_dot_reduce<<<(2 * channels + 7) / 8, 256, 0, stream>>>(partial, blocks, channels, d_stats);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_bn_forward_coeffs(const double* d_stats, double count, const void* d_gamma, const void* d_beta,
                                     void* d_running_mean, void* d_running_var, int param_dtype, float momentum,
                                     float eps, int channels, float* d_scale, float* d_shift, float* d_mean,
                                     float* d_inv, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_stats || !d_scale || !d_shift || !d_mean || !d_inv || channels < 1 ||
      (param_dtype != RMN_F32 && param_dtype != RMN_BF16))
    return RMN_ERR_BAD_ARG;
  k_bn_forward_coeffs<<<(channels + 127) / 128, 128, 0, stream>>>(d_stats, count, d_gamma, d_beta, d_running_mean,
                                                                  d_running_var, param_dtype, momentum, eps, channels,
                                                                  d_scale, d_shift, d_mean, d_inv);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_bn_backward_coeffs(const double* d_dots, const float* d_mean, const float* d_inv,
                                      const void* d_gamma, int param_dtype, double count, int channels, float* d_c_dy,
                                      float* d_c_x, float* d_c_0, float* d_dgamma, float* d_dbeta, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_dots || !d_mean || !d_inv || !d_c_dy || !d_c_x || !d_c_0 || !d_dgamma || !d_dbeta || channels < 1 ||
      (param_dtype != RMN_F32 && param_dtype != RMN_BF16))
    return RMN_ERR_BAD_ARG;
  k_bn_backward_coeffs<<<(channels + 127) / 128, 128, 0, stream>>>(d_dots, d_mean, d_inv, d_gamma, param_dtype, count,
                                                                   channels, d_c_dy, d_c_x, d_c_0, d_dgamma, d_dbeta);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_affine2(const void* d_a, const void* d_b, uint32_t n_rows, int channels, const float* d_c_a,
                           const float* d_c_b, const float* d_c_0, void* d_out, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (channels < 1 || (dtype != RMN_F32 && dtype != RMN_BF16) || !d_c_a || !d_c_b || !d_c_0) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_a || !d_b || !d_out) return RMN_ERR_BAD_ARG;
  const int vec = dtype == RMN_F32 ? 4 : 8;
  if (channels % vec || ((uintptr_t)d_a & 15) || ((uintptr_t)d_b & 15) || ((uintptr_t)d_out & 15))
    return RMN_ERR_UNSUPPORTED;
  const size_t total_vec = (size_t)n_rows * channels / vec;
  const size_t blocks = (total_vec + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  if (dtype == RMN_F32)
    k_affine2<float><<<grid, 256, 0, stream>>>((const float*)d_a, (const float*)d_b, total_vec, channels, d_c_a, d_c_b,
                                               d_c_0, (float*)d_out);
  else
    k_affine2<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)d_a, (const __nv_bfloat16*)d_b, total_vec,
                                                       channels, d_c_a, d_c_b, d_c_0, (__nv_bfloat16*)d_out);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}
