// SIMT (CUDA-core) sparse convolution over a neighbour table, fp32
// accumulation. This is the exact-arithmetic path: fp32 features (the 1e-4
// parity bar) and any channel count the tensor-core kernels do not take.
//
// All three passes are output-stationary, so there are no atomics and results
// are bit-reproducible:
//   forward         out[j]  = sum_k F[nbr[k][j]]   . W[k]
//   backward input  dF[i]   = sum_k dY[nbr_t[k][i]] . W[k]^T   (same kernel, weight strides swapped)
//   backward weight dW[k]   = sum_j F[nbr[k][j]]^T . dY[j]     (row chunks -> partials -> fixed-order reduce)
#include "rmn_common.cuh"

#include <cuda_bf16.h>

namespace rmn {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16(v);
}

constexpr int TM = 64, TN = 64, TK = 16;

// out[j, n] = sum_k sum_r src[nbr[k][j], r] * w[k*ws_k + r*ws_red + n*ws_col]
template <typename T>
__global__ void __launch_bounds__(256) k_conv_gather_gemm(
    const T* __restrict__ src, const T* __restrict__ w, const int32_t* __restrict__ nbr,
    uint32_t n_dst, int K, int c_red, int c_col, long long ws_k, int ws_red, int ws_col,
    T* __restrict__ out, const float* __restrict__ ep_scale, const float* __restrict__ ep_shift, int ep_relu) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  __shared__ int32_t s_idx[TM];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const uint32_t row0 = blockIdx.x * TM;
  const int n0 = blockIdx.y * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k = 0; k < K; ++k) {
    int32_t my = -1;
    if (tid < TM && row0 + tid < n_dst) my = __ldg(nbr + (size_t)k * n_dst + row0 + tid);
    __syncthreads();  // previous iteration finished with s_idx / As / Bs
    if (tid < TM) s_idx[tid] = my;
    if (!__syncthreads_or(my >= 0)) continue;
    for (int c0 = 0; c0 < c_red; c0 += TK) {
      {
        const int r = tid >> 2, cc = (tid & 3) * 4;
        const int32_t idx = s_idx[r];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + cc + j;
          float v = 0.f;
          if (idx >= 0 && c < c_red) v = to_f32<T>(src[(size_t)idx * c_red + c]);
          As[cc + j][r] = v;
        }
      }
      {
        const int kk = tid >> 4, nn = (tid & 15) * 4;
        const int r = c0 + kk;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + nn + j;
          float v = 0.f;
          if (r < c_red && n < c_col) v = to_f32<T>(w[k * ws_k + (long long)r * ws_red + (long long)n * ws_col]);
          Bs[kk][nn + j] = v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t row = row0 + ty * 4 + i;
    if (row >= n_dst) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < c_col) {
        // fused epilogue: out = act(acc * scale + shift)
        float f = acc[i][j];
        if (ep_scale) f *= __ldg(ep_scale + n);
        if (ep_shift) f += __ldg(ep_shift + n);
        if (ep_relu) f = fmaxf(f, 0.f);
        out[(size_t)row * c_col + n] = from_f32<T>(f);
      }
    }
  }
}

// partial[chunk][k][ci][co] = sum over rows j of the chunk: F[nbr[k][j]][ci] * dY[j][co]
template <typename T>
__global__ void __launch_bounds__(256) k_conv_wgrad_partial(
    const T* __restrict__ feats, const T* __restrict__ grad_out, const int32_t* __restrict__ nbr,
    uint32_t n_dst, int K, int c_in, int c_out, uint32_t chunk_rows, int tiles_co,
    float* __restrict__ partial) {
  __shared__ float As[TK][TM + 4];  // [row][ci]
  __shared__ float Bs[TK][TN + 4];  // [row][co]
  __shared__ int32_t s_idx[TK];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int k = blockIdx.y;
  const int ci0 = (blockIdx.z / tiles_co) * TM, co0 = (blockIdx.z % tiles_co) * TN;
  const uint32_t j_begin = blockIdx.x * chunk_rows;
  const uint32_t j_end = min(n_dst, j_begin + chunk_rows);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (uint32_t j0 = j_begin; j0 < j_end; j0 += TK) {
    int32_t my = -1;
    if (tid < TK && j0 + tid < j_end) my = __ldg(nbr + (size_t)k * n_dst + j0 + tid);
    __syncthreads();
    if (tid < TK) s_idx[tid] = my;
    if (!__syncthreads_or(my >= 0)) continue;
    {
      const int r = tid >> 4, cc = (tid & 15) * 4;
      const int32_t idx = s_idx[r];
      const uint32_t j = j0 + r;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int ci = ci0 + cc + q, co = co0 + cc + q;
        float a = 0.f, b = 0.f;
        if (idx >= 0) {
          if (ci < c_in) a = to_f32<T>(feats[(size_t)idx * c_in + ci]);
          if (co < c_out) b = to_f32<T>(grad_out[(size_t)j * c_out + co]);
        }
        As[r][cc + q] = a;
        Bs[r][cc + q] = b;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
  float* dst = partial + ((size_t)blockIdx.x * K + k) * c_in * c_out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ci = ci0 + ty * 4 + i;
    if (ci >= c_in) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int co = co0 + tx * 4 + j;
      if (co < c_out) dst[(size_t)ci * c_out + co] = acc[i][j];
    }
  }
}

__global__ void __launch_bounds__(256) k_reduce_partials(const float* __restrict__ partial,
                                                         uint32_t n_chunks, size_t elems,
                                                         float* __restrict__ out) {
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= elems) return;
  float s = 0.f;
  for (uint32_t c = 0; c < n_chunks; ++c) s += partial[(size_t)c * elems + e];
  out[e] = s;
}

inline uint32_t wgrad_chunk_rows(uint32_t n_dst) {
  // about 64 chunks, each a multiple of TK rows and at least 1024 rows
  uint32_t rows = (n_dst + 63) / 64;
  if (rows < 1024) rows = 1024;
  return (rows + TK - 1) / TK * TK;
}
inline uint32_t wgrad_chunks(uint32_t n_dst) {
  const uint32_t cr = wgrad_chunk_rows(n_dst);
  return n_dst == 0 ? 1 : (n_dst + cr - 1) / cr;
}

template <typename T>
int launch_gather_gemm(const void* src, const void* w, const int32_t* nbr, uint32_t n_dst, int K,
                       int c_red, int c_col, long long ws_k, int ws_red, int ws_col, void* out,
                       const float* ep_scale, const float* ep_shift, int ep_relu, cudaStream_t stream) {
  dim3 grid((n_dst + TM - 1) / TM, (c_col + TN - 1) / TN);
  k_conv_gather_gemm<T><<<grid, 256, 0, stream>>>((const T*)src, (const T*)w, nbr, n_dst, K, c_red,
                                                  c_col, ws_k, ws_red, ws_col, (T*)out, ep_scale, ep_shift, ep_relu);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

int simt_conv_forward(const void* feats, int c_in, const void* w, int K, int c_out,
                      const int32_t* nbr, uint32_t n_dst, void* out, int dtype, const float* ep_scale,
                      const float* ep_shift, int ep_relu, cudaStream_t stream) {
  const long long ws_k = (long long)c_in * c_out;
  if (dtype == RMN_F32)
    return launch_gather_gemm<float>(feats, w, nbr, n_dst, K, c_in, c_out, ws_k, c_out, 1, out, ep_scale, ep_shift,
                                     ep_relu, stream);
  return launch_gather_gemm<__nv_bfloat16>(feats, w, nbr, n_dst, K, c_in, c_out, ws_k, c_out, 1, out, ep_scale,
                                           ep_shift, ep_relu, stream);
}

int simt_conv_backward_input(const void* grad_out, int c_out, const void* w, int K, int c_in,
                             const int32_t* nbr_t, uint32_t n_src, void* grad_feats, int dtype,
                             cudaStream_t stream) {
  const long long ws_k = (long long)c_in * c_out;
  if (dtype == RMN_F32)
    return launch_gather_gemm<float>(grad_out, w, nbr_t, n_src, K, c_out, c_in, ws_k, 1, c_out, grad_feats, nullptr,
                                     nullptr, 0, stream);
  return launch_gather_gemm<__nv_bfloat16>(grad_out, w, nbr_t, n_src, K, c_out, c_in, ws_k, 1, c_out, grad_feats,
                                           nullptr, nullptr, 0, stream);
}

size_t simt_wgrad_workspace_bytes(uint32_t n_dst, int K, int c_in, int c_out) {
  return (size_t)wgrad_chunks(n_dst) * K * c_in * c_out * sizeof(float);
}

template <typename T>
int launch_wgrad(const void* feats, const void* grad_out, const int32_t* nbr, uint32_t n_dst, int K,
                 int c_in, int c_out, float* dw, float* partial, cudaStream_t stream) {
  const uint32_t chunks = wgrad_chunks(n_dst), chunk_rows = wgrad_chunk_rows(n_dst);
  const int tiles_ci = (c_in + TM - 1) / TM, tiles_co = (c_out + TN - 1) / TN;
  dim3 grid(chunks, K, tiles_ci * tiles_co);
  k_conv_wgrad_partial<T><<<grid, 256, 0, stream>>>((const T*)feats, (const T*)grad_out, nbr, n_dst,
                                                    K, c_in, c_out, chunk_rows, tiles_co, partial);
  RMN_LAUNCH_CHECK();
  const size_t elems = (size_t)K * c_in * c_out;
  k_reduce_partials<<<(uint32_t)((elems + 255) / 256), 256, 0, stream>>>(partial, chunks, elems, dw);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

int simt_conv_backward_weight(const void* feats, int c_in, const void* grad_out, uint32_t n_dst,
                              int c_out, const int32_t* nbr, int K, float* dw, int dtype,
                              void* workspace, cudaStream_t stream) {
  if (dtype == RMN_F32)
    return launch_wgrad<float>(feats, grad_out, nbr, n_dst, K, c_in, c_out, dw, (float*)workspace, stream);
  return launch_wgrad<__nv_bfloat16>(feats, grad_out, nbr, n_dst, K, c_in, c_out, dw, (float*)workspace, stream);
}

}  // namespace rmn
