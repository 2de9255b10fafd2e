// Local pooling on neighbour tables (sum / average / maximum), forward and backward.
//
// Replaces evaluate_pooling of the reference (engine/nn/pooling.cpp:80-144), which regroups the
// kernel-map pairs by output row on the host and reduces every row with index_select + sum /
// mean / amax. Here an output row reads its K table entries nbr[k][row] and gathers the rows
// they name: one pass over the table and the gathered rows, HBM/L2-bound, no atomics.
//
// Layout: a group of `lanes_per_row` lanes owns one row, each lane a 16-byte vector of channels
// (8 bf16 or 4 fp32), so a row is read with full-line loads; accumulation is fp32. Channel counts
// whose row is not a power-of-two number (<= 32) of 16-byte vectors take the scalar kernels
// (one warp per row, lanes striding over channels).
//
// Auxiliary arrays written by the forward pass for the backward pass:
//   average: count[n_dst]       rows present under each output row
//   maximum: argmax[n_dst][C]   input row that supplied each output value (-1: none)
// The backward pass gathers through the inverse table nbr_in[k][input row] (rmn_kmap_transpose),
// one store per input row.
#include "rmn_common.cuh"

#include <cuda_bf16.h>
#include <float.h>

namespace rmn {

enum { kPoolSum = 0, kPoolAvg = 1, kPoolMax = 2 };

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float* p, float v) { *p = v; }
__device__ __forceinline__ void from_f32(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ------------------------------------------------------------------------------------------
// forward, vector form: grid-stride over groups of rows
// ------------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(256) k_pool_fwd_vec(const T* __restrict__ feats, const int32_t* __restrict__ nbr,
                                                      uint32_t n_dst, int K, int C, int lanes_per_row,
                                                      T* __restrict__ out, int32_t* __restrict__ aux) {
  constexpr int V = Vec16<T>::N;
  const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t lane_in_row = gtid % lanes_per_row;
  const uint32_t rows_per_pass = gridDim.x * blockDim.x / lanes_per_row;
  for (uint32_t row = gtid / lanes_per_row; row < n_dst; row += rows_per_pass) {
    float acc[V];
    int32_t arg[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      acc[i] = MODE == kPoolMax ? -FLT_MAX : 0.f;
      arg[i] = -1;
    }
    int count = 0;
    for (int k = 0; k < K; ++k) {
      const int32_t idx = __ldg(nbr + (size_t)k * n_dst + row);
      if (idx < 0) continue;
      float v[V];
      Vec16<T>::load(feats + (size_t)idx * C + lane_in_row * V, v);
      ++count;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        if (MODE == kPoolMax) {
          if (v[i] > acc[i] || arg[i] < 0) {
            acc[i] = v[i];
            arg[i] = idx;
          }
        } else {
          acc[i] += v[i];
        }
      }
    }
    if (MODE == kPoolAvg && count > 1) {
      const float inv = 1.f / (float)count;
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] *= inv;
    }
    if (MODE == kPoolMax && count == 0) {
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;  // no neighbour at all: zero row, as the reference
    }
    Vec16<T>::store(out + (size_t)row * C + lane_in_row * V, acc);
    if (aux) {
      if (MODE == kPoolAvg && lane_in_row == 0) aux[row] = count;
      if (MODE == kPoolMax) {
#pragma unroll
        for (int i = 0; i < V; ++i) aux[(size_t)row * C + lane_in_row * V + i] = arg[i];
      }
    }
  }
}

// forward, scalar form: one warp per row
template <typename T, int MODE>
__global__ void __launch_bounds__(256) k_pool_fwd_scalar(const T* __restrict__ feats,
                                                         const int32_t* __restrict__ nbr, uint32_t n_dst, int K,
                                                         int C, T* __restrict__ out, int32_t* __restrict__ aux) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  for (uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_dst; row += warps) {
    int count = 0;
    for (int k = 0; k < K; ++k) count += __ldg(nbr + (size_t)k * n_dst + row) >= 0;
    for (int c = lane; c < C; c += 32) {
      float acc = MODE == kPoolMax ? -FLT_MAX : 0.f;
      int32_t arg = -1;
      for (int k = 0; k < K; ++k) {
        const int32_t idx = __ldg(nbr + (size_t)k * n_dst + row);
        if (idx < 0) continue;
        const float v = to_f32(feats[(size_t)idx * C + c]);
        if (MODE == kPoolMax) {
          if (v > acc || arg < 0) {
            acc = v;
            arg = idx;
          }
        } else {
          acc += v;
        }
      }
      if (MODE == kPoolAvg && count > 1) acc /= (float)count;
      if (MODE == kPoolMax && count == 0) acc = 0.f;
      from_f32(out + (size_t)row * C + c, acc);
      if (aux && MODE == kPoolMax) aux[(size_t)row * C + c] = arg;
    }
    if (aux && MODE == kPoolAvg && lane == 0) aux[row] = count;
  }
}

// ------------------------------------------------------------------------------------------
// backward: grad_in[i] = sum over (k, j = nbr_in[k][i]) of the share of grad_out[j] that row i gets
// ------------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(256) k_pool_bwd_vec(const T* __restrict__ grad_out,
                                                      const int32_t* __restrict__ nbr_in, uint32_t n_src, int K,
                                                      int C, int lanes_per_row, const int32_t* __restrict__ aux,
                                                      T* __restrict__ grad_in) {
  constexpr int V = Vec16<T>::N;
  const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t lane_in_row = gtid % lanes_per_row;
  const uint32_t rows_per_pass = gridDim.x * blockDim.x / lanes_per_row;
  for (uint32_t row = gtid / lanes_per_row; row < n_src; row += rows_per_pass) {
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int32_t j = __ldg(nbr_in + (size_t)k * n_src + row);
      if (j < 0) continue;
      float g[V];
      Vec16<T>::load(grad_out + (size_t)j * C + lane_in_row * V, g);
      if (MODE == kPoolSum) {
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += g[i];
      } else if (MODE == kPoolAvg) {
        const int cnt = __ldg(aux + j);
        const float inv = cnt > 1 ? 1.f / (float)cnt : 1.f;
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += g[i] * inv;
      } else {
        const int32_t* a = aux + (size_t)j * C + lane_in_row * V;
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (__ldg(a + i) == (int32_t)row) acc[i] += g[i];
      }
    }
    Vec16<T>::store(grad_in + (size_t)row * C + lane_in_row * V, acc);
  }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) k_pool_bwd_scalar(const T* __restrict__ grad_out,
                                                         const int32_t* __restrict__ nbr_in, uint32_t n_src,
                                                         int K, int C, const int32_t* __restrict__ aux,
                                                         T* __restrict__ grad_in) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  for (uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_src; row += warps) {
    for (int c = lane; c < C; c += 32) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        const int32_t j = __ldg(nbr_in + (size_t)k * n_src + row);
        if (j < 0) continue;
        const float g = to_f32(grad_out[(size_t)j * C + c]);
        if (MODE == kPoolSum) {
          acc += g;
        } else if (MODE == kPoolAvg) {
          const int cnt = __ldg(aux + j);
          acc += cnt > 1 ? g / (float)cnt : g;
        } else if (__ldg(aux + (size_t)j * C + c) == (int32_t)row) {
          acc += g;
        }
      }
      from_f32(grad_in + (size_t)row * C + c, acc);
    }
  }
}

// lanes per row of the vector form, 0 when the channel count does not fit it
template <typename T>
int pool_lanes_per_row(int C, const void* a, const void* b) {
  constexpr int V = Vec16<T>::N;
  if (C % V != 0) return 0;
  const int lanes = C / V;
  if (lanes < 1 || lanes > 32 || (lanes & (lanes - 1)) != 0) return 0;
  if (((uintptr_t)a & 15) || ((uintptr_t)b & 15)) return 0;
  return lanes;
}

inline uint32_t pool_grid(uint64_t threads_needed) {
  const uint64_t blocks = (threads_needed + 255) / 256;
  const uint64_t cap = 148ull * 8ull * 4ull;  // grid-stride beyond a few waves
  return (uint32_t)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T, int MODE>
int pool_forward_t(const void* feats, const int32_t* nbr, uint32_t n_dst, int K, int C, void* out, int32_t* aux,
                   cudaStream_t stream) {
  const int lanes = pool_lanes_per_row<T>(C, feats, out);
  if (lanes > 0) {
    k_pool_fwd_vec<T, MODE><<<pool_grid((uint64_t)n_dst * lanes), 256, 0, stream>>>(
        (const T*)feats, nbr, n_dst, K, C, lanes, (T*)out, aux);
  } else {
    k_pool_fwd_scalar<T, MODE><<<pool_grid((uint64_t)n_dst * 32), 256, 0, stream>>>((const T*)feats, nbr, n_dst, K, C,
                                                                                    (T*)out, aux);
  }
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

template <typename T, int MODE>
int pool_backward_t(const void* grad_out, const int32_t* nbr_in, uint32_t n_src, int K, int C, const int32_t* aux,
                    void* grad_in, cudaStream_t stream) {
  const int lanes = pool_lanes_per_row<T>(C, grad_out, grad_in);
  if (lanes > 0) {
    k_pool_bwd_vec<T, MODE><<<pool_grid((uint64_t)n_src * lanes), 256, 0, stream>>>(
        (const T*)grad_out, nbr_in, n_src, K, C, lanes, aux, (T*)grad_in);
  } else {
    k_pool_bwd_scalar<T, MODE><<<pool_grid((uint64_t)n_src * 32), 256, 0, stream>>>((const T*)grad_out, nbr_in, n_src,
                                                                                    K, C, aux, (T*)grad_in);
  }
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

}  // namespace rmn

using namespace rmn;

extern "C" int rmn_pool_forward(const void* d_feats, uint32_t n_src, int channels, const int32_t* d_nbr, int K,
                                uint32_t n_dst, int mode, void* d_out, int32_t* d_aux, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (channels < 1 || K < 1 || mode < kPoolSum || mode > kPoolMax || (dtype != RMN_F32 && dtype != RMN_BF16))
    return RMN_ERR_BAD_ARG;
  if (n_dst == 0) return RMN_OK;
  if (!d_nbr || !d_out || (n_src > 0 && !d_feats)) return RMN_ERR_BAD_ARG;
#define RMN_POOL_FWD(T)                                                                                    \
  (mode == kPoolSum   ? pool_forward_t<T, kPoolSum>(d_feats, d_nbr, n_dst, K, channels, d_out, d_aux, stream) \
   : mode == kPoolAvg ? pool_forward_t<T, kPoolAvg>(d_feats, d_nbr, n_dst, K, channels, d_out, d_aux, stream) \
                      : pool_forward_t<T, kPoolMax>(d_feats, d_nbr, n_dst, K, channels, d_out, d_aux, stream))
  return dtype == RMN_F32 ? RMN_POOL_FWD(float) : RMN_POOL_FWD(__nv_bfloat16);
#undef RMN_POOL_FWD
}

extern "C" int rmn_pool_backward(const void* d_grad_out, uint32_t n_dst, int channels, const int32_t* d_nbr_in, int K,
                                 uint32_t n_src, int mode, const int32_t* d_aux, void* d_grad_in, int dtype,
                                 void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (channels < 1 || K < 1 || mode < kPoolSum || mode > kPoolMax || (dtype != RMN_F32 && dtype != RMN_BF16))
    return RMN_ERR_BAD_ARG;
  if (mode != kPoolSum && !d_aux && n_dst > 0) return RMN_ERR_BAD_ARG;
  if (n_src == 0) return RMN_OK;
  if (!d_nbr_in || !d_grad_in || (n_dst > 0 && !d_grad_out)) return RMN_ERR_BAD_ARG;
#define RMN_POOL_BWD(T)                                                                                              \
  (mode == kPoolSum   ? pool_backward_t<T, kPoolSum>(d_grad_out, d_nbr_in, n_src, K, channels, d_aux, d_grad_in, stream) \
   : mode == kPoolAvg ? pool_backward_t<T, kPoolAvg>(d_grad_out, d_nbr_in, n_src, K, channels, d_aux, d_grad_in, stream) \
                      : pool_backward_t<T, kPoolMax>(d_grad_out, d_nbr_in, n_src, K, channels, d_aux, d_grad_in, stream))
  return dtype == RMN_F32 ? RMN_POOL_BWD(float) : RMN_POOL_BWD(__nv_bfloat16);
#undef RMN_POOL_BWD
}
