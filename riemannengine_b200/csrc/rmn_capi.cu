// C-ABI entry points of the convolution passes: argument checks and dispatch
// between the tensor-core (tcgen05, bf16) and SIMT (fp32 / odd shapes) kernels.
#include "rmn_common.cuh"

namespace rmn {
int simt_conv_forward(const void* feats, int c_in, const void* w, int K, int c_out,
                      const int32_t* nbr, uint32_t n_dst, void* out, int dtype, const float* ep_scale,
                      const float* ep_shift, int ep_relu, cudaStream_t stream);
int simt_conv_backward_input(const void* grad_out, int c_out, const void* w, int K, int c_in,
                             const int32_t* nbr_t, uint32_t n_src, void* grad_feats, int dtype,
                             cudaStream_t stream);
size_t simt_wgrad_workspace_bytes(uint32_t n_dst, int K, int c_in, int c_out);
int simt_conv_backward_weight(const void* feats, int c_in, const void* grad_out, uint32_t n_dst,
                              int c_out, const int32_t* nbr, int K, float* dw, int dtype,
                              void* workspace, cudaStream_t stream);
int tc_conv(const void* src, uint32_t n_src, const void* w, const int32_t* nbr, uint32_t n_dst, int K, int c_red,
            int c_col, bool transposed_weights, void* out, const float* ep_scale, const float* ep_shift, int ep_relu,
            cudaStream_t stream, const void* plan);
int tc_read_status(cudaStream_t stream, uint32_t* status);
unsigned long long tc_launch_count();
int tc_conv_wgrad(const void* feats, const void* grad_out, const int32_t* nbr, uint32_t n_dst, int K, int c_in,
                  int c_out, float* dw, void* workspace, size_t workspace_bytes, size_t* need,
                  cudaStream_t stream);
}  // namespace rmn

#include <atomic>
#include <cstdlib>

namespace rmn {
static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace rmn

using namespace rmn;

extern "C" unsigned long long rmn_launch_count(void) {
  return g_launches.load(std::memory_order_relaxed);
}

extern "C" unsigned long long rmn_tensor_core_launch_count(void) { return tc_launch_count(); }

extern "C" int rmn_version(void) { return 100; }

extern "C" const char* rmn_status_string(int status) {
  switch (status) {
    case RMN_OK: return "ok";
    case RMN_ERR_BAD_ARG: return "bad argument";
    case RMN_ERR_ALLOC: return "caller-provided buffer too small";
    case RMN_ERR_PROBE_LIMIT: return "hash probe limit reached (table full)";
    case RMN_ERR_TIMEOUT: return "bounded device wait ran out";
    case RMN_ERR_CUDA: return "CUDA runtime error";
    case RMN_ERR_RANGE: return "coordinate bounding box does not pack into 63 bits";
    case RMN_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case RMN_ERR_TOO_LARGE: return "size exceeds the fixed capacity of the allocation-free entry point";
    default: return "unknown status";
  }
}


extern "C" int rmn_device_status(void* stream_) {
  uint32_t st = 0;
  const int rc = tc_read_status((cudaStream_t)stream_, &st);
  return rc != RMN_OK ? rc : (int)st;
}

static bool conv_args_ok(const void* a, const void* w, const int32_t* nbr, const void* out, int K,
                         int c_in, int c_out, int dtype) {
  return a && w && nbr && out && K >= 1 && K <= 65535 && c_in >= 1 && c_out >= 1 &&
         c_in <= 65536 && c_out <= 65536 && (dtype == RMN_F32 || dtype == RMN_BF16);
}

extern "C" int rmn_conv_forward_fused(const void* d_feats, uint32_t n_src, int c_in, const void* d_weights, int K,
                                      int c_out, const int32_t* d_nbr, uint32_t n_dst, void* d_out, int dtype,
                                      const float* d_scale, const float* d_shift, int relu, void* stream_) {
  return rmn_conv_forward_planned(d_feats, n_src, c_in, d_weights, K, c_out, d_nbr, nullptr, n_dst, d_out, dtype,
                                  d_scale, d_shift, relu, stream_);
}

extern "C" int rmn_conv_forward_planned(const void* d_feats, uint32_t n_src, int c_in, const void* d_weights, int K,
                                        int c_out, const int32_t* d_nbr, const void* d_plan, uint32_t n_dst,
                                        void* d_out, int dtype, const float* d_scale, const float* d_shift, int relu,
                                        void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_dst == 0) return RMN_OK;
  if (!conv_args_ok(n_src ? d_feats : d_out, d_weights, d_nbr, d_out, K, c_in, c_out, dtype)) return RMN_ERR_BAD_ARG;
  if (dtype == RMN_BF16 && n_src > 0) {
    const int st = tc_conv(d_feats, n_src, d_weights, d_nbr, n_dst, K, c_in, c_out, false, d_out, d_scale, d_shift,
                           relu, stream, d_plan);
    if (st != RMN_ERR_UNSUPPORTED) return st;
  }
  // (with no source rows every neighbour entry is -1: the SIMT kernel then writes act(shift))
  return simt_conv_forward(d_feats, c_in, d_weights, K, c_out, d_nbr, n_dst, d_out, dtype, d_scale, d_shift, relu,
                           stream);
}

extern "C" int rmn_conv_forward(const void* d_feats, uint32_t n_src, int c_in,
                                const void* d_weights, int K, int c_out, const int32_t* d_nbr,
                                uint32_t n_dst, void* d_out, int dtype, void* stream_) {
  return rmn_conv_forward_fused(d_feats, n_src, c_in, d_weights, K, c_out, d_nbr, n_dst, d_out, dtype, nullptr,
                                nullptr, 0, stream_);
}

extern "C" int rmn_conv_backward_input(const void* d_grad_out, uint32_t n_dst, int c_out,
                                       const void* d_weights, int K, int c_in,
                                       const int32_t* d_nbr_t, uint32_t n_src, void* d_grad_feats,
                                       int dtype, void* stream_) {
  return rmn_conv_backward_input_planned(d_grad_out, n_dst, c_out, d_weights, K, c_in, d_nbr_t, nullptr, n_src,
                                         d_grad_feats, dtype, stream_);
}

extern "C" int rmn_conv_backward_input_planned(const void* d_grad_out, uint32_t n_dst, int c_out,
                                               const void* d_weights, int K, int c_in, const int32_t* d_nbr_t,
                                               const void* d_plan_t, uint32_t n_src, void* d_grad_feats, int dtype,
                                               void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_src == 0) return RMN_OK;
  if (n_dst == 0) {
    if (!d_grad_feats || (dtype != RMN_F32 && dtype != RMN_BF16)) return RMN_ERR_BAD_ARG;
    RMN_CUDA_TRY(cudaMemsetAsync(d_grad_feats, 0, (size_t)n_src * c_in * (dtype == RMN_F32 ? 4 : 2), stream));
    return RMN_OK;
  }
  if (!conv_args_ok(d_grad_out, d_weights, d_nbr_t, d_grad_feats, K, c_in, c_out, dtype))
    return RMN_ERR_BAD_ARG;
  if (dtype == RMN_BF16) {
    const int st = tc_conv(d_grad_out, n_dst, d_weights, d_nbr_t, n_src, K, c_out, c_in, true, d_grad_feats, nullptr, nullptr, 0,
                           stream, d_plan_t);
    if (st != RMN_ERR_UNSUPPORTED) return st;
  }
  return simt_conv_backward_input(d_grad_out, c_out, d_weights, K, c_in, d_nbr_t, n_src,
                                  d_grad_feats, dtype, stream);
}

extern "C" size_t rmn_conv_backward_weight_workspace_bytes(uint32_t n_dst, int K, int c_in,
                                                           int c_out, int dtype) {
  if (K < 1 || c_in < 1 || c_out < 1) return 0;
  size_t need = 0;
  if (dtype == RMN_BF16 &&
      tc_conv_wgrad(nullptr, nullptr, nullptr, n_dst, K, c_in, c_out, nullptr, nullptr, 0, &need, nullptr) == RMN_OK)
    return need;
  return simt_wgrad_workspace_bytes(n_dst, K, c_in, c_out);
}

extern "C" int rmn_conv_backward_weight(const void* d_feats, uint32_t n_src, int c_in,
                                        const void* d_grad_out, uint32_t n_dst, int c_out,
                                        const int32_t* d_nbr, int K, float* d_grad_weights,
                                        int dtype, void* d_workspace, size_t workspace_bytes,
                                        void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_grad_weights || K < 1 || c_in < 1 || c_out < 1) return RMN_ERR_BAD_ARG;
  if (n_dst == 0 || n_src == 0) {
    RMN_CUDA_TRY(cudaMemsetAsync(d_grad_weights, 0, (size_t)K * c_in * c_out * sizeof(float), stream));
    return RMN_OK;
  }
  if (!conv_args_ok(d_feats, d_grad_out, d_nbr, d_grad_weights, K, c_in, c_out, dtype) || !d_workspace)
    return RMN_ERR_BAD_ARG;
  if (workspace_bytes < rmn_conv_backward_weight_workspace_bytes(n_dst, K, c_in, c_out, dtype))
    return RMN_ERR_ALLOC;
  if (dtype == RMN_BF16) {
    size_t need = 0;
    const int st = tc_conv_wgrad(d_feats, d_grad_out, d_nbr, n_dst, K, c_in, c_out, d_grad_weights, d_workspace,
                                 workspace_bytes, &need, stream);
    if (st != RMN_ERR_UNSUPPORTED) return st;
  }
  return simt_conv_backward_weight(d_feats, c_in, d_grad_out, n_dst, c_out, d_nbr, K,
                                   d_grad_weights, dtype, d_workspace, stream);
}
