// riemann_cpp (B200): C++20 / LibTorch host layer of the sparse-convolution hot path.
//
// Same names, constructor argument order, defaults and exception behaviour as
// the reference's public classes, so that networks written against the
// reference compile unchanged:
//   CoordinateMapKey                 engine/grid/key.hpp:18-99
//   CoordinateManager                engine/grid/space.hpp:817-906
//   SparseTensor                     engine/tensor/sparse_tensor.hpp:16-80
//   KernelGenerator                  engine/grid/stencil.hpp:533-598
//   RiemannConvolution{,Transpose,GenerativeTranspose} (TORCH_MODULE)
//                                    engine/nn/conv.hpp:13-90
//   ConvolutionFunction / ConvolutionTransposeFunction
//                                    autodiff/compat.hpp:86-156
// Every coordinate and convolution operation is one or more calls into the C
// ABI of librmn_b200.so (include/rmn_b200.h) on the current CUDA stream; there
// is no CPU backend.
#pragma once

#include <torch/torch.h>

#include <map>
#include <memory>
#include <optional>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

namespace riemann {

using stride_type = std::vector<uint32_t>;
using size_type = uint32_t;
using coordinate_map_key_type = std::pair<stride_type, std::string>;

namespace SparseTensorQuantizationMode {
enum Type { RANDOM_SUBSAMPLE = 0, UNWEIGHTED_AVERAGE = 1, UNWEIGHTED_SUM = 2, MAX_POOL = 3, NO_QUANTIZATION = 4 };
}
namespace GPUMemoryAllocatorBackend {
enum Type { PYTORCH = 0, CUDA = 1 };
}
namespace RiemannAlgorithm {
enum Mode { DEFAULT = 0, MEMORY_EFFICIENT = 1, SPEED_OPTIMIZED = 2 };
}
namespace CoordinateMapBackend {
enum Type { CPU = 0, CUDA = 1 };
}
namespace RegionType {
enum Type { HYPER_CUBE, HYPER_CROSS, CUSTOM };
}
namespace ConvolutionMode {
enum Type { DEFAULT, DIRECT_GEMM, COPY_GEMM };
}
namespace PoolingMode {  // engine/foundation/types.hpp:121-136
enum Type {
  LOCAL_SUM_POOLING,
  LOCAL_AVG_POOLING,
  LOCAL_MAX_POOLING,
  GLOBAL_SUM_POOLING_DEFAULT,
  GLOBAL_AVG_POOLING_DEFAULT,
  GLOBAL_MAX_POOLING_DEFAULT,
  GLOBAL_SUM_POOLING_KERNEL,
  GLOBAL_AVG_POOLING_KERNEL,
  GLOBAL_MAX_POOLING_KERNEL,
  GLOBAL_SUM_POOLING_PYTORCH_INDEX,
  GLOBAL_AVG_POOLING_PYTORCH_INDEX,
  GLOBAL_MAX_POOLING_PYTORCH_INDEX
};
}

class CoordinateMapKey {
public:
  CoordinateMapKey() = delete;
  explicit CoordinateMapKey(size_type coordinate_size) : m_key_set(false), m_coordinate_size(coordinate_size) {}
  CoordinateMapKey(size_type coordinate_size, coordinate_map_key_type const& key);
  CoordinateMapKey(stride_type tensor_stride, std::string string_id = "");

  size_type get_coordinate_size() const { return m_coordinate_size; }
  void set_key(stride_type tensor_stride, std::string string_id);
  void set_key(coordinate_map_key_type const& key);
  coordinate_map_key_type get_key() const;
  uint64_t hash() const;
  bool is_key_set() const noexcept { return m_key_set; }
  stride_type get_tensor_stride() const { return m_key.first; }
  bool operator==(CoordinateMapKey const& key) const;
  std::string to_string() const;

private:
  bool m_key_set;
  size_type m_coordinate_size;
  coordinate_map_key_type m_key;
};

// One cached kernel map. nbr_out [K, N_out] holds the input row (or -1) of every (offset,
// output row); nbr_in [K, N_in] is its inverse, built on first use. The pair lists are the
// reference's representation (engine/grid/maps.hpp:19-79).
struct KernelMap {
  at::Tensor nbr_out;
  int64_t n_in = 0, n_out = 0;
  at::Tensor offset_ptr;  // int64 [K+1] device, of the probe that produced nbr_out (undefined on a swapped view)
  at::Tensor workspace;
  // offset_ptr copied to pinned host memory right after the probe, and the event after that copy:
  // by the time pair lists are asked for, the sizes are on the host without draining the stream
  at::Tensor host_offset_ptr;
  std::optional<c10::Event> offset_ptr_ready;
  std::shared_ptr<KernelMap> parent;  // set on a swapped view
  // stride-1 self map with a point-symmetric region: nbr_in[k] == nbr_out[K-1-k], so the input
  // gradient reuses nbr_out with the kernel flipped along its offset axis
  bool self_symmetric = false;

  at::Tensor const& nbr_in();
  // Host copy of the region offsets [K, D] the table was probed with (steers the row grouping of the plans)
  std::vector<int32_t> region_offsets;
  // Convolution plan (rmn_conv_plan_build) of nbr_out / of nbr_in, or an undefined tensor when the policy says
  // "not yet": a plan costs about two passes over the table, so under PlanPolicy::AUTO it is built by the pass
  // that brings the work done on the table (sum of c_in * c_out of the passes) to the point where the plan
  // repays itself. `weight` is c_in * c_out of the calling layer.
  at::Tensor plan_out(int64_t weight);
  at::Tensor plan_in(int64_t weight);
  // (offset_ptr on the host, in rows, out rows)
  std::tuple<at::Tensor, at::Tensor, at::Tensor> const& pairs();
  std::shared_ptr<KernelMap> swapped(std::shared_ptr<KernelMap> const& self);

private:
  at::Tensor build_plan(const at::Tensor& table, bool negate_offsets);
  at::Tensor nbr_in_, plan_out_, plan_in_;
  int64_t weight_out_ = 0, weight_in_ = 0;  // sum of c_in * c_out over the passes made on each table
  bool have_pairs_ = false;
  std::tuple<at::Tensor, at::Tensor, at::Tensor> pairs_;
};

// When a kernel map gets a convolution plan (see KernelMap::plan_out). No counterpart in the reference.
namespace PlanPolicy {
enum Type { AUTO = 0, ALWAYS = 1, NEVER = 2 };
}
void set_convolution_plan_policy(PlanPolicy::Type policy);
PlanPolicy::Type convolution_plan_policy();

// Data-parallel training: batches shard by sample over the ranks (one process per GPU) and the only
// collective is the sum of the weight gradients, done by rmn_allreduce_grads (NCCL over NVLink). The
// reference has no distributed code. Usage: rank 0 calls gradient_allreduce_unique_id() and sends the
// 128 bytes to the other ranks (for instance through the torch.distributed store); every rank then calls
// init_gradient_allreduce with its CUDA device current. From then on the backward pass of every
// convolution layer reduces its weight (and bias) gradient as soon as the weight-gradient kernel has
// finished, on a second stream, while the input-gradient kernel of the same layer runs: the gradients
// autograd hands on are already the sum (average = false) or the mean over the ranks.
std::string gradient_allreduce_unique_id();
void init_gradient_allreduce(const std::string& unique_id, int rank, int world_size, bool average = true);
void shutdown_gradient_allreduce();
bool gradient_allreduce_active();
int gradient_allreduce_world_size();
// In-place reduction of fp32 CUDA tensors as ONE flat bucket on the current stream (what the layers call).
void allreduce_gradients(const std::vector<at::Tensor>& gradients);

class CoordinateManager {
public:
  CoordinateManager(int D, CoordinateMapBackend::Type map_type = CoordinateMapBackend::CUDA,
                    GPUMemoryAllocatorBackend::Type alloc_type = GPUMemoryAllocatorBackend::PYTORCH,
                    RiemannAlgorithm::Mode algo = RiemannAlgorithm::DEFAULT);

  std::pair<CoordinateMapKey, std::pair<at::Tensor, at::Tensor>>
  insert_and_map(const at::Tensor& coordinates, stride_type tensor_stride, std::string string_id = "");

  CoordinateMapKey stride(const CoordinateMapKey& in_key, const stride_type& kernel_stride,
                          std::string string_id = "");
  // The origin map (engine/grid/space.hpp:817-906 `origin`, space_impl.hpp:383-421, lattice_cpu.hpp:539-558): one
  // row per batch index present in the manager's maps, spatial columns zero, tensor stride all zeros, key
  // (zeros, ""). Returns the key and whether the map was created by this call. Rows are numbered by first
  // occurrence of the batch index in the seed map (the reference numbers them in hash-iteration order).
  std::pair<CoordinateMapKey, bool> origin();
  // Union of maps of one tensor stride (engine/grid/space.hpp:862-863, space_impl.hpp:896-914): sets out_key to the
  // merged map and returns one int64 [2, N_i] tensor per input map (row in that map, row in the merged map).
  std::vector<at::Tensor> union_map(const std::vector<CoordinateMapKey>& in_keys, CoordinateMapKey& out_key);
  // New map holding every `in + offset` of a transposed region on out_tensor_stride
  // (engine/grid/lattice_cpu.hpp:499-534 through space_impl.hpp:359-381): pooling-transpose's coordinates.
  CoordinateMapKey stride_region(const CoordinateMapKey& in_key, const stride_type& kernel_size,
                                 const stride_type& kernel_dilation, const stride_type& out_tensor_stride,
                                 RegionType::Type region_type = RegionType::HYPER_CUBE,
                                 const at::Tensor& offsets = at::Tensor());

  // Continuous coordinates (float32 [N, 1 + D]) under a field key (engine/grid/space_impl.hpp:36-80), and their
  // voxelisation at a tensor stride into a new sparse map: (sparse key, (first rows, field row -> sparse row))
  // (engine/grid/space_impl.hpp:103-166).
  CoordinateMapKey insert_field(const at::Tensor& coordinates, stride_type tensor_stride, std::string string_id = "");
  std::pair<CoordinateMapKey, std::pair<at::Tensor, at::Tensor>>
  field_to_sparse_insert_and_map(const CoordinateMapKey& field_key, stride_type sparse_tensor_stride,
                                 std::string sparse_tensor_string_id = "");
  at::Tensor get_field_coordinates(const CoordinateMapKey& field_key) const;

  at::Tensor get_coordinates(const CoordinateMapKey& key) const;
  uint32_t size(const CoordinateMapKey& key) const;
  bool exists(const CoordinateMapKey& key) const;

  // Cached kernel map (engine/grid/space_impl.hpp:499-706).
  std::shared_ptr<KernelMap> kernel_map(const CoordinateMapKey& in_key, const CoordinateMapKey& out_key,
                                        const stride_type& kernel_size, const stride_type& kernel_stride,
                                        const stride_type& kernel_dilation, RegionType::Type region_type,
                                        const at::Tensor& offsets, bool is_transpose, bool is_pool);
  // {offset index -> int32 [2, P_k]} (engine/grid/space.cpp:202-228)
  std::map<int64_t, at::Tensor> kernel_map_th(const CoordinateMapKey& in_key, const CoordinateMapKey& out_key,
                                              const stride_type& kernel_size, const stride_type& kernel_stride,
                                              const stride_type& kernel_dilation, RegionType::Type region_type,
                                              const at::Tensor& offsets, bool is_transpose, bool is_pool);

  int D() const { return D_; }
  CoordinateMapBackend::Type backend() const { return map_type_; }

private:
  struct Map {
    at::Tensor table;   // uint8, device
    at::Tensor coords;  // int32 [n, W]
    stride_type tensor_stride;
    uint32_t size = 0;
  };
  Map const& find(const CoordinateMapKey& key, const char* what = "") const;
  Map build(const at::Tensor& coords, const stride_type& tensor_stride, at::Tensor* mapping, at::Tensor* inverse);

  int D_;
  CoordinateMapBackend::Type map_type_;
  std::map<coordinate_map_key_type, Map> maps_;
  std::map<std::string, std::shared_ptr<KernelMap>> kernel_maps_;
  std::map<coordinate_map_key_type, at::Tensor> fields_;
};

class SparseTensor {
public:
  SparseTensor(at::Tensor features, at::Tensor coordinates, std::shared_ptr<CoordinateManager> manager = nullptr,
               SparseTensorQuantizationMode::Type quantization_mode = SparseTensorQuantizationMode::RANDOM_SUBSAMPLE,
               GPUMemoryAllocatorBackend::Type alloc_type = GPUMemoryAllocatorBackend::PYTORCH,
               RiemannAlgorithm::Mode algo = RiemannAlgorithm::DEFAULT);
  SparseTensor(at::Tensor features, CoordinateMapKey coordinate_map_key, std::shared_ptr<CoordinateManager> manager);

  const at::Tensor& F() const noexcept { return features_; }
  at::Tensor C() const;
  const CoordinateMapKey& coordinate_map_key() const noexcept { return key_; }
  std::shared_ptr<CoordinateManager> coordinate_manager() const noexcept { return manager_; }
  stride_type tensor_stride() const { return key_.get_tensor_stride(); }
  int dimension() const noexcept { return dimension_; }
  torch::Device device() const { return features_.device(); }
  c10::ScalarType dtype() const { return features_.scalar_type(); }
  bool requires_grad() const { return features_.requires_grad(); }
  SparseTensor to(c10::ScalarType dtype) const;
  SparseTensor detach() const;

  // Element-wise arithmetic on the union of the two coordinate sets, rows a side lacks counting as zero
  // (engine/tensor/sparse_tensor.cpp:31-58, 345-395). Tensors that share manager and key (residual
  // connections) are combined row by row on that map and keep it, so cached kernel maps stay usable;
  // otherwise the result lives on a new manager, as in the reference.
  SparseTensor operator+(const SparseTensor& other) const;
  SparseTensor operator-(const SparseTensor& other) const;
  SparseTensor operator*(const SparseTensor& other) const;
  SparseTensor operator/(const SparseTensor& other) const;
  SparseTensor& operator+=(const SparseTensor& other);
  SparseTensor operator+(at::Scalar scalar) const;
  SparseTensor operator*(at::Scalar scalar) const;

private:
  at::Tensor features_;
  mutable c10::optional<at::Tensor> coordinates_;
  CoordinateMapKey key_;
  std::shared_ptr<CoordinateManager> manager_;
  int dimension_;
};

// Features on continuous coordinates (engine/tensor/field.hpp:10-53).
class TensorField {
public:
  TensorField(at::Tensor features, at::Tensor coordinates, std::shared_ptr<CoordinateManager> manager = nullptr,
              SparseTensorQuantizationMode::Type quantization_mode = SparseTensorQuantizationMode::UNWEIGHTED_AVERAGE);
  SparseTensor sparse(stride_type tensor_stride = {}, c10::optional<CoordinateMapKey> coordinate_map_key = c10::nullopt,
                      SparseTensorQuantizationMode::Type quantization_mode =
                          SparseTensorQuantizationMode::UNWEIGHTED_AVERAGE) const;
  SparseTensor splat() const;
  at::Tensor inverse_mapping(const CoordinateMapKey& sparse_key) const;

  const at::Tensor& F() const noexcept { return features_; }
  at::Tensor C() const { return coordinates_; }
  const CoordinateMapKey& coordinate_field_map_key() const noexcept { return field_key_; }
  std::shared_ptr<CoordinateManager> coordinate_manager() const noexcept { return manager_; }
  int dimension() const noexcept { return dimension_; }
  torch::Device device() const { return features_.device(); }
  c10::ScalarType dtype() const { return features_.scalar_type(); }

private:
  at::Tensor features_, coordinates_;
  CoordinateMapKey field_key_;
  std::shared_ptr<CoordinateManager> manager_;
  int dimension_;
  mutable std::map<coordinate_map_key_type, at::Tensor> inverse_mappings_;
};

// helpers/discretization.hpp:15-34
struct SparseQuantizeResult {
  at::Tensor coordinates;
  c10::optional<at::Tensor> features;
  c10::optional<at::Tensor> labels;
  at::Tensor unique_index;
  at::Tensor inverse_mapping;
};
SparseQuantizeResult sparse_quantize(at::Tensor coordinates, c10::optional<at::Tensor> features = c10::nullopt,
                                     c10::optional<at::Tensor> labels = c10::nullopt, int ignore_label = -100,
                                     c10::optional<double> quantization_size = c10::nullopt);
std::pair<at::Tensor, at::Tensor> unique_coordinate_map(at::Tensor coordinates, stride_type tensor_stride = {});

// engine/nn/operations.hpp:10-12: tensors of one coordinate map, concatenated along channels / summed / averaged
SparseTensor cat(const std::vector<SparseTensor>& tensors);
SparseTensor sum(const std::vector<SparseTensor>& tensors);
SparseTensor mean(const std::vector<SparseTensor>& tensors);

// engine/nn/activation.hpp:11-29
class RiemannReLUImpl : public torch::nn::Module {
public:
  explicit RiemannReLUImpl(bool inplace = false) : inplace_(inplace) {}
  explicit RiemannReLUImpl(torch::nn::ReLUOptions options) : inplace_(options.inplace()) {}
  SparseTensor forward(const SparseTensor& input);

private:
  bool inplace_;
};
TORCH_MODULE(RiemannReLU);

class KernelGenerator {
public:
  struct KernelParams {
    stride_type kernel_size, kernel_stride, kernel_dilation;
    RegionType::Type region_type;
    at::Tensor region_offsets;
    bool expand_coordinates;
    int D;
  };
  KernelGenerator(torch::IntArrayRef kernel_size, torch::IntArrayRef stride = {1}, torch::IntArrayRef dilation = {1},
                  bool is_transpose = false, RegionType::Type region_type = RegionType::HYPER_CUBE,
                  at::Tensor region_offsets = {}, bool expand_coordinates = false,
                  std::vector<RegionType::Type> axis_types = {}, int dimension = -1);
  int kernel_volume() const { return kernel_volume_; }
  const stride_type& kernel_size() const { return kernel_size_; }
  const stride_type& kernel_stride() const { return kernel_stride_; }
  const stride_type& kernel_dilation() const { return kernel_dilation_; }
  RegionType::Type region_type() const { return region_type_; }
  bool expand_coordinates() const { return expand_coordinates_; }
  int dimension() const { return D_; }
  KernelParams get_kernel(const stride_type& tensor_stride, bool is_transpose) const;

private:
  stride_type kernel_size_, kernel_stride_, kernel_dilation_;
  bool is_transpose_;
  RegionType::Type region_type_;
  at::Tensor region_offsets_;
  bool expand_coordinates_;
  int D_;
  int kernel_volume_;
};

// out = sum_k F[in_k] @ W[k] scattered to out_k, with a hand-written backward.
// (an optional bias [1, C_out] is added inside the kernel's epilogue)
at::Tensor sparse_convolution(const at::Tensor& features, const at::Tensor& kernel,
                              const std::shared_ptr<KernelMap>& kmap, const at::Tensor& bias = at::Tensor());

// Helpers with the reference's argument list (autodiff/compat.hpp:89-96, 125-132): run one
// (transposed) convolution over explicit keys and write the resulting key into *out_key.
struct ConvolutionFunction {
  static at::Tensor apply(at::Tensor input_features, at::Tensor kernel, stride_type kernel_size,
                          stride_type kernel_stride, stride_type kernel_dilation, RegionType::Type region_type,
                          at::Tensor region_offsets, bool expand_coordinates, ConvolutionMode::Type conv_mode,
                          std::shared_ptr<CoordinateMapKey> in_key, std::shared_ptr<CoordinateMapKey> out_key,
                          std::shared_ptr<CoordinateManager> manager);
};
struct ConvolutionTransposeFunction {
  static at::Tensor apply(at::Tensor input_features, at::Tensor kernel, stride_type kernel_size,
                          stride_type kernel_stride, stride_type kernel_dilation, RegionType::Type region_type,
                          at::Tensor region_offsets, bool expand_coordinates, ConvolutionMode::Type conv_mode,
                          std::shared_ptr<CoordinateMapKey> in_key, std::shared_ptr<CoordinateMapKey> out_key,
                          std::shared_ptr<CoordinateManager> manager);
};

class RiemannConvolutionBaseImpl : public torch::nn::Cloneable<RiemannConvolutionBaseImpl> {
public:
  RiemannConvolutionBaseImpl(int in_channels, int out_channels, int kernel_size = 3, int stride = 1,
                             int dilation = 1, bool bias = false, bool is_transpose = false,
                             bool expand_coordinates = false,
                             ConvolutionMode::Type convolution_mode = ConvolutionMode::DEFAULT, int dimension = 3,
                             RegionType::Type region_type = RegionType::HYPER_CUBE);
  void reset() override;
  void reset_parameters(bool is_transpose = false);
  SparseTensor forward(const SparseTensor& input);

  int in_channels_, out_channels_;
  bool is_transpose_, use_mm_;
  int dimension_;
  ConvolutionMode::Type convolution_mode_;
  KernelGenerator kernel_generator_;
  torch::Tensor kernel_{nullptr};
  torch::Tensor bias_{nullptr};
  // per-call epilogue fold (scale, shift, ReLU) installed by fused_conv_bn_relu; empty otherwise
  at::Tensor fold_scale_, fold_shift_;
  bool fold_relu_ = false;
};

// RiemannBatchNormImpl (engine/nn/normalization.hpp:11-34): torch's BatchNorm1d over the feature matrix.
class RiemannBatchNormImpl : public torch::nn::Module {
public:
  RiemannBatchNormImpl(int64_t num_features, double eps = 1e-5, double momentum = 0.1, bool affine = true,
                       bool track_running_stats = true);
  SparseTensor forward(const SparseTensor& input);
  torch::nn::BatchNorm1d normalization() { return normalization_; }

private:
  torch::nn::BatchNorm1d normalization_{nullptr};
};
TORCH_MODULE(RiemannBatchNorm);
using RiemannSyncBatchNormImpl = RiemannBatchNormImpl;  // as in the reference (normalization.hpp:36-37)
using RiemannSyncBatchNorm = RiemannBatchNorm;

// Inference-only conv -> batch norm -> ReLU as one kernel; `bn` may be an empty holder (bias + ReLU only).
SparseTensor fused_conv_bn_relu(const SparseTensor& input, RiemannConvolutionBaseImpl& conv,
                                torch::nn::BatchNorm1d bn = nullptr, bool relu = true);

#define RIEMANN_B200_CONV_WRAPPER(Name)                                                                   \
  class Name##Impl : public torch::nn::Cloneable<Name##Impl> {                                            \
  public:                                                                                                 \
    Name##Impl(int in_channels, int out_channels, int kernel_size = 3, int stride = 1, int dilation = 1,  \
               bool bias = false, bool expand_coordinates = false,                                        \
               ConvolutionMode::Type convolution_mode = ConvolutionMode::DEFAULT, int dimension = 3);     \
    void reset() override { base_->reset(); }                                                             \
    SparseTensor forward(const SparseTensor& input) { return base_->forward(input); }                     \
    std::shared_ptr<RiemannConvolutionBaseImpl> base() { return base_; }                                  \
                                                                                                          \
  private:                                                                                                \
    std::shared_ptr<RiemannConvolutionBaseImpl> base_{nullptr};                                           \
  };                                                                                                      \
  TORCH_MODULE(Name)

RIEMANN_B200_CONV_WRAPPER(RiemannConvolution);
RIEMANN_B200_CONV_WRAPPER(RiemannConvolutionTranspose);

class RiemannGenerativeConvolutionTransposeImpl
    : public torch::nn::Cloneable<RiemannGenerativeConvolutionTransposeImpl> {
public:
  RiemannGenerativeConvolutionTransposeImpl(int in_channels, int out_channels, int kernel_size = 3, int stride = 1,
                                            int dilation = 1, bool bias = false,
                                            ConvolutionMode::Type convolution_mode = ConvolutionMode::DEFAULT,
                                            int dimension = 3);
  void reset() override { base_->reset(); }
  SparseTensor forward(const SparseTensor& input) { return base_->forward(input); }
  std::shared_ptr<RiemannConvolutionBaseImpl> base() { return base_; }

private:
  std::shared_ptr<RiemannConvolutionBaseImpl> base_{nullptr};
};
TORCH_MODULE(RiemannGenerativeConvolutionTranspose);

// Local pooling over a kernel map (engine/nn/pooling.cpp:80-144) with a hand-written backward:
// `mode` is one of the three local pooling modes.
at::Tensor sparse_pooling(const at::Tensor& features, const std::shared_ptr<KernelMap>& kmap, PoolingMode::Type mode);

// RiemannPoolingBaseImpl and its three wrappers (engine/nn/pooling.hpp:12-77): same constructor
// arguments; the output map is the input map strided by the pooling stride.
class RiemannPoolingBaseImpl : public torch::nn::Module {
public:
  RiemannPoolingBaseImpl(int kernel_size, int stride = 1, int dilation = 1,
                         PoolingMode::Type mode = PoolingMode::LOCAL_AVG_POOLING, int dimension = 3);
  RiemannPoolingBaseImpl(KernelGenerator kernel_generator, PoolingMode::Type mode, int dimension);
  SparseTensor forward(const SparseTensor& input);

private:
  KernelGenerator kernel_generator_;
  PoolingMode::Type mode_;
  int dimension_;
};

#define RIEMANN_B200_POOL_WRAPPER(Name, Mode)                                                  \
  class Name##Impl : public torch::nn::Module {                                                \
  public:                                                                                      \
    Name##Impl(int kernel_size, int stride = 1, int dilation = 1, int dimension = 3)           \
        : pooling_(kernel_size, stride, dilation, Mode, dimension) {}                          \
    SparseTensor forward(const SparseTensor& input) { return pooling_.forward(input); }        \
                                                                                               \
  private:                                                                                     \
    RiemannPoolingBaseImpl pooling_;                                                           \
  };                                                                                           \
  TORCH_MODULE(Name)

// RiemannPoolingTransposeImpl (engine/nn/pooling.hpp:79-93): un-pooling onto generated coordinates.
class RiemannPoolingTransposeImpl : public torch::nn::Module {
public:
  RiemannPoolingTransposeImpl(int kernel_size, int stride, int dilation = 1, bool expand_coordinates = false,
                              int dimension = 3);
  RiemannPoolingTransposeImpl(KernelGenerator kernel_generator, int dimension,
                              PoolingMode::Type mode = PoolingMode::LOCAL_SUM_POOLING);
  SparseTensor forward(const SparseTensor& input);

private:
  KernelGenerator kernel_generator_;
  int dimension_;
  PoolingMode::Type mode_ = PoolingMode::LOCAL_SUM_POOLING;
};
TORCH_MODULE(RiemannPoolingTranspose);

RIEMANN_B200_POOL_WRAPPER(RiemannAvgPooling, PoolingMode::LOCAL_AVG_POOLING);
RIEMANN_B200_POOL_WRAPPER(RiemannSumPooling, PoolingMode::LOCAL_SUM_POOLING);
RIEMANN_B200_POOL_WRAPPER(RiemannMaxPooling, PoolingMode::LOCAL_MAX_POOLING);

}  // namespace riemann
