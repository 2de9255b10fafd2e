// pybind11 module `_C`: re-exports the C++ host layer with the names and keyword arguments of
// the reference's Python module (python/src/sparse_bindings.cpp:79-199,
// python/src/nn_bindings.cpp:91-117), so that the C++ classes can be driven from pytest.
#include <torch/extension.h>

#include "networks.hpp"
#include "riemann_b200.hpp"

namespace py = pybind11;
using namespace riemann;

namespace {

// local pooling layers (engine/nn/pooling.hpp:30-77): (kernel_size, stride = 1, dilation = 1, dimension = 3)
template <typename Impl>
void bind_pool(py::module_& m, const char* name) {
  py::class_<Impl, std::shared_ptr<Impl>>(m, name)
      .def(py::init([](int kernel_size, int stride, int dilation, int dimension) {
             return std::make_shared<Impl>(kernel_size, stride, dilation, dimension);
           }),
           py::arg("kernel_size"), py::arg("stride") = 1, py::arg("dilation") = 1, py::arg("dimension") = 3)
      .def("forward", [](Impl& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"),
           py::call_guard<py::gil_scoped_release>())
      .def("__call__", [](Impl& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"),
           py::call_guard<py::gil_scoped_release>());
}

template <typename Impl>
py::class_<Impl, std::shared_ptr<Impl>> bind_conv(py::module_& m, const char* name) {
  py::class_<Impl, std::shared_ptr<Impl>> cls(m, name);
  cls.def("forward", [](Impl& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"),
          py::call_guard<py::gil_scoped_release>());
  cls.def("__call__", [](Impl& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"),
          py::call_guard<py::gil_scoped_release>());
  cls.def_property_readonly("kernel", [](Impl& self) { return self.base()->kernel_; });
  cls.def_property_readonly("bias", [](Impl& self) { return self.base()->bias_; });
  cls.def("parameters", [](Impl& self) { return self.parameters(); });
  cls.def("named_parameters", [](Impl& self) {
    py::dict out;
    for (auto& p : self.named_parameters()) out[py::str(p.key())] = p.value();
    return out;
  });
  cls.def("to", [](Impl& self, py::object dtype_or_device) {
    if (THPDtype_Check(dtype_or_device.ptr()))
      self.to(reinterpret_cast<THPDtype*>(dtype_or_device.ptr())->scalar_type);
    else
      self.to(torch::Device(py::cast<std::string>(py::str(dtype_or_device))));
  });
  cls.def("zero_grad", [](Impl& self) { self.zero_grad(); });
  return cls;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "riemann_cpp (B200) host layer";

  py::enum_<CoordinateMapBackend::Type>(m, "CoordinateMapBackend")
      .value("CPU", CoordinateMapBackend::CPU)
      .value("CUDA", CoordinateMapBackend::CUDA);
  py::enum_<RiemannAlgorithm::Mode>(m, "RiemannAlgorithm")
      .value("DEFAULT", RiemannAlgorithm::DEFAULT)
      .value("MEMORY_EFFICIENT", RiemannAlgorithm::MEMORY_EFFICIENT)
      .value("SPEED_OPTIMIZED", RiemannAlgorithm::SPEED_OPTIMIZED);
  py::enum_<SparseTensorQuantizationMode::Type>(m, "SparseTensorQuantizationMode")
      .value("RANDOM_SUBSAMPLE", SparseTensorQuantizationMode::RANDOM_SUBSAMPLE)
      .value("UNWEIGHTED_AVERAGE", SparseTensorQuantizationMode::UNWEIGHTED_AVERAGE)
      .value("UNWEIGHTED_SUM", SparseTensorQuantizationMode::UNWEIGHTED_SUM)
      .value("MAX_POOL", SparseTensorQuantizationMode::MAX_POOL)
      .value("NO_QUANTIZATION", SparseTensorQuantizationMode::NO_QUANTIZATION);
  py::enum_<RegionType::Type>(m, "RegionType")
      .value("HYPER_CUBE", RegionType::HYPER_CUBE)
      .value("HYPER_CROSS", RegionType::HYPER_CROSS)
      .value("CUSTOM", RegionType::CUSTOM);
  py::enum_<ConvolutionMode::Type>(m, "ConvolutionMode")
      .value("DEFAULT", ConvolutionMode::DEFAULT)
      .value("DIRECT_GEMM", ConvolutionMode::DIRECT_GEMM)
      .value("COPY_GEMM", ConvolutionMode::COPY_GEMM);

  py::class_<CoordinateMapKey>(m, "CoordinateMapKey")
      .def(py::init<stride_type, std::string>(), py::arg("tensor_stride"), py::arg("string_id") = "")
      .def_property_readonly("tensor_stride", &CoordinateMapKey::get_tensor_stride)
      .def_property_readonly("coordinate_size", &CoordinateMapKey::get_coordinate_size)
      .def("is_key_set", &CoordinateMapKey::is_key_set)
      .def("__eq__", [](const CoordinateMapKey& a, const CoordinateMapKey& b) { return a == b; })
      .def("__hash__", &CoordinateMapKey::hash)
      .def("__repr__", &CoordinateMapKey::to_string);

  py::class_<CoordinateManager, std::shared_ptr<CoordinateManager>>(m, "CoordinateManager")
      .def(py::init([](int dimension, CoordinateMapBackend::Type backend, RiemannAlgorithm::Mode algorithm) {
             return std::make_shared<CoordinateManager>(dimension, backend, GPUMemoryAllocatorBackend::PYTORCH,
                                                        algorithm);
           }),
           py::arg("dimension"), py::arg("backend") = CoordinateMapBackend::CUDA,
           py::arg("algorithm") = RiemannAlgorithm::DEFAULT)
      .def_property_readonly("dimension", &CoordinateManager::D)
      .def("size", [](const CoordinateManager& self, const CoordinateMapKey& key) { return self.size(key); },
           py::arg("coordinate_map_key"))
      .def("get_coordinates", &CoordinateManager::get_coordinates, py::arg("coordinate_map_key"))
      .def("insert_and_map", &CoordinateManager::insert_and_map, py::arg("coordinates"), py::arg("tensor_stride"),
           py::arg("string_id") = "")
      .def("stride", &CoordinateManager::stride, py::arg("in_key"), py::arg("kernel_stride"),
           py::arg("string_id") = "")
      .def("union_map",
           [](CoordinateManager& self, const std::vector<CoordinateMapKey>& in_keys) {
             CoordinateMapKey out_key(in_keys.empty() ? 0 : in_keys.front().get_coordinate_size());
             auto maps = self.union_map(in_keys, out_key);
             return py::make_tuple(out_key, maps);
           },
           py::arg("in_keys"))
      .def("stride_region",
           [](CoordinateManager& self, const CoordinateMapKey& in_key, stride_type kernel_size,
              stride_type kernel_dilation, stride_type out_tensor_stride, RegionType::Type region_type,
              std::optional<at::Tensor> offsets) {
             return self.stride_region(in_key, kernel_size, kernel_dilation, out_tensor_stride, region_type,
                                       offsets.value_or(at::Tensor()));
           },
           py::arg("in_key"), py::arg("kernel_size"), py::arg("kernel_dilation"), py::arg("out_tensor_stride"),
           py::arg("region_type") = RegionType::HYPER_CUBE, py::arg("offsets") = py::none())
      .def("origin", &CoordinateManager::origin)
      .def("kernel_map_pairs",
           [](CoordinateManager& self, const CoordinateMapKey& in_key, const CoordinateMapKey& out_key,
              stride_type kernel_size, stride_type kernel_stride, stride_type kernel_dilation,
              RegionType::Type region_type, bool is_transpose) {
             // (offset_ptr int64 [K+1] on the host, in rows int32 [P], out rows int32 [P]) of the cached map
             auto kmap = self.kernel_map(in_key, out_key, kernel_size, kernel_stride, kernel_dilation, region_type,
                                         at::Tensor(), is_transpose, false);
             return kmap->pairs();
           },
           py::arg("in_key"), py::arg("out_key"), py::arg("kernel_size"), py::arg("kernel_stride"),
           py::arg("kernel_dilation"), py::arg("region_type") = RegionType::HYPER_CUBE,
           py::arg("is_transpose") = false, py::call_guard<py::gil_scoped_release>())
      .def("kernel_map_th",
           [](CoordinateManager& self, const CoordinateMapKey& in_key, const CoordinateMapKey& out_key,
              stride_type kernel_size, stride_type kernel_stride, stride_type kernel_dilation,
              RegionType::Type region_type, bool is_transpose) {
             return self.kernel_map_th(in_key, out_key, kernel_size, kernel_stride, kernel_dilation, region_type,
                                       at::Tensor(), is_transpose, false);
           },
           py::arg("in_key"), py::arg("out_key"), py::arg("kernel_size"), py::arg("kernel_stride"),
           py::arg("kernel_dilation"), py::arg("region_type") = RegionType::HYPER_CUBE,
           py::arg("is_transpose") = false);

  py::class_<SparseTensor>(m, "SparseTensor")
      .def(py::init([](at::Tensor features, at::Tensor coordinates, std::shared_ptr<CoordinateManager> manager,
                       SparseTensorQuantizationMode::Type quantization_mode, RiemannAlgorithm::Mode algorithm) {
             return SparseTensor(std::move(features), std::move(coordinates), std::move(manager), quantization_mode,
                                 GPUMemoryAllocatorBackend::PYTORCH, algorithm);
           }),
           py::arg("features"), py::arg("coordinates"),
           py::arg("coordinate_manager") = std::shared_ptr<CoordinateManager>(),
           py::arg("quantization_mode") = SparseTensorQuantizationMode::RANDOM_SUBSAMPLE,
           py::arg("algorithm") = RiemannAlgorithm::DEFAULT)
      .def(py::init<at::Tensor, CoordinateMapKey, std::shared_ptr<CoordinateManager>>(), py::arg("features"),
           py::arg("coordinate_map_key"), py::arg("coordinate_manager"))
      .def_property_readonly("F", &SparseTensor::F)
      .def_property_readonly("C", &SparseTensor::C)
      .def_property_readonly("features", &SparseTensor::F)
      .def_property_readonly("coordinates", &SparseTensor::C)
      .def_property_readonly("coordinate_map_key", &SparseTensor::coordinate_map_key)
      .def_property_readonly("coordinate_manager", &SparseTensor::coordinate_manager)
      .def_property_readonly("tensor_stride", &SparseTensor::tensor_stride)
      .def_property_readonly("dimension", &SparseTensor::dimension)
      .def_property_readonly("requires_grad", &SparseTensor::requires_grad)
      .def_property_readonly("shape",
                             [](const SparseTensor& self) { return py::make_tuple(self.F().size(0), self.F().size(1)); })
      .def("__len__", [](const SparseTensor& self) { return self.F().size(0); })
      .def("detach", &SparseTensor::detach)
      .def("__add__", [](const SparseTensor& a, const SparseTensor& b) { return a + b; })
      .def("__sub__", [](const SparseTensor& a, const SparseTensor& b) { return a - b; })
      .def("__mul__", [](const SparseTensor& a, const SparseTensor& b) { return a * b; })
      .def("__truediv__", [](const SparseTensor& a, const SparseTensor& b) { return a / b; })
      .def("__add__", [](const SparseTensor& a, double s) { return a + at::Scalar(s); })
      .def("__mul__", [](const SparseTensor& a, double s) { return a * at::Scalar(s); });
  // 0 = automatic (plan a kernel map from its second convolution pass on, or at once for wide layers),
  // 1 = always, 2 = never
  m.def("set_convolution_plan_policy", [](int policy) { set_convolution_plan_policy(PlanPolicy::Type(policy)); },
        py::arg("policy"));
  m.def("convolution_plan_policy", []() { return int(convolution_plan_policy()); });
  // data-parallel weight-gradient all-reduce (rmn_allreduce_grads)
  m.def("gradient_allreduce_unique_id", []() { return py::bytes(gradient_allreduce_unique_id()); });
  m.def("init_gradient_allreduce",
        [](const std::string& unique_id, int rank, int world_size, bool average) {
          init_gradient_allreduce(unique_id, rank, world_size, average);
        },
        py::arg("unique_id"), py::arg("rank"), py::arg("world_size"), py::arg("average") = true,
        py::call_guard<py::gil_scoped_release>());
  m.def("shutdown_gradient_allreduce", &shutdown_gradient_allreduce);
  m.def("gradient_allreduce_active", &gradient_allreduce_active);
  m.def("allreduce_gradients", &allreduce_gradients, py::arg("gradients"));
  m.def("cat", &cat, py::arg("tensors"));
  m.def("sum", &sum, py::arg("tensors"));
  m.def("mean", &mean, py::arg("tensors"));
  py::class_<RiemannReLUImpl, std::shared_ptr<RiemannReLUImpl>>(m, "RiemannReLU")
      .def(py::init<bool>(), py::arg("inplace") = false)
      .def("forward", &RiemannReLUImpl::forward, py::arg("input"))
      .def("__call__", &RiemannReLUImpl::forward, py::arg("input"));

  // python/src/sparse_bindings.cpp:204-233
  py::class_<TensorField>(m, "TensorField")
      .def(py::init<at::Tensor, at::Tensor, std::shared_ptr<CoordinateManager>, SparseTensorQuantizationMode::Type>(),
           py::arg("features"), py::arg("coordinates"),
           py::arg("coordinate_manager") = std::shared_ptr<CoordinateManager>(),
           py::arg("quantization_mode") = SparseTensorQuantizationMode::UNWEIGHTED_AVERAGE)
      .def("sparse",
           [](const TensorField& self, stride_type tensor_stride, c10::optional<CoordinateMapKey> key,
              SparseTensorQuantizationMode::Type mode) { return self.sparse(std::move(tensor_stride), key, mode); },
           py::arg("tensor_stride") = stride_type{}, py::arg("coordinate_map_key") = py::none(),
           py::arg("quantization_mode") = SparseTensorQuantizationMode::UNWEIGHTED_AVERAGE)
      .def("splat", &TensorField::splat)
      .def("inverse_mapping", &TensorField::inverse_mapping, py::arg("sparse_coordinate_map_key"))
      .def_property_readonly("F", &TensorField::F)
      .def_property_readonly("C", &TensorField::C)
      .def_property_readonly("features", &TensorField::F)
      .def_property_readonly("coordinates", &TensorField::C)
      .def_property_readonly("coordinate_field_map_key", &TensorField::coordinate_field_map_key)
      .def_property_readonly("coordinate_manager", &TensorField::coordinate_manager)
      .def_property_readonly("dimension", &TensorField::dimension)
      .def("__len__", [](const TensorField& self) { return self.F().size(0); });

  m.def(
      "sparse_quantize",
      [](at::Tensor coordinates, c10::optional<at::Tensor> features, c10::optional<double> quantization_size) {
        auto r = sparse_quantize(std::move(coordinates), std::move(features), c10::nullopt, -100, quantization_size);
        return py::make_tuple(r.coordinates, r.features.has_value() ? py::cast(*r.features) : py::none(),
                              r.unique_index, r.inverse_mapping);
      },
      py::arg("coordinates"), py::arg("features") = py::none(), py::arg("quantization_size") = py::none(),
      "(coordinates, features, unique_index, inverse_mapping) of the voxelised points");

  bind_conv<RiemannConvolutionImpl>(m, "RiemannConvolution")
      .def(py::init([](int in_channels, int out_channels, int kernel_size, int stride, int dilation, bool bias,
                       bool expand_coordinates, ConvolutionMode::Type convolution_mode, int dimension) {
             return std::make_shared<RiemannConvolutionImpl>(in_channels, out_channels, kernel_size, stride, dilation,
                                                             bias, expand_coordinates, convolution_mode, dimension);
           }),
           py::arg("in_channels"), py::arg("out_channels"), py::arg("kernel_size") = 3, py::arg("stride") = 1,
           py::arg("dilation") = 1, py::arg("bias") = false, py::arg("expand_coordinates") = false,
           py::arg("convolution_mode") = ConvolutionMode::DEFAULT, py::arg("dimension") = 3);
  bind_conv<RiemannConvolutionTransposeImpl>(m, "RiemannConvolutionTranspose")
      .def(py::init([](int in_channels, int out_channels, int kernel_size, int stride, int dilation, bool bias,
                       bool expand_coordinates, ConvolutionMode::Type convolution_mode, int dimension) {
             return std::make_shared<RiemannConvolutionTransposeImpl>(in_channels, out_channels, kernel_size, stride,
                                                                      dilation, bias, expand_coordinates,
                                                                      convolution_mode, dimension);
           }),
           py::arg("in_channels"), py::arg("out_channels"), py::arg("kernel_size") = 3, py::arg("stride") = 1,
           py::arg("dilation") = 1, py::arg("bias") = false, py::arg("expand_coordinates") = false,
           py::arg("convolution_mode") = ConvolutionMode::DEFAULT, py::arg("dimension") = 3);
  bind_conv<RiemannGenerativeConvolutionTransposeImpl>(m, "RiemannGenerativeConvolutionTranspose")
      .def(py::init([](int in_channels, int out_channels, int kernel_size, int stride, int dilation, bool bias,
                       ConvolutionMode::Type convolution_mode, int dimension) {
             return std::make_shared<RiemannGenerativeConvolutionTransposeImpl>(
                 in_channels, out_channels, kernel_size, stride, dilation, bias, convolution_mode, dimension);
           }),
           py::arg("in_channels"), py::arg("out_channels"), py::arg("kernel_size") = 3, py::arg("stride") = 1,
           py::arg("dilation") = 1, py::arg("bias") = false, py::arg("convolution_mode") = ConvolutionMode::DEFAULT,
           py::arg("dimension") = 3);

  // engine/nn/normalization.hpp:11-34
  {
    using BN = RiemannBatchNormImpl;
    py::class_<BN, std::shared_ptr<BN>> cls(m, "RiemannBatchNorm");
    cls.def(py::init([](int64_t num_features, double eps, double momentum) {
              return std::make_shared<BN>(num_features, eps, momentum);
            }),
            py::arg("num_features"), py::arg("eps") = 1e-5, py::arg("momentum") = 0.1);
    cls.def("forward", [](BN& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"));
    cls.def("__call__", [](BN& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"));
    cls.def_property_readonly("weight", [](BN& self) { return self.normalization()->weight; });
    cls.def_property_readonly("bias", [](BN& self) { return self.normalization()->bias; });
    cls.def_property_readonly("running_mean", [](BN& self) { return self.normalization()->running_mean; });
    cls.def_property_readonly("running_var", [](BN& self) { return self.normalization()->running_var; });
    cls.def("train", [](BN& self, bool on) { self.train(on); }, py::arg("on") = true);
    cls.def("to", [](BN& self, py::object dtype_or_device) {
      if (THPDtype_Check(dtype_or_device.ptr()))
        self.to(reinterpret_cast<THPDtype*>(dtype_or_device.ptr())->scalar_type);
      else
        self.to(torch::Device(py::cast<std::string>(py::str(dtype_or_device))));
    });
  }

  // the example encoder/decoder of networks.hpp (the network the benchmark trains)
  {
    using Net = networks::MinkUNetImpl;
    py::class_<Net, std::shared_ptr<Net>> cls(m, "MinkUNet");
    cls.def(py::init([](int in_channels, int out_channels, int width, int dimension) {
              return std::make_shared<Net>(in_channels, out_channels, width, dimension);
            }),
            py::arg("in_channels"), py::arg("out_channels"), py::arg("width") = 32, py::arg("dimension") = 3);
    cls.def("forward", [](Net& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"),
            py::call_guard<py::gil_scoped_release>());
    cls.def("__call__", [](Net& self, const SparseTensor& input) { return self.forward(input); }, py::arg("input"),
            py::call_guard<py::gil_scoped_release>());
    cls.def("parameters", [](Net& self) { return self.parameters(); });
    cls.def("named_parameters", [](Net& self) {
      py::dict out;
      for (auto& p : self.named_parameters()) out[py::str(p.key())] = p.value();
      return out;
    });
    cls.def("to", [](Net& self, py::object dtype_or_device) {
      if (THPDtype_Check(dtype_or_device.ptr()))
        self.to(reinterpret_cast<THPDtype*>(dtype_or_device.ptr())->scalar_type);
      else
        self.to(torch::Device(py::cast<std::string>(py::str(dtype_or_device))));
    });
    cls.def("zero_grad", [](Net& self) { self.zero_grad(); });
    cls.def("train", [](Net& self, bool on) { self.train(on); }, py::arg("on") = true);
  }

  // inference fold of a batch norm given by its tensors (what torch.nn.BatchNorm1d holds in eval mode)
  m.def(
      "fused_conv_bn_relu",
      [](const SparseTensor& input, std::shared_ptr<RiemannConvolutionImpl> conv, at::Tensor running_mean,
         at::Tensor running_var, at::Tensor weight, at::Tensor bias, double eps, bool relu) {
        torch::nn::BatchNorm1d bn(torch::nn::BatchNorm1dOptions(running_mean.numel()).eps(eps));
        bn->to(running_mean.device());
        {
          torch::NoGradGuard guard;
          bn->running_mean.copy_(running_mean);
          bn->running_var.copy_(running_var);
          if (weight.defined() && weight.numel()) bn->weight.copy_(weight);
          if (bias.defined() && bias.numel()) bn->bias.copy_(bias);
        }
        bn->eval();
        return fused_conv_bn_relu(input, *conv->base(), bn, relu);
      },
      py::arg("input"), py::arg("conv"), py::arg("running_mean"), py::arg("running_var"), py::arg("weight"),
      py::arg("bias"), py::arg("eps") = 1e-5, py::arg("relu") = true, py::call_guard<py::gil_scoped_release>());

  py::enum_<PoolingMode::Type>(m, "PoolingMode")
      .value("LOCAL_SUM_POOLING", PoolingMode::LOCAL_SUM_POOLING)
      .value("LOCAL_AVG_POOLING", PoolingMode::LOCAL_AVG_POOLING)
      .value("LOCAL_MAX_POOLING", PoolingMode::LOCAL_MAX_POOLING);
  py::class_<RiemannPoolingTransposeImpl, std::shared_ptr<RiemannPoolingTransposeImpl>>(m, "RiemannPoolingTranspose")
      .def(py::init([](int kernel_size, int stride, int dilation, bool expand_coordinates, int dimension) {
             return std::make_shared<RiemannPoolingTransposeImpl>(kernel_size, stride, dilation, expand_coordinates,
                                                                  dimension);
           }),
           py::arg("kernel_size"), py::arg("stride"), py::arg("dilation") = 1, py::arg("expand_coordinates") = false,
           py::arg("dimension") = 3)
      .def("forward", [](RiemannPoolingTransposeImpl& self, const SparseTensor& input) { return self.forward(input); },
           py::arg("input"), py::call_guard<py::gil_scoped_release>())
      .def("__call__", [](RiemannPoolingTransposeImpl& self, const SparseTensor& input) { return self.forward(input); },
           py::arg("input"), py::call_guard<py::gil_scoped_release>());
  bind_pool<RiemannAvgPoolingImpl>(m, "RiemannAvgPooling");
  bind_pool<RiemannSumPoolingImpl>(m, "RiemannSumPooling");
  bind_pool<RiemannMaxPoolingImpl>(m, "RiemannMaxPooling");
}
