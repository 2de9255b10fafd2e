// Driver around the UNMODIFIED reference CPU implementation of the sparse
// convolution hot path. TEST INFRASTRUCTURE ONLY: it produces golden vectors
// for the parity tests and is the CPU baseline timed by the benchmark.
//
// It is compiled (see the Makefile beside this file) together with the four
// reference translation units it needs, taken from the reference checkout
// where they lie; nothing of the reference is copied here. The driver only
// calls the reference's public API:
//   riemann::SparseTensor ctor            engine/tensor/sparse_tensor.cpp:62-99
//   riemann::CoordinateManager            engine/grid/space.hpp:817-906
//   cpu manager kernel_map                engine/grid/space_impl.hpp:499-706
//   riemann::RiemannConvolution(+Transpose) engine/nn/conv.cpp:104-171
//
// usage: ref_driver <in.rmna> <out.rmna>
// Files hold named arrays: u32 name_len, name, u32 dtype (0 i32, 1 f32,
// 2 i64, 3 f64), u32 ndim, i64 dims[ndim], raw little-endian data.
//
// Input arrays:
//   coords  i32 [N, W]      may contain duplicate rows
//   feats   f32 [N, Cin]
//   weights f32 [K, Cin, Cout]
//   params  i32 [8] = {kernel_size, stride, dilation, chain, threads, reps, timing_only, warmup}
//     chain = 1: after the first (strided) convolution run a transposed
//     convolution with the same kernel_size/stride using `weights2`
//     [K, Cout, C2] back onto the input coordinates.
//   weights2 f32 (only when chain = 1)
//   pool    i32 [3 or 4] = {mode (1 sum, 2 average, 3 maximum), kernel_size, stride[, transpose]}  (optional):
//     also run the reference's local pooling layer on the input tensor
//     (engine/nn/pooling.cpp:17-144) and write pool_coords, pool_feats and
//     pool_grad_feats (gradient of 0.5 * sum(pool_feats^2) w.r.t. the input features). With transpose = 1 the
//     pooling-transpose layer (sum; engine/nn/pooling.cpp:197-229) is applied to the convolution's output instead.
//   field   f32 [N, W] + field_params f64 [2 + D] = {quantisation mode, quantisation size, tensor stride...}
//     (optional; when present ONLY the input step is run and the arrays above other than feats are ignored):
//     riemann::TensorField(feats, field).sparse(stride, mode) (engine/tensor/field.cpp:41-59) -> field_coords,
//     field_feats, field_inverse; TensorField::splat (field.cpp:61-94) -> splat_coords, splat_feats;
//     riemann::sparse_quantize(field, feats, quantization_size) (engine/helpers/discretization.cpp:78-125) ->
//     sq_coords, sq_feats, sq_unique_index, sq_inverse.
// Output arrays: mapping, inverse, in_coords, out_coords, out_feats,
//   kmap_ptr / kmap_in / kmap_out, grad_feats, grad_weights, and for chain = 1
//   up_coords, up_feats, kmap2_ptr / kmap2_in / kmap2_out, grad_weights2;
//   times_ms f64 [4] = {SparseTensor ctor, first forward (kernel map + conv),
//   forward with cached kernel map, forward + backward}, each the median of
//   `reps` runs after `warmup` untimed ones; times_all f64 [reps, 4] holds every timed run;
//   info i32 [2] = {hardware_concurrency, torch threads}.
#include "engine/nn/conv.hpp"
#include "engine/nn/pooling.hpp"
#include "engine/tensor/field.hpp"
#include "engine/tensor/sparse_tensor.hpp"
#include "helpers/discretization.hpp"

#include <torch/torch.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <map>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Array {
  uint32_t dtype;
  std::vector<int64_t> dims;
  std::vector<char> data;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
};

size_t dtype_size(uint32_t t) { return (t == 2 || t == 3) ? 8 : 4; }

std::map<std::string, Array> read_arrays(const char* path) {
  std::map<std::string, Array> out;
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error(std::string("cannot open ") + path);
  for (;;) {
    uint32_t len;
    if (!f.read(reinterpret_cast<char*>(&len), 4)) break;
    std::string name(len, '\0');
    f.read(name.data(), len);
    Array a;
    uint32_t ndim;
    f.read(reinterpret_cast<char*>(&a.dtype), 4);
    f.read(reinterpret_cast<char*>(&ndim), 4);
    a.dims.resize(ndim);
    f.read(reinterpret_cast<char*>(a.dims.data()), 8 * ndim);
    a.data.resize(a.numel() * dtype_size(a.dtype));
    f.read(a.data.data(), a.data.size());
    out[name] = std::move(a);
  }
  return out;
}

void write_array(std::ofstream& f, const std::string& name, const at::Tensor& t_in) {
  auto t = t_in.detach().cpu().contiguous();
  uint32_t dtype;
  if (t.scalar_type() == torch::kInt32) dtype = 0;
  else if (t.scalar_type() == torch::kFloat32) dtype = 1;
  else if (t.scalar_type() == torch::kInt64) dtype = 2;
  else if (t.scalar_type() == torch::kFloat64) dtype = 3;
  else throw std::runtime_error("unsupported dtype for " + name);
  uint32_t len = name.size(), ndim = t.dim();
  f.write(reinterpret_cast<char*>(&len), 4);
  f.write(name.data(), len);
  f.write(reinterpret_cast<char*>(&dtype), 4);
  f.write(reinterpret_cast<char*>(&ndim), 4);
  for (int i = 0; i < t.dim(); ++i) {
    int64_t d = t.size(i);
    f.write(reinterpret_cast<char*>(&d), 8);
  }
  f.write(reinterpret_cast<const char*>(t.data_ptr()), t.numel() * t.element_size());
}

at::Tensor to_tensor(const Array& a) {
  auto st = a.dtype == 0 ? torch::kInt32 : a.dtype == 1 ? torch::kFloat32
            : a.dtype == 2 ? torch::kInt64 : torch::kFloat64;
  auto t = torch::empty(a.dims, torch::TensorOptions().dtype(st));
  std::memcpy(t.data_ptr(), a.data.data(), a.data.size());
  return t;
}

double now_ms() {
  return std::chrono::duration<double, std::milli>(
             std::chrono::steady_clock::now().time_since_epoch()).count();
}

double median(std::vector<double> v) {
  std::sort(v.begin(), v.end());
  return v[v.size() / 2];
}

void dump_kernel_map(std::ofstream& f, const std::string& prefix,
                     const riemann::cpu_kernel_map& map) {
  std::vector<int64_t> ptr{0};
  std::vector<int32_t> in, out;
  for (size_t k = 0; k < map.first.size(); ++k) {
    for (size_t i = 0; i < map.first[k].size(); ++i) {
      in.push_back(static_cast<int32_t>(map.first[k][i]));
      out.push_back(static_cast<int32_t>(map.second[k][i]));
    }
    ptr.push_back(static_cast<int64_t>(in.size()));
  }
  write_array(f, prefix + "_ptr", torch::tensor(ptr, torch::kInt64));
  write_array(f, prefix + "_in", torch::tensor(in, torch::kInt32));
  write_array(f, prefix + "_out", torch::tensor(out, torch::kInt32));
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 3) {
    std::fprintf(stderr, "usage: %s <in> <out>\n", argv[0]);
    return 2;
  }
  try {
    auto arrays = read_arrays(argv[1]);
    if (arrays.count("field")) {
      torch::set_num_threads(1);
      auto field = to_tensor(arrays.at("field"));
      auto ffeats = to_tensor(arrays.at("feats"));
      auto fp = to_tensor(arrays.at("field_params"));
      const int D = static_cast<int>(field.size(1)) - 1;
      const auto mode = static_cast<riemann::SparseTensorQuantizationMode::Type>(fp[0].item<double>());
      const double qsize = fp[1].item<double>();
      riemann::stride_type stride;
      for (int a = 0; a < D; ++a) stride.push_back(static_cast<uint32_t>(fp[2 + a].item<double>()));
      std::ofstream out(argv[2], std::ios::binary);
      riemann::TensorField tf(ffeats, field);
      auto sp = tf.sparse(stride, c10::nullopt, mode);
      write_array(out, "field_coords", sp.C());
      write_array(out, "field_feats", sp.F());
      write_array(out, "field_inverse", tf.inverse_mapping(sp.coordinate_map_key()));
      riemann::TensorField tf2(ffeats, field);
      auto spl = tf2.splat();
      write_array(out, "splat_coords", spl.C());
      write_array(out, "splat_feats", spl.F());
      auto sq = riemann::sparse_quantize(field, ffeats, c10::nullopt, -100,
                                         qsize > 0 ? c10::optional<double>(qsize) : c10::nullopt);
      write_array(out, "sq_coords", sq.coordinates);
      write_array(out, "sq_feats", sq.features.value());
      write_array(out, "sq_unique_index", sq.unique_index);
      write_array(out, "sq_inverse", sq.inverse_mapping);
      return 0;
    }
    auto coords = to_tensor(arrays.at("coords"));
    auto feats = to_tensor(arrays.at("feats"));
    auto weights = to_tensor(arrays.at("weights"));
    auto params = to_tensor(arrays.at("params"));
    const int ksize = params[0].item<int>(), stride = params[1].item<int>(),
              dilation = params[2].item<int>(), chain = params[3].item<int>();
    int threads = params[4].item<int>();
    const int reps = std::max(1, params[5].item<int>());
    const bool timing_only = params[6].item<int>() != 0;
    const int warmup = std::max(0, params[7].item<int>());
    const int hw = static_cast<int>(std::thread::hardware_concurrency());
    if (threads <= 0) threads = std::max(hw, 1);
    torch::set_num_threads(threads);
    const int D = static_cast<int>(coords.size(1)) - 1;
    const int cin = weights.size(1), cout = weights.size(2);

    riemann::RiemannConvolution conv(cin, cout, ksize, stride, dilation, false, false,
                                     riemann::ConvolutionMode::DEFAULT, D);
    {
      torch::NoGradGuard g;
      conv->base()->kernel_.copy_(weights);
    }
    riemann::RiemannConvolutionTranspose up(nullptr);
    if (chain) {
      auto w2 = to_tensor(arrays.at("weights2"));
      up = riemann::RiemannConvolutionTranspose(cout, static_cast<int>(w2.size(2)), ksize, stride,
                                                dilation, false, false,
                                                riemann::ConvolutionMode::DEFAULT, D);
      torch::NoGradGuard g;
      up->base()->kernel_.copy_(w2);
    }

    std::ofstream out(argv[2], std::ios::binary);

    // --- timings (median of reps); also warms everything up -----------------
    std::vector<double> t_ctor, t_first, t_cached, t_fb;
    std::vector<double> all;
    for (int r = 0; r < reps + warmup; ++r) {
      double t0, t1, t2, t3, t4;
      {  // forward-only phases run without autograd recording
        torch::NoGradGuard no_grad;
        t0 = now_ms();
        riemann::SparseTensor x(feats, coords);
        t1 = now_ms();
        auto y = conv->forward(x);
        if (chain) y = up->forward(y);
        t2 = now_ms();
        auto y2 = conv->forward(x);
        if (chain) y2 = up->forward(y2);
        t3 = now_ms();
      }
      const double t_c = t1 - t0, t_f = t2 - t1, t_k = t3 - t2;
      {  // forward + backward on a tensor whose kernel maps are already cached
        auto f = feats.clone().requires_grad_(true);
        riemann::SparseTensor x(f, coords);
        conv->forward(x);
        if (chain) up->forward(conv->forward(x));
        t3 = now_ms();
        auto y3 = conv->forward(x);
        if (chain) y3 = up->forward(y3);
        (y3.F() * y3.F()).sum().mul(0.5).backward();
        t4 = now_ms();
      }
      conv->zero_grad();
      if (chain) up->zero_grad();
      if (r < warmup) continue;
      for (double v : {t_c, t_f, t_k, t4 - t3}) all.push_back(v);
      t_ctor.push_back(t_c);
      t_first.push_back(t_f);
      t_cached.push_back(t_k);
      t_fb.push_back(t4 - t3);
    }
    write_array(out, "times_ms",
                torch::tensor({median(t_ctor), median(t_first), median(t_cached), median(t_fb)},
                              torch::kFloat64));
    write_array(out, "times_all", torch::tensor(all, torch::kFloat64).reshape({reps, 4}));
    write_array(out, "info", torch::tensor({hw, at::get_num_threads()}, torch::kInt32));
    if (timing_only) return 0;

    // --- values --------------------------------------------------------------
    auto manager = std::make_shared<riemann::CoordinateManager>(D, riemann::CoordinateMapBackend::CPU);
    riemann::stride_type unit(static_cast<size_t>(D), 1);
    auto inserted = manager->insert_and_map(coords.contiguous(), unit);
    write_array(out, "mapping", inserted.second.first);
    write_array(out, "inverse", inserted.second.second);

    auto f = feats.clone().requires_grad_(true);
    riemann::SparseTensor x(f, coords);
    write_array(out, "in_coords", x.C());
    auto y = conv->forward(x);
    write_array(out, "out_coords", y.C());
    write_array(out, "out_feats", y.F());

    auto* cpu_manager =
        x.coordinate_manager()->manager_ptr<riemann::cpu_manager_type<int32_t>>();
    auto kparams = conv->base()->kernel_generator_.get_kernel(x.tensor_stride(), false);
    const auto& kmap = cpu_manager->kernel_map(
        &x.coordinate_map_key(), &y.coordinate_map_key(), kparams.kernel_size, kparams.kernel_stride,
        kparams.kernel_dilation, kparams.region_type, kparams.region_offsets, false, false);
    dump_kernel_map(out, "kmap", kmap);

    riemann::SparseTensor last = y;
    if (chain) {
      auto z = up->forward(y);
      write_array(out, "up_coords", z.C());
      write_array(out, "up_feats", z.F());
      auto uparams = up->base()->kernel_generator_.get_kernel(y.tensor_stride(), true);
      const auto& kmap2 = cpu_manager->kernel_map(
          &y.coordinate_map_key(), &z.coordinate_map_key(), uparams.kernel_size,
          uparams.kernel_stride, uparams.kernel_dilation, uparams.region_type,
          uparams.region_offsets, true, false);
      dump_kernel_map(out, "kmap2", kmap2);
      last = z;
    }
    (last.F() * last.F()).sum().mul(0.5).backward();
    write_array(out, "grad_feats", f.grad());
    write_array(out, "grad_weights", conv->base()->kernel_.grad());
    if (chain) write_array(out, "grad_weights2", up->base()->kernel_.grad());

    if (arrays.count("pool")) {
      auto pool = to_tensor(arrays.at("pool"));
      const int pmode = pool[0].item<int>(), pk = pool[1].item<int>(), ps = pool[2].item<int>();
      const auto mode = pmode == 1   ? riemann::PoolingMode::LOCAL_SUM_POOLING
                        : pmode == 2 ? riemann::PoolingMode::LOCAL_AVG_POOLING
                                     : riemann::PoolingMode::LOCAL_MAX_POOLING;
      const bool pool_transpose = pool.numel() > 3 && pool[3].item<int>() != 0;
      auto fp = feats.clone().requires_grad_(true);
      riemann::SparseTensor xp(fp, coords);
      if (!pool_transpose) {
        riemann::RiemannPoolingBaseImpl pooling(pk, ps, 1, mode, D);
        auto yp = pooling.forward(xp);
        write_array(out, "pool_coords", yp.C());
        write_array(out, "pool_feats", yp.F());
        (yp.F() * yp.F()).sum().mul(0.5).backward();
      } else {
        // pooling-transpose (sum) of the convolution's output: un-pooling onto generated coordinates
        conv->zero_grad();
        auto yc = conv->forward(xp);
        riemann::RiemannPoolingTranspose unpool(pk, ps, 1, false, D);
        auto yp = unpool->forward(yc);
        write_array(out, "pool_coords", yp.C());
        write_array(out, "pool_feats", yp.F());
        (yp.F() * yp.F()).sum().mul(0.5).backward();
      }
      write_array(out, "pool_grad_feats", fp.grad());
    }
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ref_driver: %s\n", e.what());
    return 1;
  }
}
