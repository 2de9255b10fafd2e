// Implementation of the riemann_cpp (B200) host layer: LibTorch tensors for device memory and
// autograd, the C ABI of librmn_b200.so for every coordinate / convolution operation.
#include "riemann_b200.hpp"

#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>

#include "rmn_b200.h"

namespace riemann {
namespace {

constexpr const char* ERROR_MAP_NOT_FOUND = "CoordinateMap not found";

// status -> the exception type the reference's ASSERT throws (engine/foundation/errors.hpp:113-122)
void check(int status, const char* where) {
  if (status != RMN_OK)
    throw std::runtime_error(std::string(where) + ": " + rmn_status_string(status) + " (status " +
                             std::to_string(status) + ")");
}

void* current_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void* ptr(const at::Tensor& t) { return t.defined() && t.numel() > 0 ? t.data_ptr() : nullptr; }

int dtype_code(const at::Tensor& t) {
  if (t.scalar_type() == at::kFloat) return RMN_F32;
  if (t.scalar_type() == at::kBFloat16) return RMN_BF16;
  throw std::runtime_error("unsupported feature dtype: float32 and bfloat16 only");
}

// the checks of insert_and_map_cpp (engine/grid/space_impl.hpp:268-276)
void check_coordinates(const at::Tensor& c) {
  TORCH_CHECK(c.is_cuda(), "coordinates must be a CUDA tensor: this library has no CPU path");
  TORCH_CHECK(c.dim() == 2, "coordinates must be 2-D [N, 1 + D]");
  TORCH_CHECK(c.scalar_type() == at::kInt, "coordinates must be int32");
  TORCH_CHECK(c.is_contiguous(), "coordinates must be contiguous");
  TORCH_CHECK(c.size(1) >= 2 && c.size(1) <= RMN_MAX_W, "coordinates must have between 2 and 8 columns");
}

// (plain string appends: iostreams are avoided on purpose, the extension shares a process with
// libraries that carry their own copies of the stream templates)
std::string stride_string(const stride_type& s) {
  std::string out = "[";
  for (size_t i = 0; i < s.size(); ++i) {
    if (i) out += ", ";
    out += std::to_string(s[i]);
  }
  out += "]";
  return out;
}

std::vector<int32_t> to_i32(const stride_type& s) { return std::vector<int32_t>(s.begin(), s.end()); }

}  // namespace

// ---------------------------------------------------------------------------------------------
// CoordinateMapKey
// ---------------------------------------------------------------------------------------------
CoordinateMapKey::CoordinateMapKey(size_type coordinate_size, coordinate_map_key_type const& key)
    : m_key_set(true), m_coordinate_size(coordinate_size), m_key(key) {
  if (coordinate_size - 1 != m_key.first.size())
    throw std::runtime_error("Invalid tensor_stride: " + stride_string(m_key.first));
}

CoordinateMapKey::CoordinateMapKey(stride_type tensor_stride, std::string string_id)
    : m_key_set(true), m_coordinate_size(tensor_stride.size() + 1), m_key(std::move(tensor_stride), std::move(string_id)) {}

void CoordinateMapKey::set_key(stride_type tensor_stride, std::string string_id) {
  if (m_coordinate_size - 1 != tensor_stride.size())
    throw std::runtime_error("Invalid tensor_stride size: " + stride_string(tensor_stride));
  m_key = std::make_pair(std::move(tensor_stride), std::move(string_id));
  m_key_set = true;
}

void CoordinateMapKey::set_key(coordinate_map_key_type const& key) { set_key(key.first, key.second); }

coordinate_map_key_type CoordinateMapKey::get_key() const {
  if (!m_key_set) throw std::runtime_error("Key not set");
  return m_key;
}

uint64_t CoordinateMapKey::hash() const {
  uint64_t h = UINT64_C(14695981039346656037);  // FNV-1a over stride entries and id bytes
  for (auto s : m_key.first) { h ^= s; h *= UINT64_C(1099511628211); }
  for (unsigned char c : m_key.second) { h ^= c; h *= UINT64_C(1099511628211); }
  return h;
}

bool CoordinateMapKey::operator==(CoordinateMapKey const& key) const {
  if (!m_key_set || !key.m_key_set) return false;
  return m_key == key.m_key;
}

std::string CoordinateMapKey::to_string() const {
  std::string out = "coordinate map key:" + stride_string(m_key.first);
  if (!m_key.second.empty()) out += ":" + m_key.second;
  return out;
}

// ---------------------------------------------------------------------------------------------
// KernelMap
// ---------------------------------------------------------------------------------------------
at::Tensor const& KernelMap::nbr_in() {
  if (!nbr_in_.defined()) {
    c10::cuda::CUDAGuard guard(nbr_out.device());
    const int64_t K = nbr_out.size(0);
    nbr_in_ = at::empty({K, n_in}, nbr_out.options());
    check(rmn_kmap_transpose(static_cast<const int32_t*>(ptr(nbr_out)), static_cast<uint32_t>(n_out),
                             static_cast<int>(K), static_cast<uint32_t>(n_in),
                             static_cast<int32_t*>(ptr(nbr_in_)), current_stream()),
          "rmn_kmap_transpose");
  }
  return nbr_in_;
}

namespace {
std::atomic<int> g_plan_policy{PlanPolicy::AUTO};
}
void set_convolution_plan_policy(PlanPolicy::Type policy) { g_plan_policy.store(int(policy)); }
PlanPolicy::Type convolution_plan_policy() { return PlanPolicy::Type(g_plan_policy.load()); }

at::Tensor KernelMap::build_plan(const at::Tensor& table, bool negate_offsets) {
  const int64_t K = table.size(0), n = table.size(1);
  const size_t plan_bytes = rmn_conv_plan_bytes(static_cast<uint32_t>(n), static_cast<int>(K));
  if (n == 0 || plan_bytes == 0 || region_offsets.empty()) return at::Tensor();  // (tables beyond the plan limit run unplanned)
  c10::cuda::CUDAGuard guard(table.device());
  std::vector<int32_t> off(region_offsets);
  if (negate_offsets)
    for (auto& v : off) v = -v;
  const int D = static_cast<int>(off.size() / static_cast<size_t>(K));
  auto bytes = table.options().dtype(at::kByte);
  auto plan = at::empty({static_cast<int64_t>(plan_bytes)}, bytes);
  const size_t ws_bytes = rmn_conv_plan_workspace_bytes(static_cast<uint32_t>(n), static_cast<int>(K));
  auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, bytes);
  check(rmn_conv_plan_build(static_cast<const int32_t*>(ptr(table)), static_cast<uint32_t>(n), static_cast<int>(K),
                            off.data(), D, ptr(plan), plan_bytes, ptr(ws), ws_bytes, current_stream()),
        "rmn_conv_plan_build");
  return plan;
}

namespace {
// AUTO: a plan costs about two passes over the table (0.12 ms for 1.2 M rows x 27 offsets) and saves 10-18 % of
// every tensor-core pass over it, which for a 64 -> 64 layer is a quarter of the build. The passes over a table
// are therefore weighed by c_in * c_out and the plan is built by the pass that brings the sum to four 64 x 64
// layers' worth: at once for a 128 -> 128 layer, at the fourth pass of a 64 -> 64 network, never for a map that
// one or two narrow layers use.
bool want_plan(int64_t weight_sum, int64_t rows) {
  const int policy = g_plan_policy.load();
  if (policy == PlanPolicy::NEVER || rows < 8192) return false;
  return policy == PlanPolicy::ALWAYS || weight_sum >= 4 * 64 * 64;
}
}  // namespace

at::Tensor KernelMap::plan_out(int64_t weight) {
  if (parent) return parent->plan_in(weight);  // a swapped view: its output table is the parent's input table
  weight_out_ += weight;
  if (!plan_out_.defined() && want_plan(weight_out_, n_out)) plan_out_ = build_plan(nbr_out, false);
  return plan_out_;
}

at::Tensor KernelMap::plan_in(int64_t weight) {
  if (parent) return parent->plan_out(weight);
  if (self_symmetric) return plan_out(weight);  // the input gradient of a self map runs over the same table
  weight_in_ += weight;
  if (!plan_in_.defined() && want_plan(weight_in_, n_in)) plan_in_ = build_plan(nbr_in(), true);
  return plan_in_;
}

namespace {
// One second stream per device (pair-list kernels, early header read-back): the caching allocator keeps a pool per stream, so
// a stream picked afresh from torch's round-robin pool on every call would allocate the lists anew each time.
c10::cuda::CUDAStream pair_list_stream(c10::DeviceIndex device) {
  static std::mutex lock;
  static std::map<int, c10::cuda::CUDAStream> streams;
  std::lock_guard<std::mutex> guard(lock);
  auto it = streams.find(static_cast<int>(device));
  if (it == streams.end()) it = streams.emplace(static_cast<int>(device), c10::cuda::getStreamFromPool(false, device)).first;
  return it->second;
}
}  // namespace

std::tuple<at::Tensor, at::Tensor, at::Tensor> const& KernelMap::pairs() {
  if (have_pairs_) return pairs_;
  if (parent) {  // in <-> out of the parent's lists (engine/grid/space.cpp:104-107)
    auto const& p = parent->pairs();
    pairs_ = std::make_tuple(std::get<0>(p), std::get<2>(p), std::get<1>(p));
  } else {
    c10::cuda::CUDAGuard guard(nbr_out.device());
    at::Tensor host_ptr;
    if (offset_ptr_ready.has_value()) {
      offset_ptr_ready->synchronize();  // the copy was queued before the convolution: normally long done
      host_ptr = host_offset_ptr.clone();
    } else {
      host_ptr = offset_ptr.cpu();
    }
    const int64_t K = nbr_out.size(0);
    const int64_t total = host_ptr[K].item<int64_t>();
    // The lists are written on a second stream: nothing a convolution needs depends on them, and the
    // compaction is bound by HBM while the convolution kernels are bound by shared memory and the tensor
    // pipe, so a convolution already queued on the caller's stream and this kernel share the SMs. The
    // caller's stream waits for the lists before anything queued after this call.
    auto main_stream = c10::cuda::getCurrentCUDAStream();
    auto side_stream = pair_list_stream(main_stream.device_index());
    at::Tensor in_idx, out_idx;
    {
      c10::cuda::CUDAStreamGuard on_side(side_stream);
      in_idx = at::empty({total}, nbr_out.options());   // from the second stream's pool: memory freed on the
      out_idx = at::empty({total}, nbr_out.options());  // caller's stream may still be in use by queued kernels
      if (offset_ptr_ready.has_value()) {
        offset_ptr_ready->block(side_stream);
      } else {
        c10::Event built(c10::DeviceType::CUDA);
        built.record(main_stream);
        built.block(side_stream);
      }
      check(rmn_kmap_pairs_background(static_cast<const int32_t*>(ptr(nbr_out)), static_cast<uint32_t>(n_out),
                                      static_cast<int>(K), static_cast<const int64_t*>(ptr(offset_ptr)),
                                      ptr(workspace), static_cast<int32_t*>(ptr(in_idx)),
                                      static_cast<int32_t*>(ptr(out_idx)), static_cast<uint64_t>(total),
                                      side_stream.stream()),
            "rmn_kmap_pairs_background");
      c10::Event done(c10::DeviceType::CUDA);
      done.record(side_stream);
      done.block(main_stream);
    }
    if (total > 0) {
      c10::cuda::CUDACachingAllocator::recordStream(in_idx.storage().data_ptr(), main_stream);
      c10::cuda::CUDACachingAllocator::recordStream(out_idx.storage().data_ptr(), main_stream);
    }
    pairs_ = std::make_tuple(host_ptr, in_idx, out_idx);
  }
  have_pairs_ = true;
  return pairs_;
}

std::shared_ptr<KernelMap> KernelMap::swapped(std::shared_ptr<KernelMap> const& self) {
  auto out = std::make_shared<KernelMap>();
  out->nbr_out = nbr_in();
  out->nbr_in_ = nbr_out;
  out->n_in = n_out;
  out->n_out = n_in;
  out->parent = self;
  return out;
}

// ---------------------------------------------------------------------------------------------
// CoordinateManager
// ---------------------------------------------------------------------------------------------
namespace {
// Device copy of a region's offsets, cached per device: networks build a fresh manager per forward pass
// and ask for the same few regions every time, and a copy from pageable host memory blocks the host while
// the GPU waits for its next launch.
at::Tensor device_offsets(const std::vector<int32_t>& off, const c10::Device& device) {
  static std::mutex lock;
  static std::map<std::pair<int, std::vector<int32_t>>, at::Tensor> cache;
  std::lock_guard<std::mutex> guard(lock);
  auto key = std::make_pair(static_cast<int>(device.index()), off);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 256) cache.clear();
  auto host = at::empty({static_cast<int64_t>(off.size())}, at::TensorOptions().dtype(at::kInt));
  if (!off.empty()) std::memcpy(host.data_ptr(), off.data(), off.size() * sizeof(int32_t));
  auto dev = host.to(device);
  cache[key] = dev;
  return dev;
}
}  // namespace

CoordinateManager::CoordinateManager(int D, CoordinateMapBackend::Type map_type, GPUMemoryAllocatorBackend::Type,
                                     RiemannAlgorithm::Mode)
    : D_(D), map_type_(map_type) {
  if (map_type != CoordinateMapBackend::CUDA)
    throw std::runtime_error("riemann_cpp (B200) has no CPU coordinate-map backend");
}

CoordinateManager::Map CoordinateManager::build(const at::Tensor& coords, const stride_type& tensor_stride,
                                                at::Tensor* mapping_out, at::Tensor* inverse_out) {
  c10::cuda::CUDAGuard guard(coords.device());
  const uint32_t n = static_cast<uint32_t>(coords.size(0));
  const int W = static_cast<int>(coords.size(1));
  auto bytes = at::TensorOptions().dtype(at::kByte).device(coords.device());
  auto longs = at::TensorOptions().dtype(at::kLong).device(coords.device());
  Map m;
  m.tensor_stride = tensor_stride;
  const size_t table_bytes = rmn_table_bytes(n), ws_bytes = rmn_table_build_workspace_bytes(n);
  m.table = at::empty({static_cast<int64_t>(table_bytes)}, bytes);
  auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, bytes);
  auto mapping = at::empty({n}, longs), inverse = at::empty({n}, longs);
  auto unique = at::empty({n, W}, coords.options());
  // The header (number of unique rows) is final after the first half of the build: it is read back on the
  // second stream while the second half still runs on the caller's, so the host is already preparing the
  // next launches when the build ends.
  auto main_stream = c10::cuda::getCurrentCUDAStream();
  check(rmn_table_build_begin(static_cast<const int32_t*>(ptr(coords)), n, W, ptr(m.table), table_bytes, ptr(ws),
                              ws_bytes, main_stream.stream()),
        "rmn_table_build");
  c10::Event counted(c10::DeviceType::CUDA);
  counted.record(main_stream);
  check(rmn_table_build_finish(static_cast<const int32_t*>(ptr(coords)), n, W, ptr(m.table),
                               static_cast<int64_t*>(ptr(mapping)), static_cast<int64_t*>(ptr(inverse)),
                               static_cast<int32_t*>(ptr(unique)), ptr(ws), main_stream.stream()),
        "rmn_table_build");
  auto side_stream = pair_list_stream(main_stream.device_index());
  counted.block(side_stream);
  uint32_t info[4];
  check(rmn_table_info(ptr(m.table), info, side_stream.stream()), "rmn_table_build");
  m.size = info[0];
  m.coords = unique.narrow(0, 0, m.size);
  if (mapping_out) *mapping_out = mapping.narrow(0, 0, m.size);
  if (inverse_out) *inverse_out = inverse;
  return m;
}

CoordinateManager::Map const& CoordinateManager::find(const CoordinateMapKey& key, const char* what) const {
  auto it = maps_.find(key.get_key());
  if (it == maps_.end()) {
    std::string msg = what && *what ? std::string(what) + " " : std::string();
    throw std::runtime_error(msg + ERROR_MAP_NOT_FOUND);
  }
  return it->second;
}

bool CoordinateManager::exists(const CoordinateMapKey& key) const { return maps_.count(key.get_key()) != 0; }
uint32_t CoordinateManager::size(const CoordinateMapKey& key) const { return find(key).size; }
at::Tensor CoordinateManager::get_coordinates(const CoordinateMapKey& key) const { return find(key).coords; }

std::pair<CoordinateMapKey, std::pair<at::Tensor, at::Tensor>>
CoordinateManager::insert_and_map(const at::Tensor& coordinates, stride_type tensor_stride, std::string string_id) {
  check_coordinates(coordinates);
  const auto coordinate_size = static_cast<size_type>(coordinates.size(1));
  if (coordinate_size - 1 != tensor_stride.size())
    throw std::runtime_error("The coordinate dimension (coordinate_size - 1): " +
                             std::to_string(coordinate_size - 1) +
                             " must match the size of tensor stride: " + stride_string(tensor_stride));
  coordinate_map_key_type map_key(tensor_stride, string_id);
  while (maps_.count(map_key)) {  // key collision -> random string id (space_impl.hpp:284-289)
    std::string suffix = "-";
    for (int i = 0; i < 8; ++i) suffix.push_back(static_cast<char>('a' + std::rand() % 26));
    map_key.second = string_id + suffix;
  }
  at::Tensor mapping, inverse;
  maps_[map_key] = build(coordinates, tensor_stride, &mapping, &inverse);
  return {CoordinateMapKey(coordinate_size, map_key), {mapping, inverse}};
}

CoordinateMapKey CoordinateManager::insert_field(const at::Tensor& coordinates, stride_type tensor_stride,
                                                 std::string string_id) {
  TORCH_CHECK(coordinates.is_cuda(), "coordinates must be a CUDA tensor: this library has no CPU path");
  TORCH_CHECK(coordinates.dim() == 2 && coordinates.is_contiguous() && coordinates.scalar_type() == at::kFloat,
              "field coordinates must be a contiguous 2D float32 tensor");
  const auto coordinate_size = static_cast<size_type>(coordinates.size(1));
  if (coordinate_size - 1 != tensor_stride.size())
    throw std::runtime_error("The coordinate dimension (coordinate_size - 1): " +
                             std::to_string(coordinate_size - 1) +
                             " must match the size of tensor stride: " + stride_string(tensor_stride));
  coordinate_map_key_type map_key(tensor_stride, string_id);
  while (fields_.count(map_key)) {
    std::string suffix = "-";
    for (int i = 0; i < 8; ++i) suffix.push_back(static_cast<char>('a' + std::rand() % 26));
    map_key.second = string_id + suffix;
  }
  fields_[map_key] = coordinates;
  return CoordinateMapKey(coordinate_size, map_key);
}

at::Tensor CoordinateManager::get_field_coordinates(const CoordinateMapKey& field_key) const {
  auto it = fields_.find(field_key.get_key());
  if (it == fields_.end()) throw std::runtime_error(ERROR_MAP_NOT_FOUND);
  return it->second;
}

std::pair<CoordinateMapKey, std::pair<at::Tensor, at::Tensor>>
CoordinateManager::field_to_sparse_insert_and_map(const CoordinateMapKey& field_key, stride_type sparse_tensor_stride,
                                                  std::string sparse_tensor_string_id) {
  auto field = get_field_coordinates(field_key);
  if (static_cast<size_t>(field.size(1)) - 1 != sparse_tensor_stride.size())
    throw std::runtime_error("The coordinate dimension (coordinate_size - 1): " +
                             std::to_string(field.size(1) - 1) +
                             " must match the size of tensor stride: " + stride_string(sparse_tensor_stride));
  c10::cuda::CUDAGuard guard(field.device());
  auto voxels = at::empty(field.sizes(), field.options().dtype(at::kInt));
  auto st = to_i32(sparse_tensor_stride);
  check(rmn_field_quantize(static_cast<const float*>(ptr(field)), static_cast<uint32_t>(field.size(0)),
                           static_cast<int>(field.size(1)), st.data(), static_cast<int32_t*>(ptr(voxels)),
                           current_stream()),
        "rmn_field_quantize");
  return insert_and_map(voxels, sparse_tensor_stride, sparse_tensor_string_id);
}

CoordinateMapKey CoordinateManager::stride(const CoordinateMapKey& in_key, const stride_type& kernel_stride,
                                           std::string string_id) {
  auto const& in_map = find(in_key);
  if (in_map.tensor_stride.size() != kernel_stride.size()) throw std::runtime_error("stride size mismatch.");
  stride_type out_stride(in_map.tensor_stride);
  for (size_t i = 0; i < out_stride.size(); ++i) out_stride[i] *= kernel_stride[i];
  coordinate_map_key_type out_key(out_stride, string_id.empty() ? in_key.get_key().second : string_id);
  if (!maps_.count(out_key)) {
    c10::cuda::CUDAGuard guard(in_map.coords.device());
    auto aligned = at::empty_like(in_map.coords);
    auto st = to_i32(out_stride);
    check(rmn_coords_stride(static_cast<const int32_t*>(ptr(in_map.coords)), in_map.size,
                            static_cast<int>(in_map.coords.size(1)), st.data(),
                            static_cast<int32_t*>(ptr(aligned)), current_stream()),
          "rmn_coords_stride");
    maps_[out_key] = build(aligned, out_stride, nullptr, nullptr);
  }
  return CoordinateMapKey(in_key.get_coordinate_size(), out_key);
}

std::pair<CoordinateMapKey, bool> CoordinateManager::origin() {
  if (maps_.empty()) throw std::runtime_error("No coordinate map found");
  const size_t D = maps_.begin()->second.tensor_stride.size();
  coordinate_map_key_type origin_key(stride_type(D, 0), "");
  const bool created = !maps_.count(origin_key);
  if (created) {
    // seed: the smallest map (every map holds every batch index that has any voxel at its stride)
    const Map* seed = nullptr;
    for (auto const& kv : maps_)
      if (!seed || kv.second.size < seed->size) seed = &kv.second;
    c10::cuda::CUDAGuard guard(seed->coords.device());
    auto zeroed = at::zeros_like(seed->coords);
    zeroed.select(1, 0).copy_(seed->coords.select(1, 0));
    maps_[origin_key] = build(zeroed, origin_key.first, nullptr, nullptr);  // dedup on the batch column
  }
  return {CoordinateMapKey(static_cast<size_type>(D + 1), origin_key), created};
}

std::vector<at::Tensor> CoordinateManager::union_map(const std::vector<CoordinateMapKey>& in_keys,
                                                     CoordinateMapKey& out_key) {
  if (in_keys.empty()) throw std::runtime_error("union_map needs at least one map");
  std::vector<at::Tensor> coords;
  auto const& first = find(in_keys.front());
  for (auto const& key : in_keys) {
    auto const& m = find(key);
    if (m.tensor_stride != first.tensor_stride)
      throw std::runtime_error("all maps of a union must share one tensor stride");
    coords.push_back(m.coords);
  }
  auto inserted = insert_and_map(at::cat(coords, 0), first.tensor_stride, "");
  out_key = inserted.first;
  auto const& merged = find(out_key);
  std::vector<at::Tensor> out;
  for (auto const& c : coords) {
    c10::cuda::CUDAGuard guard(c.device());
    auto rows = at::empty({c.size(0)}, c.options());
    check(rmn_table_find(ptr(merged.table), static_cast<const int32_t*>(ptr(c)), static_cast<uint32_t>(c.size(0)),
                         static_cast<int>(c.size(1)), static_cast<int32_t*>(ptr(rows)), current_stream()),
          "rmn_table_find");
    out.push_back(at::stack({at::arange(c.size(0), rows.options().dtype(at::kLong)), rows.to(at::kLong)}));
  }
  return out;
}

CoordinateMapKey CoordinateManager::stride_region(const CoordinateMapKey& in_key, const stride_type& kernel_size,
                                                  const stride_type& kernel_dilation,
                                                  const stride_type& out_tensor_stride, RegionType::Type region_type,
                                                  const at::Tensor& offsets) {
  auto const& in_map = find(in_key, "in_map");
  const int D = static_cast<int>(kernel_size.size());
  if (kernel_dilation.size() != kernel_size.size() || out_tensor_stride.size() != kernel_size.size() ||
      static_cast<int64_t>(D) + 1 != in_map.coords.size(1))
    throw std::runtime_error("kernel size mismatch");
  std::vector<int32_t> custom;
  if (region_type == RegionType::CUSTOM) {
    TORCH_CHECK(offsets.defined(), "CUSTOM region needs offsets");
    auto host = offsets.to(at::kCPU, at::kInt).contiguous();
    custom.assign(host.data_ptr<int32_t>(), host.data_ptr<int32_t>() + host.numel());
  }
  auto ks = to_i32(kernel_size), kd = to_i32(kernel_dilation), ts = to_i32(out_tensor_stride);
  const int n_custom = D ? static_cast<int>(custom.size()) / D : 0;
  const int K = rmn_region_volume(int(region_type), D, ks.data(), n_custom);
  if (K < 0) check(-K, "rmn_region_volume");
  std::vector<int32_t> off(static_cast<size_t>(K) * D);
  const int K2 = rmn_region_offsets(int(region_type), D, ks.data(), kd.data(), ts.data(),
                                    custom.empty() ? nullptr : custom.data(), n_custom, off.data());
  if (K2 < 0) check(-K2, "rmn_region_offsets");
  c10::cuda::CUDAGuard guard(in_map.coords.device());
  auto d_off = device_offsets(off, in_map.coords.device());
  auto generated = at::empty({static_cast<int64_t>(in_map.size) * K, in_map.coords.size(1)}, in_map.coords.options());
  check(rmn_coords_expand(static_cast<const int32_t*>(ptr(in_map.coords)), in_map.size,
                          static_cast<int>(in_map.coords.size(1)), static_cast<const int32_t*>(ptr(d_off)), K,
                          static_cast<int32_t*>(ptr(generated)), current_stream()),
        "rmn_coords_expand");
  return insert_and_map(generated, out_tensor_stride, "").first;
}

std::shared_ptr<KernelMap> CoordinateManager::kernel_map(const CoordinateMapKey& in_key,
                                                         const CoordinateMapKey& out_key,
                                                         const stride_type& kernel_size,
                                                         const stride_type& kernel_stride,
                                                         const stride_type& kernel_dilation,
                                                         RegionType::Type region_type, const at::Tensor& offsets,
                                                         bool is_transpose, bool is_pool) {
  const size_t kernel_dim = kernel_size.size();
  if (kernel_dim != kernel_stride.size() || kernel_dim != kernel_dilation.size())
    throw std::runtime_error("kernel size mismatch");
  std::vector<int32_t> custom;
  if (region_type == RegionType::CUSTOM) {
    TORCH_CHECK(offsets.defined(), "CUSTOM region needs offsets");
    auto host = offsets.to(at::kCPU, at::kInt).contiguous();
    custom.assign(host.data_ptr<int32_t>(), host.data_ptr<int32_t>() + host.numel());
    for (size_t i = 0; i < kernel_dim; ++i)
      TORCH_CHECK(kernel_size[i] > 0 && kernel_stride[i] > 0 && kernel_dilation[i] > 0,
                  "CUSTOM kernel size, stride and dilation must be positive");
  }
  auto cache_key = [&](const CoordinateMapKey& a, const CoordinateMapKey& b, bool transpose) {
    std::string out = a.to_string() + "|" + b.to_string() + "|" + stride_string(kernel_size) +
                      stride_string(kernel_stride) + stride_string(kernel_dilation) + "|" +
                      std::to_string(int(region_type)) + (transpose ? "T" : "F") + (is_pool ? "P" : "C") + "|";
    for (auto v : custom) out += std::to_string(v) + ",";
    return out;
  };
  const std::string key = cache_key(in_key, out_key, is_transpose);
  if (auto it = kernel_maps_.find(key); it != kernel_maps_.end()) return it->second;

  auto const& in_map = find(in_key, "in_map");
  auto const& out_map = find(out_key, "out_map");
  const int W = static_cast<int>(in_map.coords.size(1));
  if (kernel_dim + 1 != static_cast<size_t>(W) || out_map.coords.size(1) != W)
    throw std::runtime_error("kernel size mismatch");

  std::shared_ptr<KernelMap> result;
  if (is_transpose) {
    const std::string swapped_key = cache_key(out_key, in_key, false);
    if (auto it = kernel_maps_.find(swapped_key); it != kernel_maps_.end()) result = it->second->swapped(it->second);
  }
  if (!result) {
    // forward: region on the INPUT stride, probe the input map around every output row.
    // transposed: region on the OUTPUT (fine) stride, out = in + off_k; probing the input map at
    // out - off_k gives the output-stationary table directly (space_impl.hpp:649-697 builds the same
    // pairs by probing the output map and swapping).
    auto const& region_stride = is_transpose ? out_map.tensor_stride : in_map.tensor_stride;
    auto ks = to_i32(kernel_size), kd = to_i32(kernel_dilation), ts = to_i32(region_stride);
    const int D = static_cast<int>(kernel_dim);
    const int n_custom = D ? static_cast<int>(custom.size()) / D : 0;
    const int K = rmn_region_volume(int(region_type), D, ks.data(), n_custom);
    if (K < 0) check(-K, "rmn_region_volume");
    std::vector<int32_t> off(static_cast<size_t>(K) * D);
    const int K2 = rmn_region_offsets(int(region_type), D, ks.data(), kd.data(), ts.data(),
                                      custom.empty() ? nullptr : custom.data(), n_custom, off.data());
    if (K2 < 0) check(-K2, "rmn_region_offsets");
    if (is_transpose)
      for (auto& v : off) v = -v;

    c10::cuda::CUDAGuard guard(in_map.coords.device());
    auto ints = in_map.coords.options();
    auto d_off = device_offsets(off, in_map.coords.device());
    result = std::make_shared<KernelMap>();
    result->n_in = in_map.size;
    result->n_out = out_map.size;
    result->nbr_out = at::empty({K, static_cast<int64_t>(out_map.size)}, ints);
    result->offset_ptr = at::empty({K + 1}, ints.dtype(at::kLong));
    const size_t ws_bytes = rmn_kmap_workspace_bytes(out_map.size, K);
    result->workspace = at::empty({static_cast<int64_t>(ws_bytes)}, ints.dtype(at::kByte));
    // self map (stride-1 convolution) with a point-symmetric region: half the probes
    bool self_symmetric = !is_transpose && in_key.get_key() == out_key.get_key() && (K % 2 == 1);
    for (int k = 0; self_symmetric && k < K; ++k)
      for (int a = 0; a < D; ++a)
        if (off[static_cast<size_t>(k) * D + a] != -off[static_cast<size_t>(K - 1 - k) * D + a]) self_symmetric = false;
    auto build = self_symmetric ? rmn_kmap_build_self : rmn_kmap_build;
    check(build(ptr(in_map.table), static_cast<const int32_t*>(ptr(out_map.coords)), out_map.size, W,
                static_cast<const int32_t*>(ptr(d_off)), K, static_cast<int32_t*>(ptr(result->nbr_out)),
                static_cast<int64_t*>(ptr(result->offset_ptr)), ptr(result->workspace), ws_bytes, current_stream()),
          self_symmetric ? "rmn_kmap_build_self" : "rmn_kmap_build");
    result->self_symmetric = self_symmetric;
    result->region_offsets = off;
    result->host_offset_ptr = at::empty({K + 1}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
    // stored by a kernel, not a copy engine: behind a large device-to-host copy of the caller's (the previous
    // step's result) an engine copy of these few bytes would wait for all of it
    check(rmn_readback_small(ptr(result->offset_ptr), result->host_offset_ptr.data_ptr(),
                             static_cast<size_t>(K + 1) * sizeof(int64_t), current_stream()),
          "rmn_readback_small");
    result->offset_ptr_ready.emplace(c10::DeviceType::CUDA);
    result->offset_ptr_ready->record(c10::cuda::getCurrentCUDAStream());
  }
  kernel_maps_[key] = result;
  return result;
}

std::map<int64_t, at::Tensor> CoordinateManager::kernel_map_th(
    const CoordinateMapKey& in_key, const CoordinateMapKey& out_key, const stride_type& kernel_size,
    const stride_type& kernel_stride, const stride_type& kernel_dilation, RegionType::Type region_type,
    const at::Tensor& offsets, bool is_transpose, bool is_pool) {
  auto kmap = kernel_map(in_key, out_key, kernel_size, kernel_stride, kernel_dilation, region_type, offsets,
                         is_transpose, is_pool);
  auto const& [host_ptr, in_idx, out_idx] = kmap->pairs();
  std::map<int64_t, at::Tensor> out;
  auto acc = host_ptr.accessor<int64_t, 1>();
  for (int64_t k = 0; k + 1 < host_ptr.size(0); ++k)
    if (acc[k + 1] > acc[k])
      out[k] = at::stack({in_idx.slice(0, acc[k], acc[k + 1]), out_idx.slice(0, acc[k], acc[k + 1])});
  return out;
}

// ---------------------------------------------------------------------------------------------
// SparseTensor (engine/tensor/sparse_tensor.cpp:62-120, 447-481)
// ---------------------------------------------------------------------------------------------
namespace {
at::Tensor quantize_features(const at::Tensor& features, const at::Tensor& first_rows,
                             const at::Tensor& row_to_unique, int64_t unique_count,
                             SparseTensorQuantizationMode::Type mode) {
  switch (mode) {
    case SparseTensorQuantizationMode::RANDOM_SUBSAMPLE:
      // all rows unique <=> first rows are 0..N-1 (first-occurrence numbering)
      if (features.size(0) == unique_count) return features;
      return features.index_select(0, first_rows);
    case SparseTensorQuantizationMode::NO_QUANTIZATION:
      return features;
    case SparseTensorQuantizationMode::UNWEIGHTED_SUM:
    case SparseTensorQuantizationMode::UNWEIGHTED_AVERAGE: {
      auto result = torch::zeros({unique_count, features.size(1)}, features.options());
      result.index_add_(0, row_to_unique, features);
      if (mode == SparseTensorQuantizationMode::UNWEIGHTED_SUM) return result;
      auto counts = torch::zeros({unique_count}, features.options());
      counts.index_add_(0, row_to_unique, torch::ones({features.size(0)}, features.options()));
      return result / counts.clamp_min(1).unsqueeze(1);
    }
    case SparseTensorQuantizationMode::MAX_POOL: {
      auto result = torch::zeros({unique_count, features.size(1)}, features.options());
      return at::scatter_reduce(result, 0, row_to_unique.unsqueeze(1).expand_as(features), features, "amax", false);
    }
    default:
      throw std::runtime_error("Unknown quantization mode");
  }
}
}  // namespace

SparseTensor::SparseTensor(at::Tensor features, at::Tensor coordinates, std::shared_ptr<CoordinateManager> manager,
                           SparseTensorQuantizationMode::Type quantization_mode,
                           GPUMemoryAllocatorBackend::Type alloc_type, RiemannAlgorithm::Mode algo)
    : features_(std::move(features)), key_(static_cast<size_type>(coordinates.dim() == 2 ? coordinates.size(1) : 0)),
      dimension_(0) {
  TORCH_CHECK(features_.dim() == 2, "Features must be a 2D tensor");
  TORCH_CHECK(coordinates.dim() == 2, "Coordinates must be a 2D tensor");
  TORCH_CHECK(features_.size(0) == coordinates.size(0), "Features and coordinates must have same number of rows");
  TORCH_CHECK(coordinates.size(1) >= 2, "Coordinates must contain a batch column and spatial columns");
  TORCH_CHECK(coordinates.is_cuda(), "coordinates must be a CUDA tensor: this library has no CPU path");
  dimension_ = static_cast<int>(coordinates.size(1) - 1);
  if (!manager)
    manager = std::make_shared<CoordinateManager>(dimension_, CoordinateMapBackend::CUDA, alloc_type, algo);
  TORCH_CHECK(manager->D() == dimension_, "Coordinate manager dimension does not match coordinates");
  manager_ = std::move(manager);
  stride_type unit_stride(static_cast<size_t>(dimension_), 1);
  auto inserted = manager_->insert_and_map(coordinates.contiguous(), unit_stride);
  key_ = std::move(inserted.first);
  features_ = quantize_features(features_, inserted.second.first, inserted.second.second, manager_->size(key_),
                                quantization_mode);
}

SparseTensor::SparseTensor(at::Tensor features, CoordinateMapKey coordinate_map_key,
                           std::shared_ptr<CoordinateManager> manager)
    : features_(std::move(features)), key_(std::move(coordinate_map_key)), manager_(std::move(manager)),
      dimension_(static_cast<int>(key_.get_coordinate_size()) - 1) {
  TORCH_CHECK(manager_, "Manager must not be null");
  TORCH_CHECK(features_.dim() == 2, "Features must be 2D");
  TORCH_CHECK(key_.is_key_set(), "Coordinate map key must be set");
  TORCH_CHECK(manager_->D() == dimension_, "Coordinate manager dimension does not match coordinate key");
  TORCH_CHECK(features_.size(0) == manager_->size(key_), "Feature row count must match coordinate map size");
}

at::Tensor SparseTensor::C() const {
  if (!coordinates_.has_value()) coordinates_ = manager_->get_coordinates(key_);
  return coordinates_.value();
}

// ---------------------------------------------------------------------------------------------
// TensorField (engine/tensor/field.cpp:9-142) and the discretisation helpers
// (engine/helpers/discretization.cpp:78-141)
// ---------------------------------------------------------------------------------------------
TensorField::TensorField(at::Tensor features, at::Tensor coordinates, std::shared_ptr<CoordinateManager> manager,
                         SparseTensorQuantizationMode::Type)
    : features_(std::move(features)), field_key_(static_cast<size_type>(coordinates.dim() == 2 ? coordinates.size(1) : 0)),
      dimension_(0) {
  TORCH_CHECK(features_.dim() == 2, "Features must be a 2D tensor");
  TORCH_CHECK(coordinates.dim() == 2, "Coordinates must be a 2D tensor");
  TORCH_CHECK(features_.size(0) == coordinates.size(0), "Features and coordinates must have same number of rows");
  TORCH_CHECK(coordinates.scalar_type() == at::kFloat || coordinates.scalar_type() == at::kDouble,
              "TensorField coordinates must be float or double");
  TORCH_CHECK(coordinates.size(1) >= 2, "Coordinates must contain a batch column and spatial columns");
  dimension_ = static_cast<int>(coordinates.size(1) - 1);
  if (!manager) manager = std::make_shared<CoordinateManager>(dimension_, CoordinateMapBackend::CUDA);
  TORCH_CHECK(manager->D() == dimension_, "Coordinate manager dimension does not match coordinates");
  manager_ = std::move(manager);
  coordinates_ = coordinates.contiguous();
  field_key_ = manager_->insert_field(coordinates_, stride_type(static_cast<size_t>(dimension_), 1));
}

SparseTensor TensorField::sparse(stride_type tensor_stride, c10::optional<CoordinateMapKey>,
                                 SparseTensorQuantizationMode::Type quantization_mode) const {
  if (tensor_stride.empty()) tensor_stride.assign(static_cast<size_t>(dimension_), 1);
  auto inserted = manager_->field_to_sparse_insert_and_map(field_key_, tensor_stride);
  auto const& sparse_key = inserted.first;
  auto quantized = quantize_features(features_, inserted.second.first, inserted.second.second,
                                     manager_->size(sparse_key), quantization_mode);
  inverse_mappings_[sparse_key.get_key()] = inserted.second.second;
  return SparseTensor(std::move(quantized), sparse_key, manager_);
}

SparseTensor TensorField::splat() const {
  c10::cuda::CUDAGuard guard(coordinates_.device());
  TORCH_CHECK(coordinates_.scalar_type() == at::kFloat, "field coordinates must be float32");
  auto feats = features_.contiguous();
  const int64_t n = coordinates_.size(0), W = coordinates_.size(1), C = feats.size(1);
  const int64_t rows = n << (W - 1);
  auto out_c = at::empty({rows, W}, coordinates_.options().dtype(at::kInt));
  auto out_f = at::empty({rows, C}, feats.options());
  check(rmn_field_splat(static_cast<const float*>(ptr(coordinates_)), ptr(feats), dtype_code(feats),
                        static_cast<uint32_t>(n), static_cast<int>(W), static_cast<int>(C),
                        static_cast<int32_t*>(ptr(out_c)), ptr(out_f), current_stream()),
        "rmn_field_splat");
  return SparseTensor(std::move(out_f), std::move(out_c), manager_, SparseTensorQuantizationMode::UNWEIGHTED_SUM);
}

at::Tensor TensorField::inverse_mapping(const CoordinateMapKey& sparse_key) const {
  auto it = inverse_mappings_.find(sparse_key.get_key());
  if (it != inverse_mappings_.end()) return it->second;
  auto inserted = manager_->field_to_sparse_insert_and_map(field_key_, sparse_key.get_tensor_stride());
  inverse_mappings_[sparse_key.get_key()] = inserted.second.second;
  return inserted.second.second;
}

std::pair<at::Tensor, at::Tensor> unique_coordinate_map(at::Tensor coordinates, stride_type tensor_stride) {
  TORCH_CHECK(coordinates.dim() == 2 && coordinates.size(1) >= 2,
              "Coordinates must include a batch column and spatial dimensions");
  const auto dimension = static_cast<size_t>(coordinates.size(1) - 1);
  if (tensor_stride.empty()) tensor_stride.assign(dimension, 1);
  TORCH_CHECK(tensor_stride.size() == dimension, "Tensor stride dimension must match coordinates");
  auto manager = std::make_shared<CoordinateManager>(static_cast<int>(dimension), CoordinateMapBackend::CUDA);
  return manager->insert_and_map(coordinates.contiguous(), tensor_stride).second;
}

SparseQuantizeResult sparse_quantize(at::Tensor coordinates, c10::optional<at::Tensor> features,
                                     c10::optional<at::Tensor> labels, int, c10::optional<double> quantization_size) {
  TORCH_CHECK(coordinates.dim() == 2, "Coordinates must be a 2D matrix");
  TORCH_CHECK(!features.has_value() || (features->dim() == 2 && features->size(0) == coordinates.size(0)),
              "Feature rows must match coordinate rows");
  // the reference coalesces labels in a CPU-only loop (engine/helpers/discretization.cpp:31-76)
  TORCH_CHECK(!labels.has_value(), "Label quantization currently requires CPU tensors");
  if (quantization_size.has_value())
    TORCH_CHECK(*quantization_size > 0.0 && std::isfinite(*quantization_size),
                "Quantization size must be positive and finite");
  TORCH_CHECK(coordinates.is_cuda(), "coordinates must be a CUDA tensor: this library has no CPU path");
  int in_type = coordinates.scalar_type() == at::kFloat ? 0 : coordinates.scalar_type() == at::kDouble ? 1
                : coordinates.scalar_type() == at::kInt ? 2 : -1;
  if (in_type < 0) {
    coordinates = coordinates.to(at::kDouble);
    in_type = 1;
  }
  coordinates = coordinates.contiguous();
  c10::cuda::CUDAGuard guard(coordinates.device());
  auto discrete = at::empty(coordinates.sizes(), coordinates.options().dtype(at::kInt));
  check(rmn_coords_discretize(ptr(coordinates), in_type, static_cast<uint64_t>(coordinates.numel()),
                              quantization_size.value_or(0.0), static_cast<int32_t*>(ptr(discrete)), current_stream()),
        "rmn_coords_discretize");
  auto maps = unique_coordinate_map(discrete);
  SparseQuantizeResult result;
  result.unique_index = maps.first;
  result.inverse_mapping = maps.second;
  result.coordinates = discrete.index_select(0, maps.first);
  if (features.has_value()) result.features = features->to(discrete.device()).index_select(0, maps.first);
  return result;
}

// ---------------------------------------------------------------------------------------------
// Arithmetic between sparse tensors and the same-map helpers
// ---------------------------------------------------------------------------------------------
namespace {
template <typename Operation>
SparseTensor union_binary_operation(const SparseTensor& lhs, const SparseTensor& rhs, const char* what,
                                    Operation operation) {
  TORCH_CHECK(lhs.dimension() == rhs.dimension(), "Cannot ", what, " tensors with different dimensions");
  TORCH_CHECK(lhs.F().size(1) == rhs.F().size(1), "Cannot ", what,
              " tensors with different feature channel counts");
  TORCH_CHECK(lhs.F().device() == rhs.F().device(), "Cannot ", what, " tensors on different devices");
  if (lhs.coordinate_manager() == rhs.coordinate_manager() && lhs.coordinate_map_key() == rhs.coordinate_map_key())
    return SparseTensor(operation(lhs.F(), rhs.F()), lhs.coordinate_map_key(), lhs.coordinate_manager());
  auto output_stride = lhs.tensor_stride();
  const auto other_stride = rhs.tensor_stride();
  for (size_t axis = 0; axis < output_stride.size(); ++axis)
    output_stride[axis] = std::min(output_stride[axis], other_stride[axis]);
  auto manager = std::make_shared<CoordinateManager>(lhs.dimension(), CoordinateMapBackend::CUDA);
  auto inserted = manager->insert_and_map(at::cat({lhs.C(), rhs.C()}, 0).contiguous(), std::move(output_stride));
  const int64_t union_size = manager->size(inserted.first);
  auto const& row_to_union = inserted.second.second;
  const int64_t lhs_rows = lhs.F().size(0), rhs_rows = rhs.F().size(0);
  auto align = [&](const at::Tensor& features, const at::Tensor& rows) {
    auto result = torch::zeros({union_size, features.size(1)}, features.options());
    return result.index_copy(0, rows, features);
  };
  return SparseTensor(operation(align(lhs.F(), row_to_union.slice(0, 0, lhs_rows)),
                                align(rhs.F(), row_to_union.slice(0, lhs_rows, lhs_rows + rhs_rows))),
                      inserted.first, std::move(manager));
}

void validate_same_map(const std::vector<SparseTensor>& tensors, bool same_channels) {
  TORCH_CHECK(tensors.size() > 1, "At least two sparse tensors are required");
  for (size_t i = 1; i < tensors.size(); ++i) {
    TORCH_CHECK(tensors.front().coordinate_manager() == tensors[i].coordinate_manager(),
                "Sparse tensors must share a coordinate manager");
    TORCH_CHECK(tensors.front().coordinate_map_key() == tensors[i].coordinate_map_key(),
                "Sparse tensors must share a coordinate map key");
    TORCH_CHECK(!same_channels || tensors[i].F().size(1) == tensors.front().F().size(1),
                "Sparse tensor feature widths must match");
  }
}
}  // namespace

SparseTensor SparseTensor::operator+(const SparseTensor& other) const {
  return union_binary_operation(*this, other, "add", [](const at::Tensor& a, const at::Tensor& b) { return a + b; });
}
SparseTensor SparseTensor::operator-(const SparseTensor& other) const {
  return union_binary_operation(*this, other, "subtract",
                                [](const at::Tensor& a, const at::Tensor& b) { return a - b; });
}
SparseTensor SparseTensor::operator*(const SparseTensor& other) const {
  return union_binary_operation(*this, other, "multiply",
                                [](const at::Tensor& a, const at::Tensor& b) { return a * b; });
}
SparseTensor SparseTensor::operator/(const SparseTensor& other) const {
  return union_binary_operation(*this, other, "divide", [](const at::Tensor& a, const at::Tensor& b) { return a / b; });
}
SparseTensor& SparseTensor::operator+=(const SparseTensor& other) {
  TORCH_CHECK(manager_ == other.manager_, "Cannot add tensors from different managers");
  TORCH_CHECK(key_ == other.key_, "In-place addition requires same key");
  features_ += other.features_;
  return *this;
}
SparseTensor SparseTensor::operator+(at::Scalar scalar) const { return SparseTensor(features_ + scalar, key_, manager_); }
SparseTensor SparseTensor::operator*(at::Scalar scalar) const { return SparseTensor(features_ * scalar, key_, manager_); }

SparseTensor cat(const std::vector<SparseTensor>& tensors) {
  validate_same_map(tensors, false);
  std::vector<at::Tensor> features;
  for (auto const& t : tensors) features.push_back(t.F());
  return SparseTensor(torch::cat(features, 1), tensors.front().coordinate_map_key(),
                      tensors.front().coordinate_manager());
}

SparseTensor sum(const std::vector<SparseTensor>& tensors) {
  validate_same_map(tensors, true);
  auto output = tensors.front().F();
  for (size_t i = 1; i < tensors.size(); ++i) output = output + tensors[i].F();
  return SparseTensor(std::move(output), tensors.front().coordinate_map_key(), tensors.front().coordinate_manager());
}

SparseTensor mean(const std::vector<SparseTensor>& tensors) {
  return sum(tensors) * (1.0 / static_cast<double>(tensors.size()));
}

SparseTensor RiemannReLUImpl::forward(const SparseTensor& input) {
  auto output = input.F();
  if (inplace_)
    at::relu_(output);
  else
    output = at::relu(output);
  return SparseTensor(std::move(output), input.coordinate_map_key(), input.coordinate_manager());
}

SparseTensor SparseTensor::to(c10::ScalarType dtype) const { return SparseTensor(features_.to(dtype), key_, manager_); }
SparseTensor SparseTensor::detach() const { return SparseTensor(features_.detach(), key_, manager_); }

// ---------------------------------------------------------------------------------------------
// KernelGenerator (engine/grid/stencil.cpp:81-193)
// ---------------------------------------------------------------------------------------------
namespace {
stride_type to_stride_vector(torch::IntArrayRef v) {
  stride_type out;
  for (auto x : v) {
    TORCH_CHECK(x > 0, "kernel parameters must be positive");
    out.push_back(static_cast<uint32_t>(x));
  }
  return out;
}
}  // namespace

KernelGenerator::KernelGenerator(torch::IntArrayRef kernel_size, torch::IntArrayRef stride, torch::IntArrayRef dilation,
                                 bool is_transpose, RegionType::Type region_type, at::Tensor region_offsets,
                                 bool expand_coordinates, std::vector<RegionType::Type> axis_types, int dimension)
    : kernel_size_(to_stride_vector(kernel_size)), kernel_stride_(to_stride_vector(stride)),
      kernel_dilation_(to_stride_vector(dilation)), is_transpose_(is_transpose), region_type_(region_type),
      region_offsets_(std::move(region_offsets)), expand_coordinates_(expand_coordinates), D_(dimension),
      kernel_volume_(0) {
  if (D_ <= 0) D_ = static_cast<int>(kernel_size_.size());
  if (kernel_size_.size() == 1 && D_ > 1) kernel_size_.assign(D_, kernel_size_[0]);
  if (kernel_stride_.size() == 1 && D_ > 1) kernel_stride_.assign(D_, kernel_stride_[0]);
  if (kernel_dilation_.size() == 1 && D_ > 1) kernel_dilation_.assign(D_, kernel_dilation_[0]);
  TORCH_CHECK(kernel_size_.size() == static_cast<size_t>(D_), "kernel_size dimension mismatch");
  TORCH_CHECK(kernel_stride_.size() == static_cast<size_t>(D_), "kernel_stride dimension mismatch");
  TORCH_CHECK(kernel_dilation_.size() == static_cast<size_t>(D_), "kernel_dilation dimension mismatch");
  TORCH_CHECK(axis_types.empty(), "axis_types must be empty");
  if (region_type_ == RegionType::CUSTOM) {
    TORCH_CHECK(region_offsets_.defined(), "CUSTOM region needs region_offsets");
    region_offsets_ = region_offsets_.to(at::kCPU, at::kInt).reshape({-1, D_}).contiguous();
  } else if (region_offsets_.defined()) {
    TORCH_CHECK(region_offsets_.numel() == 0, "region_offsets must be empty for HYPER_CUBE/HYPER_CROSS");
  }
  auto ks = to_i32(kernel_size_);
  kernel_volume_ = rmn_region_volume(int(region_type_), D_, ks.data(),
                                     region_type_ == RegionType::CUSTOM ? static_cast<int>(region_offsets_.size(0)) : 0);
  TORCH_CHECK(kernel_volume_ > 0, "invalid kernel region");
}

KernelGenerator::KernelParams KernelGenerator::get_kernel(const stride_type& tensor_stride, bool) const {
  TORCH_CHECK(tensor_stride.size() == static_cast<size_t>(D_), "tensor_stride dimension mismatch");
  for (auto s : tensor_stride) TORCH_CHECK(s > 0, "tensor_stride must be positive");
  KernelParams params;
  params.kernel_size = kernel_size_;
  params.kernel_stride = kernel_stride_;
  params.kernel_dilation = kernel_dilation_;
  params.region_type = region_type_;
  params.region_offsets = region_offsets_.defined() ? region_offsets_.clone() : at::Tensor{};
  params.expand_coordinates = expand_coordinates_;
  params.D = D_;
  return params;
}

// ---------------------------------------------------------------------------------------------
// Weight-gradient all-reduce over the ranks (rmn_allreduce_grads)
// ---------------------------------------------------------------------------------------------
namespace {
struct GradientReducer {
  void* comm = nullptr;
  int rank = 0, world = 1;
  bool average = true;
};
GradientReducer g_reducer;
}  // namespace

std::string gradient_allreduce_unique_id() {
  std::string id(RMN_COMM_ID_BYTES, '\0');
  check(rmn_comm_unique_id(id.data()), "rmn_comm_unique_id");
  return id;
}

void init_gradient_allreduce(const std::string& unique_id, int rank, int world_size, bool average) {
  TORCH_CHECK(unique_id.size() == RMN_COMM_ID_BYTES, "the unique id must be ", RMN_COMM_ID_BYTES, " bytes");
  TORCH_CHECK(!g_reducer.comm, "gradient all-reduce is already initialised");
  void* comm = nullptr;
  check(rmn_comm_init(unique_id.data(), rank, world_size, &comm), "rmn_comm_init");
  g_reducer = GradientReducer{comm, rank, world_size, average};
}

void shutdown_gradient_allreduce() {
  if (g_reducer.comm) check(rmn_comm_destroy(g_reducer.comm), "rmn_comm_destroy");
  g_reducer = GradientReducer{};
}

bool gradient_allreduce_active() { return g_reducer.comm != nullptr && g_reducer.world > 1; }
int gradient_allreduce_world_size() { return g_reducer.world; }

void allreduce_gradients(const std::vector<at::Tensor>& gradients) {
  if (!gradient_allreduce_active() || gradients.empty()) return;
  std::vector<float*> bufs;
  std::vector<size_t> counts;
  for (auto const& g : gradients) {
    TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kFloat && g.is_contiguous(),
                "gradients must be contiguous float32 CUDA tensors");
    bufs.push_back(static_cast<float*>(ptr(g)));
    counts.push_back(static_cast<size_t>(g.numel()));
  }
  c10::cuda::CUDAGuard guard(gradients.front().device());
  const size_t ws_bytes = rmn_allreduce_grads_workspace_bytes(counts.data(), static_cast<int>(counts.size()));
  at::Tensor ws;
  if (ws_bytes) ws = at::empty({static_cast<int64_t>(ws_bytes)}, gradients.front().options().dtype(at::kByte));
  check(rmn_allreduce_grads(g_reducer.comm, bufs.data(), counts.data(), static_cast<int>(bufs.size()), ptr(ws),
                            ws_bytes, g_reducer.average ? 1 : 0, g_reducer.world, current_stream()),
        "rmn_allreduce_grads");
}

// ---------------------------------------------------------------------------------------------
// Convolution with a hand-written backward (the reference differentiates the
// index_select / matmul / index_add_ chain through torch autograd, engine/nn/conv.cpp:47-64)
// ---------------------------------------------------------------------------------------------
namespace {

// bias (if defined) is folded into the kernel's epilogue as a per-channel shift
at::Tensor conv_forward(const at::Tensor& feats_in, const at::Tensor& kernel_in, const at::Tensor& nbr,
                        const at::Tensor& bias = at::Tensor(), const at::Tensor& scale_in = at::Tensor(),
                        bool relu = false, const at::Tensor& plan = at::Tensor()) {
  TORCH_CHECK(feats_in.is_cuda() && kernel_in.is_cuda(), "features and kernel must be CUDA tensors");
  TORCH_CHECK(feats_in.scalar_type() == kernel_in.scalar_type(), "expected features and kernel to have the same dtype");
  auto feats = feats_in.contiguous(), kernel = kernel_in.contiguous();
  c10::cuda::CUDAGuard guard(feats.device());
  const int K = static_cast<int>(kernel.size(0)), c_in = static_cast<int>(kernel.size(1)),
            c_out = static_cast<int>(kernel.size(2));
  auto out = at::empty({nbr.size(1), c_out}, feats.options());
  at::Tensor shift;
  if (bias.defined() && bias.numel() > 0) {
    shift = bias.detach().reshape({-1}).to(at::kFloat).contiguous();
    TORCH_CHECK(shift.numel() == c_out, "bias must have one entry per output channel");
  }
  at::Tensor scale;
  if (scale_in.defined() && scale_in.numel() > 0) {
    scale = scale_in.detach().reshape({-1}).to(at::kFloat).contiguous();
    TORCH_CHECK(scale.numel() == c_out, "scale must have one entry per output channel");
  }
  check(rmn_conv_forward_planned(ptr(feats), static_cast<uint32_t>(feats.size(0)), c_in, ptr(kernel), K, c_out,
                                 static_cast<const int32_t*>(ptr(nbr)), ptr(plan), static_cast<uint32_t>(nbr.size(1)),
                                 ptr(out), dtype_code(feats),
                                 scale.defined() ? static_cast<const float*>(ptr(scale)) : nullptr,
                                 static_cast<const float*>(ptr(shift)), relu ? 1 : 0, current_stream()),
        "rmn_conv_forward_planned");
  return out;
}

at::Tensor conv_backward_input(const at::Tensor& grad_in, const at::Tensor& kernel_in, const at::Tensor& nbr_t,
                               const at::Tensor& plan_t = at::Tensor()) {
  auto grad = grad_in.contiguous(), kernel = kernel_in.contiguous();
  c10::cuda::CUDAGuard guard(grad.device());
  const int K = static_cast<int>(kernel.size(0)), c_in = static_cast<int>(kernel.size(1)),
            c_out = static_cast<int>(kernel.size(2));
  auto out = at::empty({nbr_t.size(1), c_in}, grad.options());
  check(rmn_conv_backward_input_planned(ptr(grad), static_cast<uint32_t>(grad.size(0)), c_out, ptr(kernel), K, c_in,
                                        static_cast<const int32_t*>(ptr(nbr_t)), ptr(plan_t),
                                        static_cast<uint32_t>(nbr_t.size(1)), ptr(out), dtype_code(grad),
                                        current_stream()),
        "rmn_conv_backward_input_planned");
  return out;
}

// (reduction channels, output channels) with a tensor-core forward / input-gradient kernel (csrc/rmn_conv_tc.cu);
// the weight-gradient kernels cover the same pairs
bool tc_forward_shape(int64_t c_red, int64_t c_col) {
  static const int64_t shapes[][2] = {{32, 32}, {32, 64}, {64, 32}, {64, 64}, {64, 128}, {128, 64}, {128, 128},
                                      {128, 256}, {256, 128}, {256, 256}};
  for (auto const& sh : shapes)
    if (sh[0] == c_red && sh[1] == c_col) return true;
  return false;
}
// Smallest channel counts >= (c_in, c_out) that the tensor-core kernels take in the forward pass AND, with
// the roles exchanged, in the input-gradient pass; (c_in, c_out) itself when there is none.
std::pair<int64_t, int64_t> tc_legal_shape(int64_t c_in, int64_t c_out) {
  static const int64_t sizes[] = {32, 64, 128, 256};
  std::pair<int64_t, int64_t> best{c_in, c_out};
  int64_t best_cost = -1;
  for (auto ci : sizes)
    for (auto co : sizes)
      if (ci >= c_in && co >= c_out && tc_forward_shape(ci, co) && tc_forward_shape(co, ci) &&
          (best_cost < 0 || ci * co < best_cost)) {
        best = {ci, co};
        best_cost = ci * co;
      }
  return best;
}

at::Tensor conv_backward_weight(const at::Tensor& feats_in, const at::Tensor& grad_in, const at::Tensor& nbr) {
  auto feats = feats_in.contiguous(), grad = grad_in.contiguous();
  c10::cuda::CUDAGuard guard(feats.device());
  const int K = static_cast<int>(nbr.size(0)), c_in = static_cast<int>(feats.size(1)),
            c_out = static_cast<int>(grad.size(1));
  const uint32_t n_dst = static_cast<uint32_t>(nbr.size(1));
  const int code = dtype_code(feats);
  auto dw = at::empty({K, c_in, c_out}, feats.options().dtype(at::kFloat));
  const size_t ws_bytes = rmn_conv_backward_weight_workspace_bytes(n_dst, K, c_in, c_out, code);
  auto ws = at::empty({static_cast<int64_t>(ws_bytes ? ws_bytes : 16)}, feats.options().dtype(at::kByte));
  check(rmn_conv_backward_weight(ptr(feats), static_cast<uint32_t>(feats.size(0)), c_in, ptr(grad), n_dst, c_out,
                                 static_cast<const int32_t*>(ptr(nbr)), K, static_cast<float*>(ptr(dw)), code,
                                 ptr(ws), ws_bytes, current_stream()),
        "rmn_conv_backward_weight");
  return dw;
}

// The neighbour tables travel through autograd as plain (non-differentiable) int32 tensors:
// nbr_out for the forward pass and the weight gradient, nbr_in for the input gradient.
class SparseConvolutionAutograd : public torch::autograd::Function<SparseConvolutionAutograd> {
public:
  // plan_out: plan of nbr_out for this pass; plan_in: plan of nbr_in for the input gradient (empty = none)
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, at::Tensor features, at::Tensor kernel,
                            at::Tensor nbr_out, at::Tensor nbr_in, bool flip_kernel, at::Tensor bias,
                            at::Tensor plan_out, at::Tensor plan_in) {
    ctx->save_for_backward({features, kernel});
    ctx->saved_data["has_bias"] = bias.numel() > 0;
    ctx->saved_data["nbr_out"] = nbr_out;
    ctx->saved_data["nbr_in"] = nbr_in;
    ctx->saved_data["plan_in"] = plan_in;
    ctx->saved_data["flip_kernel"] = flip_kernel;
    return conv_forward(features, kernel, nbr_out, bias, at::Tensor(), false,
                        plan_out.numel() > 0 ? plan_out : at::Tensor());
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grad_outputs) {
    auto saved = ctx->get_saved_variables();
    auto nbr_out = ctx->saved_data["nbr_out"].toTensor();
    auto nbr_in = ctx->saved_data["nbr_in"].toTensor();
    auto grad = grad_outputs[0].contiguous();
    at::Tensor g_feat, g_kernel, g_bias;
    // (needs_input_grad counts the tensor arguments only: features 0, kernel 1, nbr_out 2, nbr_in 3, bias 4)
    const bool want_bias = ctx->saved_data["has_bias"].toBool() && ctx->needs_input_grad(4);
    if (gradient_allreduce_active() && (ctx->needs_input_grad(1) || want_bias)) {
      // Data-parallel: the weight gradient comes first, its all-reduce runs on the second stream and the
      // input gradient on this one; this stream waits for the reduced gradients before handing them on.
      std::vector<at::Tensor> reduce;
      if (ctx->needs_input_grad(1)) reduce.push_back(g_kernel = conv_backward_weight(saved[0], grad, nbr_out));
      if (want_bias) reduce.push_back(g_bias = grad.sum(0, /*keepdim=*/true).to(at::kFloat).contiguous());
      auto main_stream = c10::cuda::getCurrentCUDAStream();
      auto side_stream = pair_list_stream(main_stream.device_index());
      c10::Event ready(c10::DeviceType::CUDA);
      ready.record(main_stream);
      {
        c10::cuda::CUDAStreamGuard on_side(side_stream);
        ready.block(side_stream);
        allreduce_gradients(reduce);
      }
      for (auto const& t : reduce) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), side_stream);
      if (ctx->needs_input_grad(0)) {
        auto plan_in = ctx->saved_data["plan_in"].toTensor();
        g_feat = conv_backward_input(grad, ctx->saved_data["flip_kernel"].toBool() ? saved[1].flip(0) : saved[1], nbr_in,
                                     plan_in.numel() > 0 ? plan_in : at::Tensor());
      }
      c10::Event reduced(c10::DeviceType::CUDA);
      reduced.record(side_stream);
      reduced.block(main_stream);
      if (g_kernel.defined()) g_kernel = g_kernel.to(saved[1].scalar_type());
      if (g_bias.defined()) g_bias = g_bias.to(grad.scalar_type());
      return {g_feat, g_kernel, at::Tensor(), at::Tensor(), at::Tensor(), g_bias, at::Tensor(), at::Tensor()};
    }
    if (ctx->needs_input_grad(0)) {
      auto plan_in = ctx->saved_data["plan_in"].toTensor();
      g_feat = conv_backward_input(grad, ctx->saved_data["flip_kernel"].toBool() ? saved[1].flip(0) : saved[1], nbr_in,
                                   plan_in.numel() > 0 ? plan_in : at::Tensor());
    }
    if (ctx->needs_input_grad(1)) g_kernel = conv_backward_weight(saved[0], grad, nbr_out).to(saved[1].scalar_type());
    if (want_bias) g_bias = grad.sum(0, /*keepdim=*/true);
    return {g_feat, g_kernel, at::Tensor(), at::Tensor(), at::Tensor(), g_bias, at::Tensor(), at::Tensor()};
  }
};

}  // namespace

at::Tensor sparse_convolution(const at::Tensor& features_in, const at::Tensor& kernel_in,
                              const std::shared_ptr<KernelMap>& kmap, const at::Tensor& bias_in) {
  // bf16 channel counts without a tensor-core kernel (a 4-channel stem, 48 or 96 channels ...) are zero-padded
  // to the next pair that has one, with differentiable torch ops around the convolution: padded input channels
  // multiply zero weights, padded output channels are cut off again, and autograd slices the gradients back.
  at::Tensor features = features_in, kernel = kernel_in, bias = bias_in;
  const int64_t c_in = kernel.size(1), c_out = kernel.size(2);
  int64_t pad_out = 0;
  if (features.scalar_type() == at::kBFloat16 && kernel.scalar_type() == at::kBFloat16) {
    auto legal = tc_legal_shape(c_in, c_out);
    if (legal.first != c_in || legal.second != c_out) {
      pad_out = legal.second - c_out;
      features = at::constant_pad_nd(features, {0, legal.first - c_in});
      kernel = at::constant_pad_nd(kernel, {0, pad_out, 0, legal.first - c_in});
      if (bias.defined() && bias.numel() > 0 && pad_out) bias = at::constant_pad_nd(bias, {0, pad_out});
    }
  }
  if (pad_out) {
    auto padded = sparse_convolution(features, kernel, kmap, bias);
    return padded.narrow(1, 0, c_out);
  }
  // the inverse table is cached in the kernel map; it is only needed when the features want a gradient
  at::Tensor nbr_in = kmap->self_symmetric
                          ? kmap->nbr_out
                          : (features.requires_grad() ? kmap->nbr_in() : at::empty({0}, kmap->nbr_out.options()));
  // (autograd functions take defined tensors only: an empty tensor stands for "no bias")
  at::Tensor bias_arg = bias.defined() ? bias : at::empty({0}, kernel.options());
  const int64_t weight = kernel.size(1) * kernel.size(2);
  auto none = at::empty({0}, kmap->nbr_out.options().dtype(at::kByte));
  at::Tensor plan_out, plan_in;
  if (features.scalar_type() == at::kBFloat16) {  // plans serve the tensor-core kernels only
    plan_out = kmap->plan_out(weight);
    if (features.requires_grad()) plan_in = kmap->plan_in(weight);
  }
  return SparseConvolutionAutograd::apply(features, kernel, kmap->nbr_out, nbr_in, kmap->self_symmetric, bias_arg,
                                          plan_out.defined() ? plan_out : none, plan_in.defined() ? plan_in : none);
}

// ---------------------------------------------------------------------------------------------
// Layers (engine/nn/conv.cpp:70-189)
// ---------------------------------------------------------------------------------------------
RiemannConvolutionBaseImpl::RiemannConvolutionBaseImpl(int in_channels, int out_channels, int kernel_size, int stride,
                                                       int dilation, bool bias, bool is_transpose,
                                                       bool expand_coordinates, ConvolutionMode::Type convolution_mode,
                                                       int dimension, RegionType::Type region_type)
    : in_channels_(in_channels), out_channels_(out_channels), is_transpose_(is_transpose), use_mm_(false),
      dimension_(dimension), convolution_mode_(convolution_mode),
      kernel_generator_({kernel_size}, {stride}, {dilation}, is_transpose, region_type, {}, expand_coordinates, {},
                        dimension) {
  TORCH_CHECK(in_channels > 0 && out_channels > 0, "Convolution channel counts must be positive");
  const auto volume = kernel_generator_.kernel_volume();
  kernel_ = register_parameter("kernel", torch::empty({volume, in_channels_, out_channels_}));
  if (bias) bias_ = register_parameter("bias", torch::empty({1, out_channels_}));
  reset_parameters(is_transpose);
}

void RiemannConvolutionBaseImpl::reset() { reset_parameters(is_transpose_); }

void RiemannConvolutionBaseImpl::reset_parameters(bool is_transpose) {
  torch::NoGradGuard guard;
  const auto fan = (is_transpose ? out_channels_ : in_channels_) * kernel_generator_.kernel_volume();
  const auto bound = 1.0 / std::sqrt(static_cast<double>(fan));
  kernel_.uniform_(-bound, bound);
  if (bias_.defined()) bias_.uniform_(-bound, bound);
}

SparseTensor RiemannConvolutionBaseImpl::forward(const SparseTensor& input) {
  TORCH_CHECK(input.dimension() == dimension_, "Input dimension mismatch");
  TORCH_CHECK(input.F().size(1) == in_channels_, "Input channel count does not match convolution");
  const auto params = kernel_generator_.get_kernel(input.tensor_stride(), is_transpose_);
  const auto input_key = input.coordinate_map_key().get_key();
  auto output_stride = input_key.first;
  for (size_t axis = 0; axis < output_stride.size(); ++axis) {
    const auto step = params.kernel_stride[axis];
    if (is_transpose_) {
      TORCH_CHECK(step != 0 && output_stride[axis] % step == 0,
                  "Transpose convolution stride must divide tensor stride");
      output_stride[axis] /= step;
    } else {
      output_stride[axis] *= step;
    }
  }
  CoordinateMapKey output_key(static_cast<size_type>(input.coordinate_map_key().get_coordinate_size()),
                              {output_stride, input_key.second});
  auto manager = input.coordinate_manager();
  if (!is_transpose_ && params.kernel_stride != stride_type(dimension_, 1))
    output_key = manager->stride(input.coordinate_map_key(), params.kernel_stride);
  // Generative transposed convolution: the output coordinates are generated, every input voxel spawning its
  // whole kernel region on the output stride (stride_region: engine/grid/space_impl.hpp:362-380,
  // engine/grid/lattice_cpu.hpp:499-534), instead of being looked up among the maps that exist. (The
  // reference's layer carries the flag but its forward never reaches stride_region, engine/nn/conv.cpp:104-138,
  // 173-189; its pooling-transpose layer does, and this follows that path.)
  if (is_transpose_ && kernel_generator_.expand_coordinates())
    output_key = manager->stride_region(input.coordinate_map_key(), params.kernel_size, params.kernel_dilation,
                                        output_stride, params.region_type, params.region_offsets);
  auto kmap = manager->kernel_map(input.coordinate_map_key(), output_key, params.kernel_size, params.kernel_stride,
                                  params.kernel_dilation, params.region_type, params.region_offsets, is_transpose_,
                                  false);
  if (fold_scale_.defined() || fold_shift_.defined() || fold_relu_) {  // set by fused_conv_bn_relu for one call
    torch::NoGradGuard guard;
    at::Tensor plan;
    if (input.F().scalar_type() == at::kBFloat16) plan = kmap->plan_out(int64_t(in_channels_) * out_channels_);
    auto result = conv_forward(input.F(), kernel_, kmap->nbr_out, fold_shift_, fold_scale_, fold_relu_, plan);
    return SparseTensor(std::move(result), output_key, std::move(manager));
  }
  auto result = sparse_convolution(input.F(), kernel_, kmap, bias_);  // the bias add is fused into the epilogue
  return SparseTensor(std::move(result), output_key, std::move(manager));
}

// conv -> batch norm (running statistics) -> ReLU as ONE kernel (inference): the norm's affine and the
// layer's bias are folded into the convolution epilogue (engine/nn/residual.cpp:44-52 runs three modules).
SparseTensor fused_conv_bn_relu(const SparseTensor& input, RiemannConvolutionBaseImpl& conv,
                                torch::nn::BatchNorm1d bn, bool relu) {
  torch::NoGradGuard guard;
  at::Tensor scale, shift;
  at::Tensor bias = conv.bias_.defined() ? conv.bias_.reshape({-1}).to(at::kFloat) : at::Tensor();
  if (!bn.is_empty()) {
    TORCH_CHECK(!bn->is_training(), "fused_conv_bn_relu folds running statistics: call bn->eval() first");
    TORCH_CHECK(bn->running_var.defined(), "fused_conv_bn_relu needs running statistics");
    auto inv = torch::rsqrt(bn->running_var.to(at::kFloat) + bn->options.eps());
    scale = bn->weight.defined() ? inv * bn->weight.to(at::kFloat) : inv;
    shift = -bn->running_mean.to(at::kFloat) * scale;
    if (bn->bias.defined()) shift = shift + bn->bias.to(at::kFloat);
    if (bias.defined()) shift = shift + bias * scale;
  } else {
    shift = bias;
  }
  conv.fold_scale_ = scale;
  conv.fold_shift_ = shift;
  conv.fold_relu_ = relu;
  try {
    auto out = conv.forward(input);
    conv.fold_scale_ = at::Tensor();
    conv.fold_shift_ = at::Tensor();
    conv.fold_relu_ = false;
    return out;
  } catch (...) {
    conv.fold_scale_ = at::Tensor();
    conv.fold_shift_ = at::Tensor();
    conv.fold_relu_ = false;
    throw;
  }
}

RiemannBatchNormImpl::RiemannBatchNormImpl(int64_t num_features, double eps, double momentum, bool affine,
                                           bool track_running_stats)
    : normalization_(register_module(
          "normalization", torch::nn::BatchNorm1d(torch::nn::BatchNorm1dOptions(num_features)
                                                      .eps(eps)
                                                      .momentum(momentum)
                                                      .affine(affine)
                                                      .track_running_stats(track_running_stats)))) {}

namespace {
// Training-mode batch norm of a feature matrix as three streaming passes forward (sums, coefficients,
// normalise) and three backward (sums of dy and dy * x, coefficients, input gradient), in place of torch's
// BatchNorm1d kernels, which run narrow channels-last matrices at a fraction of memory speed. Same arithmetic
// (batch mean, biased variance, running statistics with momentum and the unbiased variance).
class BatchNormAutograd : public torch::autograd::Function<BatchNormAutograd> {
public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, at::Tensor x_in, at::Tensor gamma, at::Tensor beta,
                            at::Tensor running_mean, at::Tensor running_var, double momentum, double eps) {
    auto x = x_in.contiguous();
    c10::cuda::CUDAGuard guard(x.device());
    const uint32_t n = static_cast<uint32_t>(x.size(0));
    const int C = static_cast<int>(x.size(1));
    const int code = dtype_code(x);
    auto f32 = x.options().dtype(at::kFloat);
    auto stats = at::empty({2, C}, x.options().dtype(at::kDouble));
    const size_t ws_bytes = rmn_channel_dot_stats_workspace_bytes(C);
    auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, x.options().dtype(at::kByte));
    check(rmn_channel_dot_stats(ptr(x), ptr(x), n, C, code, static_cast<double*>(ptr(stats)), ptr(ws), ws_bytes,
                                current_stream()),
          "rmn_channel_dot_stats");
    auto coeffs = at::empty({4, C}, f32);  // scale, shift, mean, 1 / sqrt(var + eps)
    float* co = static_cast<float*>(ptr(coeffs));
    const at::Tensor& any_param = gamma.numel() ? gamma : (running_mean.numel() ? running_mean : beta);
    const int pcode = any_param.numel() && any_param.scalar_type() == at::kBFloat16 ? RMN_BF16 : RMN_F32;
    check(rmn_bn_forward_coeffs(static_cast<const double*>(ptr(stats)), static_cast<double>(n), ptr(gamma), ptr(beta),
                                ptr(running_mean), ptr(running_var), pcode, static_cast<float>(momentum),
                                static_cast<float>(eps), C, co, co + C, co + 2 * C, co + 3 * C, current_stream()),
          "rmn_bn_forward_coeffs");
    auto y = at::empty_like(x);
    check(rmn_affine_act(ptr(x), n, C, co, co + C, 0, ptr(y), code, current_stream()), "rmn_affine_act");
    ctx->save_for_backward({x, gamma, coeffs});
    return y;
  }

  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grad_outputs) {
    auto saved = ctx->get_saved_variables();
    auto x = saved[0], gamma = saved[1], coeffs = saved[2];
    auto dy = grad_outputs[0].contiguous();
    c10::cuda::CUDAGuard guard(x.device());
    const uint32_t n = static_cast<uint32_t>(x.size(0));
    const int C = static_cast<int>(x.size(1));
    const int code = dtype_code(x);
    auto dots = at::empty({2, C}, x.options().dtype(at::kDouble));
    const size_t ws_bytes = rmn_channel_dot_stats_workspace_bytes(C);
    auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, x.options().dtype(at::kByte));
    check(rmn_channel_dot_stats(ptr(dy), ptr(x), n, C, code, static_cast<double*>(ptr(dots)), ptr(ws), ws_bytes,
                                current_stream()),
          "rmn_channel_dot_stats");
    auto back = at::empty({5, C}, coeffs.options());  // c_dy, c_x, c_0, dgamma, dbeta
    float* bk = static_cast<float*>(ptr(back));
    const float* co = static_cast<const float*>(ptr(coeffs));
    const int pcode = gamma.numel() && gamma.scalar_type() == at::kBFloat16 ? RMN_BF16 : RMN_F32;
    check(rmn_bn_backward_coeffs(static_cast<const double*>(ptr(dots)), co + 2 * C, co + 3 * C, ptr(gamma), pcode,
                                 static_cast<double>(n), C, bk, bk + C, bk + 2 * C, bk + 3 * C, bk + 4 * C,
                                 current_stream()),
          "rmn_bn_backward_coeffs");
    auto dx = at::empty_like(x);
    check(rmn_affine2(ptr(dy), ptr(x), n, C, bk, bk + C, bk + 2 * C, ptr(dx), code, current_stream()), "rmn_affine2");
    at::Tensor dgamma, dbeta;
    if (ctx->needs_input_grad(1)) dgamma = back[3].to(gamma.scalar_type());
    if (ctx->needs_input_grad(2)) dbeta = back[4].to(gamma.numel() ? gamma.scalar_type() : x.scalar_type());
    return {dx, dgamma, dbeta, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

// shapes rmn_channel_dot_stats / rmn_affine2 take: 16-byte lanes, a power-of-two number of them (<= 32) per row
bool bn_fast_shape(const at::Tensor& x) {
  if (!x.is_cuda() || x.dim() != 2 || x.size(0) == 0) return false;
  if (x.scalar_type() != at::kFloat && x.scalar_type() != at::kBFloat16) return false;
  const int64_t lanes16 = x.size(1) * x.element_size() / 16;
  return x.size(1) * x.element_size() % 16 == 0 && lanes16 >= 1 && lanes16 <= 32 && (32 % lanes16) == 0;
}
}  // namespace

SparseTensor RiemannBatchNormImpl::forward(const SparseTensor& input) {
  auto& bn = normalization_;
  const auto momentum = bn->options.momentum();
  at::Tensor values;
  if (bn->is_training() && momentum.has_value() && bn_fast_shape(input.F())) {
    auto none = at::empty({0}, input.F().options());
    values = BatchNormAutograd::apply(input.F(), bn->weight.defined() ? bn->weight : none,
                                      bn->bias.defined() ? bn->bias : none,
                                      bn->running_mean.defined() ? bn->running_mean : none,
                                      bn->running_var.defined() ? bn->running_var : none, *momentum, bn->options.eps());
    if (bn->num_batches_tracked.defined()) {
      torch::NoGradGuard guard;
      bn->num_batches_tracked += 1;
    }
  } else {
    values = bn->forward(input.F());  // evaluation mode and shapes without a streaming kernel: torch's layer
  }
  return SparseTensor(std::move(values), input.coordinate_map_key(), input.coordinate_manager());
}

RiemannConvolutionImpl::RiemannConvolutionImpl(int in_channels, int out_channels, int kernel_size, int stride,
                                               int dilation, bool bias, bool expand_coordinates,
                                               ConvolutionMode::Type convolution_mode, int dimension) {
  base_ = std::make_shared<RiemannConvolutionBaseImpl>(in_channels, out_channels, kernel_size, stride, dilation, bias,
                                                       false, expand_coordinates, convolution_mode, dimension);
  register_module("base", base_);
}

RiemannConvolutionTransposeImpl::RiemannConvolutionTransposeImpl(int in_channels, int out_channels, int kernel_size,
                                                                 int stride, int dilation, bool bias,
                                                                 bool expand_coordinates,
                                                                 ConvolutionMode::Type convolution_mode,
                                                                 int dimension) {
  base_ = std::make_shared<RiemannConvolutionBaseImpl>(in_channels, out_channels, kernel_size, stride, dilation, bias,
                                                       true, expand_coordinates, convolution_mode, dimension);
  register_module("base", base_);
}

RiemannGenerativeConvolutionTransposeImpl::RiemannGenerativeConvolutionTransposeImpl(
    int in_channels, int out_channels, int kernel_size, int stride, int dilation, bool bias,
    ConvolutionMode::Type convolution_mode, int dimension) {
  base_ = std::make_shared<RiemannConvolutionBaseImpl>(in_channels, out_channels, kernel_size, stride, dilation, bias,
                                                       true, true, convolution_mode, dimension);
  register_module("base", base_);
}

// ---------------------------------------------------------------------------------------------
// ConvolutionFunction helpers (autodiff/compat.hpp:86-156)
// ---------------------------------------------------------------------------------------------
namespace {
std::vector<int64_t> to_int64(const stride_type& s) { return std::vector<int64_t>(s.begin(), s.end()); }

at::Tensor run_function(bool transpose, at::Tensor input_features, at::Tensor kernel, const stride_type& kernel_size,
                        const stride_type& kernel_stride, const stride_type& kernel_dilation,
                        RegionType::Type region_type, at::Tensor region_offsets, bool expand_coordinates,
                        ConvolutionMode::Type conv_mode, std::shared_ptr<CoordinateMapKey> in_key,
                        std::shared_ptr<CoordinateMapKey> out_key, std::shared_ptr<CoordinateManager> manager) {
  TORCH_CHECK(kernel.dim() == 3, "Convolution kernel must have shape [kernel, in, out]");
  TORCH_CHECK(kernel.size(1) == input_features.size(1), "Convolution kernel input channels do not match features");
  TORCH_CHECK(in_key && in_key->is_key_set(), "input key must be set");
  const int dimension = static_cast<int>(in_key->get_coordinate_size()) - 1;
  SparseTensor input(input_features, *in_key, manager);
  RiemannConvolutionBaseImpl layer(static_cast<int>(input_features.size(1)), static_cast<int>(kernel.size(2)), 1, 1,
                                   1, false, transpose, expand_coordinates, conv_mode, dimension, region_type);
  layer.kernel_generator_ = KernelGenerator(to_int64(kernel_size), to_int64(kernel_stride), to_int64(kernel_dilation),
                                            transpose, region_type, std::move(region_offsets), expand_coordinates, {},
                                            dimension);
  TORCH_CHECK(kernel.size(0) == layer.kernel_generator_.kernel_volume(),
              "Convolution kernel volume does not match its geometry");
  layer.kernel_ = std::move(kernel);
  auto output = layer.forward(input);
  if (out_key) out_key->set_key(output.coordinate_map_key().get_key());
  return output.F();
}
}  // namespace

at::Tensor ConvolutionFunction::apply(at::Tensor input_features, at::Tensor kernel, stride_type kernel_size,
                                      stride_type kernel_stride, stride_type kernel_dilation,
                                      RegionType::Type region_type, at::Tensor region_offsets, bool expand_coordinates,
                                      ConvolutionMode::Type conv_mode, std::shared_ptr<CoordinateMapKey> in_key,
                                      std::shared_ptr<CoordinateMapKey> out_key,
                                      std::shared_ptr<CoordinateManager> manager) {
  return run_function(false, std::move(input_features), std::move(kernel), kernel_size, kernel_stride, kernel_dilation,
                      region_type, std::move(region_offsets), expand_coordinates, conv_mode, std::move(in_key),
                      std::move(out_key), std::move(manager));
}

at::Tensor ConvolutionTransposeFunction::apply(at::Tensor input_features, at::Tensor kernel, stride_type kernel_size,
                                               stride_type kernel_stride, stride_type kernel_dilation,
                                               RegionType::Type region_type, at::Tensor region_offsets,
                                               bool expand_coordinates, ConvolutionMode::Type conv_mode,
                                               std::shared_ptr<CoordinateMapKey> in_key,
                                               std::shared_ptr<CoordinateMapKey> out_key,
                                               std::shared_ptr<CoordinateManager> manager) {
  return run_function(true, std::move(input_features), std::move(kernel), kernel_size, kernel_stride, kernel_dilation,
                      region_type, std::move(region_offsets), expand_coordinates, conv_mode, std::move(in_key),
                      std::move(out_key), std::move(manager));
}

}  // namespace riemann

// ---------------------------------------------------------------------------------------------
// Local pooling (engine/nn/pooling.cpp:80-144, 166-195)
// ---------------------------------------------------------------------------------------------
namespace riemann {
namespace {

int pool_code(PoolingMode::Type mode) {
  switch (mode) {
    case PoolingMode::LOCAL_SUM_POOLING: return RMN_POOL_SUM;
    case PoolingMode::LOCAL_AVG_POOLING: return RMN_POOL_AVG;
    case PoolingMode::LOCAL_MAX_POOLING: return RMN_POOL_MAX;
    default: TORCH_CHECK(false, "Local pooling requires a local pooling mode");
  }
}

class SparsePoolingAutograd : public torch::autograd::Function<SparsePoolingAutograd> {
public:
  // nbr_in is the inverse table (empty when no gradient is wanted); aux is filled by the forward kernel
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, at::Tensor features, at::Tensor nbr_out,
                            at::Tensor nbr_in, int64_t mode) {
    TORCH_CHECK(features.is_cuda(), "features must be CUDA tensors: this library has no CPU path");
    TORCH_CHECK(features.is_floating_point(), "Sparse pooling requires floating-point features");
    auto feats = features.contiguous();
    c10::cuda::CUDAGuard guard(feats.device());
    const int64_t n_dst = nbr_out.size(1), C = feats.size(1);
    auto out = at::empty({n_dst, C}, feats.options());
    at::Tensor aux;
    if (nbr_in.numel() > 0 && mode == RMN_POOL_AVG) aux = at::empty({n_dst}, nbr_out.options());
    if (nbr_in.numel() > 0 && mode == RMN_POOL_MAX) aux = at::empty({n_dst, C}, nbr_out.options());
    check(rmn_pool_forward(ptr(feats), static_cast<uint32_t>(feats.size(0)), static_cast<int>(C),
                           static_cast<const int32_t*>(ptr(nbr_out)), static_cast<int>(nbr_out.size(0)),
                           static_cast<uint32_t>(n_dst), static_cast<int>(mode), ptr(out),
                           aux.defined() ? static_cast<int32_t*>(ptr(aux)) : nullptr, dtype_code(feats),
                           current_stream()),
          "rmn_pool_forward");
    ctx->saved_data["nbr_in"] = nbr_in;
    ctx->saved_data["aux"] = aux.defined() ? aux : at::empty({0}, nbr_out.options());
    ctx->saved_data["mode"] = mode;
    return out;
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grad_outputs) {
    auto nbr_in = ctx->saved_data["nbr_in"].toTensor();
    auto aux = ctx->saved_data["aux"].toTensor();
    const int64_t mode = ctx->saved_data["mode"].toInt();
    auto grad = grad_outputs[0].contiguous();
    c10::cuda::CUDAGuard guard(grad.device());
    auto g_feat = at::empty({nbr_in.size(1), grad.size(1)}, grad.options());
    check(rmn_pool_backward(ptr(grad), static_cast<uint32_t>(grad.size(0)), static_cast<int>(grad.size(1)),
                            static_cast<const int32_t*>(ptr(nbr_in)), static_cast<int>(nbr_in.size(0)),
                            static_cast<uint32_t>(nbr_in.size(1)), static_cast<int>(mode),
                            aux.numel() ? static_cast<const int32_t*>(ptr(aux)) : nullptr, ptr(g_feat),
                            dtype_code(grad), current_stream()),
          "rmn_pool_backward");
    return {g_feat, at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

}  // namespace

at::Tensor sparse_pooling(const at::Tensor& features, const std::shared_ptr<KernelMap>& kmap, PoolingMode::Type mode) {
  at::Tensor nbr_in = features.requires_grad() ? kmap->nbr_in() : at::empty({0}, kmap->nbr_out.options());
  return SparsePoolingAutograd::apply(features, kmap->nbr_out, nbr_in, static_cast<int64_t>(pool_code(mode)));
}

RiemannPoolingBaseImpl::RiemannPoolingBaseImpl(int kernel_size, int stride, int dilation, PoolingMode::Type mode,
                                               int dimension)
    : kernel_generator_({kernel_size}, {stride}, {dilation}, false, RegionType::HYPER_CUBE, {}, false, {}, dimension),
      mode_(mode), dimension_(dimension) {
  pool_code(mode);
}

RiemannPoolingBaseImpl::RiemannPoolingBaseImpl(KernelGenerator kernel_generator, PoolingMode::Type mode, int dimension)
    : kernel_generator_(std::move(kernel_generator)), mode_(mode), dimension_(dimension) {
  pool_code(mode);
}

RiemannPoolingTransposeImpl::RiemannPoolingTransposeImpl(int kernel_size, int stride, int dilation,
                                                         bool expand_coordinates, int dimension)
    : kernel_generator_({kernel_size}, {stride}, {dilation}, true, RegionType::HYPER_CUBE, {}, expand_coordinates, {},
                        dimension),
      dimension_(dimension) {}

RiemannPoolingTransposeImpl::RiemannPoolingTransposeImpl(KernelGenerator kernel_generator, int dimension,
                                                         PoolingMode::Type mode)
    : kernel_generator_(std::move(kernel_generator)), dimension_(dimension), mode_(mode) {
  pool_code(mode);
}

SparseTensor RiemannPoolingTransposeImpl::forward(const SparseTensor& input) {
  TORCH_CHECK(input.dimension() == dimension_, "Input dimension mismatch");
  const auto params = kernel_generator_.get_kernel(input.tensor_stride(), true);
  const auto in_stride = input.tensor_stride();
  stride_type out_stride(in_stride);
  for (size_t axis = 0; axis < out_stride.size(); ++axis) {
    const auto step = params.kernel_stride[axis];
    TORCH_CHECK(step != 0 && out_stride[axis] % step == 0, "Transpose stride must divide tensor stride");
    out_stride[axis] /= step;
  }
  auto manager = input.coordinate_manager();
  // a map of the output stride that exists already (the input's own) is reused unless coordinates are expanded
  CoordinateMapKey output_key =
      (out_stride == in_stride && !kernel_generator_.expand_coordinates())
          ? input.coordinate_map_key()
          : manager->stride_region(input.coordinate_map_key(), params.kernel_size, params.kernel_dilation, out_stride,
                                   params.region_type, params.region_offsets);
  auto kmap = manager->kernel_map(input.coordinate_map_key(), output_key, params.kernel_size, params.kernel_stride,
                                  params.kernel_dilation, params.region_type, params.region_offsets, true, true);
  auto result = sparse_pooling(input.F(), kmap, mode_);
  return SparseTensor(std::move(result), output_key, std::move(manager));
}

SparseTensor RiemannPoolingBaseImpl::forward(const SparseTensor& input) {
  TORCH_CHECK(input.dimension() == dimension_, "Input dimension mismatch");
  const auto params = kernel_generator_.get_kernel(input.tensor_stride(), false);
  auto manager = input.coordinate_manager();
  auto output_key = manager->stride(input.coordinate_map_key(), params.kernel_stride);
  auto kmap = manager->kernel_map(input.coordinate_map_key(), output_key, params.kernel_size, params.kernel_stride,
                                  params.kernel_dilation, params.region_type, params.region_offsets, false, true);
  auto result = sparse_pooling(input.F(), kmap, mode_);
  return SparseTensor(std::move(result), output_key, std::move(manager));
}

}  // namespace riemann
