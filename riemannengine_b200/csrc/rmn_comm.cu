// Weight-gradient all-reduce: the one collective of the data-parallel hot path.
//
// Batches shard by sample, so the forward pass and both gradient passes are local to a rank;
// only the weight gradients [K, C_in, C_out] (fp32) are summed over the ranks. The buffers of
// a step are packed into one flat fp32 bucket by one kernel, reduced by ONE ncclAllReduce over
// NVLink (a 3^3 64 -> 64 layer is 442 KB: latency-bound, so one call, not one per tensor) and
// unpacked (optionally averaged) by one kernel. The reference has no distributed code (its
// RiemannSyncBatchNorm is an alias of the plain layer, engine/nn/normalization.hpp:36-37).
//
// NCCL is looked up at run time (dlopen of libnccl.so.2: in a process that has loaded torch it
// resolves to the copy torch already loaded), so the library itself loads on machines without
// NCCL and every other entry point works there.
#include "rmn_common.cuh"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <mutex>

namespace rmn {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  bool ok = false;
};

static const NcclApi& nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the process already uses, if any
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce;
  });
  return api;
}

constexpr int kMaxBufs = 120;  // buffers per pack / unpack launch (kernel parameter space)

struct BufList {
  float* ptr[kMaxBufs];
  unsigned long long begin[kMaxBufs + 1];  // element offsets into the flat bucket
  int n;
};

// direction 0: bufs -> flat; 1: flat * scale -> bufs. One block walks one 4096-element slice of the bucket.
__global__ void __launch_bounds__(256) k_bucket_copy(BufList list, float* __restrict__ flat, int direction,
                                                     float scale) {
  const unsigned long long base = list.begin[0];
  const unsigned long long total = list.begin[list.n] - base;
  const unsigned long long e0 = (unsigned long long)blockIdx.x * 4096ull;
  int b = 0;
  for (unsigned long long e = e0 + threadIdx.x; e < min(total, e0 + 4096ull); e += 256) {
    const unsigned long long g = base + e;
    while (g >= list.begin[b + 1]) ++b;  // monotone in e: amortised constant
    float* p = list.ptr[b] + (g - list.begin[b]);
    if (direction == 0) flat[g] = *p;
    else *p = flat[g] * scale;
  }
}

}  // namespace rmn

using namespace rmn;

extern "C" int rmn_comm_unique_id(void* id_out) {
  if (!id_out) return RMN_ERR_BAD_ARG;
  const NcclApi& api = nccl_api();
  if (!api.ok) return RMN_ERR_UNSUPPORTED;
  static_assert(sizeof(ncclUniqueId) == RMN_COMM_ID_BYTES, "unique id size");
  return api.GetUniqueId(static_cast<ncclUniqueId*>(id_out)) == ncclSuccess ? RMN_OK : RMN_ERR_CUDA;
}

extern "C" int rmn_comm_init(const void* id, int rank, int world_size, void** comm_out) {
  if (!id || !comm_out || world_size < 1 || rank < 0 || rank >= world_size) return RMN_ERR_BAD_ARG;
  const NcclApi& api = nccl_api();
  if (!api.ok) return RMN_ERR_UNSUPPORTED;
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  ncclComm_t comm = nullptr;
  if (api.CommInitRank(&comm, world_size, uid, rank) != ncclSuccess) return RMN_ERR_CUDA;
  *comm_out = comm;
  return RMN_OK;
}

extern "C" int rmn_comm_destroy(void* comm) {
  if (!comm) return RMN_OK;
  const NcclApi& api = nccl_api();
  if (!api.ok) return RMN_ERR_UNSUPPORTED;
  return api.CommDestroy(static_cast<ncclComm_t>(comm)) == ncclSuccess ? RMN_OK : RMN_ERR_CUDA;
}

extern "C" size_t rmn_allreduce_grads_workspace_bytes(const size_t* counts, int n_bufs) {
  if (!counts || n_bufs < 1) return 0;
  size_t total = 0;
  for (int i = 0; i < n_bufs; ++i) total += counts[i];
  return n_bufs == 1 ? 0 : total * sizeof(float);
}

extern "C" int rmn_allreduce_grads(void* comm, float* const* d_bufs, const size_t* counts, int n_bufs,
                                   void* d_workspace, size_t workspace_bytes, int average, int world_size,
                                   void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_bufs < 0 || world_size < 1 || (n_bufs > 0 && (!d_bufs || !counts))) return RMN_ERR_BAD_ARG;
  if (n_bufs == 0 || world_size == 1) return RMN_OK;  // one rank: the local gradients are the sum
  if (!comm) return RMN_ERR_BAD_ARG;
  const NcclApi& api = nccl_api();
  if (!api.ok) return RMN_ERR_UNSUPPORTED;
  size_t total = 0;
  for (int i = 0; i < n_bufs; ++i) {
    if (counts[i] > 0 && !d_bufs[i]) return RMN_ERR_BAD_ARG;
    total += counts[i];
  }
  if (total == 0) return RMN_OK;
  const float scale = average ? 1.0f / (float)world_size : 1.0f;
  float* flat = static_cast<float*>(d_workspace);
  if (n_bufs == 1) {
    flat = d_bufs[0];  // a single buffer is reduced in place
  } else {
    if (!d_workspace || ((uintptr_t)d_workspace & 15)) return RMN_ERR_BAD_ARG;
    if (workspace_bytes < total * sizeof(float)) return RMN_ERR_ALLOC;
  }
  auto copy_all = [&](int direction) -> int {
    size_t begin = 0;
    for (int first = 0; first < n_bufs; first += kMaxBufs) {
      BufList list;
      list.n = n_bufs - first < kMaxBufs ? n_bufs - first : kMaxBufs;
      size_t pos = begin;
      for (int i = 0; i < list.n; ++i) {
        list.ptr[i] = d_bufs[first + i];
        list.begin[i] = pos;
        pos += counts[first + i];
      }
      list.begin[list.n] = pos;
      const size_t elems = pos - begin;
      if (elems > 0) {
        k_bucket_copy<<<(unsigned)((elems + 4095) / 4096), 256, 0, stream>>>(list, flat, direction, scale);
        RMN_LAUNCH_CHECK();
      }
      begin = pos;
    }
    return RMN_OK;
  };
  if (n_bufs > 1) {
    const int rc = copy_all(0);
    if (rc != RMN_OK) return rc;
  }
  if (api.AllReduce(flat, flat, total, ncclFloat, ncclSum, static_cast<ncclComm_t>(comm), stream) != ncclSuccess)
    return RMN_ERR_CUDA;
  if (n_bufs > 1) return copy_all(1);
  if (average) {  // single buffer: scale in place
    BufList list;
    list.n = 1;
    list.ptr[0] = flat;
    list.begin[0] = 0;
    list.begin[1] = total;
    k_bucket_copy<<<(unsigned)((total + 4095) / 4096), 256, 0, stream>>>(list, flat, 1, scale);
    RMN_LAUNCH_CHECK();
  }
  return RMN_OK;
}
