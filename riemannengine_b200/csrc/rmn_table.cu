// Coordinate hash table: dedup insert with first-occurrence numbering, lookup,
// stride alignment. Integer work bound by HBM/L2 bandwidth.
//
// Build pipeline (all on the caller's stream, no host synchronisation):
//   256-byte memset of the header
//   -> fill + range (slots to the empty pattern, column min/max; the last block plans the bit packing)
//   -> insert (one 16-byte CAS on the packed key, atomicMin on the first row)
//   -> count (rows that are the first occurrence, per 256-row block; the last block scans the counts)
//   -> finalize (unique ids, mapping, unique coordinates; identity inverse when nothing was a duplicate)
//   -> inverse (only does work when there were duplicates)
// Numbering unique rows by first occurrence reproduces the reference CPU map
// (engine/grid/lattice_cpu.hpp:419-444) deterministically; the reference GPU
// map lets a CAS race pick the surviving duplicate
// (engine/grid/lattice_gpu.cu:30-51).
#include "rmn_common.cuh"

#include <cuda_bf16.h>

#include <limits.h>
#include <stddef.h>

#include <mutex>

namespace rmn {

int tc_copy_status_async(uint32_t* host_dst, cudaStream_t stream);  // rmn_conv_tc.cu
int tc_clear_status();
const uint32_t* tc_status_device_address();

constexpr int kRowsPerBlock = 256;

__device__ void plan_packing(TableHeader* h);

// First kernel of a build, on a header that a 256-byte memset has zeroed: fills the slots with the empty
// pattern (all ones) and reduces the column bounds of the rows in the same pass (the fill writes, the
// reduction reads: one launch moves both at HBM speed). The last block to finish writes the header's
// constants, decodes the bounds and plans the key packing.
template <int W>
__global__ void __launch_bounds__(256) k_fill_range(const int32_t* __restrict__ coords, uint32_t n,
                                                    TableHeader* h, uint4* __restrict__ slots, uint32_t capacity) {
  __shared__ int32_t s_mn[8][W], s_mx[8][W];
  __shared__ uint32_t s_or[8];
  const uint4 ones = make_uint4(~0u, ~0u, ~0u, ~0u);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += gridDim.x * blockDim.x)
    slots[i] = ones;
  int32_t mn[W], mx[W];
#pragma unroll
  for (int c = 0; c < W; ++c) { mn[c] = INT_MAX; mx[c] = INT_MIN; }
  // OR of (x - x of row 0) over the rows: its trailing zeros are the bits of the first spatial
  // column that all rows share
  const uint32_t x0 = n > 0 ? (uint32_t)__ldg(coords + 1) : 0u;
  uint32_t x_or = 0;
  for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    int32_t v[W];
    load_row<W>(coords, r, v);
#pragma unroll
    for (int c = 0; c < W; ++c) { mn[c] = min(mn[c], v[c]); mx[c] = max(mx[c], v[c]); }
    x_or |= (uint32_t)v[1] - x0;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int c = 0; c < W; ++c) {
    const int32_t a = __reduce_min_sync(0xFFFFFFFFu, mn[c]);
    const int32_t b = __reduce_max_sync(0xFFFFFFFFu, mx[c]);
    if (lane == 0) { s_mn[warp][c] = a; s_mx[warp][c] = b; }
  }
  x_or = __reduce_or_sync(0xFFFFFFFFu, x_or);
  if (lane == 0) s_or[warp] = x_or;
  __syncthreads();
  // one atomic per block and column (per-warp atomics on eight addresses serialise badly); blocks that
  // saw no row leave the zero ("no row yet") in place
  if (threadIdx.x < W && blockIdx.x * blockDim.x < n) {
    int32_t a = s_mn[0][threadIdx.x], b = s_mx[0][threadIdx.x];
#pragma unroll
    for (int w2 = 1; w2 < 8; ++w2) { a = min(a, s_mn[w2][threadIdx.x]); b = max(b, s_mx[w2][threadIdx.x]); }
    atomicMax(&h->mn_enc[threadIdx.x], ~((uint32_t)a ^ 0x80000000u));
    atomicMax(&h->mx_enc[threadIdx.x], (uint32_t)b ^ 0x80000000u);
  }
  if (threadIdx.x == 32 && blockIdx.x * blockDim.x < n) {
    uint32_t o = 0;
#pragma unroll
    for (int w2 = 0; w2 < 8; ++w2) o |= s_or[w2];
    if (o) atomicOr(&h->x_or, o);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(&h->range_blocks_done, 1u) == gridDim.x - 1) {
    __threadfence();
    h->magic = kTableMagic;
    h->W = W;
    h->n_rows = n;
    h->capacity = capacity;
    for (int c = 0; c < RMN_MAX_W; ++c) {
      // volatile: the bounds were written by other blocks' atomics
      const uint32_t en = *(volatile uint32_t*)&h->mn_enc[c], ex = *(volatile uint32_t*)&h->mx_enc[c];
      h->mn[c] = (c < W && n > 0) ? (int32_t)(~en ^ 0x80000000u) : 0;
      h->mx[c] = (c < W && n > 0) ? (int32_t)(ex ^ 0x80000000u) : 0;
      h->bits[c] = 0;
      h->shift[c] = 0;
    }
    {
      const uint32_t o = *(volatile uint32_t*)&h->x_or;
      h->pos_shift = o ? (uint32_t)(__ffs((int)o) - 1) : 0u;
    }
    plan_packing(h);
  }
}

// One thread: bit widths and shifts of the packed key from the bounding box in the header.
__device__ void plan_packing(TableHeader* h) {
  uint32_t total = 0;
  // packing order: spatial columns first (column 1 in the lowest bits: its low three bits pick
  // the position inside a bucket), the batch column last
  for (uint32_t i = 0; i < h->W; ++i) {
    const uint32_t c = i + 1 < h->W ? i + 1 : 0;
    uint32_t b = 0;
    if (h->n_rows > 0) {
      const uint32_t span = (uint32_t)h->mx[c] - (uint32_t)h->mn[c];
      b = span == 0 ? 0 : 32 - __clz(span);
    }  // empty table: bounds are zero and every probe ends on a free slot
    h->bits[c] = b;
    h->shift[c] = total > 63 ? 63 : total;
    total += b;
  }
  h->total_bits = total;
  if (total > 63) h->status = RMN_ERR_RANGE;
}

// 16-byte atomic compare-and-swap of a whole slot against the empty pattern (all ones); returns
// the slot's previous content.
__device__ __forceinline__ void cas_slot(Slot* slot, unsigned long long key, unsigned long long rows,
                                         unsigned long long& old_key, unsigned long long& old_rows) {
  asm volatile(
      "{\n\t.reg .b128 c, d, o;\n\t"
      "mov.b128 c, {%2, %2};\n\t"
      "mov.b128 d, {%3, %4};\n\t"
      "atom.relaxed.gpu.global.cas.b128 o, [%5], c, d;\n\t"
      "mov.b128 {%0, %1}, o;\n\t}"
      : "=l"(old_key), "=l"(old_rows)
      : "l"(~0ull), "l"(key), "l"(rows), "l"(slot)
      : "memory");
}

template <int W>
__global__ void __launch_bounds__(256) k_insert(const int32_t* __restrict__ coords, uint32_t n,
                                                TableHeader* h, Slot* slots,
                                                uint32_t* __restrict__ slot_of_row) {
  if (h->status != RMN_OK) return;
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  Packer<W> pk;
  pk.load(h);
  const uint32_t capacity = h->capacity;
  int32_t c[W];
  load_row<W>(coords, row, c);
  unsigned long long key;
  pk.pack(c, key);
  uint32_t s = hash_key(key, capacity, h->pos_shift);
  bool placed = false;
  // One 16-byte compare-and-swap claims a free slot (all ones) with {key, first_row = row,
  // uid = row}: without duplicates the unique numbering is the row numbering and the slot is
  // final after this single memory operation. A row that finds its key taken lowers first_row
  // and counts itself as a duplicate (k_finalize then renumbers).
  const unsigned long long mine = (unsigned long long)row | ((unsigned long long)row << 32);
  for (uint32_t probe = 0; probe < (capacity >> 3); ++probe) {
    unsigned long long cur_key, cur_rows;
    cas_slot(&slots[s], key, mine, cur_key, cur_rows);
    if (cur_key == kEmptyKey || cur_key == key) {
      if (cur_key == key) {
        atomicMin(&slots[s].first_row, row);
        atomicAdd(&h->n_dups, 1u);
      }
      slot_of_row[row] = s;
      placed = true;
      break;
    }
    // another key lives here and this one walks on: leave word for the lookups (kPassedBit)
    if (!((uint32_t)(cur_rows >> 32) & kPassedBit)) atomicOr(&slots[s].uid, kPassedBit);
    s = next_slot(s, capacity);
  }
  if (!placed) atomicExch(&h->status, (uint32_t)RMN_ERR_PROBE_LIMIT);
}

// In-place exclusive scan of counts[n] by ONE block (any multiple of 32 threads up to 1024); the total goes
// to *total_out. Reads bypass the L1: the counts may have been written by other blocks of the same launch.
__device__ __forceinline__ void scan_u32_block(uint32_t* __restrict__ counts, uint32_t n, uint32_t* total_out) {
  __shared__ uint32_t warp_sums[32];
  const uint32_t nthreads = blockDim.x, nwarps = nthreads >> 5;
  const uint32_t per = (n + nthreads - 1u) / nthreads;
  const uint32_t begin = min(n, threadIdx.x * per), end = min(n, begin + per);
  uint32_t sum = 0;
  for (uint32_t i = begin; i < end; ++i) sum += __ldcg(counts + i);
  // block exclusive scan of `sum`
  uint32_t incl = sum;
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if (lane >= (uint32_t)d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < nwarps ? warp_sums[lane] : 0u, wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xFFFFFFFFu, wi, d);
      if (lane >= (uint32_t)d) wi += t;
    }
    warp_sums[lane] = wi - w;  // exclusive
    if (lane == 31 && total_out) *total_out = wi;
  }
  __syncthreads();
  uint32_t run = warp_sums[warp] + incl - sum;
  for (uint32_t i = begin; i < end; ++i) {
    uint32_t v = __ldcg(counts + i);
    counts[i] = run;
    run += v;
  }
}

// Rows that are the first occurrence of their key, counted per 256-row block; the last block to finish
// turns the counts into block offsets (exclusive scan) and writes n_unique. Returns at once when the
// insert pass met no duplicate: nothing is compacted then (see k_finalize).
__global__ void __launch_bounds__(kRowsPerBlock) k_count_first(const Slot* __restrict__ slots,
                                                              const uint32_t* __restrict__ slot_of_row,
                                                              uint32_t n, TableHeader* h,
                                                              uint32_t* __restrict__ block_counts) {
  if (h->status != RMN_OK) return;
  if (h->n_dups == 0) {  // every row is its own first occurrence: publish the count, nothing to compact
    if (blockIdx.x == 0 && threadIdx.x == 0) h->n_unique = n;
    return;
  }
  __shared__ uint32_t s_last;
  const uint32_t row = blockIdx.x * kRowsPerBlock + threadIdx.x;
  int flag = 0;
  if (row < n) flag = slots[slot_of_row[row]].first_row == row;
  int total = __syncthreads_count(flag);
  if (threadIdx.x == 0) {
    block_counts[blockIdx.x] = (uint32_t)total;
    __threadfence();
    s_last = atomicAdd(&h->count_blocks_done, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  scan_u32_block(block_counts, gridDim.x, &h->n_unique);
}

template <int W>
__global__ void __launch_bounds__(kRowsPerBlock) k_finalize(
    const int32_t* __restrict__ coords, uint32_t n, const TableHeader* h, Slot* slots,
    const uint32_t* __restrict__ slot_of_row, const uint32_t* __restrict__ block_offsets,
    int64_t* __restrict__ mapping, int32_t* __restrict__ unique_coords, int64_t* __restrict__ inverse) {
  __shared__ uint32_t warp_counts[kRowsPerBlock / 32];
  if (h->status != RMN_OK) return;
  const uint32_t row = blockIdx.x * kRowsPerBlock + threadIdx.x;
  if (h->n_dups == 0) {
    // Fast path (all rows distinct): unique row == input row, already stored in the slots by
    // k_insert; only the identity mapping and the coordinate copy remain (both streaming).
    if (row < n) {
      mapping[row] = (int64_t)row;
      if (inverse) inverse[row] = (int64_t)row;
      if (unique_coords) {
        int32_t c[W];
        load_row<W>(coords, row, c);
#pragma unroll
        for (int i = 0; i < W; ++i) unique_coords[(size_t)row * W + i] = c[i];
      }
    }
    if (row == 0) const_cast<TableHeader*>(h)->n_unique = n;
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t s = 0;
  int flag = 0;
  if (row < n) {
    s = slot_of_row[row];
    flag = slots[s].first_row == row;
  }
  const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, flag);
  if (lane == 0) warp_counts[warp] = __popc(ballot);
  __syncthreads();
  uint32_t base = block_offsets[blockIdx.x];
  for (int w = 0; w < warp; ++w) base += warp_counts[w];
  if (flag) {
    const uint32_t uid = base + __popc(ballot & ((1u << lane) - 1u));
    slots[s].uid = uid | (slots[s].uid & kPassedBit);
    mapping[uid] = (int64_t)row;
    if (unique_coords) {
      int32_t c[W];
      load_row<W>(coords, row, c);
#pragma unroll
      for (int i = 0; i < W; ++i) unique_coords[(size_t)uid * W + i] = c[i];
    }
  }
}

__global__ void __launch_bounds__(256) k_inverse(const Slot* __restrict__ slots,
                                                 const uint32_t* __restrict__ slot_of_row,
                                                 uint32_t n, const TableHeader* h,
                                                 int64_t* __restrict__ inverse) {
  // without duplicates k_finalize has already written the identity
  if (h->n_dups == 0 || h->status != RMN_OK) return;
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  inverse[row] = (int64_t)(slots[slot_of_row[row]].uid & ~kPassedBit);
}

template <int W>
__global__ void __launch_bounds__(256) k_find(const TableHeader* __restrict__ h,
                                              const Slot* __restrict__ slots,
                                              const int32_t* __restrict__ query, uint32_t n,
                                              int32_t* __restrict__ rows) {
  const uint32_t q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  Packer<W> pk;
  pk.load(h);
  const uint32_t capacity = h->capacity;
  int32_t c[W];
  load_row<W>(query, q, c);
  unsigned long long key;
  uint32_t uid = 0xFFFFFFFFu;
  if (pk.pack(c, key)) uid = table_find(slots, capacity, h->pos_shift, key);
  rows[q] = (int32_t)uid;
}

struct StrideArg {
  int32_t s[RMN_MAX_W];
};

__global__ void __launch_bounds__(256) k_stride(const int32_t* __restrict__ coords, uint64_t total,
                                                int W, StrideArg st, int32_t* __restrict__ out) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int col = (int)(i % (uint64_t)W);
  int32_t c = coords[i];
  if (col > 0) {
    const int32_t s = st.s[col - 1];
    int32_t q = c / s;
    if ((c % s != 0) && (c < 0)) --q;  // floor for negative coordinates
    c = q * s;
  }
  out[i] = c;
}

// Continuous (field) coordinates -> integer voxel coordinates, the reference's rule in float32:
// batch column lroundf(v), spatial column j: stride_j * (int)floor(v / stride_j)
// (engine/grid/lattice_cpu.hpp:944-984, engine/grid/lattice_gpu.cu:78-151). One thread per element, streaming.
__global__ void __launch_bounds__(256) k_field_quantize(const float* __restrict__ field, uint64_t total, int W,
                                                        StrideArg st, int32_t* __restrict__ out) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int col = (int)(i % (uint64_t)W);
  const float v = field[i];
  int32_t c;
  if (col == 0) {
    c = (int32_t)lroundf(v);
  } else {
    const int32_t s = st.s[col - 1];
    c = s == 1 ? (int32_t)floorf(v) : s * (int32_t)floorf(__fdiv_rn(v, (float)s));
  }
  out[i] = c;
}

// out = (int32)floor((double)v / q) on EVERY column (q <= 0: floor only): the discretisation step of
// sparse_quantize (engine/helpers/discretization.cpp:97-102), computed in float64 as there.
template <typename T>
__global__ void __launch_bounds__(256) k_discretize(const T* __restrict__ in, uint64_t total, double q,
                                                    int32_t* __restrict__ out) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  double v = (double)in[i];
  if (q > 0.0) v = __ddiv_rn(v, q);
  out[i] = (int32_t)floor(v);
}

// Multilinear splat of a field onto the 2^D lattice corners around every point
// (engine/tensor/field.cpp:61-94): corner-major rows (row = corner * n + point), coordinates
// floor(v) + corner bit per spatial axis (batch column floor(v)), features scaled by
// prod_axis (bit ? frac : 1 - frac). One thread per (output row, 4-channel group).
template <typename T>
__global__ void __launch_bounds__(256) k_field_splat(const float* __restrict__ field, const T* __restrict__ feats,
                                                     uint32_t n, int W, int C, int32_t* __restrict__ out_coords,
                                                     T* __restrict__ out_feats) {
  const int groups = (C + 3) / 4;
  const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t rows = (uint64_t)n << (W - 1);
  if (t >= rows * groups) return;
  const uint64_t row = t / groups;
  const int g = (int)(t % groups);
  const uint32_t corner = (uint32_t)(row / n), point = (uint32_t)(row % n);
  float w = 1.0f;
  for (int a = 0; a < W; ++a) {
    const float v = field[(size_t)point * W + a];
    const float fl = floorf(v);
    int32_t c = (int32_t)fl;
    if (a > 0) {
      const float frac = v - fl;
      const bool upper = (corner >> (a - 1)) & 1u;
      w *= upper ? frac : 1.0f - frac;
      c += upper ? 1 : 0;
    }
    if (g == 0) out_coords[row * W + a] = c;
  }
  for (int ch = g * 4; ch < min(C, g * 4 + 4); ++ch)
    out_feats[row * C + ch] = (T)((float)feats[(size_t)point * C + ch] * w);
}

// out[(row * K + k)] = coords[row] + offsets[k] on the spatial columns (batch column copied)
__global__ void __launch_bounds__(256) k_expand(const int32_t* __restrict__ coords, uint64_t total, int W, int K,
                                                const int32_t* __restrict__ offsets, int32_t* __restrict__ out) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int col = (int)(i % (uint64_t)W);
  const uint64_t rk = i / (uint64_t)W;
  const int k = (int)(rk % (uint64_t)K);
  const uint64_t row = rk / (uint64_t)K;
  int32_t c = __ldg(coords + row * W + col);
  if (col > 0) c += __ldg(offsets + (size_t)k * (W - 1) + (col - 1));
  out[i] = c;
}

}  // namespace rmn

using namespace rmn;

extern "C" int rmn_coords_expand(const int32_t* d_coords, uint32_t n_rows, int W, const int32_t* d_offsets, int K,
                                 int32_t* d_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (W < 2 || W > RMN_MAX_W || K < 1) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_coords || !d_offsets || !d_out) return RMN_ERR_BAD_ARG;
  const uint64_t total = (uint64_t)n_rows * (uint64_t)K * (uint64_t)W;
  if ((uint64_t)n_rows * (uint64_t)K >= 0x7FFFFFFFull) return RMN_ERR_TOO_LARGE;
  k_expand<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(d_coords, total, W, K, d_offsets, d_out);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_field_quantize(const float* d_field, uint32_t n_rows, int W, const int32_t* tensor_stride,
                                  int32_t* d_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (W < 2 || W > RMN_MAX_W || !tensor_stride) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_field || !d_out) return RMN_ERR_BAD_ARG;
  StrideArg st;
  for (int a = 0; a < RMN_MAX_W; ++a) st.s[a] = 1;
  for (int a = 0; a < W - 1; ++a) {
    if (tensor_stride[a] <= 0) return RMN_ERR_BAD_ARG;
    st.s[a] = tensor_stride[a];
  }
  const uint64_t total = (uint64_t)n_rows * W;
  k_field_quantize<<<(uint32_t)((total + 255) / 256), 256, 0, stream>>>(d_field, total, W, st, d_out);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_coords_discretize(const void* d_in, int in_type, uint64_t n_elems, double quantization_size,
                                     int32_t* d_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_elems == 0) return RMN_OK;
  if (!d_in || !d_out || n_elems >= ((uint64_t)1 << 39)) return RMN_ERR_BAD_ARG;
  if (quantization_size != quantization_size) return RMN_ERR_BAD_ARG;  // NaN
  const uint32_t nb = (uint32_t)((n_elems + 255) / 256);
  switch (in_type) {
    case 0: k_discretize<float><<<nb, 256, 0, stream>>>((const float*)d_in, n_elems, quantization_size, d_out); break;
    case 1: k_discretize<double><<<nb, 256, 0, stream>>>((const double*)d_in, n_elems, quantization_size, d_out); break;
    case 2: k_discretize<int32_t><<<nb, 256, 0, stream>>>((const int32_t*)d_in, n_elems, quantization_size, d_out); break;
    default: return RMN_ERR_UNSUPPORTED;
  }
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_field_splat(const float* d_field, const void* d_feats, int dtype, uint32_t n_rows, int W, int C,
                               int32_t* d_out_coords, void* d_out_feats, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (W < 2 || W > RMN_MAX_W || C < 1) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_field || !d_feats || !d_out_coords || !d_out_feats) return RMN_ERR_BAD_ARG;
  const uint64_t rows = (uint64_t)n_rows << (W - 1);
  if (rows >= 0x7FFFFFFFull) return RMN_ERR_TOO_LARGE;
  const uint64_t threads = rows * (uint64_t)((C + 3) / 4);
  const uint32_t nb = (uint32_t)((threads + 255) / 256);
  if (dtype == RMN_F32)
    k_field_splat<float><<<nb, 256, 0, stream>>>(d_field, (const float*)d_feats, n_rows, W, C, d_out_coords,
                                                 (float*)d_out_feats);
  else if (dtype == RMN_BF16)
    k_field_splat<__nv_bfloat16><<<nb, 256, 0, stream>>>(d_field, (const __nv_bfloat16*)d_feats, n_rows, W, C,
                                                         d_out_coords, (__nv_bfloat16*)d_out_feats);
  else
    return RMN_ERR_UNSUPPORTED;
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" size_t rmn_table_bytes(uint32_t n_rows) {
  return sizeof(TableHeader) + sizeof(Slot) * (size_t)table_capacity(n_rows);
}

extern "C" size_t rmn_table_build_workspace_bytes(uint32_t n_rows) {
  const size_t nb = (n_rows + kRowsPerBlock - 1) / kRowsPerBlock;
  return (size_t)n_rows * 4 + (nb + 1) * 4 + 256;
}

// First half of a build: header, slot fill + bounding box, insert, first-occurrence counts. When it has
// run, the header is final (number of unique rows, status): a caller may read it back while the second
// half is still running.
extern "C" int rmn_table_build_begin(const int32_t* d_coords, uint32_t n_rows, int W, void* d_table,
                                     size_t table_bytes, void* d_workspace, size_t workspace_bytes,
                                     void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_table || W < 2 || W > RMN_MAX_W || n_rows >= 0x7FFFFFFFu) return RMN_ERR_BAD_ARG;
  if (n_rows > 0 && (!d_coords || !d_workspace)) return RMN_ERR_BAD_ARG;
  if (((uintptr_t)d_table & 15) || !coords_aligned(d_coords, W)) return RMN_ERR_BAD_ARG;
  if (table_bytes < rmn_table_bytes(n_rows) ||
      (n_rows > 0 && workspace_bytes < rmn_table_build_workspace_bytes(n_rows)))
    return RMN_ERR_ALLOC;
  auto* h = reinterpret_cast<TableHeader*>(d_table);
  auto* slots = reinterpret_cast<Slot*>(reinterpret_cast<char*>(d_table) + sizeof(TableHeader));
  const uint32_t capacity = table_capacity(n_rows);
  RMN_CUDA_TRY(cudaMemsetAsync(h, 0, sizeof(TableHeader), stream));
  {
    const uint32_t fill_blocks = (capacity + 255u) / 256u;
    const uint32_t blocks = fill_blocks < 148u * 8u ? fill_blocks : 148u * 8u;
    RMN_DISPATCH_W(W, k_fill_range<kW><<<blocks, 256, 0, stream>>>(d_coords, n_rows, h,
                                                                    reinterpret_cast<uint4*>(slots), capacity));
    RMN_LAUNCH_CHECK();
  }
  if (n_rows == 0) return RMN_OK;
  uint32_t* slot_of_row = reinterpret_cast<uint32_t*>(d_workspace);
  uint32_t* block_counts = slot_of_row + n_rows;
  const uint32_t nb = (n_rows + kRowsPerBlock - 1) / kRowsPerBlock;
  RMN_DISPATCH_W(W, k_insert<kW><<<nb, 256, 0, stream>>>(d_coords, n_rows, h, slots, slot_of_row));
  RMN_LAUNCH_CHECK();
  k_count_first<<<nb, kRowsPerBlock, 0, stream>>>(slots, slot_of_row, n_rows, h, block_counts);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

// Second half: unique ids, mapping, unique coordinates, inverse. Same table, coordinates and workspace as
// the first half, on the same stream.
extern "C" int rmn_table_build_finish(const int32_t* d_coords, uint32_t n_rows, int W, void* d_table,
                                      int64_t* d_mapping, int64_t* d_inverse, int32_t* d_unique_coords,
                                      void* d_workspace, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_table || W < 2 || W > RMN_MAX_W || n_rows >= 0x7FFFFFFFu) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_coords || !d_mapping || !d_workspace) return RMN_ERR_BAD_ARG;
  auto* h = reinterpret_cast<TableHeader*>(d_table);
  auto* slots = reinterpret_cast<Slot*>(reinterpret_cast<char*>(d_table) + sizeof(TableHeader));
  uint32_t* slot_of_row = reinterpret_cast<uint32_t*>(d_workspace);
  uint32_t* block_counts = slot_of_row + n_rows;
  const uint32_t nb = (n_rows + kRowsPerBlock - 1) / kRowsPerBlock;
  RMN_DISPATCH_W(W, k_finalize<kW><<<nb, kRowsPerBlock, 0, stream>>>(
                        d_coords, n_rows, h, slots, slot_of_row, block_counts, d_mapping,
                        d_unique_coords, d_inverse));
  RMN_LAUNCH_CHECK();
  if (d_inverse) {  // optional: only the quantisation modes that average or sample features read it
    k_inverse<<<nb, 256, 0, stream>>>(slots, slot_of_row, n_rows, h, d_inverse);
    RMN_LAUNCH_CHECK();
  }
  return RMN_OK;
}

extern "C" int rmn_table_build(const int32_t* d_coords, uint32_t n_rows, int W, void* d_table,
                               size_t table_bytes, int64_t* d_mapping, int64_t* d_inverse,
                               int32_t* d_unique_coords, void* d_workspace,
                               size_t workspace_bytes, void* stream_) {
  if (n_rows > 0 && n_rows < 0x7FFFFFFFu && !d_mapping) return RMN_ERR_BAD_ARG;
  const int rc = rmn_table_build_begin(d_coords, n_rows, W, d_table, table_bytes, d_workspace, workspace_bytes,
                                       stream_);
  if (rc != RMN_OK) return rc;
  return rmn_table_build_finish(d_coords, n_rows, W, d_table, d_mapping, d_inverse, d_unique_coords, d_workspace,
                                stream_);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of rmn_table_build.
//
// Some hosts may not allocate device memory once they are running: a perception
// loop with a fixed memory plan treats cudaMalloc as forbidden because it
// synchronises the whole device and can fail from fragmentation in the middle
// of a drive, and a plug-in loaded into somebody else's process may be handed
// input and output buffers but no allocator to ask for scratch. Such callers
// own the table, mapping and inverse buffers (they are outputs) yet have
// nowhere to put the build's scratch (slot-of-row array + block counters).
// Here that scratch lives in a file-scope device array of fixed size, so the
// call needs nothing beyond its inputs and outputs. The price is a hard row
// limit and 4 MiB of device memory held by every GPU that loads the library.
//
// The host symbol below is only a handle: kernels must be given the device
// address obtained with cudaGetSymbolAddress, which is looked up once per
// device (with that device current) on the first call made on it.
// ---------------------------------------------------------------------------
constexpr uint32_t kStaticMaxRows = 1u << 20;
constexpr size_t kStaticScratchBytes =
    (size_t)kStaticMaxRows * 4 + ((kStaticMaxRows + rmn::kRowsPerBlock - 1) / rmn::kRowsPerBlock + 1) * 4 + 256;
static __device__ __align__(256) unsigned char g_table_static_scratch[kStaticScratchBytes];

static int static_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static void* address[kMaxDevices] = {};
  static std::mutex lock;
  int dev = 0;
  RMN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return RMN_ERR_BAD_ARG;
  std::lock_guard<std::mutex> guard(lock);
  if (!address[dev]) {
    void* p = nullptr;
    // the current device is `dev`: the address returned belongs to this device's copy of the array
    RMN_CUDA_TRY(cudaGetSymbolAddress(&p, g_table_static_scratch));
    if (!p) return RMN_ERR_CUDA;
    address[dev] = p;
  }
  *out = address[dev];
  return RMN_OK;
}

extern "C" uint32_t rmn_table_build_static_max_rows(void) { return kStaticMaxRows; }

extern "C" int rmn_table_build_static(const int32_t* d_coords, uint32_t n_rows, int W, void* d_table,
                                      size_t table_bytes, int64_t* d_mapping, int64_t* d_inverse,
                                      int32_t* d_unique_coords, void* stream_) {
  if (n_rows > kStaticMaxRows) return RMN_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != RMN_OK) return rc;
  // Nothing in the scratch has to start at zero: the insert pass writes the slot of every row
  // and the count pass writes every block counter before anything reads them, so whatever an
  // earlier call left behind is overwritten.
  return rmn_table_build(d_coords, n_rows, W, d_table, table_bytes, d_mapping, d_inverse,
                         d_unique_coords, scratch, kStaticScratchBytes, stream_);
}

// Small read-backs go through a kernel that stores into page-locked host memory, not through a copy
// engine: a device-to-host cudaMemcpyAsync waits its turn behind every copy already queued on that
// engine, on whatever stream, so the 256-byte header of a table build would sit behind the previous
// step's 150 MB result on its way to the host (measured: 6 ms behind two such copies, 14 us on an idle
// link) and the step behind it. Stores from an SM share the link but not the queue.
__global__ void k_words_to_host(const uint32_t* __restrict__ src, uint32_t n_words, const uint32_t* __restrict__ extra,
                                volatile uint32_t* __restrict__ dst) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += gridDim.x * blockDim.x) dst[i] = src[i];
  if (extra && blockIdx.x == 0 && threadIdx.x == 0) dst[n_words] = *extra;
  __threadfence_system();
}

// device-side alias of a page-locked host block, or NULL when the block is not mapped into the device
static void* device_alias(void* host_block) {
  void* d = nullptr;
  if (cudaHostGetDevicePointer(&d, host_block, 0) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return d;
}

extern "C" int rmn_readback_small(const void* d_src, void* h_dst_pinned, size_t bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (bytes == 0) return RMN_OK;
  if (!d_src || !h_dst_pinned || (bytes & 3) || ((uintptr_t)d_src & 3) || ((uintptr_t)h_dst_pinned & 3) ||
      bytes > (1u << 20))
    return RMN_ERR_BAD_ARG;
  void* alias = device_alias(h_dst_pinned);
  if (!alias) {  // not page-locked / not mapped: the copy engine it is
    RMN_CUDA_TRY(cudaMemcpyAsync(h_dst_pinned, d_src, bytes, cudaMemcpyDeviceToHost, stream));
    return RMN_OK;
  }
  const uint32_t n_words = (uint32_t)(bytes / 4);
  k_words_to_host<<<(n_words + 255) / 256 < 64 ? (n_words + 255) / 256 : 64, 256, 0, stream>>>(
      static_cast<const uint32_t*>(d_src), n_words, nullptr, static_cast<volatile uint32_t*>(alias));
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_table_info(const void* d_table, uint32_t info[4], void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_table || !info) return RMN_ERR_BAD_ARG;
  // The header is read back through a page-locked staging block owned by the calling thread: a copy into
  // pageable memory is staged by the driver and costs several microseconds more, and this read-back is the
  // one host synchronisation of a table build.
  // The same wait also brings back the status word of the convolution kernels (a bounded wait that ran out
  // in a kernel queued before this read-back on a stream this one is ordered after): every table build
  // of a host thus checks the convolutions that went before it without a synchronisation of its own.
  struct Staging {
    TableHeader header;
    uint32_t conv_status;  // directly behind the header: k_words_to_host stores it as word n_words
  };
  static_assert(sizeof(TableHeader) % 4 == 0 && offsetof(Staging, conv_status) == sizeof(TableHeader), "layout");
  thread_local Staging* staging = nullptr;
  if (!staging) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, sizeof(Staging), cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    staging = static_cast<Staging*>(p);
  }
  TableHeader pageable;
  TableHeader* dst = staging ? &staging->header : &pageable;
  void* alias = staging ? device_alias(staging) : nullptr;
  const uint32_t* d_conv_status = alias ? tc_status_device_address() : nullptr;
  if (alias && d_conv_status) {
    // header and status word in one launch, stored by the SM (see k_words_to_host)
    staging->header.magic = 0;
    staging->conv_status = 0;
    k_words_to_host<<<1, 64, 0, stream>>>(static_cast<const uint32_t*>(d_table), (uint32_t)(sizeof(TableHeader) / 4),
                                          d_conv_status, reinterpret_cast<volatile uint32_t*>(alias));
    RMN_LAUNCH_CHECK();
  } else {
    RMN_CUDA_TRY(cudaMemcpyAsync(dst, d_table, sizeof(TableHeader), cudaMemcpyDeviceToHost, stream));
    if (staging) {
      staging->conv_status = 0;
      RMN_CUDA_TRY(tc_copy_status_async(&staging->conv_status, stream) == RMN_OK ? cudaSuccess : cudaErrorUnknown);
    }
  }
  RMN_CUDA_TRY(cudaStreamSynchronize(stream));
  const TableHeader h = *dst;
  if (h.magic != kTableMagic) return RMN_ERR_BAD_ARG;
  info[0] = h.n_unique;
  info[1] = h.status;
  info[2] = h.capacity;
  info[3] = h.n_rows;
  if (h.status == RMN_OK && staging && staging->conv_status != 0) {
    const int st = (int)staging->conv_status;
    tc_clear_status();
    return st;
  }
  return (int)h.status;
}

extern "C" int rmn_table_find(const void* d_table, const int32_t* d_query, uint32_t n_query, int W,
                              int32_t* d_rows, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!d_table || W < 2 || W > RMN_MAX_W) return RMN_ERR_BAD_ARG;
  if (n_query == 0) return RMN_OK;
  if (!d_query || !d_rows || !coords_aligned(d_query, W)) return RMN_ERR_BAD_ARG;
  auto* h = reinterpret_cast<const TableHeader*>(d_table);
  auto* slots =
      reinterpret_cast<const Slot*>(reinterpret_cast<const char*>(d_table) + sizeof(TableHeader));
  const uint32_t nb = (n_query + 255) / 256;
  RMN_DISPATCH_W(W, k_find<kW><<<nb, 256, 0, stream>>>(h, slots, d_query, n_query, d_rows));
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}

extern "C" int rmn_coords_stride(const int32_t* d_coords, uint32_t n_rows, int W,
                                 const int32_t* out_tensor_stride, int32_t* d_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (W < 2 || W > RMN_MAX_W || !out_tensor_stride) return RMN_ERR_BAD_ARG;
  if (n_rows == 0) return RMN_OK;
  if (!d_coords || !d_out) return RMN_ERR_BAD_ARG;
  StrideArg st;
  for (int a = 0; a < RMN_MAX_W; ++a) st.s[a] = 1;
  for (int a = 0; a < W - 1; ++a) {
    if (out_tensor_stride[a] <= 0) return RMN_ERR_BAD_ARG;
    st.s[a] = out_tensor_stride[a];
  }
  const uint64_t total = (uint64_t)n_rows * W;
  const uint32_t nb = (uint32_t)((total + 255) / 256);
  k_stride<<<nb, 256, 0, stream>>>(d_coords, total, W, st, d_out);
  RMN_LAUNCH_CHECK();
  return RMN_OK;
}
