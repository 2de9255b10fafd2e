/*
 * CPU restatement of RiemannEngine's sparse-convolution hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the parity checker for the CUDA
 * library: tests, the smoke check and the benchmark's cpu_baseline leg may
 * call it; no product code path may. Plain C, single-threaded, scalar.
 *
 * Parity status: pinned. The convolution arithmetic is checked against the
 * three known-answer tests of the reference
 * (tests/convolution/test_cpu_convolution.cpp:15-61) and every map/convolution
 * function is checked against outputs of the reference's own CPU build
 * (golden fixtures produced by the reference driver that sits beside this
 * file).
 *
 * Each function cites the reference code it follows (paths relative to the
 * reference project root, RiemannEngine/engine/...).
 *
 * Row-numbering rule used where the reference's own numbering is an artefact
 * of hash-table iteration order (strided maps, grid/lattice_cpu.hpp:475-493):
 * unique rows are numbered by first occurrence when the source rows are
 * visited in row order. Comparisons against the reference for those maps are
 * made in coordinate space.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_EMPTY 0xFFFFFFFFu

/* ------------------------------------------------------------------------
 * MurmurHash3 x86-32, seed 0, over the raw bytes of one coordinate row.
 * Follows foundation/hashing.hpp:205-276 (coordinate_murmur3): little-endian
 * byte-wise block loads, len = W*4 so the tail switch is never taken.
 * ---------------------------------------------------------------------- */
static inline uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }

uint32_t orc_murmur3_row(const int32_t *row, int W) {
  const uint8_t *data = (const uint8_t *)row;
  const uint32_t len = (uint32_t)W * 4u;
  uint32_t h1 = 0;
  for (int i = 0; i < W; ++i) {
    const uint8_t *q = data + 4 * i;
    uint32_t k1 = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) |
                  ((uint32_t)q[3] << 24);
    k1 *= 0xcc9e2d51u;
    k1 = rotl32(k1, 15);
    k1 *= 0x1b873593u;
    h1 ^= k1;
    h1 = rotl32(h1, 13);
    h1 = h1 * 5u + 0xe6546b64u;
  }
  h1 ^= len;
  h1 ^= h1 >> 16;
  h1 *= 0x85ebca6bu;
  h1 ^= h1 >> 13;
  h1 *= 0xc2b2ae35u;
  h1 ^= h1 >> 16;
  return h1;
}

/* ------------------------------------------------------------------------
 * Coordinate hash map: key = a coordinate row (W int32), value = uint32 row
 * id. The reference uses robin_hood::unordered_flat_map keyed by a pointer
 * to the row with coordinate_murmur3 / coordinate_equal_to
 * (grid/lattice_cpu.hpp:356-398, foundation/hashing.hpp:182-200). Only the
 * map semantics (insert-if-absent, find) are observable, so a linear-probing
 * table at <= 50 % load stands in for robin_hood.
 * ---------------------------------------------------------------------- */
typedef struct {
  const int32_t *keys; /* borrowed [n_keys, W] */
  int W;
  uint32_t cap; /* power of two */
  uint32_t *slot_row; /* row of `keys` held by the slot, ORC_EMPTY if free */
  uint32_t *slot_val;
} orc_map;

static int orc_map_init(orc_map *m, const int32_t *keys, int W, uint64_t n) {
  uint64_t cap = 16;
  while (cap < 2 * n + 2) cap <<= 1;
  m->keys = keys;
  m->W = W;
  m->cap = (uint32_t)cap;
  m->slot_row = (uint32_t *)malloc(cap * sizeof(uint32_t));
  m->slot_val = (uint32_t *)malloc(cap * sizeof(uint32_t));
  if (!m->slot_row || !m->slot_val) return -1;
  memset(m->slot_row, 0xFF, cap * sizeof(uint32_t));
  return 0;
}

static void orc_map_free(orc_map *m) {
  free(m->slot_row);
  free(m->slot_val);
}

static inline int row_eq(const int32_t *a, const int32_t *b, int W) {
  for (int i = 0; i < W; ++i)
    if (a[i] != b[i]) return 0;
  return 1;
}

/* insert-if-absent; returns 1 when inserted, value of the resident entry in *val */
static inline int orc_map_insert(orc_map *m, uint32_t key_row, uint32_t value, uint32_t *val) {
  const int32_t *key = m->keys + (size_t)key_row * m->W;
  uint32_t s = orc_murmur3_row(key, m->W) & (m->cap - 1);
  for (;;) {
    uint32_t r = m->slot_row[s];
    if (r == ORC_EMPTY) {
      m->slot_row[s] = key_row;
      m->slot_val[s] = value;
      *val = value;
      return 1;
    }
    if (row_eq(m->keys + (size_t)r * m->W, key, m->W)) {
      *val = m->slot_val[s];
      return 0;
    }
    s = (s + 1) & (m->cap - 1);
  }
}

static inline int orc_map_find(const orc_map *m, const int32_t *key, uint32_t *val) {
  uint32_t s = orc_murmur3_row(key, m->W) & (m->cap - 1);
  for (;;) {
    uint32_t r = m->slot_row[s];
    if (r == ORC_EMPTY) return 0;
    if (row_eq(m->keys + (size_t)r * m->W, key, m->W)) {
      *val = m->slot_val[s];
      return 1;
    }
    s = (s + 1) & (m->cap - 1);
  }
}

/* ------------------------------------------------------------------------
 * insert_and_map<remap = true>: dedup coordinate rows.
 * Follows grid/lattice_cpu.hpp:419-444: rows are visited in order; a row
 * that inserts gets the next unique id and its row index is appended to
 * `mapping` (first-occurrence rows); `inverse[i]` is the unique id of row i.
 * Returns the number of unique rows, or -1 on allocation failure.
 * ---------------------------------------------------------------------- */
int64_t orc_insert_and_map(const int32_t *coords, int64_t n, int W, int64_t *mapping,
                           int64_t *inverse) {
  orc_map m;
  if (orc_map_init(&m, coords, W, (uint64_t)n)) return -1;
  uint32_t value = 0;
  for (int64_t row = 0; row < n; ++row) {
    uint32_t resident;
    int inserted = orc_map_insert(&m, (uint32_t)row, value, &resident);
    if (inserted) {
      mapping[value] = row;
      inverse[row] = value;
      value += 1;
    } else {
      inverse[row] = resident;
    }
  }
  orc_map_free(&m);
  return (int64_t)value;
}

/* ------------------------------------------------------------------------
 * stride_coordinate: floor-align spatial columns to the OUTPUT tensor
 * stride; the batch column passes through.
 * Follows grid/stencil.hpp:35-43, including its float arithmetic
 * (floor((float)c / s) * s), which is exact for |c| < 2^24.
 * ---------------------------------------------------------------------- */
void orc_stride_coords(const int32_t *coords, int64_t n, int W, const int32_t *out_stride,
                       int32_t *dst) {
  for (int64_t r = 0; r < n; ++r) {
    dst[r * W] = coords[r * W];
    for (int a = 0; a < W - 1; ++a) {
      float s = (float)out_stride[a];
      dst[r * W + a + 1] = (int32_t)(floorf((float)coords[r * W + a + 1] / s) * s);
    }
  }
}

/* ------------------------------------------------------------------------
 * kernel_region::coordinate_at restated as an offset table.
 * Follows grid/stencil.hpp:223-278. region_type: 0 HYPER_CUBE, 1 HYPER_CROSS,
 * 2 CUSTOM (foundation/types.hpp RegionType). Writes offsets[K][D] such that
 * neighbour = centre + offsets[k]; returns K.
 *  - HYPER_CUBE: axis 0 varies fastest; odd sizes are centred
 *    ((i - k/2) * dil * ts), even sizes enumerate 0..k-1 (i * dil * ts).
 *  - HYPER_CROSS: index 0 is the centre, then per axis (k_a - 1) entries:
 *    the first r = (k_a-1)/2 are +1..+r, the rest are -r..-1... exactly as
 *    the reference computes them (ind < r ? ind + 1 : ind - 2r).
 *  - CUSTOM: user offsets scaled by ts * dil.
 * ---------------------------------------------------------------------- */
int orc_region_volume(int region_type, int D, const int32_t *ksize, int n_custom) {
  if (region_type == 0) {
    int v = 1;
    for (int a = 0; a < D; ++a) v *= ksize[a];
    return v;
  }
  if (region_type == 1) {
    int v = 1;
    for (int a = 0; a < D; ++a) v += ksize[a] - 1;
    return v;
  }
  return n_custom;
}

int orc_region_offsets(int region_type, int D, const int32_t *ksize, const int32_t *dilation,
                       const int32_t *tensor_stride, const int32_t *custom, int n_custom,
                       int32_t *offsets) {
  const int K = orc_region_volume(region_type, D, ksize, n_custom);
  for (int k = 0; k < K; ++k) {
    int32_t *o = offsets + (size_t)k * D;
    for (int a = 0; a < D; ++a) o[a] = 0;
    if (region_type == 0) {
      uint32_t idx = (uint32_t)k;
      for (int a = 0; a < D; ++a) {
        uint32_t ks = (uint32_t)ksize[a];
        uint32_t cur = idx % ks;
        if (ks % 2 == 0)
          o[a] = (int32_t)(dilation[a] * tensor_stride[a] * (int32_t)cur);
        else
          o[a] = ((int32_t)cur - (int32_t)(ks / 2)) * dilation[a] * tensor_stride[a];
        idx /= ks;
      }
    } else if (region_type == 1) {
      if (k == 0) continue;
      int ind = k - 1, axis = 0;
      while (axis < D) {
        if (ind < ksize[axis] - 1) break;
        ind -= ksize[axis] - 1;
        axis += 1;
      }
      int r = (ksize[axis] - 1) / 2;
      int co = (ind < r) ? (ind + 1) : (ind - 2 * r);
      o[axis] = co * dilation[axis] * tensor_stride[axis];
    } else {
      for (int a = 0; a < D; ++a)
        o[a] = (int32_t)((int64_t)custom[(size_t)k * D + a] * tensor_stride[a] * dilation[a]);
    }
  }
  return K;
}

/* ------------------------------------------------------------------------
 * kernel_map: for every query row q and offset k, look coords_q[q] +
 * offsets[k] up in the map over coords_a; on a hit append (a_row, q_row) to
 * offset k. Follows grid/lattice_cpu.hpp:606-673 (the map being queried is
 * `this`, the iterated map is out_coordinate_map). The reference appends
 * through an atomic slot counter from several threads, so order inside an
 * offset is unspecified there; here queries are visited in row order, which
 * yields pairs sorted by q_row.
 * a_idx / q_idx: [K][n_q] preallocated like the reference (lattice_cpu.hpp:
 * 613-615); counts[K] receives the used length of each offset.
 * For a forward (non-transposed) map a = input, q = output. For a transposed
 * map the reference queries the OUTPUT map with the input rows and swaps
 * (grid/space_impl.hpp:649-697): call with a = output coords, q = input
 * coords and read (q_idx, a_idx) as (in, out).
 * Returns total pairs, -1 on allocation failure.
 * ---------------------------------------------------------------------- */
int64_t orc_kernel_map(const int32_t *coords_a, int64_t n_a, const int32_t *coords_q, int64_t n_q,
                       int W, const int32_t *offsets, int K, int32_t *a_idx, int32_t *q_idx,
                       int64_t *counts) {
  orc_map m;
  if (orc_map_init(&m, coords_a, W, (uint64_t)n_a)) return -1;
  for (int64_t r = 0; r < n_a; ++r) {
    uint32_t resident;
    orc_map_insert(&m, (uint32_t)r, (uint32_t)r, &resident);
  }
  for (int k = 0; k < K; ++k) counts[k] = 0;
  int32_t tmp[16];
  int64_t total = 0;
  for (int64_t q = 0; q < n_q; ++q) {
    const int32_t *c = coords_q + q * W;
    for (int k = 0; k < K; ++k) {
      tmp[0] = c[0];
      for (int a = 0; a < W - 1; ++a) tmp[a + 1] = c[a + 1] + offsets[(size_t)k * (W - 1) + a];
      uint32_t hit;
      if (orc_map_find(&m, tmp, &hit)) {
        int64_t slot = counts[k]++;
        a_idx[(size_t)k * n_q + slot] = (int32_t)hit;
        q_idx[(size_t)k * n_q + slot] = (int32_t)q;
        total += 1;
      }
    }
  }
  orc_map_free(&m);
  return total;
}

/* ------------------------------------------------------------------------
 * Sparse convolution forward over a kernel map in CSR-over-offsets form
 * (offset_ptr[K+1], in_idx[P], out_idx[P]).
 * Follows ops/convolution_cpu.hpp:27-52 (same loop nest and summation order:
 * offsets, then pairs, then in-channel, then out-channel; out-of-range pairs
 * are skipped). `output` is accumulated into, as in the reference.
 * weights: [K, c_in, c_out] row-major (nn/conv.cpp:83-84).
 * ---------------------------------------------------------------------- */
void orc_conv_fwd_f32(const float *input, int c_in, float *output, int c_out, int64_t n_in,
                      int64_t n_out, const float *weights, int K, const int64_t *offset_ptr,
                      const int32_t *in_idx, const int32_t *out_idx) {
  for (int k = 0; k < K; ++k) {
    const float *w = weights + (size_t)k * c_in * c_out;
    for (int64_t p = offset_ptr[k]; p < offset_ptr[k + 1]; ++p) {
      int64_t i = in_idx[p], o = out_idx[p];
      if (i < 0 || i >= n_in || o < 0 || o >= n_out) continue;
      const float *f = input + i * c_in;
      float *r = output + o * c_out;
      for (int ci = 0; ci < c_in; ++ci)
        for (int co = 0; co < c_out; ++co) r[co] += f[ci] * w[ci * c_out + co];
    }
  }
}

/* Backward: grad_input[in] += grad_out[out] . W[k]^T ; grad_w[k] += f^T . g.
 * Follows ops/convolution_cpu.hpp:54-88. Both outputs are accumulated into. */
void orc_conv_bwd_f32(const float *input, float *grad_input, int c_in, const float *grad_output,
                      int c_out, int64_t n_in, int64_t n_out, const float *weights,
                      float *grad_weights, int K, const int64_t *offset_ptr, const int32_t *in_idx,
                      const int32_t *out_idx) {
  for (int k = 0; k < K; ++k) {
    const float *w = weights + (size_t)k * c_in * c_out;
    float *gw = grad_weights + (size_t)k * c_in * c_out;
    for (int64_t p = offset_ptr[k]; p < offset_ptr[k + 1]; ++p) {
      int64_t i = in_idx[p], o = out_idx[p];
      if (i < 0 || i >= n_in || o < 0 || o >= n_out) continue;
      const float *f = input + i * c_in;
      const float *g = grad_output + o * c_out;
      float *gi = grad_input + i * c_in;
      for (int ci = 0; ci < c_in; ++ci)
        for (int co = 0; co < c_out; ++co) {
          gi[ci] += g[co] * w[ci * c_out + co];
          gw[ci * c_out + co] += f[ci] * g[co];
        }
    }
  }
}

/* Same sums in double precision: the tolerance reference for fp32/bf16 GPU
 * results (the reference's own fp32 summation order is not pinned because its
 * layer runs LibTorch index_select/matmul/index_add_, nn/conv.cpp:47-64). */
void orc_conv_fwd_f64(const float *input, int c_in, double *output, int c_out, int64_t n_in,
                      int64_t n_out, const float *weights, int K, const int64_t *offset_ptr,
                      const int32_t *in_idx, const int32_t *out_idx) {
  for (int k = 0; k < K; ++k) {
    const float *w = weights + (size_t)k * c_in * c_out;
    for (int64_t p = offset_ptr[k]; p < offset_ptr[k + 1]; ++p) {
      int64_t i = in_idx[p], o = out_idx[p];
      if (i < 0 || i >= n_in || o < 0 || o >= n_out) continue;
      const float *f = input + i * c_in;
      double *r = output + o * c_out;
      for (int ci = 0; ci < c_in; ++ci) {
        double fv = f[ci];
        for (int co = 0; co < c_out; ++co) r[co] += fv * (double)w[ci * c_out + co];
      }
    }
  }
}

void orc_conv_bwd_f64(const float *input, double *grad_input, int c_in, const float *grad_output,
                      int c_out, int64_t n_in, int64_t n_out, const float *weights,
                      double *grad_weights, int K, const int64_t *offset_ptr,
                      const int32_t *in_idx, const int32_t *out_idx) {
  for (int k = 0; k < K; ++k) {
    const float *w = weights + (size_t)k * c_in * c_out;
    double *gw = grad_weights + (size_t)k * c_in * c_out;
    for (int64_t p = offset_ptr[k]; p < offset_ptr[k + 1]; ++p) {
      int64_t i = in_idx[p], o = out_idx[p];
      if (i < 0 || i >= n_in || o < 0 || o >= n_out) continue;
      const float *f = input + i * c_in;
      const float *g = grad_output + o * c_out;
      double *gi = grad_input + i * c_in;
      for (int ci = 0; ci < c_in; ++ci)
        for (int co = 0; co < c_out; ++co) {
          gi[ci] += (double)g[co] * (double)w[ci * c_out + co];
          gw[ci * c_out + co] += (double)f[ci] * (double)g[co];
        }
    }
  }
}
