/*
 * rmn_b200 — C ABI of the B200 (sm_100a) sparse-convolution hot path:
 * coordinate hashing, kernel-map generation and gather-GEMM-scatter
 * convolution (forward / backward, plain, strided-down and transposed).
 *
 * This is the boundary a host binding (C++/LibTorch, Python ctypes, ...) links
 * against. The reference project has no C ABI; every entry point below names
 * the reference C++ interface it stands in for (paths relative to the
 * reference project root).
 *
 * Conventions
 *  - Every function returns an int status (RMN_OK == 0). No exceptions cross
 *    the boundary.
 *  - All `d_*` pointers are DEVICE pointers on the current CUDA device; all
 *    buffers are allocated by the caller. `*_bytes` queries say how large.
 *    The library never allocates device memory.
 *  - `stream` is a cudaStream_t passed as void*. Calls only enqueue work;
 *    they do not synchronise unless the comment says so.
 *  - Coordinates are int32 rows [N, W], W = 1 + D, batch index first,
 *    contiguous (reference: engine/grid/space_impl.hpp:268-276).
 *  - Row counts are < 2^31.
 *  - There is no CPU fallback: without a CUDA device every compute entry
 *    point returns RMN_ERR_CUDA.
 */
#ifndef RMN_B200_H
#define RMN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define RMN_OK 0
#define RMN_ERR_BAD_ARG 1      /* null pointer, bad size, unsupported W/K/channels */
#define RMN_ERR_ALLOC 2        /* a caller-provided buffer is too small */
#define RMN_ERR_PROBE_LIMIT 3  /* a hash probe sequence hit its bound (table full) */
#define RMN_ERR_TIMEOUT 4      /* a bounded device-side wait ran out */
#define RMN_ERR_CUDA 5         /* a CUDA runtime call failed */
#define RMN_ERR_RANGE 6        /* coordinate bounding box does not pack into 63 bits */
#define RMN_ERR_UNSUPPORTED 7  /* shape / dtype combination has no kernel */
#define RMN_ERR_TOO_LARGE 8    /* size exceeds the fixed capacity of an allocation-free entry point */

/* ---- feature element types -------------------------------------------- */
#define RMN_F32 0
#define RMN_BF16 1

/* ---- region types (reference: engine/foundation/types.hpp RegionType) -- */
#define RMN_HYPER_CUBE 0
#define RMN_HYPER_CROSS 1
#define RMN_CUSTOM 2

#define RMN_MAX_W 8 /* batch column + up to 7 spatial/temporal axes */

/* Library version (major*10000 + minor*100 + patch) and status text. */
int rmn_version(void);
const char *rmn_status_string(int status);
/* Number of CUDA kernels this library has launched in this process so far
 * (telemetry for benchmarks; no counterpart in the reference). */
unsigned long long rmn_launch_count(void);
/* Of those, launches of the tcgen05 convolution kernels (forward, input gradient, weight gradient): tells a
 * host that a convolution ran on the tensor cores and not on the SIMT kernels. No counterpart in the reference. */
unsigned long long rmn_tensor_core_launch_count(void);
/* Synchronises `stream` and returns the device-side status of the convolution
 * kernels: RMN_OK, or RMN_ERR_TIMEOUT when a bounded wait inside a kernel ran
 * out (the kernel then returned early and its output is invalid). The status
 * is ONE word per device, shared by all streams; a non-zero value is returned
 * once and reset by the call that returns it. rmn_table_info returns the same
 * status (and resets it) when the table itself is fine, so a host that builds
 * a coordinate map per step checks its earlier convolutions at the read-back
 * it makes anyway. No counterpart in the reference. */
int rmn_device_status(void *stream);

/* =======================================================================
 * Coordinate hash table
 * Replaces: CoordinateMapCPU / CoordinateMapGPU storage
 *   (engine/grid/lattice_cpu.hpp:356-398, engine/grid/lattice_gpu.cuh:519-678)
 *   and the vendored concurrent_unordered_map
 *   (vendor/concurrent_unordered_map.cuh:305-391).
 * An open-addressing table of 16-byte slots {packed key, first row, unique
 * row} with 4 * n_rows + 64 slots (load <= 1/4; 3 * n_rows + 64 once that would exceed
 * 120 MiB: ask rmn_table_bytes), preceded by a 256-byte header.
 * ===================================================================== */

/* Bytes of device memory a table for `n_rows` input rows needs. */
size_t rmn_table_bytes(uint32_t n_rows);
/* Bytes of scratch rmn_table_build needs for `n_rows` rows. */
size_t rmn_table_build_workspace_bytes(uint32_t n_rows);

/*
 * Dedup-insert `n_rows` coordinate rows and number the unique rows in
 * first-occurrence order.
 * Replaces: CoordinateMapCPU::insert_and_map<true>
 *   (engine/grid/lattice_cpu.hpp:419-444), CoordinateMapGPU::insert<true>
 *   (engine/grid/lattice_gpu.cu:160-230) and the uint32->int64 widening of
 *   engine/grid/space.cu:60-80.
 *  d_mapping  [n_rows] int64: first n_unique entries = first-occurrence rows
 *  d_inverse  [n_rows] int64: unique row of every input row; may be NULL (not produced)
 *  d_unique_coords [n_rows, W] int32 or NULL: unique rows in map order
 *    (what CoordinateMapManager::get_coordinates returns,
 *     engine/grid/space_impl.hpp:947-975)
 * n_unique and the device-side status are read back with rmn_table_info.
 */
int rmn_table_build(const int32_t *d_coords, uint32_t n_rows, int W, void *d_table,
                    size_t table_bytes, int64_t *d_mapping, int64_t *d_inverse,
                    int32_t *d_unique_coords, void *d_workspace, size_t workspace_bytes,
                    void *stream);

/*
 * rmn_table_build in two calls on one stream, for hosts that want the number of unique rows as early as
 * possible: after rmn_table_build_begin (header, slot fill, insert, first-occurrence counts) the header is
 * final, so an event recorded between the two calls lets a second stream run rmn_table_info while
 * rmn_table_build_finish (unique ids, mapping, unique coordinates, inverse) still runs on the first.
 * Arguments as in rmn_table_build; both calls take the same table, coordinates and workspace.
 * rmn_table_build is exactly begin followed by finish. Replaces: as rmn_table_build.
 */
int rmn_table_build_begin(const int32_t *d_coords, uint32_t n_rows, int W, void *d_table, size_t table_bytes,
                          void *d_workspace, size_t workspace_bytes, void *stream);
int rmn_table_build_finish(const int32_t *d_coords, uint32_t n_rows, int W, void *d_table, int64_t *d_mapping,
                           int64_t *d_inverse, int32_t *d_unique_coords, void *d_workspace, void *stream);

/*
 * rmn_table_build for callers that cannot allocate device memory. It has no
 * counterpart in the reference. Same inputs, outputs and results as
 * rmn_table_build, but there is no workspace argument: the build's scratch is
 * a fixed device array inside the library (4 MiB per GPU, held from the moment
 * the library is loaded on that GPU until the process exits).
 * Meant for hosts with a frozen memory plan (real-time loops where cudaMalloc
 * is banned because it synchronises the device and may fail mid-run) and for
 * plug-ins that receive input/output buffers from their host but no allocator.
 *  - n_rows must not exceed rmn_table_build_static_max_rows() (1 048 576);
 *    larger inputs return RMN_ERR_TOO_LARGE and enqueue nothing.
 *  - The first call on each device looks up the device address of the scratch
 *    array (with that device current); make that first call outside any stream
 *    capture. Later calls on the same device only enqueue kernels. The address is kept for the life of
 *    the process: do not call cudaDeviceReset (or otherwise destroy the device's primary context) while
 *    the library is loaded and then call this entry point again.
 *  - The call itself performs no cudaMalloc / cudaFree and calls no allocating
 *    library routine.
 *  - All calls on one GPU share the one scratch array, which keeps the
 *    previous call's contents (every word is rewritten before it is read, so
 *    stale contents are harmless). Two calls whose kernels overlap on the same
 *    GPU (different streams, different threads) race on it: serialise them.
 */
uint32_t rmn_table_build_static_max_rows(void);
int rmn_table_build_static(const int32_t *d_coords, uint32_t n_rows, int W, void *d_table,
                           size_t table_bytes, int64_t *d_mapping, int64_t *d_inverse,
                           int32_t *d_unique_coords, void *stream);

/*
 * Synchronising read-back: info[0] = n_unique, info[1] = device status
 * (RMN_OK / RMN_ERR_PROBE_LIMIT / RMN_ERR_RANGE), info[2] = slot count,
 * info[3] = n_rows. Returns info[1] when it is non-zero; otherwise the pending
 * status of earlier convolution kernels (see rmn_device_status), normally RMN_OK.
 */
int rmn_table_info(const void *d_table, uint32_t info[4], void *stream);

/*
 * Queue a read-back of `bytes` (a multiple of 4, at most 1 MiB) from device memory into PAGE-LOCKED host
 * memory on `stream`, carried out by a kernel that stores into the host block instead of by a copy engine:
 * a device-to-host cudaMemcpyAsync queues behind every copy already running on that engine on any stream
 * (a step's few bytes of bookkeeping behind the previous step's result on its way to the host), SM stores
 * do not. The host reads the block after synchronising the stream or an event recorded behind the call.
 * rmn_table_info reads the header this way. A block that is not mapped into the device falls back to
 * cudaMemcpyAsync. No counterpart in the reference (its maps live on the host).
 */
int rmn_readback_small(const void *d_src, void *h_dst_pinned, size_t bytes, void *stream);

/*
 * Look rows up: d_rows[i] = unique row of d_query[i] or -1.
 * Replaces: CoordinateMapCPU::find (engine/grid/lattice_cpu.hpp:449-470),
 *   remap_inverse_map (engine/grid/lattice_gpu.cu:58-71).
 */
int rmn_table_find(const void *d_table, const int32_t *d_query, uint32_t n_query, int W,
                   int32_t *d_rows, void *stream);

/*
 * Floor-align the spatial columns of `d_coords` to `out_tensor_stride[D]`
 * (host array; batch column copied). Integer floor; equal to the reference's
 * float floor for |c| < 2^24.
 * Replaces: detail::stride_coordinate (engine/grid/stencil.hpp:35-53),
 *   stride_copy (engine/grid/lattice_gpu.cu:309-336).
 * Feeding the result to rmn_table_build gives the strided-down map of
 * CoordinateMapCPU::stride (engine/grid/lattice_cpu.hpp:475-493); its
 * d_inverse is the stride map of lattice_cpu.hpp:679-710.
 */
int rmn_coords_stride(const int32_t *d_coords, uint32_t n_rows, int W,
                      const int32_t *out_tensor_stride, int32_t *d_out, void *stream);

/*
 * Continuous (field) coordinates -> integer voxel coordinates at a tensor stride, in float32 as the
 * reference computes it: batch column lroundf(v); spatial column j
 * tensor_stride[j] * (int)floor(v / tensor_stride[j]). d_field float32 [n_rows, W] (device),
 * tensor_stride int32 [W-1] (host), d_out int32 [n_rows, W] (device). Feeding d_out to rmn_table_build gives
 * the sparse map of a field and its d_inverse is the field-to-sparse map.
 * Replaces: CoordinateFieldMapCPU::quantize_coordinates (engine/grid/lattice_cpu.hpp:944-984),
 *   quantize_coordinates_kernel (engine/grid/lattice_gpu.cu:78-151), as called by
 *   field_to_sparse_insert_and_map_cpp (engine/grid/space_impl.hpp:103-166) under TensorField::sparse
 *   (engine/tensor/field.cpp:41-59).
 */
int rmn_field_quantize(const float *d_field, uint32_t n_rows, int W, const int32_t *tensor_stride,
                       int32_t *d_out, void *stream);

/*
 * d_out[i] = (int32)floor((double)d_in[i] / quantization_size) over ALL n_elems elements (every column,
 * the batch column included, as the reference does); quantization_size <= 0 means floor only.
 * in_type: 0 float32, 1 float64, 2 int32.
 * Replaces: the discretisation of sparse_quantize (engine/helpers/discretization.cpp:97-102), which the
 *   reference runs as torch ops in float64.
 */
int rmn_coords_discretize(const void *d_in, int in_type, uint64_t n_elems, double quantization_size,
                          int32_t *d_out, void *stream);

/*
 * Multilinear splat of a field onto the 2^D lattice corners around every point: output row
 * corner * n_rows + point has coordinates floor(v) (+1 on spatial axis a when bit a of `corner` is set; batch
 * column floor(v)) and features feats[point] * prod_a (bit ? frac_a : 1 - frac_a). d_out_coords int32
 * [n_rows << (W-1), W], d_out_feats [n_rows << (W-1), C] in `dtype` (RMN_F32 / RMN_BF16). Deduplicating
 * d_out_coords with rmn_table_build and summing the features of equal rows gives the splatted tensor.
 * Replaces: TensorField::splat (engine/tensor/field.cpp:61-94), a per-corner loop of torch ops there.
 */
int rmn_field_splat(const float *d_field, const void *d_feats, int dtype, uint32_t n_rows, int W, int C,
                    int32_t *d_out_coords, void *d_out_feats, void *stream);

/*
 * Region expansion: d_out[(row * K + k)] = d_coords[row] + d_offsets[k] on the spatial columns (batch
 * column copied), d_out int32 [n_rows * K, W]; d_offsets device int32 [K, W-1]. Deduplicating the result
 * with rmn_table_build gives the coordinate map that
 * Replaces: CoordinateMapCPU::stride_region for transposed regions (engine/grid/lattice_cpu.hpp:499-534;
 *   GPU: engine/grid/lattice_gpu.cu:434-601), the coordinate generation of pooling-transpose and generative
 *   transposed layers. (Rows come out numbered by first occurrence over (row, k); the reference numbers
 *   them in hash-iteration order.)
 */
int rmn_coords_expand(const int32_t *d_coords, uint32_t n_rows, int W, const int32_t *d_offsets, int K,
                      int32_t *d_out, void *stream);

/* =======================================================================
 * Kernel regions and kernel maps
 * ===================================================================== */

/* Number of offsets of a region. Replaces kernel_region::set_volume
 * (engine/grid/stencil.hpp:283-303). */
int rmn_region_volume(int region_type, int D, const int32_t *kernel_size, int n_custom);

/*
 * HOST helper: offsets[K, D] with neighbour = centre + offsets[k], in the
 * reference's enumeration order (axis 0 fastest; odd sizes centred, even
 * sizes 0..k-1; cross = centre then per-axis; custom scaled by stride*dil).
 * Replaces: kernel_region::coordinate_at (engine/grid/stencil.hpp:223-278).
 * Returns K, or a negative status.
 */
int rmn_region_offsets(int region_type, int D, const int32_t *kernel_size,
                       const int32_t *dilation, const int32_t *tensor_stride,
                       const int32_t *custom_offsets, int n_custom, int32_t *offsets);

/* Scratch bytes of rmn_kmap_build / rmn_kmap_pairs for n_query rows, K offsets. */
size_t rmn_kmap_workspace_bytes(uint32_t n_query, int K);

/*
 * For every query row q and offset k: d_nbr[k * n_query + q] = unique row a
 * of the table with coords_a == d_query[q] + d_offsets[k], else -1.
 * d_offset_ptr [K+1] int64 (device) receives the CSR row pointer of the pair
 * lists (pairs of offset k occupy [ptr[k], ptr[k+1])).
 * Replaces: CoordinateMapCPU::kernel_map (engine/grid/lattice_cpu.hpp:606-673),
 *   CoordinateMapGPU::kernel_map + direct_kernel_map / count_kernel
 *   (engine/grid/lattice_gpu.cu:1145-1549).
 * Forward convolution: table = input map, query = output coordinates,
 * offsets on the input tensor stride -> d_nbr is [K, N_out] of input rows.
 * Transposed convolution: table = output (fine) map, query = input (coarse)
 * coordinates, offsets on the output tensor stride
 * (engine/grid/space_impl.hpp:649-697) -> d_nbr is [K, N_in] of output rows.
 * d_offsets: DEVICE [K, D] int32.
 */
int rmn_kmap_build(const void *d_table, const int32_t *d_query, uint32_t n_query, int W,
                   const int32_t *d_offsets, int K, int32_t *d_nbr, int64_t *d_offset_ptr,
                   void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * rmn_kmap_build for the self map of a stride-1 convolution: `d_coords` must be exactly the
 * unique coordinates of `d_table` in row order (row q of the query IS row q of the table), K
 * must be odd and the offsets point-symmetric (offsets[K-1-k] == -offsets[k], offsets[K/2] == 0;
 * the caller checks this on its host copy). Same outputs as rmn_kmap_build, about half the
 * probes: a hit (q -> a) at offset k also fills (a -> q) at offset K-1-k, and the centre offset
 * is the identity. The workspace records that the map is a self map: rmn_kmap_pairs then emits the
 * pairs of offset K-1-k as the pairs of offset k with input and output row exchanged.
 * Every region of CoordinateMapCPU::kernel_map
 * (engine/grid/lattice_cpu.hpp:606-673) with odd kernel sizes is of this kind when input and
 * output maps coincide (engine/nn/conv.cpp:111-125).
 */
int rmn_kmap_build_self(const void *d_table, const int32_t *d_coords, uint32_t n_rows, int W,
                        const int32_t *d_offsets, int K, int32_t *d_nbr, int64_t *d_offset_ptr,
                        void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * Materialise the pair lists of the last rmn_kmap_build (same d_nbr,
 * d_offset_ptr and d_workspace): d_a_idx[p], d_q_idx[p] for p < ptr[K],
 * pairs of one offset sorted by query row (for a map built by
 * rmn_kmap_build_self the offsets above the centre are the exchanged lists of
 * their mirror offsets and therefore sorted by table row instead; the order is
 * deterministic either way, the reference's is not: engine/grid/lattice_cpu.hpp:657-659).
 * `capacity` = entries available in each index array (K * n_query always
 * suffices; ptr[K] is exact).
 * Replaces: the per-offset in/out vectors of cpu_kernel_map
 *   (engine/grid/maps.hpp:19-79) and gpu_kernel_map::decompose
 *   (engine/grid/lattice_gpu.cuh:440-488). Passing the arrays in the other
 *   order is the in/out swap of swap_in_out_map_functor
 *   (engine/grid/space.cpp:104-107).
 */
int rmn_kmap_pairs(const int32_t *d_nbr, uint32_t n_query, int K, const int64_t *d_offset_ptr,
                   const void *d_workspace, int32_t *d_a_idx, int32_t *d_q_idx,
                   uint64_t capacity, void *stream);

/*
 * Synchronising check after rmn_kmap_pairs / rmn_kmap_pairs_background on the same workspace: RMN_OK, or
 * RMN_ERR_ALLOC when `capacity` was smaller than the number of pairs (the lists are then truncated). A
 * caller that sizes the lists from d_offset_ptr[K] never needs it. No counterpart in the reference, whose
 * lists are std::vectors preallocated for every (offset, row) and shrunk afterwards
 * (engine/grid/lattice_cpu.hpp:606-673).
 */
int rmn_kmap_pairs_status(const void *d_workspace, uint32_t n_query, int K, void *stream);

/*
 * rmn_kmap_pairs built to run in the shadow of a convolution: same arguments and the same lists, bit for
 * bit, from blocks of 128 threads x 32 registers that become resident beside a convolution CTA already
 * running on the SM (launch it on a second stream after the convolution has been queued on the first). Alone
 * it is slower than rmn_kmap_pairs; use it only for that overlap. No counterpart in the reference, whose
 * kernel map IS the pair lists and is always built before the convolution.
 */
int rmn_kmap_pairs_background(const int32_t *d_nbr, uint32_t n_query, int K, const int64_t *d_offset_ptr,
                              const void *d_workspace, int32_t *d_a_idx, int32_t *d_q_idx, uint64_t capacity,
                              void *stream);

/*
 * Invert a neighbour table: d_nbr_t[k * n_a + a] = q where
 * d_nbr[k * n_query + q] == a, else -1. Used for the input-gradient pass and
 * for running a transposed convolution output-stationary.
 */
int rmn_kmap_transpose(const int32_t *d_nbr, uint32_t n_query, int K, uint32_t n_a,
                       int32_t *d_nbr_t, void *stream);

/* =======================================================================
 * Convolution over a neighbour table
 * Replaces: evaluate_sparse_convolution (engine/nn/conv.cpp:9-66), its torch
 *   autograd (index_select / matmul / index_add_ chain) and the scalar
 *   kernels of engine/ops/convolution_cpu.hpp:27-88.
 * Weights are [K, c_in, c_out] row-major, of the feature dtype
 * (engine/nn/conv.cpp:83-84). Accumulation is fp32.
 * ===================================================================== */

/* out[j, :] = sum_k feats[nbr[k, j], :] @ weights[k]      (rows with -1 skipped)
 * d_nbr: [K, n_dst]; d_feats: [n_src, c_in]; d_out: [n_dst, c_out] (overwritten). */
int rmn_conv_forward(const void *d_feats, uint32_t n_src, int c_in, const void *d_weights, int K,
                     int c_out, const int32_t *d_nbr, uint32_t n_dst, void *d_out, int dtype,
                     void *stream);

/* rmn_conv_forward with a fused per-channel epilogue:
 *   out[j, c] = act((sum_k feats[nbr[k, j], :] @ weights[k])[c] * scale[c] + shift[c])
 * d_scale / d_shift: fp32 [c_out] device arrays or NULL (1 / 0); relu != 0 applies max(., 0).
 * shift alone is the layer's bias add (engine/nn/conv.cpp:135-136); scale + shift is an
 * inference-mode batch norm folded with the bias (engine/nn/normalization.hpp:11-34), relu the
 * activation that follows it in the reference's blocks (engine/nn/residual.cpp:44-52). The
 * reference runs these as separate passes over [N, C]. */
int rmn_conv_forward_fused(const void *d_feats, uint32_t n_src, int c_in, const void *d_weights, int K,
                           int c_out, const int32_t *d_nbr, uint32_t n_dst, void *d_out, int dtype,
                           const float *d_scale, const float *d_shift, int relu, void *stream);

/* grad_feats[i, :] = sum_k grad_out[nbr_t[k, i], :] @ weights[k]^T
 * d_nbr_t: [K, n_src] of destination rows (rmn_kmap_transpose of the forward table). */
int rmn_conv_backward_input(const void *d_grad_out, uint32_t n_dst, int c_out,
                            const void *d_weights, int K, int c_in, const int32_t *d_nbr_t,
                            uint32_t n_src, void *d_grad_feats, int dtype, void *stream);

/* Scratch bytes of rmn_conv_backward_weight. */
size_t rmn_conv_backward_weight_workspace_bytes(uint32_t n_dst, int K, int c_in, int c_out,
                                                int dtype);

/* grad_weights[k] = sum_j feats[nbr[k, j], :]^T @ grad_out[j, :]   -> fp32 [K, c_in, c_out]
 * (fp32 for either feature dtype, so that gradients can be all-reduced
 * across GPUs without a cast). Deterministic: partial sums are reduced in a
 * fixed order through the workspace. */
int rmn_conv_backward_weight(const void *d_feats, uint32_t n_src, int c_in,
                             const void *d_grad_out, uint32_t n_dst, int c_out,
                             const int32_t *d_nbr, int K, float *d_grad_weights, int dtype,
                             void *d_workspace, size_t workspace_bytes, void *stream);

/* --------------------------- convolution plans ---------------------------------------------
 * Output rows of a sparse tensor arrive in arbitrary order, so every 128-row tile of the
 * output-stationary kernels has some neighbour at every kernel offset and nothing can be skipped,
 * although more than half of all (row, offset) entries of a surface scan are empty. A plan is an
 * internal row order for ONE neighbour table - rows sorted by which sides of the kernel region they
 * have neighbours on (a stable counting sort) - with, per 128-row tile, the set of offsets that hold
 * any neighbour, and a copy of the table in that order. The *_planned entry points then skip
 * (tile, offset) pairs without neighbours: no gather, no zero fill, no MMA. Public row numbering is
 * unchanged (the kernels store row perm[p]) and the results are bit-identical to the plain entry
 * points'. A plan costs about two passes over the table and is meant to be built once per kernel map
 * and shared by every convolution on that map (forward; input gradient of a stride-1 self map, whose
 * table is the same). No counterpart in the reference, whose convolution loops over per-offset pair
 * lists in torch (engine/nn/conv.cpp:47-64).
 */

/* Bytes of a plan / of the scratch rmn_conv_plan_build needs, for a table [K, n_dst]; 0 when K exceeds the
 * plan limit of 32 offsets (such tables are run unplanned). */
size_t rmn_conv_plan_bytes(uint32_t n_dst, int K);
size_t rmn_conv_plan_workspace_bytes(uint32_t n_dst, int K);

/*
 * Build the plan of neighbour table d_nbr [K, n_dst] (device). `offsets` is the HOST array [K, D] of the
 * region (rmn_region_offsets) the table was built with; it only steers the grouping of rows, any values give
 * correct results. d_plan: device, 256-byte aligned, rmn_conv_plan_bytes large. Returns RMN_ERR_UNSUPPORTED
 * for K > 32 (pass NULL as the plan then).
 */
int rmn_conv_plan_build(const int32_t *d_nbr, uint32_t n_dst, int K, const int32_t *offsets, int D, void *d_plan,
                        size_t plan_bytes, void *d_workspace, size_t workspace_bytes, void *stream);

/* rmn_conv_forward_fused / rmn_conv_backward_input / rmn_conv_forward_stats with a plan of the table they are
 * given (d_plan built from d_nbr, d_plan_t from d_nbr_t; NULL = no plan). The table itself is still passed: shapes
 * and dtypes that the tensor-core kernels do not take run on it unplanned. Replaces: as the plain entry points. */
int rmn_conv_forward_planned(const void *d_feats, uint32_t n_src, int c_in, const void *d_weights, int K,
                             int c_out, const int32_t *d_nbr, const void *d_plan, uint32_t n_dst, void *d_out,
                             int dtype, const float *d_scale, const float *d_shift, int relu, void *stream);
int rmn_conv_backward_input_planned(const void *d_grad_out, uint32_t n_dst, int c_out, const void *d_weights, int K,
                                    int c_in, const int32_t *d_nbr_t, const void *d_plan_t, uint32_t n_src,
                                    void *d_grad_feats, int dtype, void *stream);
int rmn_conv_forward_stats_planned(const void *d_feats, uint32_t n_src, int c_in, const void *d_weights, int K,
                                   int c_out, const int32_t *d_nbr, const void *d_plan, uint32_t n_dst, void *d_out,
                                   int dtype, const float *d_scale, const float *d_shift, int relu, double *d_stats,
                                   void *d_workspace, size_t workspace_bytes, void *stream);

/* ------------------- batch-normalisation pieces beside the convolution -------------------
 * The reference normalises with torch::nn::BatchNorm1d on the feature matrix after every convolution
 * (engine/nn/normalization.hpp:11-34; conv -> norm -> ReLU in engine/nn/residual.cpp:44-52). */

/* Bytes of workspace for rmn_channel_stats / rmn_conv_forward_stats with `channels` (output) channels. */
size_t rmn_channel_stats_workspace_bytes(int channels);

/*
 * d_stats[0][c] = sum over rows of x[r][c], d_stats[1][c] = sum of squares (double [2, channels]);
 * partial sums are added in a fixed order. Replaces: the statistics pass of BatchNorm1d in training mode.
 */
int rmn_channel_stats(const void *d_x, uint32_t n_rows, int channels, int dtype, double *d_stats,
                      void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * rmn_conv_forward_fused that also returns the channel statistics of the values it stores (d_stats as in
 * rmn_channel_stats, over the n_dst output rows): the tensor-core kernel accumulates them in its epilogue,
 * so the batch statistics of a following normalisation cost no pass over the output.
 * Replaces: evaluate_sparse_convolution (engine/nn/conv.cpp:9-66) + the statistics pass of the
 *   BatchNorm1d that follows it.
 */
int rmn_conv_forward_stats(const void *d_feats, uint32_t n_src, int c_in, const void *d_weights, int K,
                           int c_out, const int32_t *d_nbr, uint32_t n_dst, void *d_out, int dtype,
                           const float *d_scale, const float *d_shift, int relu, double *d_stats,
                           void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * out[r][c] = act(x[r][c] * scale[c] + shift[c]) (scale / shift may be NULL; act = ReLU when relu != 0);
 * in place when d_out == d_x. With scale = gamma / sqrt(var + eps) and shift = beta - mean * scale this is
 * the normalise + affine + ReLU of conv -> norm -> ReLU as one pass.
 */
int rmn_affine_act(const void *d_x, uint32_t n_rows, int channels, const float *d_scale,
                   const float *d_shift, int relu, void *d_out, int dtype, void *stream);

/* ------------------- training-mode batch normalisation as streaming passes -------------------
 * Replaces: torch::nn::BatchNorm1d on the feature matrix (engine/nn/normalization.hpp:11-34) in training mode,
 * forward and backward. Forward: rmn_channel_dot_stats(x, x) -> rmn_bn_forward_coeffs -> rmn_affine_act(x, scale,
 * shift). Backward: rmn_channel_dot_stats(dy, x) -> rmn_bn_backward_coeffs -> rmn_affine2(dy, x). */

/* Scratch bytes of rmn_channel_dot_stats. */
size_t rmn_channel_dot_stats_workspace_bytes(int channels);
/*
 * d_stats[0][c] = sum_r a[r][c], d_stats[1][c] = sum_r a[r][c] * b[r][c] (double [2, channels]); a == b gives the
 * sum and the sum of squares. Rows are read 16 bytes per lane at memory speed, partial sums are combined in a
 * fixed order. RMN_ERR_UNSUPPORTED unless channels * element size / 16 is a power of two <= 32 (bf16: 8 ... 256
 * channels, fp32: 4 ... 128) and both pointers are 16-byte aligned: use rmn_channel_stats then.
 */
int rmn_channel_dot_stats(const void *d_a, const void *d_b, uint32_t n_rows, int channels, int dtype,
                          double *d_stats, void *d_workspace, size_t workspace_bytes, void *stream);
/*
 * One tiny kernel: from d_stats (sum, sum of squares over `count` rows) the batch mean and 1 / sqrt(var + eps)
 * (fp32 [channels] each, kept for the backward pass), the affine y = x * scale + shift that normalises and applies
 * gamma / beta (NULL: 1 / 0), and the update of the running statistics in place (NULL: none; momentum and the
 * unbiased variance as torch.nn.BatchNorm1d). gamma, beta and the running statistics are `param_dtype` arrays.
 */
int rmn_bn_forward_coeffs(const double *d_stats, double count, const void *d_gamma, const void *d_beta,
                          void *d_running_mean, void *d_running_var, int param_dtype, float momentum, float eps,
                          int channels, float *d_scale, float *d_shift, float *d_mean, float *d_inv, void *stream);
/*
 * One tiny kernel: from d_dots = rmn_channel_dot_stats(dy, x) the gradients of gamma and beta (fp32) and the
 * coefficients of dx = c_dy * dy + c_x * x + c_0 (the batch-norm input gradient, to be applied by rmn_affine2).
 */
int rmn_bn_backward_coeffs(const double *d_dots, const float *d_mean, const float *d_inv, const void *d_gamma,
                           int param_dtype, double count, int channels, float *d_c_dy, float *d_c_x, float *d_c_0,
                           float *d_dgamma, float *d_dbeta, void *stream);
/* out[r][c] = c_a[c] * a[r][c] + c_b[c] * b[r][c] + c_0[c]; channels * element size a multiple of 16 bytes, pointers
 * 16-byte aligned (else RMN_ERR_UNSUPPORTED). */
int rmn_affine2(const void *d_a, const void *d_b, uint32_t n_rows, int channels, const float *d_c_a,
                const float *d_c_b, const float *d_c_0, void *d_out, int dtype, void *stream);

/* ------------------- weight-gradient all-reduce (data-parallel training) -------------------
 * Batches shard by sample: every rank hashes, maps and convolves its own samples, and the one
 * collective of a training step is the sum of the fp32 weight gradients over the ranks (NCCL over
 * NVLink). No counterpart in the reference, which has no distributed code (its RiemannSyncBatchNorm
 * is an alias of the plain layer, engine/nn/normalization.hpp:36-37). NCCL is looked up at run time
 * (libnccl.so.2); without it these entry points return RMN_ERR_UNSUPPORTED and the rest of the
 * library is unaffected. */
#define RMN_COMM_ID_BYTES 128

/* Rank 0: fill id_out[RMN_COMM_ID_BYTES] (ncclGetUniqueId); the host sends it to the other ranks by
 * whatever channel it has (a torch.distributed store, MPI, a file). */
int rmn_comm_unique_id(void *id_out);
/* Every rank, with its CUDA device current: join the communicator (ncclCommInitRank). *comm_out is an
 * ncclComm_t; a communicator created elsewhere with the same NCCL library may be passed to
 * rmn_allreduce_grads instead. Collective: returns when all ranks have called it. */
int rmn_comm_init(const void *id, int rank, int world_size, void **comm_out);
int rmn_comm_destroy(void *comm);

/* Scratch bytes of rmn_allreduce_grads for n_bufs buffers of counts[i] floats (0 for a single buffer,
 * which is reduced in place). */
size_t rmn_allreduce_grads_workspace_bytes(const size_t *counts, int n_bufs);

/*
 * In-place sum (average != 0: mean) over the ranks of n_bufs fp32 device buffers - the weight and bias
 * gradients of a step, d_bufs[i] holding counts[i] floats (d_bufs and counts are HOST arrays). The buffers
 * are packed into one flat bucket in d_workspace, reduced by ONE ncclAllReduce on `stream` and unpacked;
 * every rank must pass the same counts in the same order (a rank without a gradient for some buffer passes
 * zeros). With world_size == 1 it returns at once. Enqueue-only: run it on a second stream behind the
 * weight-gradient kernel and it overlaps the input-gradient kernel of the same layer.
 */
int rmn_allreduce_grads(void *comm, float *const *d_bufs, const size_t *counts, int n_bufs, void *d_workspace,
                        size_t workspace_bytes, int average, int world_size, void *stream);

/* ----------------------------- local pooling --------------------------------
 * Pooling modes of rmn_pool_forward / rmn_pool_backward: the three local modes of
 * PoolingMode (engine/foundation/types.hpp), i.e. RiemannSumPooling / RiemannAvgPooling /
 * RiemannMaxPooling (engine/nn/pooling.hpp:30-77). */
#define RMN_POOL_SUM 0
#define RMN_POOL_AVG 1
#define RMN_POOL_MAX 2

/*
 * out[j][c] = reduce over the offsets k with d_nbr[k][j] >= 0 of feats[d_nbr[k][j]][c]
 * (sum, mean over the rows present, or maximum); an output row without any neighbour is zero.
 * d_nbr is the neighbour table of rmn_kmap_build for (input map, output map, pooling region).
 * d_aux (may be NULL when no backward pass follows): average -> int32 [n_dst] rows present;
 * maximum -> int32 [n_dst, channels] input row that supplied each value (-1 none); unused for sum.
 * Features fp32 or bf16 (accumulated in fp32).
 * Replaces: evaluate_pooling (engine/nn/pooling.cpp:80-144): regrouping of the kernel-map pairs by
 *   output row on the host and one index_select + sum / mean / amax per output row.
 */
int rmn_pool_forward(const void *d_feats, uint32_t n_src, int channels, const int32_t *d_nbr, int K,
                     uint32_t n_dst, int mode, void *d_out, int32_t *d_aux, int dtype, void *stream);

/*
 * Gradient of rmn_pool_forward w.r.t. the input features: grad_in[i] = sum over (k, j = d_nbr_in[k][i])
 * of grad_out[j] (sum), grad_out[j] / count[j] (average) or grad_out[j][c] where row i supplied the
 * maximum (ties: the first offset wins; torch's amax splits ties evenly). d_nbr_in is the inverse
 * table (rmn_kmap_transpose of the forward table), d_aux the array the forward pass wrote.
 * Replaces: torch autograd through the index_select / sum / mean / amax chain of
 *   engine/nn/pooling.cpp:113-126.
 */
int rmn_pool_backward(const void *d_grad_out, uint32_t n_dst, int channels, const int32_t *d_nbr_in, int K,
                      uint32_t n_src, int mode, const int32_t *d_aux, void *d_grad_in, int dtype,
                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RMN_B200_H */
