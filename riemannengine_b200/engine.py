"""Host-side mirror of the reference's sparse-convolution interface.

Same names, argument order, defaults and error behaviour as the reference's
Python module (python/src/sparse_bindings.cpp:79-199, nn_bindings.cpp:91-117),
which re-exports the C++ classes of engine/grid/key.hpp,
engine/grid/space.hpp, engine/tensor/sparse_tensor.hpp and engine/nn/conv.hpp.
Every coordinate and convolution operation runs in the CUDA library through
:mod:`riemannengine_b200.ops`; CPU tensors are rejected.
"""
from __future__ import annotations

import builtins
import math
import random
import string
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops


# --- enums (engine/foundation/types.hpp:87-151) ------------------------------------------
class SparseTensorQuantizationMode:
    RANDOM_SUBSAMPLE, UNWEIGHTED_AVERAGE, UNWEIGHTED_SUM, MAX_POOL, NO_QUANTIZATION = range(5)


class GPUMemoryAllocatorBackend:
    PYTORCH, CUDA = 0, 1


class RiemannAlgorithm:
    DEFAULT, MEMORY_EFFICIENT, SPEED_OPTIMIZED = 0, 1, 2


class CoordinateMapBackend:
    CPU, CUDA = 0, 1


class RegionType:
    HYPER_CUBE, HYPER_CROSS, CUSTOM = 0, 1, 2


class PoolingMode:
    """engine/foundation/types.hpp:121-136 (same numbering)."""
    LOCAL_SUM_POOLING = 0
    LOCAL_AVG_POOLING = 1
    LOCAL_MAX_POOLING = 2
    GLOBAL_SUM_POOLING_DEFAULT = 3
    GLOBAL_AVG_POOLING_DEFAULT = 4
    GLOBAL_MAX_POOLING_DEFAULT = 5
    GLOBAL_SUM_POOLING_KERNEL = 6
    GLOBAL_AVG_POOLING_KERNEL = 7
    GLOBAL_MAX_POOLING_KERNEL = 8
    GLOBAL_SUM_POOLING_PYTORCH_INDEX = 9
    GLOBAL_AVG_POOLING_PYTORCH_INDEX = 10
    GLOBAL_MAX_POOLING_PYTORCH_INDEX = 11


class ConvolutionMode:
    DEFAULT, DIRECT_GEMM, COPY_GEMM = 0, 1, 2


ERROR_MAP_NOT_FOUND = "CoordinateMap not found"


def _stride_list(v, dimension: int) -> List[int]:
    if isinstance(v, int):
        return [int(v)] * dimension
    v = [int(x) for x in v]
    if len(v) == 1 and dimension > 1:
        v = v * dimension
    return v


class CoordinateMapKey:
    """(tensor stride, string id) handle of one coordinate map (engine/grid/key.hpp:18-99)."""

    def __init__(self, tensor_stride: Sequence[int], string_id: str = ""):
        self._stride = tuple(int(s) for s in tensor_stride)
        self._id = str(string_id)

    @property
    def tensor_stride(self) -> List[int]:
        return list(self._stride)

    def get_tensor_stride(self) -> List[int]:
        return list(self._stride)

    @property
    def coordinate_size(self) -> int:
        return len(self._stride) + 1

    def get_coordinate_size(self) -> int:
        return len(self._stride) + 1

    def get_key(self) -> Tuple[Tuple[int, ...], str]:
        return (self._stride, self._id)

    def is_key_set(self) -> bool:
        return True

    def __eq__(self, other) -> bool:
        return isinstance(other, CoordinateMapKey) and self.get_key() == other.get_key()

    def __hash__(self) -> int:
        return hash(self.get_key())

    def __repr__(self) -> str:
        s = "coordinate map key:" + str(list(self._stride))
        return s + (":" + self._id if self._id else "")


class KernelMap:
    """One cached kernel map.

    ``nbr_out`` [K, N_out] holds, for every output row and offset, the input row
    (or -1): the output-stationary form the convolution kernels consume.
    ``nbr_in`` [K, N_in] is its inverse (built on first use; the input-gradient
    pass and the in/out swap of a transposed map use it). ``pairs()`` gives the
    reference's representation: per-offset (in, out) lists.
    """

    def __init__(self, nbr_out: torch.Tensor, n_in: int, n_out: int, table_result=None,
                 nbr_in: Optional[torch.Tensor] = None, parent: Optional["KernelMap"] = None):
        self.nbr_out = nbr_out
        self.n_in = n_in
        self.n_out = n_out
        self.K = int(nbr_out.size(0))
        self._table_result = table_result   # ops.NeighbourTable (table = input map, query = output map)
        self._nbr_in = nbr_in
        self._parent = parent               # set on a swapped view
        self._pairs = None
        # stride-1 self map with a point-symmetric region: nbr_in[k] == nbr_out[K-1-k], so the
        # input-gradient pass reuses nbr_out with the kernel flipped along its offset axis
        self.self_symmetric = False
        self.region_offsets: Optional[np.ndarray] = None   # host [K, D] offsets the table was probed with
        self._plan_out = self._plan_in = None
        self._uses_out = self._uses_in = 0

    # Convolution plans (ops.conv_plan_build), built lazily under the same rule as the C++ host layer
    # (KernelMap::plan_out in riemann_cpp): by the pass that brings the work done on the table (sum of
    # c_in * c_out over the passes) to four 64 x 64 layers' worth, where the plan repays its build.
    plan_policy = 0  # 0 automatic, 1 always, 2 never

    @staticmethod
    def _want_plan(weight_sum: int, rows: int) -> bool:
        if KernelMap.plan_policy == 2 or rows < 8192:
            return False
        return KernelMap.plan_policy == 1 or weight_sum >= 4 * 64 * 64

    def plan_out(self, weight: int):
        if self._parent is not None:
            return self._parent.plan_in(weight)
        self._uses_out += weight
        if (self._plan_out is None and self.region_offsets is not None
                and self._want_plan(self._uses_out, self.n_out)):
            self._plan_out = ops.conv_plan_build(self.nbr_out, self.region_offsets)
        return self._plan_out

    def plan_in(self, weight: int):
        if self._parent is not None:
            return self._parent.plan_out(weight)
        if self.self_symmetric:
            return self.plan_out(weight)
        self._uses_in += weight
        if (self._plan_in is None and self.region_offsets is not None
                and self._want_plan(self._uses_in, self.n_in)):
            self._plan_in = ops.conv_plan_build(self.nbr_in, -self.region_offsets)
        return self._plan_in

    @property
    def nbr_in(self) -> torch.Tensor:
        if self._nbr_in is None:
            self._nbr_in = ops.kmap_transpose(self.nbr_out, self.n_in)
        return self._nbr_in

    def swapped(self) -> "KernelMap":
        """in <-> out (engine/grid/space.cpp:104-107)."""
        return KernelMap(self.nbr_in, self.n_out, self.n_in, None, self.nbr_out, parent=self)

    def pairs(self):
        """(offset_ptr int64 [K+1] (host), in_idx int32 [P], out_idx int32 [P]) on the device."""
        if self._pairs is None:
            if self._parent is not None:
                ptr, i, o = self._parent.pairs()
                self._pairs = (ptr, o, i)
            else:
                self._pairs = self._table_result.pairs()
        return self._pairs

    def total_pairs(self) -> int:
        return int(self.pairs()[0][-1])


class _CoordinateMap:
    def __init__(self, table: "ops.CoordinateTable", tensor_stride: Tuple[int, ...]):
        self.table = table
        self.tensor_stride = tensor_stride

    @property
    def coords(self) -> torch.Tensor:
        return self.table.coords

    @property
    def size(self) -> int:
        return self.table.n_unique


class CoordinateManager:
    """Owns coordinate maps and cached kernel maps (engine/grid/space.hpp:817-906).

    Only the CUDA backend exists here. ``GPUMemoryAllocatorBackend`` and
    ``RiemannAlgorithm`` are accepted and ignored: device memory always comes
    from torch's caching allocator and there is a single kernel-map algorithm.
    """

    def __init__(self, dimension: int, backend: int = CoordinateMapBackend.CUDA,
                 allocator: int = GPUMemoryAllocatorBackend.PYTORCH, algorithm: int = RiemannAlgorithm.DEFAULT):
        if backend != CoordinateMapBackend.CUDA:
            raise RuntimeError("riemannengine_b200 has no CPU coordinate-map backend")
        self._D = int(dimension)
        self._backend = backend
        self._maps: Dict[Tuple[Tuple[int, ...], str], _CoordinateMap] = {}
        self._kernel_maps: Dict[tuple, KernelMap] = {}
        self._fields: Dict[Tuple[Tuple[int, ...], str], torch.Tensor] = {}
        self._field_to_sparse: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}

    # -- introspection -------------------------------------------------------------------
    @property
    def dimension(self) -> int:
        return self._D

    def D(self) -> int:
        return self._D

    def backend(self) -> int:
        return self._backend

    def exists(self, key: CoordinateMapKey) -> bool:
        return key.get_key() in self._maps

    def _map(self, key: CoordinateMapKey, what: str = "") -> _CoordinateMap:
        m = self._maps.get(key.get_key())
        if m is None:
            raise RuntimeError((what + " " if what else "") + ERROR_MAP_NOT_FOUND)
        return m

    def size(self, coordinate_map_key: CoordinateMapKey) -> int:
        return self._map(coordinate_map_key).size

    def get_coordinates(self, coordinate_map_key: CoordinateMapKey) -> torch.Tensor:
        """[N, 1 + D] int32 coordinates in row order (engine/grid/space_impl.hpp:947-975)."""
        return self._map(coordinate_map_key).coords

    # -- insertion -------------------------------------------------------------------------
    def _fresh_id(self, stride: Tuple[int, ...], string_id: str) -> str:
        # key collision -> random string id (engine/grid/space_impl.hpp:284-289)
        while True:
            cand = string_id + "-" + "".join(random.choice(string.ascii_lowercase) for _ in range(8))
            if (stride, cand) not in self._maps:
                return cand

    def insert_and_map(self, coordinates: torch.Tensor, tensor_stride: Sequence[int], string_id: str = ""):
        """Returns (key, (mapping, inverse_mapping)), int64 tensors
        (engine/grid/space_impl.hpp:262-302, engine/grid/lattice_cpu.hpp:419-444)."""
        ops._check_coords(coordinates)
        stride = tuple(int(s) for s in tensor_stride)
        if coordinates.size(1) - 1 != len(stride):
            raise RuntimeError(f"The coordinate dimension (coordinate_size - 1): {coordinates.size(1) - 1} "
                               f"must match the size of tensor stride: {list(stride)}")
        if (stride, string_id) in self._maps:
            string_id = self._fresh_id(stride, string_id)
        table = ops.table_build(coordinates)
        self._maps[(stride, string_id)] = _CoordinateMap(table, stride)
        return CoordinateMapKey(stride, string_id), (table.mapping, table.inverse)

    def insert_field(self, coordinates: torch.Tensor, tensor_stride: Sequence[int],
                     string_id: str = "") -> CoordinateMapKey:
        """Registers continuous coordinates (float32 [N, 1 + D]) under a field key
        (engine/grid/space_impl.hpp:36-80)."""
        ops._check_field(coordinates)
        stride = tuple(int(s) for s in tensor_stride)
        if coordinates.size(1) - 1 != len(stride):
            raise RuntimeError(f"The coordinate dimension (coordinate_size - 1): {coordinates.size(1) - 1} "
                               f"must match the size of tensor stride: {list(stride)}")
        while (stride, string_id) in self._fields:
            string_id = string_id + "-" + "".join(random.choice(string.ascii_lowercase) for _ in range(8))
        self._fields[(stride, string_id)] = coordinates
        return CoordinateMapKey(stride, string_id)

    def get_field_coordinates(self, field_key: CoordinateMapKey) -> torch.Tensor:
        f = self._fields.get(field_key.get_key())
        if f is None:
            raise RuntimeError(ERROR_MAP_NOT_FOUND)
        return f

    def field_to_sparse_insert_and_map(self, field_key: CoordinateMapKey, sparse_tensor_stride: Sequence[int],
                                       sparse_tensor_string_id: str = ""):
        """Quantises a field at ``sparse_tensor_stride`` and inserts the voxels as a new sparse map; returns
        (sparse key, (first rows, field-row -> sparse-row)) (engine/grid/space_impl.hpp:103-166)."""
        field = self.get_field_coordinates(field_key)
        stride = [int(s) for s in sparse_tensor_stride]
        if field.size(1) - 1 != len(stride):
            raise RuntimeError(f"The coordinate dimension (coordinate_size - 1): {field.size(1) - 1} "
                               f"must match the size of tensor stride: {stride}")
        voxels = ops.field_quantize(field, stride)
        key, maps = self.insert_and_map(voxels, stride, sparse_tensor_string_id)
        self._field_to_sparse[(field_key.get_key(), key.get_key())] = maps
        return key, maps

    def get_field_to_sparse_map(self, field_key: CoordinateMapKey, sparse_key: CoordinateMapKey):
        maps = self._field_to_sparse.get((field_key.get_key(), sparse_key.get_key()))
        if maps is None:
            raise RuntimeError("Field To Sparse Map doesn't exist")
        return maps

    def stride(self, in_key: CoordinateMapKey, kernel_stride: Sequence[int], string_id: str = "") -> CoordinateMapKey:
        """Strided-down map, created if absent (engine/grid/space_impl.hpp:331-350). Coarse rows
        are numbered by first occurrence over the input rows."""
        in_map = self._map(in_key)
        ks = _stride_list(kernel_stride, self._D)
        if len(ks) != len(in_map.tensor_stride):
            raise RuntimeError("stride size mismatch.")
        out_stride = tuple(a * b for a, b in zip(in_map.tensor_stride, ks))
        out_key = (out_stride, string_id if string_id else in_key.get_key()[1])
        if out_key not in self._maps:
            aligned = ops.coords_stride(in_map.coords, out_stride)
            self._maps[out_key] = _CoordinateMap(ops.table_build(aligned), out_stride)
        return CoordinateMapKey(*out_key)

    def stride_region(self, in_key: CoordinateMapKey, kernel_size: Sequence[int], kernel_dilation: Sequence[int],
                      out_tensor_stride: Sequence[int], region_type: int = RegionType.HYPER_CUBE,
                      offsets: Optional[torch.Tensor] = None, string_id: str = "") -> CoordinateMapKey:
        """New coordinate map holding every ``in + offset`` of a transposed region on ``out_tensor_stride``
        (engine/grid/lattice_cpu.hpp:499-534 through space_impl.hpp:359-381): the coordinate generation of
        pooling-transpose. Rows are numbered by first occurrence over (input row, offset); the reference's
        numbering follows its hash iteration order, so results are compared by coordinate. A key that already
        exists gets a random suffix, as insert_and_map does."""
        in_map = self._map(in_key)
        custom = None
        if region_type == RegionType.CUSTOM:
            if offsets is None:
                raise RuntimeError("CUSTOM region needs offsets")
            custom = np.ascontiguousarray(offsets.detach().cpu().numpy(), np.int32).reshape(-1, len(kernel_size))
        off = ops.region_offsets(region_type, list(kernel_size), list(kernel_dilation), list(out_tensor_stride), custom)
        generated = ops.coords_expand(in_map.coords, off)
        key, _ = self.insert_and_map(generated, list(out_tensor_stride), string_id)
        return key

    def union_map(self, in_keys: Sequence[CoordinateMapKey]):
        """Union of several maps of one tensor stride (engine/grid/space_impl.hpp:896-914,
        lattice_cpu.hpp:801-833): returns (key of the merged map, one int64 [2, N_i] tensor per input
        map: row in that map, row in the merged map). Merged rows are numbered by first occurrence over
        the concatenated inputs."""
        if not in_keys:
            raise RuntimeError("union_map needs at least one map")
        maps = [self._map(k) for k in in_keys]
        stride = maps[0].tensor_stride
        if any(m.tensor_stride != stride for m in maps):
            raise RuntimeError("all maps of a union must share one tensor stride")
        merged = torch.cat([m.coords for m in maps], 0)
        key, _ = self.insert_and_map(merged, list(stride), "")
        table = self._map(key).table
        out = []
        for m in maps:
            rows = ops.table_find(table, m.coords).to(torch.int64)
            out.append(torch.stack([torch.arange(m.size, dtype=torch.int64, device=rows.device), rows]))
        return key, out

    def stride_map(self, in_key: CoordinateMapKey, out_key: CoordinateMapKey) -> torch.Tensor:
        """Row of ``out_key`` that every row of ``in_key`` floor-aligns to
        (engine/grid/lattice_cpu.hpp:679-710)."""
        in_map, out_map = self._map(in_key), self._map(out_key)
        aligned = ops.coords_stride(in_map.coords, out_map.tensor_stride)
        return ops.table_find(out_map.table, aligned)

    # -- kernel maps -----------------------------------------------------------------------
    def kernel_map(self, in_key: CoordinateMapKey, out_key: CoordinateMapKey, kernel_size: Sequence[int],
                   kernel_stride: Sequence[int], kernel_dilation: Sequence[int],
                   region_type: int = RegionType.HYPER_CUBE, offsets: Optional[torch.Tensor] = None,
                   is_transpose: bool = False, is_pool: bool = False) -> KernelMap:
        """Cached kernel map between two coordinate maps (engine/grid/space_impl.hpp:499-706)."""
        ks, kst, kd = list(kernel_size), list(kernel_stride), list(kernel_dilation)
        if not (len(ks) == len(kst) == len(kd)):
            raise RuntimeError("kernel size mismatch")
        custom = None
        if region_type == RegionType.CUSTOM:
            if offsets is None:
                raise RuntimeError("CUSTOM region needs offsets")
            custom = np.ascontiguousarray(offsets.detach().cpu().numpy(), np.int32).reshape(-1, len(ks))
            if min(ks + kst + kd) <= 0:
                raise RuntimeError("CUSTOM kernel size, stride and dilation must be positive")
        cache_key = (in_key.get_key(), out_key.get_key(), tuple(ks), tuple(kst), tuple(kd), region_type,
                     bool(is_transpose), bool(is_pool), None if custom is None else custom.tobytes())
        hit = self._kernel_maps.get(cache_key)
        if hit is not None:
            return hit
        in_map, out_map = self._map(in_key, "in_map"), self._map(out_key, "out_map")
        if len(ks) + 1 != in_map.table.width or len(ks) + 1 != out_map.table.width:
            raise RuntimeError("kernel size mismatch")
        if not is_transpose:
            # region on the INPUT tensor stride; probe the input map around every output row
            off = ops.region_offsets(region_type, ks, kd, in_map.tensor_stride, custom)
            res = ops.kmap_build(in_map.table, out_map.coords, off, self_map=in_map is out_map)
            kmap = KernelMap(res.nbr, in_map.size, out_map.size, res)
            kmap.self_symmetric = in_map is out_map and ops.offsets_point_symmetric(off)
            kmap.region_offsets = np.asarray(off, np.int32)
        else:
            swapped_key = (out_key.get_key(), in_key.get_key(), tuple(ks), tuple(kst), tuple(kd), region_type,
                           False, bool(is_pool), None if custom is None else custom.tobytes())
            fwd = self._kernel_maps.get(swapped_key)
            if fwd is not None:
                kmap = fwd.swapped()
            else:
                # region on the OUTPUT (fine) tensor stride: out = in + off_k. Probing the input
                # map at out - off_k yields the output-stationary table directly.
                off = ops.region_offsets(region_type, ks, kd, out_map.tensor_stride, custom)
                res = ops.kmap_build(in_map.table, out_map.coords, -off)
                kmap = KernelMap(res.nbr, in_map.size, out_map.size, res)
                kmap.region_offsets = -np.asarray(off, np.int32)
        self._kernel_maps[cache_key] = kmap
        return kmap

    def kernel_map_th(self, *args, **kwargs) -> Dict[int, torch.Tensor]:
        """{offset index -> int32 [2, P_k]} with rows (in, out); empty offsets omitted
        (engine/grid/space.cpp:202-228)."""
        ptr, a, q = self.kernel_map(*args, **kwargs).pairs()
        out = {}
        for k in range(len(ptr) - 1):
            lo, hi = int(ptr[k]), int(ptr[k + 1])
            if hi > lo:
                out[k] = torch.stack([a[lo:hi], q[lo:hi]])
        return out


class SparseTensor:
    """Features [N, C] + coordinate map key + manager (engine/tensor/sparse_tensor.hpp:16-80)."""

    def __init__(self, features: torch.Tensor, coordinates: Optional[torch.Tensor] = None,
                 coordinate_manager: Optional[CoordinateManager] = None,
                 quantization_mode: int = SparseTensorQuantizationMode.RANDOM_SUBSAMPLE,
                 algorithm: int = RiemannAlgorithm.DEFAULT, *, coordinate_map_key: Optional[CoordinateMapKey] = None):
        if isinstance(coordinates, CoordinateMapKey):  # (features, key, manager) form
            coordinate_map_key, coordinates = coordinates, None
        if features.dim() != 2:
            raise RuntimeError("Features must be a 2D tensor")
        self._coords_cache = None
        if coordinate_map_key is not None:
            if coordinate_manager is None:
                raise RuntimeError("Manager must not be null")
            self._manager = coordinate_manager
            self._key = coordinate_map_key
            self._dimension = coordinate_map_key.get_coordinate_size() - 1
            if coordinate_manager.D() != self._dimension:
                raise RuntimeError("Coordinate manager dimension does not match coordinate key")
            if features.size(0) != coordinate_manager.size(coordinate_map_key):
                raise RuntimeError("Feature row count must match coordinate map size")
            self._features = features
            return
        if coordinates is None or coordinates.dim() != 2:
            raise RuntimeError("Coordinates must be a 2D tensor")
        if features.size(0) != coordinates.size(0):
            raise RuntimeError("Features and coordinates must have same number of rows")
        if coordinates.size(1) < 2:
            raise RuntimeError("Coordinates must contain a batch column and spatial columns")
        self._dimension = int(coordinates.size(1)) - 1
        if coordinate_manager is None:
            coordinate_manager = CoordinateManager(self._dimension, CoordinateMapBackend.CUDA)
        if coordinate_manager.D() != self._dimension:
            raise RuntimeError("Coordinate manager dimension does not match coordinates")
        self._manager = coordinate_manager
        key, (first_rows, row_to_unique) = coordinate_manager.insert_and_map(
            coordinates.contiguous(), [1] * self._dimension)
        self._key = key
        self._features = self._quantize(features, first_rows, row_to_unique,
                                        coordinate_manager.size(key), quantization_mode)

    # engine/tensor/sparse_tensor.cpp:447-481
    @staticmethod
    def _quantize(features, first_rows, row_to_unique, unique_count, mode):
        M = SparseTensorQuantizationMode
        if mode == M.RANDOM_SUBSAMPLE:
            if features.size(0) == unique_count:  # all rows unique => first rows are 0..N-1
                return features
            return features.index_select(0, first_rows)
        if mode == M.NO_QUANTIZATION:
            return features
        if mode in (M.UNWEIGHTED_SUM, M.UNWEIGHTED_AVERAGE):
            result = torch.zeros((unique_count, features.size(1)), dtype=features.dtype, device=features.device)
            result.index_add_(0, row_to_unique, features)
            if mode == M.UNWEIGHTED_SUM:
                return result
            counts = torch.zeros(unique_count, dtype=features.dtype, device=features.device)
            counts.index_add_(0, row_to_unique, torch.ones(features.size(0), dtype=features.dtype,
                                                           device=features.device))
            return result / counts.clamp_min(1).unsqueeze(1)
        if mode == M.MAX_POOL:
            result = torch.zeros((unique_count, features.size(1)), dtype=features.dtype, device=features.device)
            return result.scatter_reduce(0, row_to_unique.unsqueeze(1).expand_as(features), features, "amax",
                                         include_self=False)
        raise RuntimeError("Unknown quantization mode")

    @property
    def F(self) -> torch.Tensor:
        return self._features

    features = F

    @property
    def C(self) -> torch.Tensor:
        if self._coords_cache is None:
            self._coords_cache = self._manager.get_coordinates(self._key)
        return self._coords_cache

    coordinates = C

    @property
    def coordinate_map_key(self) -> CoordinateMapKey:
        return self._key

    @property
    def coordinate_manager(self) -> CoordinateManager:
        return self._manager

    @property
    def tensor_stride(self) -> List[int]:
        return self._key.get_tensor_stride()

    @property
    def dimension(self) -> int:
        return self._dimension

    @property
    def device(self):
        return self._features.device

    @property
    def dtype(self):
        return self._features.dtype

    @property
    def requires_grad(self) -> bool:
        return self._features.requires_grad

    @property
    def shape(self):
        return (self._features.size(0), self._features.size(1))

    def __len__(self) -> int:
        return int(self._features.size(0))

    def to(self, arg) -> "SparseTensor":
        if isinstance(arg, torch.dtype):
            return SparseTensor(self._features.to(arg), self._key, self._manager)
        dev = torch.device(arg)
        if dev.type != "cuda":
            raise RuntimeError("riemannengine_b200 tensors live on CUDA devices only")
        return SparseTensor(self._features.to(dev), self._key, self._manager)

    def float(self) -> "SparseTensor":
        return self.to(torch.float32)

    def detach(self) -> "SparseTensor":
        return SparseTensor(self._features.detach(), self._key, self._manager)

    # -- arithmetic (engine/tensor/sparse_tensor.cpp:31-58, 345-395) ---------------------------
    def _binary(self, other: "SparseTensor", what: str, op) -> "SparseTensor":
        """Element-wise ``op`` on the union of the two coordinate sets (rows a side lacks count as zero).
        Tensors on one coordinate map are combined row by row and keep manager and key; otherwise the
        result lives on a new manager, as in the reference."""
        if self._dimension != other._dimension:
            raise RuntimeError(f"Cannot {what} tensors with different dimensions")
        if self.F.size(1) != other.F.size(1):
            raise RuntimeError(f"Cannot {what} tensors with different feature channel counts")
        if self.F.device != other.F.device:
            raise RuntimeError(f"Cannot {what} tensors on different devices")
        if self._manager is other._manager and self._key == other._key:
            return SparseTensor(op(self.F, other.F), coordinate_map_key=self._key, coordinate_manager=self._manager)
        stride = [min(a, b) for a, b in zip(self.tensor_stride, other.tensor_stride)]
        manager = CoordinateManager(self._dimension, CoordinateMapBackend.CUDA)
        key, (_, row_to_union) = manager.insert_and_map(torch.cat([self.C, other.C], 0).contiguous(), stride)
        size, n_l = manager.size(key), self.F.size(0)

        def align(feats, rows):
            return torch.zeros((size, feats.size(1)), dtype=feats.dtype, device=feats.device).index_copy(0, rows, feats)

        return SparseTensor(op(align(self.F, row_to_union[:n_l]), align(other.F, row_to_union[n_l:])),
                            coordinate_map_key=key, coordinate_manager=manager)

    def __add__(self, other):
        if isinstance(other, SparseTensor):
            return self._binary(other, "add", torch.add)
        return SparseTensor(self.F + other, coordinate_map_key=self._key, coordinate_manager=self._manager)

    def __sub__(self, other: "SparseTensor"):
        return self._binary(other, "subtract", torch.sub)

    def __mul__(self, other):
        if isinstance(other, SparseTensor):
            return self._binary(other, "multiply", torch.mul)
        return SparseTensor(self.F * other, coordinate_map_key=self._key, coordinate_manager=self._manager)

    def __truediv__(self, other: "SparseTensor"):
        return self._binary(other, "divide", torch.div)

    def __iadd__(self, other: "SparseTensor"):
        if self._manager is not other._manager:
            raise RuntimeError("Cannot add tensors from different managers")
        if self._key != other._key:
            raise RuntimeError("In-place addition requires same key")
        self._features += other.F
        return self

    def __repr__(self) -> str:
        return (f"SparseTensor(N={self._features.size(0)}, C={self._features.size(1)}, D={self._dimension}, "
                f"device={self._features.device})")


class TensorField:
    """Features on continuous coordinates; ``sparse()`` voxelises them (engine/tensor/field.hpp:10-53,
    engine/tensor/field.cpp:9-142)."""

    def __init__(self, features: torch.Tensor, coordinates: torch.Tensor,
                 coordinate_manager: Optional[CoordinateManager] = None,
                 quantization_mode: int = SparseTensorQuantizationMode.UNWEIGHTED_AVERAGE):
        if features.dim() != 2:
            raise RuntimeError("Features must be a 2D tensor")
        if coordinates.dim() != 2:
            raise RuntimeError("Coordinates must be a 2D tensor")
        if features.size(0) != coordinates.size(0):
            raise RuntimeError("Features and coordinates must have same number of rows")
        if coordinates.dtype not in (torch.float32, torch.float64):
            raise RuntimeError("TensorField coordinates must be float or double")
        if coordinates.size(1) < 2:
            raise RuntimeError("Coordinates must contain a batch column and spatial columns")
        self._dimension = int(coordinates.size(1)) - 1
        if coordinate_manager is None:
            coordinate_manager = CoordinateManager(self._dimension, CoordinateMapBackend.CUDA)
        if coordinate_manager.D() != self._dimension:
            raise RuntimeError("Coordinate manager dimension does not match coordinates")
        self._manager = coordinate_manager
        self._features = features
        # the reference's manager takes float32 fields only (engine/grid/space_impl.hpp:47)
        self._coordinates = coordinates.contiguous()
        self._field_key = coordinate_manager.insert_field(self._coordinates, [1] * self._dimension)
        self._inverse_mappings: Dict[tuple, torch.Tensor] = {}

    def sparse(self, tensor_stride: Optional[Sequence[int]] = None,
               coordinate_map_key: Optional[CoordinateMapKey] = None,
               quantization_mode: int = SparseTensorQuantizationMode.UNWEIGHTED_AVERAGE) -> "SparseTensor":
        stride = _stride_list(tensor_stride if tensor_stride else 1, self._dimension)
        key, (first_rows, row_to_unique) = self._manager.field_to_sparse_insert_and_map(self._field_key, stride)
        feats = SparseTensor._quantize(self._features, first_rows, row_to_unique, self._manager.size(key),
                                       quantization_mode)
        self._inverse_mappings[key.get_key()] = row_to_unique
        return SparseTensor(feats, coordinate_map_key=key, coordinate_manager=self._manager)

    def splat(self) -> "SparseTensor":
        coords, feats = ops.field_splat(self._coordinates, self._features)
        return SparseTensor(feats, coords, self._manager, SparseTensorQuantizationMode.UNWEIGHTED_SUM)

    def inverse_mapping(self, sparse_key: CoordinateMapKey) -> torch.Tensor:
        found = self._inverse_mappings.get(sparse_key.get_key())
        if found is None:
            _, (_, found) = self._manager.field_to_sparse_insert_and_map(self._field_key,
                                                                         sparse_key.get_tensor_stride())
            self._inverse_mappings[sparse_key.get_key()] = found
        return found

    def slice(self, sparse: "SparseTensor") -> torch.Tensor:
        """Features of ``sparse`` read back at the field's points (rows of the sparse tensor gathered
        through the field-to-sparse map)."""
        return sparse.F.index_select(0, self.inverse_mapping(sparse.coordinate_map_key))

    @property
    def F(self) -> torch.Tensor:
        return self._features

    @property
    def C(self) -> torch.Tensor:
        return self._coordinates

    @property
    def coordinate_field_map_key(self) -> CoordinateMapKey:
        return self._field_key

    @property
    def coordinate_manager(self) -> CoordinateManager:
        return self._manager

    @property
    def dimension(self) -> int:
        return self._dimension

    @property
    def device(self):
        return self._features.device

    @property
    def dtype(self):
        return self._features.dtype


class SparseQuantizeResult:
    """Fields of the reference's struct (helpers/discretization.hpp:15-21)."""

    def __init__(self, coordinates, features, labels, unique_index, inverse_mapping):
        self.coordinates = coordinates
        self.features = features
        self.labels = labels
        self.unique_index = unique_index
        self.inverse_mapping = inverse_mapping


def unique_coordinate_map(coordinates: torch.Tensor, tensor_stride: Optional[Sequence[int]] = None):
    """(first rows, row -> unique row) of int32 coordinates (engine/helpers/discretization.cpp:127-141)."""
    if coordinates.dim() != 2 or coordinates.size(1) < 2:
        raise RuntimeError("Coordinates must include a batch column and spatial dimensions")
    dimension = int(coordinates.size(1)) - 1
    stride = list(tensor_stride) if tensor_stride else [1] * dimension
    if len(stride) != dimension:
        raise RuntimeError("Tensor stride dimension must match coordinates")
    manager = CoordinateManager(dimension, CoordinateMapBackend.CUDA)
    return manager.insert_and_map(coordinates.contiguous(), stride)[1]


def quantize_th(coordinates: torch.Tensor):
    """[first rows, inverse] (engine/helpers/discretization.cpp:24-29)."""
    if coordinates.dtype != torch.int32:
        raise RuntimeError("Coordinates must have int32 dtype")
    unique, inverse = unique_coordinate_map(coordinates)
    return [unique, inverse]


def sparse_quantize(coordinates: torch.Tensor, features: Optional[torch.Tensor] = None,
                    labels: Optional[torch.Tensor] = None, ignore_label: int = -100,
                    quantization_size: Optional[float] = None, device=None) -> SparseQuantizeResult:
    """Voxelise points: ``floor(coordinates / quantization_size)`` on every column, deduplicate, keep the
    first point of every voxel (engine/helpers/discretization.cpp:78-125). The label-coalescing branch is a
    CPU-only loop in the reference (discretization.cpp:31-76) and has no device path here."""
    if coordinates.dim() != 2:
        raise RuntimeError("Coordinates must be a 2D matrix")
    if features is not None and (features.dim() != 2 or features.size(0) != coordinates.size(0)):
        raise RuntimeError("Feature rows must match coordinate rows")
    if labels is not None:
        raise RuntimeError("Label quantization currently requires CPU tensors")
    if quantization_size is not None and not (quantization_size > 0.0 and math.isfinite(quantization_size)):
        raise RuntimeError("Quantization size must be positive and finite")
    if device is not None:
        coordinates = coordinates.to(device)
    discrete = ops.coords_discretize(coordinates, quantization_size)
    if discrete.size(1) < 2:
        raise RuntimeError("Coordinates must include a batch column and spatial dimensions")
    unique, inverse = unique_coordinate_map(discrete)
    out_feats = None
    if features is not None:
        out_feats = features.to(discrete.device).index_select(0, unique)
    return SparseQuantizeResult(discrete.index_select(0, unique), out_feats, None, unique, inverse)


class KernelGenerator:
    """Normalised kernel hyper-parameters (engine/grid/stencil.hpp:533-598, stencil.cpp:81-193)."""

    class KernelParams:
        def __init__(self, kernel_size, kernel_stride, kernel_dilation, region_type, region_offsets,
                     expand_coordinates, D):
            self.kernel_size, self.kernel_stride, self.kernel_dilation = kernel_size, kernel_stride, kernel_dilation
            self.region_type, self.region_offsets = region_type, region_offsets
            self.expand_coordinates, self.D = expand_coordinates, D

    def __init__(self, kernel_size, stride=1, dilation=1, is_transpose: bool = False,
                 region_type: int = RegionType.HYPER_CUBE, region_offsets: Optional[torch.Tensor] = None,
                 expand_coordinates: bool = False, axis_types=None, dimension: int = -1):
        ks = [kernel_size] if isinstance(kernel_size, int) else list(kernel_size)
        D = dimension if dimension > 0 else len(ks)
        self._D = D
        self._ks, self._st, self._dl = _stride_list(ks, D), _stride_list(stride, D), _stride_list(dilation, D)
        for name, v in (("kernel_size", self._ks), ("kernel_stride", self._st), ("kernel_dilation", self._dl)):
            if len(v) != D:
                raise RuntimeError(f"{name} dimension mismatch")
        if axis_types:
            raise RuntimeError("axis_types must be empty")
        self._is_transpose = is_transpose
        self._region_type = region_type
        self._offsets = region_offsets
        if region_type == RegionType.CUSTOM:
            if region_offsets is None:
                raise RuntimeError("CUSTOM region needs region_offsets")
            self._offsets = region_offsets.to(torch.int32).reshape(-1, D).cpu()
        elif region_offsets is not None and region_offsets.numel() != 0:
            raise RuntimeError("region_offsets must be empty for HYPER_CUBE/HYPER_CROSS")
        self._expand = expand_coordinates
        if region_type == RegionType.HYPER_CUBE:
            self._volume = int(np.prod(self._ks))
        elif region_type == RegionType.HYPER_CROSS:
            self._volume = 1 + builtins.sum(k - 1 for k in self._ks)
        else:
            self._volume = int(self._offsets.size(0))

    def kernel_volume(self) -> int:
        return self._volume

    def kernel_size(self):
        return list(self._ks)

    def kernel_stride(self):
        return list(self._st)

    def kernel_dilation(self):
        return list(self._dl)

    def region_type(self):
        return self._region_type

    def expand_coordinates(self):
        return self._expand

    def dimension(self):
        return self._D

    def get_kernel(self, tensor_stride: Sequence[int], is_transpose: bool) -> "KernelGenerator.KernelParams":
        ts = list(tensor_stride)
        if len(ts) != self._D:
            raise RuntimeError("tensor_stride dimension mismatch")
        if any(s <= 0 for s in ts):
            raise RuntimeError("tensor_stride must be positive")
        return KernelGenerator.KernelParams(list(self._ks), list(self._st), list(self._dl), self._region_type,
                                            self._offsets, self._expand, self._D)


class _SparseConvolutionFunction(torch.autograd.Function):
    """out = sum_k F[in_k] @ W[k] scattered to out_k, with hand-written backward
    (the reference relies on torch autograd of index_select/matmul/index_add_,
    engine/nn/conv.cpp:47-64)."""

    @staticmethod
    def forward(ctx, features, kernel, kmap: KernelMap, bias=None):
        ctx.kmap = kmap
        ctx.has_bias = bias is not None
        ctx.save_for_backward(features, kernel)
        # the bias add is fused into the convolution's epilogue
        bf16 = features.dtype == torch.bfloat16  # plans serve the tensor-core kernels only
        ctx.weight = int(kernel.size(1) * kernel.size(2)) if bf16 else -1
        plan = kmap.plan_out(ctx.weight) if bf16 else None
        return ops.conv_forward(features, kernel, kmap.nbr_out, shift=bias, plan=plan)

    @staticmethod
    def backward(ctx, grad_out):
        features, kernel = ctx.saved_tensors
        kmap: KernelMap = ctx.kmap
        grad_out = grad_out.contiguous()
        g_feat = g_kernel = None
        if ctx.needs_input_grad[0]:
            plan = kmap.plan_in(ctx.weight) if ctx.weight >= 0 else None
            if kmap.self_symmetric:
                g_feat = ops.conv_backward_input(grad_out, kernel.flip(0), kmap.nbr_out, plan=plan)
            else:
                g_feat = ops.conv_backward_input(grad_out, kernel, kmap.nbr_in, plan=plan)
        if ctx.needs_input_grad[1]:
            g_kernel = ops.conv_backward_weight(features, grad_out, kmap.nbr_out).to(kernel.dtype)
        g_bias = None
        if ctx.has_bias and ctx.needs_input_grad[3]:
            g_bias = grad_out.sum(0, keepdim=True)
        return g_feat, g_kernel, None, g_bias


_TC_FORWARD_SHAPES = {(32, 32), (32, 64), (64, 32), (64, 64), (64, 128), (128, 64), (128, 128), (128, 256),
                      (256, 128), (256, 256)}


def tc_legal_shape(c_in: int, c_out: int) -> Tuple[int, int]:
    """Smallest channel counts >= (c_in, c_out) that the tensor-core kernels take in the forward pass and,
    with the roles exchanged, in the input-gradient pass; (c_in, c_out) itself when there is none."""
    best, cost = (c_in, c_out), None
    for ci in (32, 64, 128, 256):
        for co in (32, 64, 128, 256):
            if (ci >= c_in and co >= c_out and (ci, co) in _TC_FORWARD_SHAPES and (co, ci) in _TC_FORWARD_SHAPES
                    and (cost is None or ci * co < cost)):
                best, cost = (ci, co), ci * co
    return best


def sparse_convolution(features: torch.Tensor, kernel: torch.Tensor, kmap: KernelMap,
                       bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 channel counts without a tensor-core kernel (a 4-channel stem ...) are zero-padded to the next pair
    that has one with differentiable torch ops around the convolution (as riemann_cpp's sparse_convolution does)."""
    c_in, c_out = int(kernel.size(1)), int(kernel.size(2))
    if features.dtype == torch.bfloat16 and kernel.dtype == torch.bfloat16:
        ci, co = tc_legal_shape(c_in, c_out)
        if (ci, co) != (c_in, c_out):
            features = torch.nn.functional.pad(features, (0, ci - c_in))
            kernel = torch.nn.functional.pad(kernel, (0, co - c_out, 0, ci - c_in))
            if bias is not None and co != c_out:
                bias = torch.nn.functional.pad(bias, (0, co - c_out))
            out = _SparseConvolutionFunction.apply(features, kernel, kmap, bias)
            return out[:, :c_out] if co != c_out else out
    return _SparseConvolutionFunction.apply(features, kernel, kmap, bias)


class _ConvBNActFunction(torch.autograd.Function):
    """conv -> batch norm with batch statistics -> optional ReLU (training mode).

    The per-channel sums come out of the convolution's epilogue (ops.conv_forward_stats), the
    moments are merged over the ranks of ``group`` (whole-batch statistics: the sync batch norm the
    reference aliases to the plain layer, engine/nn/normalization.hpp:36-37), and normalise + affine
    + ReLU is one pass (ops.affine_act). The backward pass is the textbook batch-norm gradient
    followed by the convolution's input and weight gradients."""

    @staticmethod
    def forward(ctx, features, kernel, bias, gamma, beta, kmap: KernelMap, eps: float, relu: bool, group):
        from . import distributed as D
        z, stats = ops.conv_forward_stats(features, kernel, kmap.nbr_out, shift=bias)
        mean, var, count = D.merge_batch_stats(stats, z.size(0), group)
        inv = torch.rsqrt(var + eps)
        g = gamma.detach().double() if gamma is not None else torch.ones_like(inv)
        b = beta.detach().double() if beta is not None else torch.zeros_like(inv)
        scale = g * inv
        y = ops.affine_act(z, scale, b - mean * scale, relu)
        ctx.save_for_backward(features, kernel, z, y if relu else None, mean, inv, gamma)
        ctx.kmap, ctx.relu, ctx.count, ctx.group = kmap, relu, count, group
        ctx.has_bias, ctx.has_beta = bias is not None, beta is not None
        total = torch.tensor(float(count), dtype=torch.float64, device=y.device)
        ctx.mark_non_differentiable(mean, var, total)
        return y, mean, var, total

    @staticmethod
    def backward(ctx, grad_y, _gm, _gv, _gc):
        from . import distributed as D
        features, kernel, z, y, mean, inv, gamma = ctx.saved_tensors
        dy = grad_y.float()
        if ctx.relu:
            dy = dy * (y > 0)
        zhat = (z.float() - mean.float()) * inv.float()
        dbeta = dy.sum(0, dtype=torch.float64)
        dgamma = (dy * zhat).sum(0, dtype=torch.float64)
        D.allreduce_sum_([dbeta, dgamma], ctx.group)
        n = float(max(ctx.count, 1))
        g = gamma.detach().float() if gamma is not None else torch.ones_like(inv, dtype=torch.float32)
        dz = (g * inv.float()) * (dy - (dbeta / n).float() - zhat * (dgamma / n).float())
        dz = dz.to(z.dtype)
        kmap = ctx.kmap
        g_feat = g_kernel = None
        if ctx.needs_input_grad[0]:
            if kmap.self_symmetric:
                g_feat = ops.conv_backward_input(dz, kernel.flip(0), kmap.nbr_out)
            else:
                g_feat = ops.conv_backward_input(dz, kernel, kmap.nbr_in)
        if ctx.needs_input_grad[1]:
            g_kernel = ops.conv_backward_weight(features, dz, kmap.nbr_out).to(kernel.dtype)
        g_bias = dz.sum(0, keepdim=True).to(kernel.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        g_gamma = dgamma.to(gamma.dtype) if gamma is not None and ctx.needs_input_grad[3] else None
        g_beta = dbeta.to(gamma.dtype if gamma is not None else torch.float32) if ctx.has_beta and ctx.needs_input_grad[4] else None
        return g_feat, g_kernel, g_bias, g_gamma, g_beta, None, None, None, None


def fused_conv_bn_relu(input: "SparseTensor", conv, bn: Optional[torch.nn.BatchNorm1d] = None,
                       relu: bool = True, process_group=None) -> "SparseTensor":
    """conv -> batch norm -> ReLU (the reference's blocks run these as three modules and four passes
    over the features, engine/nn/residual.cpp:44-52).

    ``bn`` in eval mode: the norm's running statistics and affine and the layer's bias are folded
    into the convolution epilogue: ONE kernel, inference only.
    ``bn`` in training mode: batch statistics from the convolution epilogue, merged over
    ``process_group`` when one is initialised (sync batch norm), then one normalise + ReLU pass;
    differentiable; running statistics are updated as torch.nn.BatchNorm1d does."""
    base = conv.base if hasattr(conv, "base") else conv
    if bn is not None and bn.training:
        out_key, kmap = base._output_key_and_map(input)
        bias = base.bias.reshape(-1) if base.bias is not None else None
        y, mean, var, total = _ConvBNActFunction.apply(input.F, base.kernel, bias, bn.weight, bn.bias, kmap, bn.eps,
                                                       relu, process_group)
        if bn.track_running_stats and bn.running_mean is not None:
            with torch.no_grad():
                bn.num_batches_tracked += 1
                m = bn.momentum if bn.momentum is not None else 1.0 / float(bn.num_batches_tracked)
                count = float(total.item())
                unbiased = var * (count / max(count - 1.0, 1.0))
                bn.running_mean.mul_(1 - m).add_(mean.to(bn.running_mean.dtype), alpha=m)
                bn.running_var.mul_(1 - m).add_(unbiased.to(bn.running_var.dtype), alpha=m)
        return SparseTensor(y, out_key, input.coordinate_manager)
    with torch.no_grad():
        scale = shift = None
        bias = base.bias.reshape(-1).float() if base.bias is not None else None
        if bn is not None:
            inv = torch.rsqrt(bn.running_var.float() + bn.eps)
            scale = inv * (bn.weight.float() if bn.weight is not None else 1.0)
            shift = -bn.running_mean.float() * scale
            if bn.bias is not None:
                shift = shift + bn.bias.float()
            if bias is not None:
                shift = shift + bias * scale
        else:
            shift = bias
        out_key, kmap = base._output_key_and_map(input)
        feats = ops.conv_forward(input.F, base.kernel, kmap.nbr_out, scale=scale, shift=shift, relu=relu)
    return SparseTensor(feats, out_key, input.coordinate_manager)


class RiemannBatchNorm(torch.nn.Module):
    """RiemannBatchNormImpl (engine/nn/normalization.hpp:11-34): torch's BatchNorm1d over the feature
    matrix of a SparseTensor. ``normalization`` is the wrapped module (same attribute name as the
    reference's registered sub-module); pass it to ``fused_conv_bn_relu`` to fuse it with the
    preceding convolution."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 track_running_stats: bool = True):
        super().__init__()
        self.normalization = torch.nn.BatchNorm1d(num_features, eps=eps, momentum=momentum, affine=affine,
                                                  track_running_stats=track_running_stats)

    def forward(self, input: "SparseTensor") -> "SparseTensor":
        return SparseTensor(self.normalization(input.F), input.coordinate_map_key, input.coordinate_manager)


RiemannSyncBatchNorm = RiemannBatchNorm  # the reference's alias (engine/nn/normalization.hpp:36-37)


class RiemannConvolutionBase(torch.nn.Module):
    """engine/nn/conv.hpp:13-37, conv.cpp:70-138."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size=3, stride=1, dilation=1, bias: bool = False,
                 is_transpose: bool = False, expand_coordinates: bool = False,
                 convolution_mode: int = ConvolutionMode.DEFAULT, dimension: int = 3,
                 region_type: int = RegionType.HYPER_CUBE):
        super().__init__()
        if in_channels <= 0 or out_channels <= 0:
            raise RuntimeError("Convolution channel counts must be positive")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.is_transpose = is_transpose
        self.dimension = dimension
        self.convolution_mode = convolution_mode
        self.kernel_generator = KernelGenerator(kernel_size, stride, dilation, is_transpose, region_type, None,
                                                expand_coordinates, None, dimension)
        volume = self.kernel_generator.kernel_volume()
        self.kernel = torch.nn.Parameter(torch.empty(volume, in_channels, out_channels))
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(1, out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        # U(-1/sqrt(fan), 1/sqrt(fan)), fan = (C_out if transpose else C_in) * K  (conv.cpp:94-102)
        fan = (self.out_channels if self.is_transpose else self.in_channels) * self.kernel_generator.kernel_volume()
        bound = 1.0 / math.sqrt(fan)
        with torch.no_grad():
            self.kernel.uniform_(-bound, bound)
            if self.bias is not None:
                self.bias.uniform_(-bound, bound)

    def _output_key_and_map(self, input: SparseTensor):
        """Key arithmetic of conv.cpp:104-132 plus the (cached) kernel map."""
        if input.dimension != self.dimension:
            raise RuntimeError("Input dimension mismatch")
        if input.F.size(1) != self.in_channels:
            raise RuntimeError("Input channel count does not match convolution")
        params = self.kernel_generator.get_kernel(input.tensor_stride, self.is_transpose)
        in_stride, string_id = input.coordinate_map_key.get_key()
        out_stride = list(in_stride)
        for axis, step in enumerate(params.kernel_stride):
            if self.is_transpose:
                if step == 0 or out_stride[axis] % step != 0:
                    raise RuntimeError("Transpose convolution stride must divide tensor stride")
                out_stride[axis] //= step
            else:
                out_stride[axis] *= step
        out_key = CoordinateMapKey(out_stride, string_id)
        manager = input.coordinate_manager
        if not self.is_transpose and any(s != 1 for s in params.kernel_stride):
            out_key = manager.stride(input.coordinate_map_key, params.kernel_stride)
        if self.is_transpose and self.kernel_generator.expand_coordinates():
            # generative layer: the output coordinates are generated (as riemann_cpp's layer does)
            out_key = manager.stride_region(input.coordinate_map_key, params.kernel_size, params.kernel_dilation,
                                            out_stride, params.region_type, params.region_offsets)
        kmap = manager.kernel_map(input.coordinate_map_key, out_key, params.kernel_size, params.kernel_stride,
                                  params.kernel_dilation, params.region_type, params.region_offsets,
                                  self.is_transpose, False)
        return out_key, kmap

    def forward(self, input: SparseTensor) -> SparseTensor:
        out_key, kmap = self._output_key_and_map(input)
        result = sparse_convolution(input.F, self.kernel, kmap, self.bias)
        return SparseTensor(result, out_key, input.coordinate_manager)


class _ConvWrapper(torch.nn.Module):
    _transpose = False
    _expand_default = False

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 1, dilation: int = 1,
                 bias: bool = False, expand_coordinates: bool = False,
                 convolution_mode: int = ConvolutionMode.DEFAULT, dimension: int = 3):
        super().__init__()
        self.base = RiemannConvolutionBase(in_channels, out_channels, kernel_size, stride, dilation, bias,
                                           self._transpose, expand_coordinates or self._expand_default,
                                           convolution_mode, dimension)

    @property
    def kernel(self) -> torch.nn.Parameter:
        return self.base.kernel

    @property
    def bias(self):
        return self.base.bias

    def forward(self, input: SparseTensor) -> SparseTensor:
        return self.base(input)


class RiemannConvolution(_ConvWrapper):
    """engine/nn/conv.hpp:39-55."""


class RiemannConvolutionTranspose(_ConvWrapper):
    """engine/nn/conv.hpp:57-72; the output map must already exist in the manager."""
    _transpose = True


class RiemannGenerativeConvolutionTranspose(_ConvWrapper):
    """engine/nn/conv.hpp:74-88 with the coordinate expansion the flag stands for: the output coordinates are
    generated by ``stride_region`` (the reference's own forward, conv.cpp:104-138, never reaches it)."""
    _transpose = True
    _expand_default = True

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 1, dilation: int = 1,
                 bias: bool = False, convolution_mode: int = ConvolutionMode.DEFAULT, dimension: int = 3):
        super().__init__(in_channels, out_channels, kernel_size, stride, dilation, bias, True, convolution_mode,
                         dimension)


# ---------------------------------------------------------------------------------------------
# Local pooling (engine/nn/pooling.hpp:12-77, pooling.cpp:80-144, 166-195)
# ---------------------------------------------------------------------------------------------
class _SparsePoolingFunction(torch.autograd.Function):
    """out[j] = reduce over the kernel-map neighbours of output row j; the backward pass gathers
    through the inverse neighbour table (one store per input row, no atomics)."""

    @staticmethod
    def forward(ctx, features, kmap: KernelMap, mode: int):
        out, aux = ops.pool_forward(features, kmap.nbr_out, mode, want_aux=features.requires_grad)
        ctx.kmap, ctx.mode, ctx.aux = kmap, mode, aux
        return out

    @staticmethod
    def backward(ctx, grad_out):
        return ops.pool_backward(grad_out, ctx.kmap.nbr_in, ctx.mode, ctx.aux), None, None


_LOCAL_POOL_MODES = {PoolingMode.LOCAL_SUM_POOLING: ops.POOL_SUM, PoolingMode.LOCAL_AVG_POOLING: ops.POOL_AVG,
                     PoolingMode.LOCAL_MAX_POOLING: ops.POOL_MAX}


class RiemannPoolingBase(torch.nn.Module):
    """RiemannPoolingBaseImpl (engine/nn/pooling.cpp:166-195): the output map is the input map strided
    by the pooling stride; every output row reduces the input rows of its kernel region that exist
    (average = mean over the rows present; an output row without neighbours is zero)."""

    def __init__(self, kernel_size=3, stride=1, dilation=1, mode: int = PoolingMode.LOCAL_AVG_POOLING,
                 dimension: int = 3, kernel_generator: Optional["KernelGenerator"] = None):
        super().__init__()
        if mode not in _LOCAL_POOL_MODES:
            raise RuntimeError("Local pooling requires a local pooling mode")
        self.kernel_generator = kernel_generator if kernel_generator is not None else KernelGenerator(
            kernel_size, stride, dilation, False, RegionType.HYPER_CUBE, None, False, dimension=dimension)
        self.mode = mode
        self.dimension = dimension

    def forward(self, input: SparseTensor) -> SparseTensor:
        if input.dimension != self.dimension:
            raise RuntimeError("Input dimension mismatch")
        params = self.kernel_generator.get_kernel(input.tensor_stride, False)
        manager = input.coordinate_manager
        out_key = manager.stride(input.coordinate_map_key, params.kernel_stride)
        kmap = manager.kernel_map(input.coordinate_map_key, out_key, params.kernel_size, params.kernel_stride,
                                  params.kernel_dilation, params.region_type, params.region_offsets, False, True)
        result = _SparsePoolingFunction.apply(input.F, kmap, _LOCAL_POOL_MODES[self.mode])
        return SparseTensor(result, out_key, manager)


class RiemannAvgPooling(RiemannPoolingBase):
    def __init__(self, kernel_size: int, stride: int = 1, dilation: int = 1, dimension: int = 3):
        super().__init__(kernel_size, stride, dilation, PoolingMode.LOCAL_AVG_POOLING, dimension)


class RiemannSumPooling(RiemannPoolingBase):
    def __init__(self, kernel_size: int, stride: int = 1, dilation: int = 1, dimension: int = 3):
        super().__init__(kernel_size, stride, dilation, PoolingMode.LOCAL_SUM_POOLING, dimension)


class RiemannMaxPooling(RiemannPoolingBase):
    def __init__(self, kernel_size: int, stride: int = 1, dilation: int = 1, dimension: int = 3):
        super().__init__(kernel_size, stride, dilation, PoolingMode.LOCAL_MAX_POOLING, dimension)


def cat(tensors: Sequence[SparseTensor]) -> SparseTensor:
    """Channel concatenation of tensors that share one coordinate map (riemann::cat,
    engine/nn/operations.cpp:56-64): the skip connections of encoder/decoder networks."""
    tensors = list(tensors)
    if not tensors:
        raise RuntimeError("cat needs at least one tensor")
    first = tensors[0]
    for t in tensors[1:]:
        if t.coordinate_manager is not first.coordinate_manager or t.coordinate_map_key != first.coordinate_map_key:
            raise RuntimeError("Sparse tensors must share the same coordinate map")
    return SparseTensor(torch.cat([t.F for t in tensors], 1), first.coordinate_map_key, first.coordinate_manager)


def sum(tensors: Sequence[SparseTensor]) -> SparseTensor:  # noqa: A001 - the reference's name
    """Feature sum of tensors on one coordinate map (engine/nn/operations.cpp:66-73)."""
    out = cat(tensors)
    first = tensors[0]
    if any(t.F.size(1) != first.F.size(1) for t in tensors):
        raise RuntimeError("Sparse tensor feature widths must match")
    total = first.F
    for t in tensors[1:]:
        total = total + t.F
    return SparseTensor(total, out.coordinate_map_key, out.coordinate_manager)


def mean(tensors: Sequence[SparseTensor]) -> SparseTensor:
    """engine/nn/operations.cpp:75-77"""
    return sum(tensors) * (1.0 / len(tensors))


class RiemannReLU(torch.nn.Module):
    """ReLU on the features; the coordinate map is shared (engine/nn/activation.hpp:11-29)."""

    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = inplace

    def forward(self, input: SparseTensor) -> SparseTensor:
        out = torch.relu_(input.F) if self.inplace else torch.relu(input.F)
        return SparseTensor(out, input.coordinate_map_key, input.coordinate_manager)


class RiemannPoolingTranspose(torch.nn.Module):
    """RiemannPoolingTransposeImpl (engine/nn/pooling.cpp:197-229, maps: pooling.cpp:49-70): un-pooling
    onto GENERATED coordinates. The output map holds every input coordinate expanded through the
    kernel region on the finer tensor stride (stride_region); every output row then reduces (sum by
    default) the input rows whose region reaches it."""

    def __init__(self, kernel_size=2, stride=2, dilation=1, expand_coordinates: bool = False, dimension: int = 3,
                 kernel_generator: Optional["KernelGenerator"] = None, mode: int = PoolingMode.LOCAL_SUM_POOLING):
        super().__init__()
        if mode not in _LOCAL_POOL_MODES:
            raise RuntimeError("Transpose pooling requires a local pooling mode")
        self.kernel_generator = kernel_generator if kernel_generator is not None else KernelGenerator(
            kernel_size, stride, dilation, True, RegionType.HYPER_CUBE, None, expand_coordinates, dimension=dimension)
        self.mode = mode
        self.dimension = dimension

    def forward(self, input: SparseTensor) -> SparseTensor:
        if input.dimension != self.dimension:
            raise RuntimeError("Input dimension mismatch")
        params = self.kernel_generator.get_kernel(input.tensor_stride, True)
        in_stride = input.tensor_stride
        out_stride = []
        for s, step in zip(in_stride, params.kernel_stride):
            if step == 0 or s % step != 0:
                raise RuntimeError("Transpose stride must divide tensor stride")
            out_stride.append(s // step)
        manager = input.coordinate_manager
        if list(out_stride) == list(in_stride) and not params.expand_coordinates:
            # a map of the output stride exists (the input's own): it is reused, not regenerated
            # (engine/grid/space_impl.hpp:366-380 inside the layer's private manager)
            out_key = input.coordinate_map_key
        else:
            out_key = manager.stride_region(input.coordinate_map_key, params.kernel_size, params.kernel_dilation,
                                            out_stride, params.region_type, params.region_offsets)
        kmap = manager.kernel_map(input.coordinate_map_key, out_key, params.kernel_size, params.kernel_stride,
                                  params.kernel_dilation, params.region_type, params.region_offsets, True, True)
        result = _SparsePoolingFunction.apply(input.F, kmap, _LOCAL_POOL_MODES[self.mode])
        return SparseTensor(result, out_key, manager)
