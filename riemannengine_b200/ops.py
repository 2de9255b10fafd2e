"""Tensor-level wrappers of the C ABI: torch CUDA tensors in, torch CUDA tensors out.

torch is used for device memory and streams only; every operation here is one
or more calls into ``librmn_b200.so`` on the current CUDA stream. Nothing in
this module computes on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from . import capi


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[ctypes.c_void_p]:
    if t is None or t.numel() == 0:
        return None
    return ctypes.c_void_p(t.data_ptr())


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: this library has no CPU path")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return capi.F32
    if t.dtype == torch.bfloat16:
        return capi.BF16
    raise RuntimeError(f"unsupported feature dtype {t.dtype}: float32 and bfloat16 only")


def _check_coords(coords: torch.Tensor, what: str = "coordinates") -> None:
    # same checks as the reference's insert_and_map_cpp (engine/grid/space_impl.hpp:268-276)
    _require_cuda(coords, what)
    if coords.dim() != 2:
        raise RuntimeError(f"{what} must be 2-D [N, 1 + D]")
    if coords.dtype != torch.int32:
        raise RuntimeError(f"{what} must be int32")
    if not coords.is_contiguous():
        raise RuntimeError(f"{what} must be contiguous")
    if not 2 <= coords.size(1) <= capi.MAX_W:
        raise RuntimeError(f"{what} must have between 2 and {capi.MAX_W} columns")


class CoordinateTable:
    """Device hash table over the unique rows of a coordinate list."""

    def __init__(self, buffer, n_rows, width, n_unique, mapping, inverse, coords):
        self.buffer = buffer          # uint8 [rmn_table_bytes]
        self.n_rows = n_rows
        self.width = width
        self.n_unique = n_unique
        self.mapping = mapping        # int64 [n_unique]  first-occurrence rows
        self.inverse = inverse        # int64 [n_rows]    unique row of every input row
        self.coords = coords          # int32 [n_unique, W] unique rows in map order


def table_build(coords: torch.Tensor) -> CoordinateTable:
    """Dedup-insert ``coords`` [N, W] (rmn_table_build). Synchronises once to read n_unique."""
    _check_coords(coords)
    lib = capi.lib()
    n, w = int(coords.size(0)), int(coords.size(1))
    dev = coords.device
    with torch.cuda.device(dev):
        tbytes = lib.rmn_table_bytes(n)
        buf = torch.empty(tbytes, dtype=torch.uint8, device=dev)
        mapping = torch.empty(n, dtype=torch.int64, device=dev)
        inverse = torch.empty(n, dtype=torch.int64, device=dev)
        uniq = torch.empty((n, w), dtype=torch.int32, device=dev)
        wbytes = lib.rmn_table_build_workspace_bytes(n)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        capi.check(lib.rmn_table_build(_ptr(coords), n, w, _ptr(buf), tbytes, _ptr(mapping), _ptr(inverse),
                                       _ptr(uniq), _ptr(ws), wbytes, _stream()), "rmn_table_build")
        info = (ctypes.c_uint32 * 4)()
        capi.check(lib.rmn_table_info(_ptr(buf), info, _stream()), "rmn_table_build")
    nu = int(info[0])
    return CoordinateTable(buf, n, w, nu, mapping[:nu], inverse, uniq[:nu])


def table_find(table: CoordinateTable, query: torch.Tensor) -> torch.Tensor:
    """Unique row of every query row, -1 when absent (rmn_table_find)."""
    _check_coords(query, "query coordinates")
    if query.size(1) != table.width:
        raise RuntimeError("query width does not match the table")
    rows = torch.empty(query.size(0), dtype=torch.int32, device=query.device)
    with torch.cuda.device(query.device):
        capi.check(capi.lib().rmn_table_find(_ptr(table.buffer), _ptr(query), int(query.size(0)), table.width,
                                             _ptr(rows), _stream()), "rmn_table_find")
    return rows


def coords_stride(coords: torch.Tensor, out_tensor_stride: Sequence[int]) -> torch.Tensor:
    """Floor-align spatial columns to ``out_tensor_stride`` (rmn_coords_stride)."""
    _check_coords(coords)
    st = np.ascontiguousarray(out_tensor_stride, dtype=np.int32)
    if st.size != coords.size(1) - 1:
        raise RuntimeError("Invalid stride")
    out = torch.empty_like(coords)
    with torch.cuda.device(coords.device):
        capi.check(capi.lib().rmn_coords_stride(_ptr(coords), int(coords.size(0)), int(coords.size(1)),
                                                st.ctypes.data_as(ctypes.c_void_p), _ptr(out), _stream()),
                   "rmn_coords_stride")
    return out


def region_offsets(region_type: int, kernel_size: Sequence[int], dilation: Sequence[int],
                   tensor_stride: Sequence[int], custom: Optional[np.ndarray] = None) -> np.ndarray:
    """Host offsets [K, D] of a kernel region (rmn_region_offsets)."""
    ks = np.ascontiguousarray(kernel_size, dtype=np.int32)
    dl = np.ascontiguousarray(dilation, dtype=np.int32)
    ts = np.ascontiguousarray(tensor_stride, dtype=np.int32)
    d = ks.size
    if dl.size != d or ts.size != d:
        raise RuntimeError("kernel size mismatch")
    cu = np.ascontiguousarray(custom, dtype=np.int32).reshape(-1, d) if custom is not None else np.zeros((0, d), np.int32)
    lib = capi.lib()
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
    k = lib.rmn_region_volume(region_type, d, vp(ks), int(cu.shape[0]))
    if k < 0:
        raise capi.RmnError(-k, "rmn_region_volume")
    out = np.zeros((k, d), dtype=np.int32)
    k2 = lib.rmn_region_offsets(region_type, d, vp(ks), vp(dl), vp(ts), vp(cu), int(cu.shape[0]), vp(out))
    if k2 < 0:
        raise capi.RmnError(-k2, "rmn_region_offsets")
    return out


class NeighbourTable:
    """Result of rmn_kmap_build: nbr[K, n_query] plus the CSR pointer of the pair lists."""

    def __init__(self, nbr, offset_ptr, workspace, n_query, K, n_table_rows):
        self.nbr = nbr                  # int32 [K, n_query]: table row per (offset, query) or -1
        self.offset_ptr = offset_ptr    # int64 [K + 1] device
        self.workspace = workspace
        self.n_query = n_query
        self.K = K
        self.n_table_rows = n_table_rows

    def pairs(self, background: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(offset_ptr int64 [K+1] host, a_idx int32 [P], q_idx int32 [P]); synchronises. ``background``
        picks the variant built to run beside a convolution (rmn_kmap_pairs_background): same lists."""
        ptr_host = self.offset_ptr.cpu()
        total = int(ptr_host[-1])
        dev = self.nbr.device
        a = torch.empty(total, dtype=torch.int32, device=dev)
        q = torch.empty(total, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            fn = capi.lib().rmn_kmap_pairs_background if background else capi.lib().rmn_kmap_pairs
            capi.check(fn(_ptr(self.nbr), self.n_query, self.K, _ptr(self.offset_ptr), _ptr(self.workspace), _ptr(a),
                          _ptr(q), total, _stream()), "rmn_kmap_pairs")
        return ptr_host, a, q


_OFFSET_CACHE: dict = {}


def _device_offsets(off: np.ndarray, dev: torch.device) -> torch.Tensor:
    """Device copy of a region's offsets; cached so that repeated kernel-map builds with the same
    region do not pay a synchronous host-to-device copy each time."""
    key = (dev.index, off.shape, off.tobytes())
    hit = _OFFSET_CACHE.get(key)
    if hit is None:
        if len(_OFFSET_CACHE) > 256:
            _OFFSET_CACHE.clear()
        hit = torch.from_numpy(off.reshape(-1).copy()).to(dev)
        _OFFSET_CACHE[key] = hit
    return hit


def offsets_point_symmetric(offsets: np.ndarray) -> bool:
    """True when K is odd, offsets[K-1-k] == -offsets[k] and the centre offset is zero."""
    off = np.asarray(offsets)
    k = off.shape[0]
    return k % 2 == 1 and bool((off[::-1] == -off).all()) and not off[k // 2].any()


def kmap_build(table: CoordinateTable, query: torch.Tensor, offsets: np.ndarray,
               self_map: bool = False) -> NeighbourTable:
    """Probe ``table`` at ``query[q] + offsets[k]`` for all (k, q) (rmn_kmap_build).

    ``self_map=True`` promises that ``query`` is ``table.coords`` itself; with point-symmetric
    offsets the half-probe builder (rmn_kmap_build_self) is used."""
    _check_coords(query, "query coordinates")
    if query.size(1) != table.width:
        raise RuntimeError("kernel size mismatch")
    off = np.ascontiguousarray(offsets, dtype=np.int32)
    K = int(off.shape[0])
    nq = int(query.size(0))
    dev = query.device
    lib = capi.lib()
    with torch.cuda.device(dev):
        d_off = _device_offsets(off, dev)
        nbr = torch.empty((K, nq), dtype=torch.int32, device=dev)
        ptr = torch.empty(K + 1, dtype=torch.int64, device=dev)
        wbytes = lib.rmn_kmap_workspace_bytes(nq, K)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        fn, name = lib.rmn_kmap_build, "rmn_kmap_build"
        if self_map and nq == table.n_unique and offsets_point_symmetric(off):
            fn, name = lib.rmn_kmap_build_self, "rmn_kmap_build_self"
        capi.check(fn(_ptr(table.buffer), _ptr(query), nq, table.width, _ptr(d_off), K, _ptr(nbr), _ptr(ptr),
                      _ptr(ws), wbytes, _stream()), name)
    return NeighbourTable(nbr, ptr, ws, nq, K, table.n_unique)


def kmap_transpose(nbr: torch.Tensor, n_a: int) -> torch.Tensor:
    """nbr_t[k, a] = q where nbr[k, q] == a (rmn_kmap_transpose)."""
    K, nq = int(nbr.size(0)), int(nbr.size(1))
    out = torch.empty((K, n_a), dtype=torch.int32, device=nbr.device)
    with torch.cuda.device(nbr.device):
        capi.check(capi.lib().rmn_kmap_transpose(_ptr(nbr), nq, K, int(n_a), _ptr(out), _stream()),
                   "rmn_kmap_transpose")
    return out


def _check_conv(feats: torch.Tensor, weights: torch.Tensor, what: str) -> None:
    _require_cuda(feats, what)
    _require_cuda(weights, "weights")
    if feats.dim() != 2 or weights.dim() != 3:
        raise RuntimeError("features must be [N, C] and weights [K, C_in, C_out]")
    if feats.dtype != weights.dtype:
        raise RuntimeError(f"expected {what} and weights to have the same dtype, got {feats.dtype} and {weights.dtype}")


def conv_plan_build(nbr: torch.Tensor, offsets: np.ndarray) -> Optional[torch.Tensor]:
    """Convolution plan of neighbour table ``nbr`` [K, n_dst] (rmn_conv_plan_build): an internal row order in
    which (128-row tile, offset) pairs without neighbours are skipped by the tensor-core kernels. ``offsets``
    [K, D] is the host array of the region the table was built with. Returns the plan buffer (uint8), or
    None when the table has no rows or more offsets than a plan covers."""
    _require_cuda(nbr, "neighbour table")
    K, n_dst = int(nbr.size(0)), int(nbr.size(1))
    lib = capi.lib()
    pbytes = lib.rmn_conv_plan_bytes(n_dst, K)
    if n_dst == 0 or pbytes == 0:
        return None
    off = np.ascontiguousarray(offsets, dtype=np.int32).reshape(K, -1)
    plan = torch.empty(pbytes, dtype=torch.uint8, device=nbr.device)
    wbytes = lib.rmn_conv_plan_workspace_bytes(n_dst, K)
    ws = torch.empty(wbytes, dtype=torch.uint8, device=nbr.device)
    with torch.cuda.device(nbr.device):
        capi.check(lib.rmn_conv_plan_build(_ptr(nbr), n_dst, K, off.ctypes.data, int(off.shape[1]), _ptr(plan), pbytes,
                                           _ptr(ws), wbytes, _stream()), "rmn_conv_plan_build")
    return plan


def conv_forward(feats: torch.Tensor, weights: torch.Tensor, nbr: torch.Tensor,
                 scale: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
                 relu: bool = False, plan: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[j] = act((sum_k feats[nbr[k, j]] @ weights[k]) * scale + shift) (rmn_conv_forward_planned);
    ``scale`` / ``shift`` are per-output-channel vectors (any float dtype, used as fp32) or None;
    ``plan`` is the table's convolution plan (``conv_plan_build``) or None."""
    _check_conv(feats, weights, "features")
    feats, weights = feats.contiguous(), weights.contiguous()
    K, c_in, c_out = (int(s) for s in weights.shape)
    if feats.size(1) != c_in or nbr.size(0) != K:
        raise RuntimeError("Input channel count does not match convolution")
    n_dst = int(nbr.size(1))
    out = torch.empty((n_dst, c_out), dtype=feats.dtype, device=feats.device)

    def vec(v):
        if v is None:
            return None
        v = v.detach().reshape(-1).to(device=feats.device, dtype=torch.float32).contiguous()
        if v.numel() != c_out:
            raise RuntimeError("epilogue vectors must have one entry per output channel")
        return v

    sc, sh = vec(scale), vec(shift)
    with torch.cuda.device(feats.device):
        capi.check(capi.lib().rmn_conv_forward_planned(_ptr(feats), int(feats.size(0)), c_in, _ptr(weights), K, c_out,
                                                       _ptr(nbr), _ptr(plan), n_dst, _ptr(out), _dtype_code(feats),
                                                       _ptr(sc), _ptr(sh), int(bool(relu)), _stream()),
                   "rmn_conv_forward_planned")
    return out


def conv_backward_input(grad_out: torch.Tensor, weights: torch.Tensor, nbr_t: torch.Tensor,
                        plan: Optional[torch.Tensor] = None) -> torch.Tensor:
    """grad_feats[i] = sum_k grad_out[nbr_t[k, i]] @ weights[k]^T (rmn_conv_backward_input_planned);
    ``plan`` is the convolution plan of ``nbr_t`` or None."""
    _check_conv(grad_out, weights, "grad_out")
    grad_out, weights = grad_out.contiguous(), weights.contiguous()
    K, c_in, c_out = (int(s) for s in weights.shape)
    n_src = int(nbr_t.size(1))
    out = torch.empty((n_src, c_in), dtype=grad_out.dtype, device=grad_out.device)
    with torch.cuda.device(grad_out.device):
        capi.check(capi.lib().rmn_conv_backward_input_planned(_ptr(grad_out), int(grad_out.size(0)), c_out,
                                                              _ptr(weights), K, c_in, _ptr(nbr_t), _ptr(plan), n_src,
                                                              _ptr(out), _dtype_code(grad_out), _stream()),
                   "rmn_conv_backward_input_planned")
    return out


def conv_backward_weight(feats: torch.Tensor, grad_out: torch.Tensor, nbr: torch.Tensor) -> torch.Tensor:
    """grad_weights[k] = sum_j feats[nbr[k, j]]^T @ grad_out[j]; fp32 [K, C_in, C_out]."""
    _require_cuda(feats, "features")
    feats, grad_out = feats.contiguous(), grad_out.contiguous()
    if feats.dtype != grad_out.dtype:
        raise RuntimeError("features and grad_out must have the same dtype")
    K, n_dst = int(nbr.size(0)), int(nbr.size(1))
    c_in, c_out = int(feats.size(1)), int(grad_out.size(1))
    lib = capi.lib()
    code = _dtype_code(feats)
    dw = torch.empty((K, c_in, c_out), dtype=torch.float32, device=feats.device)
    with torch.cuda.device(feats.device):
        wbytes = lib.rmn_conv_backward_weight_workspace_bytes(n_dst, K, c_in, c_out, code)
        ws = torch.empty(max(wbytes, 16), dtype=torch.uint8, device=feats.device)
        capi.check(lib.rmn_conv_backward_weight(_ptr(feats), int(feats.size(0)), c_in, _ptr(grad_out), n_dst, c_out,
                                                _ptr(nbr), K, _ptr(dw), code, _ptr(ws), wbytes, _stream()),
                   "rmn_conv_backward_weight")
    return dw


POOL_SUM, POOL_AVG, POOL_MAX = 0, 1, 2


def pool_forward(feats: torch.Tensor, nbr: torch.Tensor, mode: int, want_aux: bool = True):
    """Local pooling over a neighbour table (rmn_pool_forward): returns (out [N_out, C], aux).

    ``aux`` is what the backward pass needs: None for sum, int32 counts [N_out] for average,
    int32 argmax rows [N_out, C] for maximum (None when ``want_aux`` is false)."""
    _require_cuda(feats, "features")
    if feats.dim() != 2 or nbr.dim() != 2:
        raise RuntimeError("features must be [N, C] and the neighbour table [K, N_out]")
    if not feats.is_floating_point():
        raise RuntimeError("Sparse pooling requires floating-point features")
    feats = feats.contiguous()
    K, n_dst = int(nbr.size(0)), int(nbr.size(1))
    c = int(feats.size(1))
    out = torch.empty((n_dst, c), dtype=feats.dtype, device=feats.device)
    aux = None
    if want_aux and mode == POOL_AVG:
        aux = torch.empty(n_dst, dtype=torch.int32, device=feats.device)
    elif want_aux and mode == POOL_MAX:
        aux = torch.empty((n_dst, c), dtype=torch.int32, device=feats.device)
    with torch.cuda.device(feats.device):
        capi.check(capi.lib().rmn_pool_forward(_ptr(feats), int(feats.size(0)), c, _ptr(nbr), K, n_dst, int(mode),
                                               _ptr(out), _ptr(aux), _dtype_code(feats), _stream()),
                   "rmn_pool_forward")
    return out, aux


def pool_backward(grad_out: torch.Tensor, nbr_in: torch.Tensor, mode: int, aux: Optional[torch.Tensor]) -> torch.Tensor:
    """Gradient of pool_forward w.r.t. the input features (rmn_pool_backward); ``nbr_in`` [K, N_in] is the
    inverse neighbour table."""
    _require_cuda(grad_out, "output gradient")
    grad_out = grad_out.contiguous()
    K, n_src = int(nbr_in.size(0)), int(nbr_in.size(1))
    c = int(grad_out.size(1))
    grad_in = torch.empty((n_src, c), dtype=grad_out.dtype, device=grad_out.device)
    with torch.cuda.device(grad_out.device):
        capi.check(capi.lib().rmn_pool_backward(_ptr(grad_out), int(grad_out.size(0)), c, _ptr(nbr_in), K, n_src,
                                                int(mode), _ptr(aux), _ptr(grad_in), _dtype_code(grad_out),
                                                _stream()), "rmn_pool_backward")
    return grad_in


def channel_stats(x: torch.Tensor) -> torch.Tensor:
    """float64 [2, C]: per-channel sum and sum of squares of ``x`` [N, C] (rmn_channel_stats)."""
    _require_cuda(x, "features")
    x = x.contiguous()
    n, c = int(x.size(0)), int(x.size(1))
    lib = capi.lib()
    stats = torch.empty((2, c), dtype=torch.float64, device=x.device)
    wbytes = lib.rmn_channel_stats_workspace_bytes(c)
    ws = torch.empty(wbytes, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        capi.check(lib.rmn_channel_stats(_ptr(x), n, c, _dtype_code(x), _ptr(stats), _ptr(ws), wbytes, _stream()),
                   "rmn_channel_stats")
    return stats


def conv_forward_stats(feats: torch.Tensor, weights: torch.Tensor, nbr: torch.Tensor,
                       scale: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
                       relu: bool = False, plan: Optional[torch.Tensor] = None):
    """conv_forward that also returns float64 [2, C_out] channel sums / sums of squares of the output it
    stores, accumulated in the tensor-core kernel's epilogue (rmn_conv_forward_stats)."""
    _check_conv(feats, weights, "features")
    feats, weights = feats.contiguous(), weights.contiguous()
    K, c_in, c_out = (int(s) for s in weights.shape)
    if feats.size(1) != c_in or nbr.size(0) != K:
        raise RuntimeError("Input channel count does not match convolution")
    n_dst = int(nbr.size(1))
    out = torch.empty((n_dst, c_out), dtype=feats.dtype, device=feats.device)
    stats = torch.empty((2, c_out), dtype=torch.float64, device=feats.device)

    def vec(v):
        return None if v is None else v.detach().reshape(-1).to(device=feats.device, dtype=torch.float32).contiguous()

    sc, sh = vec(scale), vec(shift)
    lib = capi.lib()
    wbytes = lib.rmn_channel_stats_workspace_bytes(c_out)
    ws = torch.empty(wbytes, dtype=torch.uint8, device=feats.device)
    with torch.cuda.device(feats.device):
        capi.check(lib.rmn_conv_forward_stats_planned(_ptr(feats), int(feats.size(0)), c_in, _ptr(weights), K, c_out,
                                                      _ptr(nbr), _ptr(plan), n_dst, _ptr(out), _dtype_code(feats),
                                                      _ptr(sc), _ptr(sh), int(bool(relu)), _ptr(stats), _ptr(ws),
                                                      wbytes, _stream()),
                   "rmn_conv_forward_stats_planned")
    return out, stats


def affine_act(x: torch.Tensor, scale: Optional[torch.Tensor], shift: Optional[torch.Tensor], relu: bool = False,
               inplace: bool = False) -> torch.Tensor:
    """act(x * scale + shift) per channel in one pass (rmn_affine_act)."""
    _require_cuda(x, "features")
    x = x.contiguous()
    out = x if inplace else torch.empty_like(x)

    def vec(v):
        return None if v is None else v.detach().reshape(-1).to(device=x.device, dtype=torch.float32).contiguous()

    sc, sh = vec(scale), vec(shift)
    with torch.cuda.device(x.device):
        capi.check(capi.lib().rmn_affine_act(_ptr(x), int(x.size(0)), int(x.size(1)), _ptr(sc), _ptr(sh),
                                             int(bool(relu)), _ptr(out), _dtype_code(x), _stream()), "rmn_affine_act")
    return out


def coords_expand(coords: torch.Tensor, offsets: np.ndarray) -> torch.Tensor:
    """[N * K, W] coordinates ``coords[row] + offsets[k]`` (rmn_coords_expand), row-major over (row, k)."""
    _check_coords(coords)
    off = np.ascontiguousarray(offsets, dtype=np.int32)
    K = int(off.shape[0])
    n, w = int(coords.size(0)), int(coords.size(1))
    if off.ndim != 2 or off.shape[1] != w - 1:
        raise RuntimeError("kernel size mismatch")
    out = torch.empty((n * K, w), dtype=torch.int32, device=coords.device)
    with torch.cuda.device(coords.device):
        d_off = _device_offsets(off, coords.device)
        capi.check(capi.lib().rmn_coords_expand(_ptr(coords), n, w, _ptr(d_off), K, _ptr(out), _stream()),
                   "rmn_coords_expand")
    return out


def _check_field(field: torch.Tensor) -> None:
    _require_cuda(field, "coordinates")
    if field.dim() != 2 or field.dtype != torch.float32 or not field.is_contiguous():
        raise RuntimeError("field coordinates must be a contiguous 2D float32 tensor")
    if not 2 <= field.size(1) <= capi.MAX_W:
        raise RuntimeError("Coordinates must contain a batch column and spatial columns")


def field_quantize(field: torch.Tensor, tensor_stride: Sequence[int]) -> torch.Tensor:
    """int32 voxel coordinates of continuous ``field`` rows at ``tensor_stride`` (rmn_field_quantize)."""
    _check_field(field)
    st = np.ascontiguousarray(tensor_stride, dtype=np.int32)
    if st.size != field.size(1) - 1 or (st <= 0).any():
        raise RuntimeError("Invalid stride")
    out = torch.empty(field.shape, dtype=torch.int32, device=field.device)
    with torch.cuda.device(field.device):
        capi.check(capi.lib().rmn_field_quantize(_ptr(field), int(field.size(0)), int(field.size(1)),
                                                 st.ctypes.data_as(ctypes.c_void_p), _ptr(out), _stream()),
                   "rmn_field_quantize")
    return out


def coords_discretize(coords: torch.Tensor, quantization_size: Optional[float] = None) -> torch.Tensor:
    """``floor(float64(coords) / quantization_size)`` as int32 on every column (rmn_coords_discretize)."""
    _require_cuda(coords, "coordinates")
    codes = {torch.float32: 0, torch.float64: 1, torch.int32: 2}
    if coords.dtype not in codes:
        coords = coords.to(torch.float64)
    coords = coords.contiguous()
    out = torch.empty(coords.shape, dtype=torch.int32, device=coords.device)
    q = 0.0 if quantization_size is None else float(quantization_size)
    with torch.cuda.device(coords.device):
        capi.check(capi.lib().rmn_coords_discretize(_ptr(coords), codes[coords.dtype], coords.numel(), q, _ptr(out),
                                                    _stream()), "rmn_coords_discretize")
    return out


def field_splat(field: torch.Tensor, feats: torch.Tensor):
    """Corner-major lattice coordinates [N * 2^D, W] and weighted features [N * 2^D, C] (rmn_field_splat)."""
    _check_field(field)
    _require_cuda(feats, "features")
    if feats.dim() != 2 or feats.size(0) != field.size(0):
        raise RuntimeError("Features and coordinates must have same number of rows")
    feats = feats.contiguous()
    n, w, c = int(field.size(0)), int(field.size(1)), int(feats.size(1))
    rows = n << (w - 1)
    out_c = torch.empty((rows, w), dtype=torch.int32, device=field.device)
    out_f = torch.empty((rows, c), dtype=feats.dtype, device=field.device)
    with torch.cuda.device(field.device):
        capi.check(capi.lib().rmn_field_splat(_ptr(field), _ptr(feats), _dtype_code(feats), n, w, c, _ptr(out_c),
                                              _ptr(out_f), _stream()), "rmn_field_splat")
    return out_c, out_f
