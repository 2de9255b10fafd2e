"""numpy front end of the CPU oracle (``rmn_oracle.c``).

TEST INFRASTRUCTURE ONLY: the parity checker for the CUDA library. Only the
test-suite, the smoke check and the benchmark's ``cpu_baseline`` /
``--impl reference`` legs may import this module; the product package never
does.

The C file is compiled with gcc on first use into ``oracle/_build/`` (built
artefacts are not tracked). Every function returns plain numpy arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "rmn_oracle.c")
_LIB_DIR = os.path.join(_HERE, "_build")
_LIB = os.path.join(_LIB_DIR, "librmn_oracle.so")

HYPER_CUBE, HYPER_CROSS, CUSTOM = 0, 1, 2

_lib = None


def build(force: bool = False) -> str:
    """Compile the C restatement (gcc -O2) if the shared object is stale."""
    os.makedirs(_LIB_DIR, exist_ok=True)
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        tmp = _LIB + f".tmp{os.getpid()}"
        subprocess.check_call(
            ["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-o", tmp, _SRC, "-lm"]
        )
        os.replace(tmp, _LIB)
    return _LIB


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_murmur3_row.restype = ctypes.c_uint32
        _lib.orc_insert_and_map.restype = ctypes.c_int64
        _lib.orc_kernel_map.restype = ctypes.c_int64
        _lib.orc_region_offsets.restype = ctypes.c_int
        _lib.orc_region_volume.restype = ctypes.c_int
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def murmur3_row(row: Sequence[int]) -> int:
    r = _i32(row)
    return int(_load().orc_murmur3_row(_p(r), ctypes.c_int(r.size)))


def insert_and_map(coords: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Dedup rows of ``coords`` [N, W]; returns (mapping, inverse), both int64.

    ``coords[mapping]`` are the unique rows in first-occurrence order and
    ``coords[mapping][inverse] == coords``.
    """
    c = _i32(coords)
    n, w = c.shape if c.ndim == 2 else (0, 1)
    mapping = np.empty(max(n, 1), dtype=np.int64)
    inverse = np.empty(max(n, 1), dtype=np.int64)
    nu = _load().orc_insert_and_map(_p(c), ctypes.c_int64(n), ctypes.c_int(w), _p(mapping), _p(inverse))
    if nu < 0:
        raise MemoryError("oracle allocation failed")
    return mapping[:nu].copy(), inverse[:n].copy()


def stride_coords(coords: np.ndarray, out_tensor_stride: Sequence[int]) -> np.ndarray:
    """Floor-align the spatial columns to ``out_tensor_stride`` (batch column kept)."""
    c = _i32(coords)
    s = _i32(out_tensor_stride)
    assert c.shape[1] - 1 == s.size
    dst = np.empty_like(c)
    _load().orc_stride_coords(_p(c), ctypes.c_int64(c.shape[0]), ctypes.c_int(c.shape[1]), _p(s), _p(dst))
    return dst


def stride_map(coords: np.ndarray, out_tensor_stride: Sequence[int]):
    """Strided-down coordinate map: returns (coarse_coords, in_to_coarse).

    Coarse rows are numbered by first occurrence over the input rows in order.
    """
    aligned = stride_coords(coords, out_tensor_stride)
    mapping, inverse = insert_and_map(aligned)
    return aligned[mapping], inverse


def region_offsets(region_type: int, kernel_size: Sequence[int], dilation: Sequence[int],
                   tensor_stride: Sequence[int], custom: Optional[np.ndarray] = None) -> np.ndarray:
    """Offsets [K, D] of a kernel region, in the reference's enumeration order."""
    ks, dl, ts = _i32(kernel_size), _i32(dilation), _i32(tensor_stride)
    d = ks.size
    cu = _i32(custom).reshape(-1, d) if custom is not None else np.zeros((0, d), np.int32)
    lib = _load()
    k = lib.orc_region_volume(ctypes.c_int(region_type), ctypes.c_int(d), _p(ks), ctypes.c_int(cu.shape[0]))
    out = np.zeros((k, d), dtype=np.int32)
    lib.orc_region_offsets(ctypes.c_int(region_type), ctypes.c_int(d), _p(ks), _p(dl), _p(ts), _p(cu),
                           ctypes.c_int(cu.shape[0]), _p(out))
    return out


def kernel_map(coords_a: np.ndarray, coords_q: np.ndarray, offsets: np.ndarray):
    """Pairs (a_row, q_row) per offset with coords_a[a] == coords_q[q] + offsets[k].

    Returns (offset_ptr int64 [K+1], a_idx int32 [P], q_idx int32 [P]); pairs of
    one offset are sorted by q_row.
    """
    a, q, off = _i32(coords_a), _i32(coords_q), _i32(offsets)
    k = off.shape[0]
    nq = q.shape[0]
    a_idx = np.empty((k, max(nq, 1)), dtype=np.int32)
    q_idx = np.empty((k, max(nq, 1)), dtype=np.int32)
    counts = np.zeros(k, dtype=np.int64)
    w = a.shape[1] if a.ndim == 2 else q.shape[1]
    total = _load().orc_kernel_map(_p(a), ctypes.c_int64(a.shape[0]), _p(q), ctypes.c_int64(nq),
                                   ctypes.c_int(w), _p(off), ctypes.c_int(k), _p(a_idx), _p(q_idx), _p(counts))
    if total < 0:
        raise MemoryError("oracle allocation failed")
    ptr = np.zeros(k + 1, dtype=np.int64)
    np.cumsum(counts, out=ptr[1:])
    a_flat = np.concatenate([a_idx[i, :counts[i]] for i in range(k)]) if k else np.zeros(0, np.int32)
    q_flat = np.concatenate([q_idx[i, :counts[i]] for i in range(k)]) if k else np.zeros(0, np.int32)
    return ptr, a_flat.astype(np.int32), q_flat.astype(np.int32)


def conv_kernel_map(in_coords: np.ndarray, out_coords: np.ndarray, offsets: np.ndarray,
                    transposed: bool = False):
    """Kernel map of a (transposed) convolution as (offset_ptr, in_idx, out_idx).

    Forward: out + off_k == in, offsets on the input tensor stride.
    Transposed: in + off_k == out, offsets on the output tensor stride; the
    output map is the one queried and the result is swapped, as the reference
    does.
    """
    if not transposed:
        ptr, a, q = kernel_map(in_coords, out_coords, offsets)
        return ptr, a, q
    ptr, a, q = kernel_map(out_coords, in_coords, offsets)
    return ptr, q, a


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def conv_forward(feats, weights, offset_ptr, in_idx, out_idx, n_out: int, f64: bool = False) -> np.ndarray:
    f, w = _f32(feats), _f32(weights)
    k, cin, cout = w.shape
    ptr = np.ascontiguousarray(offset_ptr, dtype=np.int64)
    ii, oi = _i32(in_idx), _i32(out_idx)
    out = np.zeros((n_out, cout), dtype=np.float64 if f64 else np.float32)
    fn = _load().orc_conv_fwd_f64 if f64 else _load().orc_conv_fwd_f32
    fn(_p(f), ctypes.c_int(cin), _p(out), ctypes.c_int(cout), ctypes.c_int64(f.shape[0]),
       ctypes.c_int64(n_out), _p(w), ctypes.c_int(k), _p(ptr), _p(ii), _p(oi))
    return out


def conv_backward(feats, grad_out, weights, offset_ptr, in_idx, out_idx, f64: bool = False):
    """Returns (grad_input [N_in, C_in], grad_weights [K, C_in, C_out])."""
    f, g, w = _f32(feats), _f32(grad_out), _f32(weights)
    k, cin, cout = w.shape
    ptr = np.ascontiguousarray(offset_ptr, dtype=np.int64)
    ii, oi = _i32(in_idx), _i32(out_idx)
    dt = np.float64 if f64 else np.float32
    gi = np.zeros((f.shape[0], cin), dtype=dt)
    gw = np.zeros((k, cin, cout), dtype=dt)
    fn = _load().orc_conv_bwd_f64 if f64 else _load().orc_conv_bwd_f32
    fn(_p(f), _p(gi), ctypes.c_int(cin), _p(g), ctypes.c_int(cout), ctypes.c_int64(f.shape[0]),
       ctypes.c_int64(g.shape[0]), _p(w), _p(gw), ctypes.c_int(k), _p(ptr), _p(ii), _p(oi))
    return gi, gw


# ---------------------------------------------------------------------------------------------
# Local pooling (reference engine/nn/pooling.cpp:80-144): every output row reduces the input rows
# its kernel-map pairs name, over all offsets; an output row without pairs is zero. Average divides
# by the number of rows present (values.mean(0)), not by the kernel volume.
# ---------------------------------------------------------------------------------------------
POOL_SUM, POOL_AVG, POOL_MAX = 0, 1, 2


def pool_forward(feats, in_idx, out_idx, n_out: int, mode: int) -> np.ndarray:
    f = np.asarray(feats, dtype=np.float64)
    ii, oi = _i32(in_idx).astype(np.int64), _i32(out_idx).astype(np.int64)
    c = f.shape[1]
    if mode == POOL_MAX:
        out = np.full((n_out, c), -np.inf)
        np.maximum.at(out, oi, f[ii])
        out[np.isneginf(out)] = 0.0  # rows without any pair
        return out
    out = np.zeros((n_out, c))
    np.add.at(out, oi, f[ii])
    if mode == POOL_AVG:
        cnt = np.bincount(oi, minlength=n_out).astype(np.float64)
        out /= np.maximum(cnt, 1.0)[:, None]
    return out


def pool_backward(feats, grad_out, in_idx, out_idx, mode: int) -> np.ndarray:
    """Gradient w.r.t. the input features (what torch autograd yields through the reference's
    index_select / sum / mean / amax chain; amax ties are assumed absent)."""
    f = np.asarray(feats, dtype=np.float64)
    g = np.asarray(grad_out, dtype=np.float64)
    ii, oi = _i32(in_idx).astype(np.int64), _i32(out_idx).astype(np.int64)
    n_out = g.shape[0]
    gi = np.zeros_like(f)
    if mode == POOL_SUM:
        np.add.at(gi, ii, g[oi])
    elif mode == POOL_AVG:
        cnt = np.maximum(np.bincount(oi, minlength=n_out).astype(np.float64), 1.0)
        np.add.at(gi, ii, g[oi] / cnt[oi][:, None])
    else:
        mx = pool_forward(f, in_idx, out_idx, n_out, POOL_MAX)
        np.add.at(gi, ii, g[oi] * (f[ii] == mx[oi]))
    return gi


# --- input step: field quantisation, sparse_quantize, splat (numpy restatements) ---------------------------
def field_quantize(field: np.ndarray, tensor_stride: Sequence[int]) -> np.ndarray:
    """int32 voxel coordinates of float32 field rows, computed in float32: batch column lroundf, spatial
    column j ``stride_j * (int)floor(v / stride_j)`` (engine/grid/lattice_cpu.hpp:944-984)."""
    f = np.ascontiguousarray(field, dtype=np.float32)
    out = np.empty(f.shape, np.int32)
    b = f[:, 0]
    out[:, 0] = (np.sign(b) * np.floor(np.abs(b) + np.float32(0.5))).astype(np.int32)  # half away from zero
    for j, s in enumerate(tensor_stride):
        col = f[:, j + 1]
        if int(s) == 1:
            out[:, j + 1] = np.floor(col).astype(np.int32)
        else:
            out[:, j + 1] = np.int32(s) * np.floor(col / np.float32(s)).astype(np.int32)
    return out


def quantize_features(feats: np.ndarray, mapping: np.ndarray, inverse: np.ndarray, mode: int) -> np.ndarray:
    """engine/tensor/field.cpp:109-140 (same rule as engine/tensor/sparse_tensor.cpp:447-481); mode 0 first row,
    1 average, 2 sum, 3 maximum, 4 none. Sums run in float64 here."""
    f = np.asarray(feats, np.float64)
    nu = len(mapping)
    if mode == 0:
        return f[mapping]
    if mode == 4:
        return f
    if mode in (1, 2):
        acc = np.zeros((nu, f.shape[1]))
        np.add.at(acc, inverse, f)
        if mode == 2:
            return acc
        cnt = np.bincount(inverse, minlength=nu).astype(np.float64)
        return acc / np.maximum(cnt, 1)[:, None]
    if mode == 3:
        acc = np.full((nu, f.shape[1]), -np.inf)
        np.maximum.at(acc, inverse, f)
        return acc
    raise ValueError("Unknown quantization mode")


def field_sparse(field: np.ndarray, feats: np.ndarray, tensor_stride: Sequence[int], mode: int):
    """TensorField::sparse (engine/tensor/field.cpp:41-59): (voxel coords, features, field row -> voxel row)."""
    q = field_quantize(field, tensor_stride)
    mapping, inverse = insert_and_map(q)
    return q[mapping], quantize_features(feats, mapping, inverse, mode), inverse


def sparse_quantize(coords: np.ndarray, feats: Optional[np.ndarray], quantization_size: Optional[float] = None):
    """engine/helpers/discretization.cpp:78-125 without labels: float64 floor-divide on every column, first
    point per voxel. Returns (coords, features, unique_index, inverse)."""
    d = np.asarray(coords, np.float64)
    if quantization_size:
        d = d / float(quantization_size)
    d = np.floor(d).astype(np.int32)
    mapping, inverse = insert_and_map(d)
    return d[mapping], (None if feats is None else np.asarray(feats)[mapping]), mapping, inverse


def field_splat(field: np.ndarray, feats: np.ndarray):
    """TensorField::splat (engine/tensor/field.cpp:61-94): corner-major lattice points and weighted features
    (before the summing SparseTensor constructor)."""
    f = np.ascontiguousarray(field, dtype=np.float32)
    D = f.shape[1] - 1
    fl = np.floor(f)
    frac = f - fl
    base = fl.astype(np.int32)
    pts, fs = [], []
    for corner in range(1 << D):
        off = np.zeros(D + 1, np.int32)
        w = np.ones(len(f), np.float32)
        for a in range(D):
            up = (corner >> a) & 1
            off[a + 1] = up
            w = w * (frac[:, a + 1] if up else np.float32(1) - frac[:, a + 1])
        pts.append(base + off)
        fs.append(np.asarray(feats, np.float32) * w[:, None])
    return np.concatenate(pts, 0), np.concatenate(fs, 0)
