"""Shared parity helpers: the convolution pipeline stated once over an abstract
backend, and the comparison rules against reference outputs.

A backend provides the five primitives of the hot path on numpy arrays:
``insert_and_map, stride_map, region_offsets, conv_kernel_map, conv_forward,
conv_backward``. ``OracleBackend`` is the CPU oracle; the GPU tests supply one
that calls the CUDA library through its C ABI.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GOLDEN_CASES = ["d3_k3_s1", "d3_k2_s2_chain", "d3_k3_s2_chain", "d4_k3_s1", "d2_k3_s1_dil2",
                "d3_k1_s1", "d3_k5_s1"]


def load_golden(name: str) -> Dict[str, np.ndarray]:
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


class OracleBackend:
    """The CPU oracle behind the backend interface."""

    def __init__(self, f64: bool = False):
        from oracle import oracle as O
        self.O = O
        self.f64 = f64

    def insert_and_map(self, coords):
        return self.O.insert_and_map(coords)

    def stride_map(self, coords, out_stride):
        return self.O.stride_map(coords, out_stride)

    def region_offsets(self, ksize, dilation, tensor_stride):
        return self.O.region_offsets(self.O.HYPER_CUBE, ksize, dilation, tensor_stride)

    def conv_kernel_map(self, in_coords, out_coords, offsets, transposed=False):
        return self.O.conv_kernel_map(in_coords, out_coords, offsets, transposed)

    def conv_forward(self, feats, weights, kmap, n_in, n_out):
        return self.O.conv_forward(feats, weights, *kmap, n_out, f64=self.f64)

    def conv_backward(self, feats, grad_out, weights, kmap, n_in, n_out):
        return self.O.conv_backward(feats, grad_out, weights, *kmap, f64=self.f64)


def run_pipeline(be, coords, feats, weights, D, kernel, stride, dilation,
                 weights2: Optional[np.ndarray] = None) -> Dict[str, np.ndarray]:
    """SparseTensor ctor -> conv [-> transposed conv] -> backward of 0.5*sum(y^2).

    Mirrors what the reference driver runs (engine/tensor/sparse_tensor.cpp:62-99,
    engine/nn/conv.cpp:104-138) so that outputs carry the same names.
    """
    res: Dict[str, np.ndarray] = {}
    mapping, inverse = be.insert_and_map(coords)
    res["mapping"], res["inverse"] = mapping, inverse
    in_coords = coords[mapping]
    F = np.ascontiguousarray(feats[mapping], np.float32)
    res["in_coords"] = in_coords
    ts_in = [1] * D
    ks, dl = [kernel] * D, [dilation] * D
    if stride > 1:
        ts_out = [stride] * D
        out_coords, _ = be.stride_map(in_coords, ts_out)
    else:
        ts_out = ts_in
        out_coords = in_coords
    res["out_coords"] = out_coords
    kmap = be.conv_kernel_map(in_coords, out_coords, be.region_offsets(ks, dl, ts_in), False)
    res["kmap_ptr"], res["kmap_in"], res["kmap_out"] = kmap
    y = be.conv_forward(F, weights, kmap, len(in_coords), len(out_coords))
    res["out_feats"] = y
    if weights2 is None:
        gF, gW = be.conv_backward(F, np.asarray(y, np.float32), weights, kmap, len(in_coords), len(out_coords))
    else:
        # transposed conv back onto the (existing) fine map: region on the OUTPUT stride
        up_coords = in_coords
        kmap2 = be.conv_kernel_map(out_coords, up_coords, be.region_offsets(ks, dl, ts_in), True)
        res["kmap2_ptr"], res["kmap2_in"], res["kmap2_out"] = kmap2
        y32 = np.ascontiguousarray(y, np.float32)
        z = be.conv_forward(y32, weights2, kmap2, len(out_coords), len(up_coords))
        res["up_coords"], res["up_feats"] = up_coords, z
        gY, gW2 = be.conv_backward(y32, np.asarray(z, np.float32), weights2, kmap2, len(out_coords), len(up_coords))
        res["grad_weights2"] = gW2
        gF, gW = be.conv_backward(F, np.asarray(gY, np.float32), weights, kmap, len(in_coords), len(out_coords))
    res["grad_weights"] = gW
    # gradient w.r.t. the raw (pre-dedup) feature rows: dropped duplicates get zero
    g_raw = np.zeros((len(coords), F.shape[1]), dtype=np.asarray(gF).dtype)
    g_raw[mapping] = gF
    res["grad_feats"] = g_raw
    return res


def row_permutation(my_coords: np.ndarray, ref_coords: np.ndarray) -> np.ndarray:
    """perm with ref_coords[perm[i]] == my_coords[i]; asserts the row SETS are equal."""
    assert my_coords.shape == ref_coords.shape, (my_coords.shape, ref_coords.shape)
    lut = {tuple(r): i for i, r in enumerate(ref_coords.tolist())}
    assert len(lut) == len(ref_coords), "reference coordinates are not unique"
    perm = np.array([lut[tuple(r)] for r in my_coords.tolist()], dtype=np.int64)
    assert len(np.unique(perm)) == len(perm)
    return perm


def sorted_pairs(ptr, a, b, k):
    s = slice(int(ptr[k]), int(ptr[k + 1]))
    p = np.stack([np.asarray(a[s], np.int64), np.asarray(b[s], np.int64)], 1)
    return p[np.lexsort((p[:, 1], p[:, 0]))] if len(p) else p


def assert_kernel_maps_equal(my, ref, in_perm=None, out_perm=None):
    """Bit-exact comparison as per-offset sorted (in, out) pair sets; ``*_perm`` map my rows
    to reference rows where the reference's row numbering is a hash-order artefact."""
    my_ptr, my_in, my_out = my
    ref_ptr, ref_in, ref_out = ref
    assert len(my_ptr) == len(ref_ptr)
    assert (np.diff(my_ptr) == np.diff(ref_ptr)).all(), "per-offset pair counts differ"
    mi = np.asarray(my_in, np.int64) if in_perm is None else in_perm[np.asarray(my_in, np.int64)]
    mo = np.asarray(my_out, np.int64) if out_perm is None else out_perm[np.asarray(my_out, np.int64)]
    for k in range(len(my_ptr) - 1):
        a, b = sorted_pairs(my_ptr, mi, mo, k), sorted_pairs(ref_ptr, ref_in, ref_out, k)
        assert a.shape == b.shape and (a == b).all(), f"offset {k}: pair sets differ"


def rel_max(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)) if a.size else 0.0


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)) if a.size else 0.0


def check_against_reference(res, gold, tol=1e-4, metric=rel_max):
    """Compare a pipeline result with the reference outputs stored in a golden fixture."""
    g = {k[4:]: v for k, v in gold.items() if k.startswith("ref_")}
    assert (res["mapping"] == g["mapping"]).all()
    assert (res["inverse"] == g["inverse"]).all()
    assert (res["in_coords"] == g["in_coords"]).all()
    out_perm = row_permutation(res["out_coords"], g["out_coords"])
    assert_kernel_maps_equal((res["kmap_ptr"], res["kmap_in"], res["kmap_out"]),
                             (g["kmap_ptr"], g["kmap_in"], g["kmap_out"]), None, out_perm)
    assert metric(res["out_feats"], g["out_feats"][out_perm]) <= tol
    if "up_feats" in g:
        up_perm = row_permutation(res["up_coords"], g["up_coords"])
        assert_kernel_maps_equal((res["kmap2_ptr"], res["kmap2_in"], res["kmap2_out"]),
                                 (g["kmap2_ptr"], g["kmap2_in"], g["kmap2_out"]), out_perm, up_perm)
        assert metric(res["up_feats"], g["up_feats"][up_perm]) <= tol
        assert metric(res["grad_weights2"], g["grad_weights2"]) <= tol
    assert metric(res["grad_weights"], g["grad_weights"]) <= tol
    assert metric(res["grad_feats"], g["grad_feats"]) <= tol


# ---------------------------------------------------------------------------------------------
# local pooling fixtures (reference engine/nn/pooling.cpp, generated by tests/golden/make_golden.py)
# ---------------------------------------------------------------------------------------------
POOL_GOLDEN_CASES = ["pool_d3_sum_k2_s2", "pool_d3_avg_k2_s2", "pool_d3_max_k2_s2", "pool_d3_max_k3_s1",
                     "pool_d3_avg_k3_s2", "pool_d2_sum_k3_s1"]


def oracle_pool_case(gold: Dict[str, np.ndarray]):
    """The oracle's pooled output for a pooling fixture: (out_coords, out_feats, grad w.r.t. the raw features)
    for the loss 0.5 * sum(out^2)."""
    from oracle import oracle as O

    D, kernel, stride, mode = (int(v) for v in gold["spec"])
    coords, feats = gold["in_coords_raw"], gold["in_feats_raw"]
    mapping, _ = O.insert_and_map(coords)
    in_coords, in_feats = coords[mapping], feats[mapping]
    if stride > 1:
        out_coords, _ = O.stride_map(in_coords, [stride] * D)
    else:
        out_coords = in_coords
    offsets = O.region_offsets(O.HYPER_CUBE, [kernel] * D, [1] * D, [1] * D)
    _, in_idx, out_idx = O.conv_kernel_map(in_coords, out_coords, offsets)
    out = O.pool_forward(in_feats, in_idx, out_idx, len(out_coords), mode - 1)
    g_unique = O.pool_backward(in_feats, out, in_idx, out_idx, mode - 1)
    g_raw = np.zeros(feats.shape, np.float64)
    g_raw[mapping] = g_unique
    return out_coords, out, g_raw


def check_pool_against_reference(out_coords, out_feats, grad_raw, gold, tol: float) -> None:
    """Pooled rows are matched to the reference's by coordinate (strided maps number rows differently)."""
    ref_c, ref_f, ref_g = gold["ref_pool_coords"], gold["ref_pool_feats"], gold["ref_pool_grad_feats"]
    assert out_coords.shape == ref_c.shape
    order = np.lexsort(np.asarray(out_coords).T[::-1])
    ref_order = np.lexsort(ref_c.T[::-1])
    assert np.array_equal(np.asarray(out_coords)[order], ref_c[ref_order])
    scale = max(float(np.abs(ref_f).max()), 1e-30)
    err = float(np.abs(np.asarray(out_feats, np.float64)[order] - ref_f[ref_order]).max()) / scale
    assert err <= tol, f"pooled features differ: {err}"
    gscale = max(float(np.abs(ref_g).max()), 1e-30)
    gerr = float(np.abs(np.asarray(grad_raw, np.float64) - ref_g).max()) / gscale
    assert gerr <= tol, f"pooling gradient differs: {gerr}"


UNPOOL_GOLDEN_CASES = ["unpool_d3_k3_s2", "unpool_d2_k2_s1"]


def oracle_unpool_case(gold: Dict[str, np.ndarray]):
    """Oracle result of a (strided) convolution followed by the pooling-transpose layer (sum) with the same
    kernel size and stride (reference engine/nn/pooling.cpp:49-70, 197-229; coordinate generation
    engine/grid/lattice_cpu.hpp:499-534): (out_coords, out_feats, grad w.r.t. the raw features) for the loss
    0.5 * sum(out^2)."""
    from oracle import oracle as O

    D, kernel, stride, _ = (int(v) for v in gold["spec"])
    coords, feats, weights = gold["in_coords_raw"], gold["in_feats_raw"], gold["weights"]
    mapping, _ = O.insert_and_map(coords)
    fine, f_in = coords[mapping], feats[mapping]
    coarse = O.stride_map(fine, [stride] * D)[0] if stride > 1 else fine
    kc = O.conv_kernel_map(fine, coarse, O.region_offsets(O.HYPER_CUBE, [kernel] * D, [1] * D, [1] * D))
    y = O.conv_forward(f_in, weights, *kc, len(coarse), f64=True)
    # un-pooling region on the output (finer) tensor stride: out = in + off
    off = O.region_offsets(O.HYPER_CUBE, [kernel] * D, [1] * D, [1] * D)
    if stride > 1:
        expanded = (coarse[:, None, :].astype(np.int64)
                    + np.concatenate([np.zeros((len(off), 1), np.int64), off.astype(np.int64)], 1)[None]).reshape(
                        -1, coords.shape[1]).astype(np.int32)
        generated = expanded[O.insert_and_map(expanded)[0]]
    else:
        generated = coarse  # a map of the output stride exists already and is reused
    ku = O.conv_kernel_map(coarse, generated, off, transposed=True)
    out = O.pool_forward(y, ku[1], ku[2], len(generated), O.POOL_SUM)
    g_y = O.pool_backward(y, out, ku[1], ku[2], O.POOL_SUM)
    g_in, _ = O.conv_backward(f_in, g_y.astype(np.float32), weights, *kc, f64=True)
    g_raw = np.zeros(feats.shape, np.float64)
    g_raw[mapping] = g_in
    return generated, out, g_raw
