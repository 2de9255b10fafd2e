"""Generate the golden fixtures in this directory from the reference itself.

Runs the unmodified reference CPU path (``oracle/_ref/ref_driver``, built by
``make -C oracle ref`` from the reference checkout) on small seeded inputs and
stores inputs + reference outputs as ``<case>.npz``. The parity tests load the
fixtures only; they never need the reference at run time.

    python tests/golden/make_golden.py [--pool-only | --unpool-only | --field-only]
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import refrun  # noqa: E402

# name: (seed, D, n_rows, batches, lo, hi, c_in, c_out, kernel, stride, dilation, chain c2)
CASES = {
    "d3_k3_s1": (11, 3, 400, 2, -6, 6, 5, 7, 3, 1, 1, None),
    "d3_k2_s2_chain": (12, 3, 500, 2, -7, 7, 4, 6, 2, 2, 1, 3),
    "d3_k3_s2_chain": (13, 3, 500, 3, -7, 8, 3, 5, 3, 2, 1, 4),
    "d4_k3_s1": (14, 4, 300, 2, -3, 3, 3, 4, 3, 1, 1, None),
    "d2_k3_s1_dil2": (15, 2, 300, 2, -10, 10, 2, 3, 3, 1, 2, None),
    "d3_k1_s1": (16, 3, 200, 1, -4, 4, 6, 2, 1, 1, 1, None),
    "d3_k5_s1": (17, 3, 350, 1, 0, 7, 2, 2, 5, 1, 1, None),
}

# local pooling (reference engine/nn/pooling.cpp): name: (seed, D, n_rows, batches, lo, hi, channels, mode, kernel, stride)
# mode 1 sum, 2 average, 3 maximum
POOL_CASES = {
    "pool_d3_sum_k2_s2": (21, 3, 500, 2, -7, 7, 6, 1, 2, 2),
    "pool_d3_avg_k2_s2": (22, 3, 500, 2, -7, 7, 6, 2, 2, 2),
    "pool_d3_max_k2_s2": (23, 3, 500, 2, -7, 7, 6, 3, 2, 2),
    "pool_d3_max_k3_s1": (24, 3, 400, 2, -5, 5, 5, 3, 3, 1),
    "pool_d3_avg_k3_s2": (25, 3, 500, 3, -7, 8, 4, 2, 3, 2),
    "pool_d2_sum_k3_s1": (26, 2, 300, 2, -9, 9, 3, 1, 3, 1),
}

UNPOOL_CASES = {
    "unpool_d3_k3_s2": (31, 3, 500, 2, -7, 7, 4, 6, 3, 2),
    "unpool_d2_k2_s1": (32, 2, 300, 2, -12, 12, 3, 5, 2, 1),
}


# input step on continuous coordinates (reference engine/tensor/field.cpp, engine/helpers/discretization.cpp):
# name: (seed, D, n_rows, batches, extent, channels, tensor stride, quantisation mode, quantisation size)
# mode: 0 first point, 1 average, 2 sum, 3 maximum (engine/foundation/types.hpp:88-93)
FIELD_CASES = {
    "field_d3_s1_avg": (41, 3, 400, 2, 4.0, 5, [1, 1, 1], 1, 0.5),
    "field_d3_s2_sum": (42, 3, 400, 3, 6.0, 4, [2, 2, 2], 2, 0.0),
    "field_d2_s42_max": (43, 2, 300, 2, 9.0, 3, [4, 2], 3, 0.25),
    "field_d3_s123_first": (44, 3, 350, 1, 5.0, 6, [1, 2, 3], 0, 1.5),
    "field_d4_s1_avg": (45, 4, 250, 2, 2.0, 3, [1, 1, 1, 1], 1, 0.0),
}


def make_field_inputs(seed, D, n, batches, extent, channels):
    rng = np.random.default_rng(seed)
    field = np.concatenate([rng.integers(0, batches, (n, 1)).astype(np.float32),
                            rng.uniform(-extent, extent, (n, D)).astype(np.float32)], axis=1)
    field[::7, 1:] = np.round(field[::7, 1:])           # points exactly on voxel boundaries
    k = len(field[1::9])
    field[1::9] = field[2::9][:k]                        # exact duplicate points
    feats = rng.standard_normal((n, channels)).astype(np.float32)
    return field, feats


def make_inputs(seed, D, n, batches, lo, hi, c_in, c_out, kernel, stride, dilation, c2):
    rng = np.random.default_rng(seed)
    spatial = rng.integers(lo, hi + 1, size=(n, D), dtype=np.int32)
    batch = rng.integers(0, batches, size=(n, 1), dtype=np.int32)
    coords = np.concatenate([batch, spatial], axis=1)
    # force some exact duplicate rows (dedup path)
    dup = rng.integers(0, n, size=n // 10)
    coords[rng.integers(0, n, size=n // 10)] = coords[dup]
    feats = rng.standard_normal((n, c_in)).astype(np.float32)
    K = kernel ** D
    bound = 1.0 / np.sqrt(c_in * K)
    weights = rng.uniform(-bound, bound, size=(K, c_in, c_out)).astype(np.float32)
    weights2 = None
    if c2 is not None:
        bound2 = 1.0 / np.sqrt(c2 * K)
        weights2 = rng.uniform(-bound2, bound2, size=(K, c_out, c2)).astype(np.float32)
    return coords, feats, weights, weights2


def main_field() -> None:
    for name, (seed, D, n, batches, extent, channels, stride, mode, qsize) in FIELD_CASES.items():
        field, feats = make_field_inputs(seed, D, n, batches, extent, channels)
        ref = refrun.run_field(field, feats, stride, mode, qsize)
        arrays = {"field": field, "feats": feats, "stride": np.array(stride, np.int32),
                  "spec": np.array([D, mode], np.int32), "qsize": np.array([qsize], np.float64)}
        for k, v in ref.items():
            arrays["ref_" + k] = v
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(name, {k: v.shape for k, v in ref.items()}, os.path.getsize(path), "bytes")


def main() -> None:
    if "--field-only" in sys.argv:
        return main_field()
    only_pool = "--pool-only" in sys.argv or "--unpool-only" in sys.argv
    for name, spec in ({} if only_pool else CASES).items():
        coords, feats, weights, weights2 = make_inputs(*spec)
        _, D, _, _, _, _, _, _, kernel, stride, dilation, _ = spec
        ref = refrun.run(coords, feats, weights, kernel, stride, dilation, weights2=weights2, threads=1)
        ref.pop("times_ms", None)
        ref.pop("info", None)
        arrays = {"in_coords_raw": coords, "in_feats_raw": feats, "weights": weights,
                  "spec": np.array([D, kernel, stride, dilation], np.int32)}
        if weights2 is not None:
            arrays["weights2"] = weights2
        for k, v in ref.items():
            arrays["ref_" + k] = v
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(name, {k: v.shape for k, v in ref.items()}, os.path.getsize(path), "bytes")
    # pooling-transpose after a (strided) convolution with the same kernel size and stride:
    # name: (seed, D, n_rows, batches, lo, hi, c_in, c_out, kernel, stride). The reference's layer fails an
    # assertion of its own when kernel == stride > 1 (its pooling kernel map takes the stride_map shortcut,
    # engine/grid/lattice_cpu.hpp:679-710), so the fixtures use kernel != stride.
    for name, (seed, D, n, batches, lo, hi, c_in, c_out, ks, st) in UNPOOL_CASES.items():
        coords, feats, weights, _ = make_inputs(seed, D, n, batches, lo, hi, c_in, c_out, ks, st, 1, None)
        ref = refrun.run(coords, feats, weights, ks, st, 1, threads=1, pool=(1, ks, st, 1))
        arrays = {"in_coords_raw": coords, "in_feats_raw": feats, "weights": weights,
                  "spec": np.array([D, ks, st, 1], np.int32)}
        for k in ("mapping", "in_coords", "out_coords", "pool_coords", "pool_feats", "pool_grad_feats"):
            arrays["ref_" + k] = ref[k]
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(name, {k: v.shape for k, v in arrays.items() if k.startswith("ref_")}, os.path.getsize(path), "bytes")
    if "--unpool-only" in sys.argv:
        return
    if not only_pool:
        main_field()
    for name, (seed, D, n, batches, lo, hi, C, mode, kernel, stride) in POOL_CASES.items():
        coords, feats, _, _ = make_inputs(seed, D, n, batches, lo, hi, C, 1, 1, 1, 1, None)
        ident = np.ones((1, C, 1), np.float32)  # the driver always runs a convolution first: 1^D kernel, unused here
        ref = refrun.run(coords, feats, ident, 1, 1, 1, threads=1, pool=(mode, kernel, stride))
        arrays = {"in_coords_raw": coords, "in_feats_raw": feats,
                  "spec": np.array([D, kernel, stride, mode], np.int32)}
        for k in ("mapping", "in_coords", "pool_coords", "pool_feats", "pool_grad_feats"):
            arrays["ref_" + k] = ref[k]
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(name, {k: v.shape for k, v in arrays.items() if k.startswith("ref_")}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
