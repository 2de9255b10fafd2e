"""CPU tests that pin the oracle: the reference's known-answer tests, its
measured constants for the sphere-shell cloud, and the golden fixtures produced
by the reference's own CPU build."""
import numpy as np
import pytest

from oracle import oracle as O
from tests import parity


def test_kat_forward_identity_map():
    # reference: tests/convolution/test_cpu_convolution.cpp:15-26
    out = O.conv_forward([[1, 2], [3, 4], [5, 6]], np.array([[[1, 2], [3, 4]]]), [0, 3], [0, 1, 2], [0, 1, 2], 3)
    assert out.ravel().tolist() == [7, 10, 15, 22, 23, 34]


def test_kat_backward_identity_map():
    # reference: tests/convolution/test_cpu_convolution.cpp:28-46
    gi, gw = O.conv_backward([[1, 2], [3, 4], [5, 6]], [[1, 2], [3, 4], [5, 6]], np.array([[[1, 2], [3, 4]]]),
                             [0, 3], [0, 1, 2], [0, 1, 2])
    assert gi.ravel().tolist() == [5, 11, 11, 25, 17, 39]
    assert gw.ravel().tolist() == [35, 44, 44, 56]


def test_kat_forward_permuted_map():
    # reference: tests/convolution/test_cpu_convolution.cpp:48-61
    out = O.conv_forward([[1], [3], [5]], np.array([[[2]]]), [0, 3], [2, 0, 1], [1, 2, 0], 3)
    assert out.ravel().tolist() == [6, 10, 2]


def test_murmur3_known_values():
    # MurmurHash3 x86-32, seed 0: published check values for 4-byte little-endian inputs
    assert O.murmur3_row([0]) == 0x2362F9DE
    assert O.murmur3_row([1]) == 0xFBF1402A


def shell_cloud():
    r = np.arange(-65, 66)
    g = np.stack(np.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 3)
    nrm = np.sqrt((g.astype(np.float64) ** 2).sum(1))
    g = g[np.abs(nrm - 64) < 1]
    return np.concatenate([np.zeros((len(g), 1), np.int32), g.astype(np.int32)], 1)


def test_sphere_shell_constants():
    """Counts measured from the reference CPU build on the sphere-shell cloud."""
    c = shell_cloud()
    assert len(c) == 101930
    m, inv = O.insert_and_map(c)
    assert len(m) == 101930 and (inv == np.arange(len(c))).all()
    ptr, _, _ = O.conv_kernel_map(c, c, O.region_offsets(O.HYPER_CUBE, [3] * 3, [1] * 3, [1] * 3))
    assert ptr[-1] == 1804802
    coarse, inv = O.stride_map(c, [2, 2, 2])
    assert len(coarse) == 22376
    off2 = O.region_offsets(O.HYPER_CUBE, [2] * 3, [1] * 3, [1] * 3)
    ptr, _, _ = O.conv_kernel_map(c, coarse, off2)
    assert ptr[-1] == 101930
    ptr, _, _ = O.conv_kernel_map(coarse, c, off2, transposed=True)
    assert ptr[-1] == 101930 and len(ptr) == 9


def test_region_enumeration():
    off = O.region_offsets(O.HYPER_CUBE, [3, 3, 3], [1, 1, 1], [2, 2, 2])
    assert off[0].tolist() == [-2, -2, -2] and off[1].tolist() == [0, -2, -2] and off[13].tolist() == [0, 0, 0]
    off = O.region_offsets(O.HYPER_CUBE, [2, 2], [1, 1], [4, 4])
    assert off.tolist() == [[0, 0], [4, 0], [0, 4], [4, 4]]
    off = O.region_offsets(O.HYPER_CROSS, [3, 3], [1, 1], [1, 1])
    assert off.tolist() == [[0, 0], [1, 0], [-1, 0], [0, 1], [0, -1]]
    off = O.region_offsets(O.CUSTOM, [1, 1], [2, 2], [3, 3], custom=np.array([[1, -1], [0, 2]]))
    assert off.tolist() == [[6, -6], [0, 12]]


def test_stride_floor_negative():
    c = np.array([[0, -65, -1, 3], [1, 5, 4, -4]], np.int32)
    assert O.stride_coords(c, [2, 2, 2]).tolist() == [[0, -66, -2, 2], [1, 4, 4, -4]]


def test_empty_and_single():
    m, inv = O.insert_and_map(np.zeros((0, 4), np.int32))
    assert len(m) == 0 and len(inv) == 0
    c = np.array([[0, 1, 2, 3]], np.int32)
    ptr, a, q = O.conv_kernel_map(c, c, O.region_offsets(O.HYPER_CUBE, [3] * 3, [1] * 3, [1] * 3))
    assert ptr[-1] == 1 and a.tolist() == [0] and q.tolist() == [0] and ptr[13] == 0 and ptr[14] == 1


@pytest.mark.parametrize("name", parity.GOLDEN_CASES)
@pytest.mark.parametrize("f64", [False, True])
def test_oracle_matches_reference_golden(name, f64):
    gold = parity.load_golden(name)
    D, kernel, stride, dilation = gold["spec"].tolist()
    res = parity.run_pipeline(parity.OracleBackend(f64=f64), gold["in_coords_raw"], gold["in_feats_raw"],
                              gold["weights"], D, kernel, stride, dilation, gold.get("weights2"))
    parity.check_against_reference(res, gold, tol=1e-5)


@pytest.mark.parametrize("name", parity.POOL_GOLDEN_CASES)
def test_oracle_pooling_matches_reference_golden(name):
    gold = parity.load_golden(name)
    out_coords, out, g_raw = parity.oracle_pool_case(gold)
    parity.check_pool_against_reference(out_coords, out, g_raw, gold, tol=1e-5)


@pytest.mark.parametrize("name", parity.UNPOOL_GOLDEN_CASES)
def test_oracle_pooling_transpose_matches_reference_golden(name):
    gold = parity.load_golden(name)
    out_coords, out, g_raw = parity.oracle_unpool_case(gold)
    parity.check_pool_against_reference(out_coords, out, g_raw, gold, tol=1e-5)


FIELD_CASES = ["field_d3_s1_avg", "field_d3_s2_sum", "field_d2_s42_max", "field_d3_s123_first", "field_d4_s1_avg"]


@pytest.mark.parametrize("name", FIELD_CASES)
def test_field_oracle_matches_reference_fixture(name):
    """Input step (TensorField.sparse / splat, sparse_quantize) against fixtures the reference produced."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    field, feats, stride = g["field"], g["feats"], g["stride"].tolist()
    mode, q = int(g["spec"][1]), float(g["qsize"][0])
    c, f, inv = O.field_sparse(field, feats, stride, mode)
    assert np.array_equal(c, g["ref_field_coords"]) and np.array_equal(inv, g["ref_field_inverse"])
    assert np.abs(f - g["ref_field_feats"]).max() <= 1e-5 * max(1.0, np.abs(f).max())
    sc, sf = O.field_splat(field, feats)
    m, i = O.insert_and_map(sc)
    assert np.array_equal(sc[m], g["ref_splat_coords"])
    assert np.abs(O.quantize_features(sf, m, i, 2) - g["ref_splat_feats"]).max() <= 1e-5
    qc, qf, qu, qi = O.sparse_quantize(field, feats, q if q > 0 else None)
    assert np.array_equal(qc, g["ref_sq_coords"]) and np.array_equal(qf, g["ref_sq_feats"])
    assert np.array_equal(qu, g["ref_sq_unique_index"]) and np.array_equal(qi, g["ref_sq_inverse"])
