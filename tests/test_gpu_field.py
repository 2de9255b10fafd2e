"""GPU parity of the input step on continuous coordinates: field quantisation, TensorField.sparse / splat /
inverse_mapping and sparse_quantize, against fixtures produced by the reference (tests/golden/field_*.npz)
and against the oracle on larger seeded clouds. Coordinates and index maps are compared bit for bit; features
within 1e-5 (fp32 sums in a different order)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = ["field_d3_s1_avg", "field_d3_s2_sum", "field_d2_s42_max", "field_d3_s123_first", "field_d4_s1_avg"]


def _engine():
    from riemannengine_b200 import engine as E
    return E


@pytest.mark.parametrize("name", CASES)
def test_tensor_field_matches_reference_fixture(name):
    E = _engine()
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    stride, mode, q = g["stride"].tolist(), int(g["spec"][1]), float(g["qsize"][0])
    field = torch.from_numpy(g["field"]).cuda()
    feats = torch.from_numpy(g["feats"]).cuda()
    tf = E.TensorField(feats, field)
    sp = tf.sparse(stride, None, mode)
    assert sp.tensor_stride == stride
    assert np.array_equal(sp.C.cpu().numpy(), g["ref_field_coords"])
    assert np.array_equal(tf.inverse_mapping(sp.coordinate_map_key).cpu().numpy(), g["ref_field_inverse"])
    assert np.abs(sp.F.cpu().numpy() - g["ref_field_feats"]).max() <= 1e-5 * max(1.0, np.abs(g["ref_field_feats"]).max())
    # reading the voxel features back at the points
    back = tf.slice(sp).cpu().numpy()
    assert np.array_equal(back, sp.F.cpu().numpy()[g["ref_field_inverse"]])
    spl = E.TensorField(feats, field).splat()
    assert np.array_equal(spl.C.cpu().numpy(), g["ref_splat_coords"])
    assert np.abs(spl.F.cpu().numpy() - g["ref_splat_feats"]).max() <= 1e-5
    sq = E.sparse_quantize(field, feats, quantization_size=q if q > 0 else None)
    assert np.array_equal(sq.coordinates.cpu().numpy(), g["ref_sq_coords"])
    assert np.array_equal(sq.features.cpu().numpy(), g["ref_sq_feats"])
    assert np.array_equal(sq.unique_index.cpu().numpy(), g["ref_sq_unique_index"])
    assert np.array_equal(sq.inverse_mapping.cpu().numpy(), g["ref_sq_inverse"])


@pytest.mark.parametrize("stride", [[1, 1, 1], [2, 2, 2], [3, 1, 5]])
def test_field_quantize_against_oracle_large(stride):
    """LiDAR-like points (metres / 0.1 m voxels) incl. negative values, exact integers and half-way batch values."""
    from riemannengine_b200 import ops
    rng = np.random.default_rng(7)
    n = 300_000
    pts = (rng.uniform(-70, 70, (n, 3)) / 0.1).astype(np.float32)
    pts[::11] = np.round(pts[::11])
    batch = rng.integers(0, 16, (n, 1)).astype(np.float32)
    batch[::5] += np.float32(0.5)    # lroundf rounds half away from zero
    batch[1::5] -= np.float32(0.25)
    field = np.concatenate([batch, pts], 1)
    got = ops.field_quantize(torch.from_numpy(field).cuda(), stride).cpu().numpy()
    assert np.array_equal(got, O.field_quantize(field, stride))
    d = ops.coords_discretize(torch.from_numpy(field).cuda(), 0.37).cpu().numpy()
    assert np.array_equal(d, np.floor(field.astype(np.float64) / 0.37).astype(np.int32))
    d64 = ops.coords_discretize(torch.from_numpy(field.astype(np.float64) * 1.1).cuda(), None).cpu().numpy()
    assert np.array_equal(d64, np.floor(field.astype(np.float64) * 1.1).astype(np.int32))


def test_field_sparse_then_convolution_bf16():
    """Points -> voxels (average) -> 3^3 convolution -> features read back at the points."""
    E = _engine()
    rng = np.random.default_rng(3)
    n = 20_000
    field = np.concatenate([rng.integers(0, 2, (n, 1)).astype(np.float32),
                            rng.uniform(0, 24, (n, 3)).astype(np.float32)], 1)
    feats = rng.standard_normal((n, 32)).astype(np.float32)
    tf = E.TensorField(torch.from_numpy(feats).cuda(), torch.from_numpy(field).cuda())
    sp = tf.sparse()
    c, f, inv = O.field_sparse(field, feats, [1, 1, 1], 1)
    assert np.array_equal(sp.C.cpu().numpy(), c)
    assert np.abs(sp.F.cpu().numpy() - f).max() <= 1e-5
    conv = E.RiemannConvolution(32, 64, kernel_size=3, dimension=3).cuda()
    y = conv(sp)
    ptr, a, qq = O.conv_kernel_map(c, c, O.region_offsets(O.HYPER_CUBE, [3] * 3, [1] * 3, [1] * 3))
    want = O.conv_forward(f.astype(np.float32), conv.kernel.detach().cpu().numpy(), ptr, a, qq, len(c), f64=True)
    got = y.F.detach().cpu().numpy()
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
    at_points = tf.slice(y).detach().cpu().numpy()
    assert np.array_equal(at_points, got[inv])


def test_field_empty_and_errors():
    E = _engine()
    from riemannengine_b200 import ops
    empty = torch.empty((0, 4), dtype=torch.float32, device="cuda")
    assert ops.field_quantize(empty, [1, 1, 1]).shape == (0, 4)
    with pytest.raises(RuntimeError):
        E.TensorField(torch.zeros((3, 2), device="cuda"), torch.zeros((3, 4), dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError):
        E.TensorField(torch.zeros((2, 2), device="cuda"), torch.zeros((3, 4), device="cuda"))
    with pytest.raises(RuntimeError):
        E.sparse_quantize(torch.zeros((3, 4), device="cuda"), quantization_size=-1.0)
    with pytest.raises(RuntimeError):
        ops.field_quantize(torch.zeros((3, 4), device="cuda"), [1, 0, 1])
