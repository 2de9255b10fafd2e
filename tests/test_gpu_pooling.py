"""GPU parity of local pooling (RiemannSumPooling / RiemannAvgPooling / RiemannMaxPooling) with the
fixtures the reference produced (engine/nn/pooling.cpp), with the oracle in bf16, and through
size-independent properties at the benchmark's size."""
import numpy as np
import pytest
import torch

from tests import parity

pytestmark = pytest.mark.gpu

_LAYER = {1: "RiemannSumPooling", 2: "RiemannAvgPooling", 3: "RiemannMaxPooling"}


def _run_engine(gold, dtype=torch.float32):
    from riemannengine_b200 import engine as E
    D, kernel, stride, mode = (int(v) for v in gold["spec"])
    feats = torch.from_numpy(gold["in_feats_raw"]).cuda().to(dtype).requires_grad_(True)
    x = E.SparseTensor(feats, torch.from_numpy(gold["in_coords_raw"]).cuda())
    layer = getattr(E, _LAYER[mode])(kernel, stride, 1, dimension=D)
    y = layer(x)
    (y.F.float() * y.F.float()).sum().mul(0.5).backward()
    return y, feats.grad


@pytest.mark.parametrize("name", parity.POOL_GOLDEN_CASES)
def test_pooling_matches_reference_golden_fp32(name):
    gold = parity.load_golden(name)
    y, grad = _run_engine(gold)
    parity.check_pool_against_reference(y.C.cpu().numpy(), y.F.detach().cpu().numpy(), grad.cpu().numpy(), gold,
                                        tol=1e-4)  # fp32 bar: 1e-4 relative


@pytest.mark.parametrize("name", ["pool_d3_avg_k2_s2", "pool_d3_sum_k3_s1_wide"])
def test_pooling_bf16_against_oracle(name):
    # bf16 bar: 1e-2 relative L2 against the fp64 oracle on bf16-rounded inputs
    from oracle import oracle as O
    from riemannengine_b200 import engine as E
    rng = np.random.default_rng(5)
    if name.endswith("wide"):
        D, kernel, stride, mode, C = 3, 3, 1, 1, 64   # 128-byte rows: the vector kernels
    else:
        D, kernel, stride, mode, C = 3, 2, 2, 2, 24   # 48-byte rows: the scalar kernels
    n = 3000
    coords = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-8, 9, (n, D))], 1).astype(np.int32)
    feats = torch.from_numpy(rng.standard_normal((n, C)).astype(np.float32)).bfloat16()
    gold = {"spec": np.array([D, kernel, stride, mode]), "in_coords_raw": coords,
            "in_feats_raw": feats.float().numpy()}
    out_coords, out_ref, _ = parity.oracle_pool_case(gold)
    x = E.SparseTensor(feats.cuda(), torch.from_numpy(coords).cuda())
    y = getattr(E, _LAYER[mode])(kernel, stride, 1, dimension=D)(x)
    got_c, got = y.C.cpu().numpy(), y.F.float().cpu().numpy()
    o1, o2 = np.lexsort(got_c.T[::-1]), np.lexsort(out_coords.T[::-1])
    assert np.array_equal(got_c[o1], out_coords[o2])
    err = np.linalg.norm(got[o1] - out_ref[o2]) / max(np.linalg.norm(out_ref), 1e-30)
    assert err <= 1e-2, err


def test_pooling_properties_at_benchmark_size():
    """1.2 M-voxel indoor batch, 3^3 stride-1 region: sum pooling equals the convolution whose 27 kernels
    are identity matrices; average * count == sum; maximum >= average; the sum-pooling gradient of
    ones is the neighbour count of every input row."""
    from riemannengine_b200 import engine as E, ops, synthetic
    coords = torch.from_numpy(np.ascontiguousarray(synthetic.indoor_batch(8, 150_000), np.int32)).cuda()
    C = 32
    g = torch.Generator(device="cpu").manual_seed(3)
    feats = torch.randn(coords.size(0), C, generator=g).cuda().requires_grad_(True)
    x = E.SparseTensor(feats, coords)
    s = E.RiemannSumPooling(3, 1, 1, dimension=3)(x)
    a = E.RiemannAvgPooling(3, 1, 1, dimension=3)(x)
    m = E.RiemannMaxPooling(3, 1, 1, dimension=3)(x)
    kmap = x.coordinate_manager.kernel_map(x.coordinate_map_key, x.coordinate_map_key, [3] * 3, [1] * 3, [1] * 3,
                                           is_pool=True)
    eye = torch.eye(C, device="cuda").repeat(27, 1, 1).contiguous()
    conv = ops.conv_forward(x.F.detach(), eye, kmap.nbr_out)
    assert torch.allclose(s.F, conv, rtol=1e-5, atol=1e-5)
    count = (kmap.nbr_out >= 0).sum(0).float().unsqueeze(1)
    assert count.min() >= 1  # the centre offset always hits
    assert torch.allclose(a.F * count, s.F, rtol=1e-4, atol=1e-4)
    assert (m.F >= a.F - 1e-5).all()
    s.F.sum().backward()
    assert torch.equal(feats.grad, count.expand(-1, C))  # symmetric region: in-degree == out-degree


@pytest.mark.parametrize("name", parity.UNPOOL_GOLDEN_CASES)
def test_pooling_transpose_matches_reference_golden_fp32(name):
    """(strided) convolution -> RiemannPoolingTranspose: generated coordinates, values and the gradient back to
    the raw features equal the reference's (fixtures from engine/nn/pooling.cpp:197-229); fp32 bar 1e-4."""
    from riemannengine_b200 import engine as E
    gold = parity.load_golden(name)
    D, kernel, stride, _ = (int(v) for v in gold["spec"])
    w = torch.from_numpy(gold["weights"]).cuda()
    conv = E.RiemannConvolution(w.size(1), w.size(2), kernel_size=kernel, stride=stride, dimension=D).cuda()
    with torch.no_grad():
        conv.kernel.copy_(w)
    feats = torch.from_numpy(gold["in_feats_raw"]).cuda().requires_grad_(True)
    x = E.SparseTensor(feats, torch.from_numpy(gold["in_coords_raw"]).cuda())
    y = E.RiemannPoolingTranspose(kernel, stride, 1, False, dimension=D)(conv(x))
    assert y.tensor_stride == [1] * D
    (y.F * y.F).sum().mul(0.5).backward()
    parity.check_pool_against_reference(y.C.cpu().numpy(), y.F.detach().cpu().numpy(), feats.grad.cpu().numpy(), gold,
                                        tol=1e-4)


def test_empty_inputs_through_pooling_and_statistics():
    """Zero voxels: every layer returns an empty tensor of the right width, nothing is launched on no data."""
    from riemannengine_b200 import engine as E, ops
    coords = torch.zeros((0, 4), dtype=torch.int32, device="cuda")
    feats = torch.zeros((0, 6), device="cuda")
    x = E.SparseTensor(feats, coords)
    assert len(x) == 0
    for layer in (E.RiemannSumPooling(2, 2, 1, dimension=3), E.RiemannMaxPooling(3, 1, 1, dimension=3)):
        y = layer(x)
        assert tuple(y.F.shape) == (0, 6) and len(y) == 0
    y = E.RiemannConvolution(6, 5, kernel_size=3, dimension=3).cuda()(x)
    assert tuple(y.F.shape) == (0, 5)
    assert torch.equal(ops.channel_stats(feats), torch.zeros(2, 6, dtype=torch.float64, device="cuda"))
    assert ops.affine_act(feats, None, None, relu=True).shape == (0, 6)
    # an output row without any neighbour pools to zero (isolated voxel, region that misses the centre)
    c1 = torch.tensor([[0, 0, 0, 0], [0, 10, 10, 10]], dtype=torch.int32, device="cuda")
    f1 = torch.tensor([[1.0, -2.0], [3.0, 4.0]], device="cuda")
    t = ops.table_build(c1)
    res = ops.kmap_build(t, t.coords, np.array([[1, 0, 0], [0, 1, 0]], np.int32))
    for mode in (ops.POOL_SUM, ops.POOL_AVG, ops.POOL_MAX):
        out, _ = ops.pool_forward(f1, res.nbr, mode)
        assert torch.equal(out, torch.zeros_like(f1))
