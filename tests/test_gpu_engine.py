"""GPU tests of the host interface (SparseTensor / CoordinateManager / RiemannConvolution):
the checks the reference's own layer tests make (tests/engine/test_layers.cpp:132-148,
python/tests/test_bindings.py:73-124) plus parity of values and gradients with the oracle."""
import numpy as np
import pytest
import torch

from tests import parity
from tests.parity import OracleBackend, rel_max

pytestmark = pytest.mark.gpu


def _make(n=600, c=4, seed=7, requires_grad=False, dup=True):
    from riemannengine_b200 import engine as E
    rng = np.random.default_rng(seed)
    coords = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-6, 7, (n, 3))], 1).astype(np.int32)
    if not dup:
        coords = coords[OracleBackend().insert_and_map(coords)[0]]
    feats = rng.standard_normal((len(coords), c)).astype(np.float32)
    f = torch.from_numpy(feats).cuda().requires_grad_(requires_grad)
    return E.SparseTensor(f, torch.from_numpy(coords).cuda()), coords, feats, f


def test_sparse_tensor_dedup_matches_oracle():
    x, coords, feats, _ = _make()
    m, inv = OracleBackend().insert_and_map(coords)
    assert len(x) == len(m)
    assert (x.C.cpu().numpy() == coords[m]).all()
    assert (x.F.cpu().numpy() == feats[m]).all()
    assert x.tensor_stride == [1, 1, 1] and x.dimension == 3


def test_quantization_modes():
    from riemannengine_b200 import engine as E
    coords = torch.tensor([[0, 0, 0, 0], [0, 1, 0, 0], [0, 0, 0, 0]], dtype=torch.int32).cuda()
    feats = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 8.0]]).cuda()
    M = E.SparseTensorQuantizationMode
    assert E.SparseTensor(feats, coords).F.tolist() == [[1, 2], [3, 4]]
    assert E.SparseTensor(feats, coords, quantization_mode=M.UNWEIGHTED_SUM).F.tolist() == [[6, 10], [3, 4]]
    assert E.SparseTensor(feats, coords, quantization_mode=M.UNWEIGHTED_AVERAGE).F.tolist() == [[3, 5], [3, 4]]
    assert E.SparseTensor(feats, coords, quantization_mode=M.MAX_POOL).F.tolist() == [[5, 8], [3, 4]]


def test_strided_then_transposed_structure():
    # reference: tests/engine/test_layers.cpp:132-148
    from riemannengine_b200 import engine as E
    x, _, _, _ = _make(c=3)
    down = E.RiemannConvolution(3, 5, kernel_size=2, stride=2, dimension=3).cuda()
    up = E.RiemannConvolutionTranspose(5, 2, kernel_size=2, stride=2, dimension=3).cuda()
    y = down(x)
    assert y.F.size(1) == 5 and y.tensor_stride == [2, 2, 2] and len(y) < len(x)
    z = up(y)
    assert z.F.size(1) == 2 and z.tensor_stride == [1, 1, 1] and len(z) == len(x)
    assert torch.isfinite(z.F).all()
    assert z.coordinate_map_key == x.coordinate_map_key


def test_transposed_without_existing_map_raises():
    from riemannengine_b200 import engine as E
    x, _, _, _ = _make(c=3)
    up = E.RiemannConvolutionTranspose(3, 2, kernel_size=2, stride=2, dimension=3).cuda()
    with pytest.raises(RuntimeError, match="must divide"):
        up(x)
    mgr = E.CoordinateManager(3)
    key, _ = mgr.insert_and_map(x.C, [2, 2, 2])
    with pytest.raises(RuntimeError, match="CoordinateMap not found"):
        up(E.SparseTensor(x.F, key, mgr))


@pytest.mark.parametrize("ksize,stride,bias", [(3, 1, False), (3, 1, True), (2, 2, False), (3, 2, True)])
def test_layer_values_and_gradients_match_oracle(ksize, stride, bias):
    from riemannengine_b200 import engine as E
    x, coords, feats, leaf = _make(n=900, c=6, seed=11, requires_grad=True)
    conv = E.RiemannConvolution(6, 9, kernel_size=ksize, stride=stride, bias=bias, dimension=3).cuda()
    y = conv(x)
    loss = (y.F * y.F).sum() * 0.5
    loss.backward()
    w = conv.kernel.detach().cpu().numpy()
    O = OracleBackend(f64=True)
    r = parity.run_pipeline(O, coords, feats, w, 3, ksize, stride, 1)
    assert (y.C.cpu().numpy() == r["out_coords"]).all()
    want = r["out_feats"] + (conv.bias.detach().cpu().numpy().astype(np.float64) if bias else 0.0)
    assert rel_max(y.F.detach().cpu().numpy(), want) <= 1e-4
    if not bias:
        assert rel_max(leaf.grad.cpu().numpy(), r["grad_feats"]) <= 1e-4
        assert rel_max(conv.kernel.grad.cpu().numpy(), r["grad_weights"]) <= 1e-4
    else:
        assert conv.bias.grad is not None and torch.isfinite(conv.bias.grad).all()
    ptr, a, q = x.coordinate_manager.kernel_map(x.coordinate_map_key, y.coordinate_map_key, [ksize] * 3,
                                                [stride] * 3, [1] * 3).pairs()
    parity.assert_kernel_maps_equal((ptr.numpy(), a.cpu().numpy(), q.cpu().numpy()),
                                    (r["kmap_ptr"], r["kmap_in"], r["kmap_out"]))


def test_down_up_chain_gradients_match_oracle():
    from riemannengine_b200 import engine as E
    x, coords, feats, leaf = _make(n=900, c=4, seed=13, requires_grad=True)
    down = E.RiemannConvolution(4, 7, kernel_size=2, stride=2, dimension=3).cuda()
    up = E.RiemannConvolutionTranspose(7, 3, kernel_size=2, stride=2, dimension=3).cuda()
    z = up(down(x))
    ((z.F * z.F).sum() * 0.5).backward()
    r = parity.run_pipeline(OracleBackend(f64=True), coords, feats, down.kernel.detach().cpu().numpy(), 3, 2, 2, 1,
                            up.kernel.detach().cpu().numpy())
    assert rel_max(z.F.detach().cpu().numpy(), r["up_feats"]) <= 1e-4
    assert rel_max(leaf.grad.cpu().numpy(), r["grad_feats"]) <= 1e-4
    assert rel_max(down.kernel.grad.cpu().numpy(), r["grad_weights"]) <= 1e-4
    assert rel_max(up.kernel.grad.cpu().numpy(), r["grad_weights2"]) <= 1e-4
    th = x.coordinate_manager.kernel_map_th(down(x).coordinate_map_key, x.coordinate_map_key, [2] * 3, [2] * 3,
                                            [1] * 3, is_transpose=True)
    assert sum(v.size(1) for v in th.values()) == int(r["kmap2_ptr"][-1])


def test_optimizer_step_changes_kernel_and_reduces_loss():
    # reference: python/tests/test_bindings.py:104-124, tests/engine/test_pipeline.cpp:71-107
    from riemannengine_b200 import engine as E
    torch.manual_seed(0)
    x, _, _, _ = _make(n=500, c=4, seed=17)
    conv = E.RiemannConvolution(4, 4, kernel_size=3, dimension=3).cuda()
    target = torch.randn(len(x), 4, device="cuda") * 0.1
    opt = torch.optim.Adam(conv.parameters(), lr=1e-2)
    before = conv.kernel.detach().clone()
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(conv(x).F, target)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert not torch.equal(before, conv.kernel.detach())
    assert losses[-1] < losses[0]


def test_kernel_map_cache_is_reused():
    from riemannengine_b200 import engine as E
    x, _, _, _ = _make(c=2)
    conv = E.RiemannConvolution(2, 2, kernel_size=3, dimension=3).cuda()
    conv(x)
    mgr = x.coordinate_manager
    n = len(mgr._kernel_maps)
    conv(x)
    assert len(mgr._kernel_maps) == n == 1


def test_state_dict_round_trip_reproduces_output():
    # reference: tests/engine/test_pipeline.cpp:178-194
    from riemannengine_b200 import engine as E
    x, _, _, _ = _make(c=3)
    a = E.RiemannConvolution(3, 4, kernel_size=3, bias=True, dimension=3).cuda()
    b = E.RiemannConvolution(3, 4, kernel_size=3, bias=True, dimension=3).cuda()
    assert set(a.state_dict()) == {"base.kernel", "base.bias"}
    b.load_state_dict(a.state_dict())
    assert torch.allclose(a(x).F, b(x).F, atol=1e-6)


@pytest.mark.parametrize("dtype,c_in,c_out,tol", [(torch.float32, 6, 10, 1e-5), (torch.bfloat16, 64, 64, 2e-2),
                                                  (torch.bfloat16, 32, 128, 2e-2)])
def test_fused_conv_bn_relu_matches_unfused(dtype, c_in, c_out, tol):
    """conv -> BatchNorm1d(eval) -> ReLU folded into the convolution epilogue equals the three
    separate passes (reference blocks: engine/nn/residual.cpp:44-52)."""
    from riemannengine_b200 import engine as E
    torch.manual_seed(1)
    x, _, _, _ = _make(n=2500, c=c_in, seed=21)
    x = x.to(dtype)
    conv = E.RiemannConvolution(c_in, c_out, kernel_size=3, bias=True, dimension=3).cuda().to(dtype)
    bn = torch.nn.BatchNorm1d(c_out).cuda()
    with torch.no_grad():
        bn.running_mean.uniform_(-0.5, 0.5)
        bn.running_var.uniform_(0.5, 2.0)
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.uniform_(-0.3, 0.3)
    bn.eval()
    with torch.no_grad():
        plain = E.RiemannConvolution(c_in, c_out, kernel_size=3, bias=False, dimension=3).cuda().to(dtype)
        plain.kernel.copy_(conv.kernel)
        acc = plain(x).F.float() + conv.bias.float()
        want = torch.relu(bn(acc))
        got = E.fused_conv_bn_relu(x, conv, bn, relu=True)
        assert got.coordinate_map_key == x.coordinate_map_key
        err = (got.F.float() - want).norm() / want.norm()
        assert float(err) <= tol
        # bias-only epilogue is what the layer's own forward uses
        y = conv(x).F.float()
        assert float((y - acc).norm() / acc.norm()) <= tol
    # training mode takes the batch-statistics path (checked against torch's BatchNorm1d in
    # tests/test_gpu_norm.py): it runs, and it moves the running statistics
    bn.train()
    before = bn.running_mean.clone()
    out = E.fused_conv_bn_relu(x, conv, bn)
    assert torch.isfinite(out.F.float()).all() and not torch.equal(before, bn.running_mean)


def test_union_map_and_stride_region():
    """union_map (engine/grid/space_impl.hpp:896-914): merged map == set union, per-map rows point at equal
    coordinates; stride_region: generated map == set of in + offset. Checked on both host layers."""
    from riemannengine_b200 import cpp, engine as E
    rng = np.random.default_rng(17)

    def cloud(n):
        c = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-5, 6, (n, 3))], 1).astype(np.int32)
        return np.unique(c, axis=0)[rng.permutation(len(np.unique(c, axis=0)))]

    a, b = cloud(700), cloud(900)
    want = {tuple(r) for r in np.concatenate([a, b]).tolist()}
    off = np.array([[dx, dy, dz] for dz in (0, 1) for dy in (0, 1) for dx in (0, 1)], np.int32)
    want_region = {tuple(r) for r in (a[:, None, :] + np.concatenate([np.zeros((8, 1), np.int32), off], 1)[None])
                   .reshape(-1, 4).tolist()}
    for host in (E, cpp.load()):
        m = host.CoordinateManager(3)
        ka, _ = m.insert_and_map(torch.from_numpy(a).cuda(), [1, 1, 1], "a")
        kb, _ = m.insert_and_map(torch.from_numpy(b).cuda(), [1, 1, 1], "b")
        ku, maps = m.union_map([ka, kb])
        cu = m.get_coordinates(ku).cpu().numpy()
        assert len(cu) == len(want) and {tuple(r) for r in cu.tolist()} == want
        for src, mp in zip((a, b), maps):
            mp = mp.cpu().numpy()
            assert mp.shape == (2, len(src)) and (mp[0] == np.arange(len(src))).all()
            assert (cu[mp[1]] == src).all()
        kr = m.stride_region(ka, [2, 2, 2], [1, 1, 1], [1, 1, 1])
        cr = m.get_coordinates(kr).cpu().numpy()
        assert len(cr) == len(want_region) and {tuple(r) for r in cr.tolist()} == want_region


def _two_clouds(seed=5, n=600, c=4):
    rng = np.random.default_rng(seed)
    a = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-5, 6, (n, 3))], 1).astype(np.int32)
    b = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-5, 6, (n, 3))], 1).astype(np.int32)
    return a, b, rng.standard_normal((n, c)).astype(np.float32), rng.standard_normal((n, c)).astype(np.float32)


@pytest.mark.parametrize("host", ["py", "cpp"])
def test_sparse_tensor_arithmetic_on_the_union(host):
    """x + y, x - y, x * y on different coordinate sets: coordinates are the first occurrences of
    cat(x.C, y.C), rows a side lacks count as zero (engine/tensor/sparse_tensor.cpp:31-58, 345-379)."""
    from oracle import oracle as O
    if host == "py":
        from riemannengine_b200 import engine as H
    else:
        from riemannengine_b200 import cpp
        H = cpp.load()
    ca, cb, fa, fb = _two_clouds()
    x = H.SparseTensor(torch.from_numpy(fa).cuda(), torch.from_numpy(ca).cuda())
    y = H.SparseTensor(torch.from_numpy(fb).cuda(), torch.from_numpy(cb).cuda())
    ma, _ = O.insert_and_map(ca)
    mb, _ = O.insert_and_map(cb)
    ua, ub = ca[ma], cb[mb]
    mu, inv = O.insert_and_map(np.concatenate([ua, ub], 0))
    want_c = np.concatenate([ua, ub], 0)[mu]
    la = np.zeros((len(mu), fa.shape[1]), np.float32)
    lb = np.zeros_like(la)
    la[inv[:len(ua)]] = fa[ma]
    lb[inv[len(ua):]] = fb[mb]
    for got, want in ((x + y, la + lb), (x - y, la - lb), (x * y, la * lb)):
        assert np.array_equal(got.C.cpu().numpy(), want_c)
        assert np.allclose(got.F.cpu().numpy(), want, rtol=0, atol=1e-6)
    # same map: row by row on that map, manager and key kept (residual connection)
    z = x + x
    assert z.coordinate_map_key == x.coordinate_map_key
    assert np.allclose(z.F.cpu().numpy(), 2 * fa[ma])
    s = x * 0.5
    assert np.allclose(s.F.cpu().numpy(), 0.5 * fa[ma])
    relu = H.RiemannReLU()
    assert np.array_equal(relu(x).F.cpu().numpy(), np.maximum(fa[ma], 0))
    both = H.cat([x, z])
    assert both.F.shape[1] == 2 * fa.shape[1] and both.coordinate_map_key == x.coordinate_map_key
    assert np.allclose(H.sum([x, z]).F.cpu().numpy(), 3 * fa[ma])
    assert np.allclose(H.mean([x, z]).F.cpu().numpy(), 1.5 * fa[ma])
    with pytest.raises(RuntimeError):
        H.cat([x, y])
