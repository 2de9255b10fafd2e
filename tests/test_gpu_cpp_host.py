"""GPU tests of the C++20 / LibTorch host layer (riemann_cpp) through its pybind11 module: the
same structural checks the reference makes on its layers (tests/engine/test_layers.cpp:132-148,
python/tests/test_bindings.py:73-124) and value/gradient parity with the oracle."""
import numpy as np
import pytest
import torch

from tests import parity
from tests.parity import OracleBackend, rel_max

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from riemannengine_b200 import cpp
    return cpp.load()


def _inputs(n=800, c=5, seed=3):
    rng = np.random.default_rng(seed)
    coords = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-6, 7, (n, 3))], 1).astype(np.int32)
    feats = rng.standard_normal((n, c)).astype(np.float32)
    return coords, feats


def test_cpp_sparse_tensor_and_conv_match_oracle(C):
    coords, feats = _inputs()
    f = torch.from_numpy(feats).cuda().requires_grad_(True)
    x = C.SparseTensor(f, torch.from_numpy(coords).cuda())
    conv = C.RiemannConvolution(5, 7, kernel_size=3, dimension=3)
    conv.to("cuda")
    y = conv(x)
    ((y.F * y.F).sum() * 0.5).backward()
    w = conv.kernel.detach().cpu().numpy()
    r = parity.run_pipeline(OracleBackend(f64=True), coords, feats, w, 3, 3, 1, 1)
    assert (x.C.cpu().numpy() == r["in_coords"]).all()
    assert rel_max(y.F.detach().cpu().numpy(), r["out_feats"]) <= 1e-4
    assert rel_max(f.grad.cpu().numpy(), r["grad_feats"]) <= 1e-4
    assert rel_max(conv.kernel.grad.cpu().numpy(), r["grad_weights"]) <= 1e-4
    th = x.coordinate_manager.kernel_map_th(x.coordinate_map_key, y.coordinate_map_key, [3] * 3, [1] * 3, [1] * 3)
    assert sum(v.shape[1] for v in th.values()) == int(r["kmap_ptr"][-1])
    for k, v in th.items():
        want = parity.sorted_pairs(r["kmap_ptr"], r["kmap_in"], r["kmap_out"], k)
        got = v.cpu().numpy().T.astype(np.int64)
        got = got[np.lexsort((got[:, 1], got[:, 0]))]
        assert (got == want).all()


def test_cpp_down_up_chain(C):
    coords, feats = _inputs(c=4, seed=5)
    f = torch.from_numpy(feats).cuda().requires_grad_(True)
    x = C.SparseTensor(f, torch.from_numpy(coords).cuda())
    down = C.RiemannConvolution(4, 6, kernel_size=2, stride=2, dimension=3)
    up = C.RiemannConvolutionTranspose(6, 3, kernel_size=2, stride=2, dimension=3)
    down.to("cuda")
    up.to("cuda")
    y = down(x)
    assert y.tensor_stride == [2, 2, 2] and len(y) < len(x) and y.F.shape[1] == 6
    z = up(y)
    assert z.tensor_stride == [1, 1, 1] and len(z) == len(x) and z.coordinate_map_key == x.coordinate_map_key
    ((z.F * z.F).sum() * 0.5).backward()
    r = parity.run_pipeline(OracleBackend(f64=True), coords, feats, down.kernel.detach().cpu().numpy(), 3, 2, 2, 1,
                            up.kernel.detach().cpu().numpy())
    assert (y.C.cpu().numpy() == r["out_coords"]).all()
    assert rel_max(z.F.detach().cpu().numpy(), r["up_feats"]) <= 1e-4
    assert rel_max(f.grad.cpu().numpy(), r["grad_feats"]) <= 1e-4
    assert rel_max(down.kernel.grad.cpu().numpy(), r["grad_weights"]) <= 1e-4
    assert rel_max(up.kernel.grad.cpu().numpy(), r["grad_weights2"]) <= 1e-4


def test_cpp_transposed_needs_existing_map(C):
    coords, feats = _inputs(c=3)
    x = C.SparseTensor(torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda())
    up = C.RiemannConvolutionTranspose(3, 2, kernel_size=2, stride=2, dimension=3)
    up.to("cuda")
    with pytest.raises(RuntimeError, match="must divide"):
        up(x)


def test_cpp_bf16_layer(C):
    coords, feats = _inputs(n=3000, c=32, seed=9)
    x = C.SparseTensor(torch.from_numpy(feats).cuda().bfloat16(), torch.from_numpy(coords).cuda())
    conv = C.RiemannConvolution(32, 64, kernel_size=3, dimension=3)
    conv.to("cuda")
    conv.to(torch.bfloat16)
    y = conv(x)
    w = conv.kernel.detach().float().cpu().numpy()
    fb = torch.from_numpy(feats).bfloat16().float().numpy()
    r = parity.run_pipeline(OracleBackend(f64=True), coords, fb, w, 3, 3, 1, 1)
    assert parity.rel_l2(y.F.detach().float().cpu().numpy(), r["out_feats"]) <= 1e-2


def test_cpp_bias_is_fused_and_has_gradient(C):
    coords, feats = _inputs(c=4, seed=12)
    f = torch.from_numpy(feats).cuda().requires_grad_(True)
    x = C.SparseTensor(f, torch.from_numpy(coords).cuda())
    conv = C.RiemannConvolution(4, 6, kernel_size=3, bias=True, dimension=3)
    conv.to("cuda")
    y = conv(x)
    y.F.sum().backward()
    r = parity.run_pipeline(OracleBackend(f64=True), coords, feats, conv.kernel.detach().cpu().numpy(), 3, 3, 1, 1)
    want = r["out_feats"] + conv.bias.detach().cpu().numpy().astype(np.float64)
    assert rel_max(y.F.detach().cpu().numpy(), want) <= 1e-4
    assert torch.allclose(conv.bias.grad, torch.full_like(conv.bias.grad, float(len(y))))


@pytest.mark.parametrize("name", parity.POOL_GOLDEN_CASES)
def test_cpp_pooling_matches_reference_golden(C, name):
    # fixtures produced by the reference's pooling layers (engine/nn/pooling.cpp); fp32 bar 1e-4
    gold = parity.load_golden(name)
    D, kernel, stride, mode = (int(v) for v in gold["spec"])
    layer = {1: C.RiemannSumPooling, 2: C.RiemannAvgPooling, 3: C.RiemannMaxPooling}[mode](kernel, stride, 1, D)
    f = torch.from_numpy(gold["in_feats_raw"]).cuda().requires_grad_(True)
    x = C.SparseTensor(f, torch.from_numpy(gold["in_coords_raw"]).cuda())
    y = layer(x)
    ((y.F * y.F).sum() * 0.5).backward()
    parity.check_pool_against_reference(y.C.cpu().numpy(), y.F.detach().cpu().numpy(), f.grad.cpu().numpy(), gold,
                                        tol=1e-4)


def test_cpp_fused_conv_bn_relu_inference(C):
    """One-kernel conv -> batch norm (running statistics) -> ReLU equals the three separate steps."""
    coords, feats = _inputs(n=1500, c=6, seed=9)
    x = C.SparseTensor(torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda())
    conv = C.RiemannConvolution(6, 10, kernel_size=3, bias=True, dimension=3)
    conv.to("cuda")
    bn = torch.nn.BatchNorm1d(10).cuda().eval()
    with torch.no_grad():
        bn.running_mean.uniform_(-0.5, 0.5)
        bn.running_var.uniform_(0.5, 2.0)
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.uniform_(-0.5, 0.5)
        want = torch.relu(bn(conv(x).F))
        got = C.fused_conv_bn_relu(x, conv, bn.running_mean, bn.running_var, bn.weight, bn.bias, bn.eps, True).F
    assert rel_max(got.cpu().numpy(), want.cpu().numpy()) <= 1e-4


@pytest.mark.parametrize("name", parity.UNPOOL_GOLDEN_CASES)
def test_cpp_pooling_transpose_matches_reference_golden(C, name):
    gold = parity.load_golden(name)
    D, kernel, stride, _ = (int(v) for v in gold["spec"])
    w = torch.from_numpy(gold["weights"]).cuda()
    conv = C.RiemannConvolution(w.size(1), w.size(2), kernel_size=kernel, stride=stride, dimension=D)
    conv.to("cuda")
    with torch.no_grad():
        conv.kernel.copy_(w)
    f = torch.from_numpy(gold["in_feats_raw"]).cuda().requires_grad_(True)
    x = C.SparseTensor(f, torch.from_numpy(gold["in_coords_raw"]).cuda())
    y = C.RiemannPoolingTranspose(kernel, stride, 1, False, D)(conv(x))
    ((y.F * y.F).sum() * 0.5).backward()
    parity.check_pool_against_reference(y.C.cpu().numpy(), y.F.detach().cpu().numpy(), f.grad.cpu().numpy(), gold,
                                        tol=1e-4)


@pytest.mark.parametrize("name", ["field_d3_s1_avg", "field_d3_s2_sum", "field_d2_s42_max", "field_d3_s123_first",
                                  "field_d4_s1_avg"])
def test_cpp_tensor_field_matches_reference_fixture(C, name):
    """TensorField.sparse / splat / inverse_mapping and sparse_quantize of the C++ host against fixtures the
    reference produced (engine/tensor/field.cpp, engine/helpers/discretization.cpp)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    stride, mode, q = g["stride"].tolist(), int(g["spec"][1]), float(g["qsize"][0])
    field = torch.from_numpy(g["field"]).cuda()
    feats = torch.from_numpy(g["feats"]).cuda()
    tf = C.TensorField(feats, field)
    sp = tf.sparse(stride, None, C.SparseTensorQuantizationMode(mode))
    assert list(sp.tensor_stride) == stride
    assert np.array_equal(sp.C.cpu().numpy(), g["ref_field_coords"])
    assert np.array_equal(tf.inverse_mapping(sp.coordinate_map_key).cpu().numpy(), g["ref_field_inverse"])
    assert np.abs(sp.F.cpu().numpy() - g["ref_field_feats"]).max() <= 1e-5 * max(1.0, np.abs(g["ref_field_feats"]).max())
    spl = C.TensorField(feats, field).splat()
    assert np.array_equal(spl.C.cpu().numpy(), g["ref_splat_coords"])
    assert np.abs(spl.F.cpu().numpy() - g["ref_splat_feats"]).max() <= 1e-5
    coords, fq, unique, inverse = C.sparse_quantize(field, feats, q if q > 0 else None)
    assert np.array_equal(coords.cpu().numpy(), g["ref_sq_coords"])
    assert np.array_equal(fq.cpu().numpy(), g["ref_sq_feats"])
    assert np.array_equal(unique.cpu().numpy(), g["ref_sq_unique_index"])
    assert np.array_equal(inverse.cpu().numpy(), g["ref_sq_inverse"])


@pytest.mark.parametrize("host", ["cpp", "python"])
@pytest.mark.parametrize("c_in,c_out", [(4, 32), (16, 16), (48, 96), (256, 128), (256, 256), (32, 128)])
def test_bf16_channel_counts_without_a_kernel_run_padded_on_the_tensor_cores(C, host, c_in, c_out):
    """A 4-channel stem, 16 -> 16, 48 -> 96 ...: the host layers zero-pad the channels to a shape the tcgen05
    kernels take (and split a 256-channel weight gradient into two halves); values and gradients against the
    fp64 oracle on the same bf16-rounded inputs, and the tensor-core launch counter must move (forward, input
    gradient and weight gradient = at least 3 launches, none on the SIMT kernels)."""
    from riemannengine_b200 import capi, engine as E, synthetic
    O = OracleBackend(f64=True)
    pts = synthetic.indoor_scene(91, 12000)
    c = np.concatenate([np.zeros((len(pts), 1), np.int32), pts], 1)
    f = synthetic.features(92, len(c), c_in)
    w = synthetic.conv_weights(93, 27, c_in, c_out)
    fb = torch.from_numpy(f).bfloat16()
    wb = torch.from_numpy(w).bfloat16()
    feats = fb.cuda().requires_grad_(True)
    if host == "cpp":
        x = C.SparseTensor(feats, torch.from_numpy(c).cuda())
        conv = C.RiemannConvolution(c_in, c_out, kernel_size=3, dimension=3)
        conv.to("cuda")
        conv.to(torch.bfloat16)
    else:
        x = E.SparseTensor(feats, torch.from_numpy(c).cuda())
        conv = E.RiemannConvolution(c_in, c_out, kernel_size=3, dimension=3).cuda().bfloat16()
    with torch.no_grad():
        conv.kernel.copy_(wb.cuda())
    lib = capi.lib()
    tc0, all0 = lib.rmn_tensor_core_launch_count(), lib.rmn_launch_count()
    y = conv(x)
    g = torch.from_numpy(synthetic.features(94, len(c), c_out)).bfloat16()
    y.F.backward(g.cuda())
    torch.cuda.synchronize()
    assert lib.rmn_tensor_core_launch_count() - tc0 >= 3
    off = O.region_offsets([3] * 3, [1] * 3, [1] * 3)
    k0 = O.conv_kernel_map(c, c, off)
    y0 = O.conv_forward(fb.float().numpy(), wb.float().numpy(), k0, len(c), len(c))
    gi0, gw0 = O.conv_backward(fb.float().numpy(), g.float().numpy(), wb.float().numpy(), k0, len(c), len(c))
    assert tuple(y.F.shape) == (len(c), c_out)
    assert parity.rel_l2(y.F.detach().float().cpu().numpy(), y0) <= 1e-2
    assert parity.rel_l2(feats.grad.float().cpu().numpy(), gi0) <= 1e-2
    assert parity.rel_l2(conv.kernel.grad.float().cpu().numpy(), gw0) <= 1e-2
    assert tuple(conv.kernel.grad.shape) == (27, c_in, c_out)


def test_cpp_origin_map_has_one_row_per_batch_index(C):
    """CoordinateManager::origin (engine/grid/space_impl.hpp:383-421): rows (b, 0, 0, 0) for the batch indices
    present, tensor stride zero, created once."""
    rng = np.random.default_rng(8)
    coords = np.concatenate([rng.choice([0, 2, 5], (500, 1)), rng.integers(-6, 7, (500, 3))], 1).astype(np.int32)
    x = C.SparseTensor(torch.zeros(500, 3, device="cuda"), torch.from_numpy(coords).cuda())
    m = x.coordinate_manager
    key, created = m.origin()
    assert created and key.tensor_stride == [0, 0, 0]
    got = m.get_coordinates(key).cpu().numpy()
    assert sorted(got[:, 0].tolist()) == [0, 2, 5] and (got[:, 1:] == 0).all()
    key2, created2 = m.origin()
    assert not created2 and key2.tensor_stride == [0, 0, 0] and m.size(key2) == 3


def test_cpp_example_unet_runs_and_is_reproducible(C):
    """The MinkUNet-style network of riemann_cpp/networks.hpp (written in the reference's layer API): a forward
    and backward pass on a small cloud gives one output row per input voxel, finite values and gradients for
    every parameter, and the same numbers when repeated."""
    from riemannengine_b200 import synthetic
    pts = synthetic.indoor_scene(95, 20000)
    c = torch.from_numpy(np.concatenate([np.zeros((len(pts), 1), np.int32), pts], 1)).cuda()
    f = torch.from_numpy(synthetic.features(96, len(pts), 4)).cuda().bfloat16()
    torch.manual_seed(3)
    net = C.MinkUNet(4, 20, width=32, dimension=3)
    net.to("cuda")
    net.to(torch.bfloat16)
    net.train(True)
    outs = []
    for _ in range(2):
        net.zero_grad()
        y = net(C.SparseTensor(f, c))
        assert tuple(y.F.shape) == (len(pts), 20) and y.tensor_stride == [1, 1, 1]
        (y.F.float() ** 2).mean().backward()
        grads = {k: p.grad.float().clone() for k, p in net.named_parameters().items()}
        assert all(torch.isfinite(g).all() for g in grads.values()) and len(grads) > 60
        assert torch.isfinite(y.F.float()).all()
        outs.append((y.F.detach().clone(), grads))
    assert torch.equal(outs[0][0], outs[1][0])
    assert all(torch.allclose(outs[0][1][k], outs[1][1][k], rtol=1e-2, atol=1e-4) for k in outs[0][1])


@pytest.mark.parametrize("kernel,stride", [(2, 2), (3, 2), (3, 1)])
def test_cpp_generative_transposed_convolution_expands_coordinates(C, kernel, stride):
    """RiemannGenerativeConvolutionTranspose generates its output coordinates (every coarse voxel spawns its
    kernel region on the finer stride) and convolves onto them. Bar: the oracle's composition of the same two
    steps - region expansion + first-occurrence dedup, which the pooling-transpose fixtures of the reference pin
    (tests/golden/unpool_*.npz), and the transposed kernel map + convolution - values and gradients in fp32."""
    from oracle import oracle as O
    rng = np.random.default_rng(40 + kernel + stride)
    raw = np.concatenate([rng.integers(0, 2, (600, 1)), rng.integers(-6, 7, (600, 3)) * stride], 1).astype(np.int32)
    coarse = raw[O.insert_and_map(raw)[0]]
    feats = rng.standard_normal((len(coarse), 5)).astype(np.float32)
    # a tensor on the coarse stride: insert the aligned coordinates under that tensor stride
    m = C.CoordinateManager(3)
    key, _ = m.insert_and_map(torch.from_numpy(coarse).cuda(), [stride] * 3, "")
    f = torch.from_numpy(feats).cuda().requires_grad_(True)
    x = C.SparseTensor(f, key, m)
    layer = C.RiemannGenerativeConvolutionTranspose(5, 4, kernel_size=kernel, stride=stride, dimension=3)
    layer.to("cuda")
    y = layer(x)
    assert y.tensor_stride == [1, 1, 1]
    (y.F * y.F).sum().mul(0.5).backward()
    # oracle: out = in + off on the output stride (1), deduplicated in first-occurrence order over (row, offset)
    off = O.region_offsets(O.HYPER_CUBE, [kernel] * 3, [1] * 3, [1] * 3)
    expanded = (coarse[:, None, :].astype(np.int64)
                + np.concatenate([np.zeros((len(off), 1), np.int64), off.astype(np.int64)], 1)[None]).reshape(-1, 4)
    expanded = expanded.astype(np.int32)
    generated = expanded[O.insert_and_map(expanded)[0]]
    assert (y.C.cpu().numpy() == generated).all()
    kmap = O.conv_kernel_map(coarse, generated, off, transposed=True)
    w = layer.kernel.detach().cpu().numpy()
    want = O.conv_forward(feats, w, *kmap, len(generated), f64=True)
    assert rel_max(y.F.detach().cpu().numpy(), want) <= 1e-4
    gi, gw = O.conv_backward(feats, want.astype(np.float32), w, *kmap, f64=True)
    assert rel_max(f.grad.cpu().numpy(), gi) <= 1e-4
    assert rel_max(layer.kernel.grad.cpu().numpy(), gw) <= 1e-4
