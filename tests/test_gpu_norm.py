"""GPU tests of the batch-normalisation pieces beside the convolution: channel statistics out of the
convolution epilogue, the one-pass affine + ReLU, and the training-mode fused conv -> norm -> ReLU
against torch's BatchNorm1d (what the reference runs, engine/nn/normalization.hpp:11-34)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cloud(n, seed=1, lo=-9, hi=9):
    rng = np.random.default_rng(seed)
    c = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(lo, hi + 1, (n, 3))], 1).astype(np.int32)
    return np.unique(c, axis=0)


@pytest.mark.parametrize("dtype,c_in,c_out", [(torch.bfloat16, 64, 64), (torch.bfloat16, 32, 128),
                                              (torch.bfloat16, 24, 40), (torch.float32, 16, 24)])
def test_conv_forward_stats_equal_a_pass_over_the_output(dtype, c_in, c_out):
    """Statistics from the epilogue (tensor-core shapes) or the fallback pass == sums over the stored output;
    the output itself is bit-identical to rmn_conv_forward_fused."""
    from riemannengine_b200 import ops
    coords = torch.from_numpy(_cloud(9000)).cuda()
    t = ops.table_build(coords)
    nbr = ops.kmap_build(t, t.coords, ops.region_offsets(0, [3] * 3, [1] * 3, [1] * 3), self_map=True).nbr
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(t.n_unique, c_in, device="cuda", generator=g).to(dtype)
    w = (torch.randn(27, c_in, c_out, device="cuda", generator=g) * 0.1).to(dtype)
    shift = torch.randn(c_out, device="cuda", generator=g)
    y0 = ops.conv_forward(x, w, nbr, shift=shift)
    y1, stats = ops.conv_forward_stats(x, w, nbr, shift=shift)
    assert torch.equal(y0, y1)
    ref = torch.stack([y0.double().sum(0), (y0.double() ** 2).sum(0)])
    assert float((stats - ref).abs().max() / ref.abs().max()) < 1e-6
    assert float((ops.channel_stats(y0) - ref).abs().max() / ref.abs().max()) < 1e-6


def test_conv_forward_stats_at_benchmark_size():
    from riemannengine_b200 import ops, synthetic
    coords = torch.from_numpy(np.ascontiguousarray(synthetic.indoor_batch(8, 150_000), np.int32)).cuda()
    t = ops.table_build(coords)
    nbr = ops.kmap_build(t, t.coords, ops.region_offsets(0, [3] * 3, [1] * 3, [1] * 3), self_map=True).nbr
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(t.n_unique, 64, device="cuda", generator=g).bfloat16()
    w = (torch.randn(27, 64, 64, device="cuda", generator=g) * 0.05).bfloat16()
    y, stats = ops.conv_forward_stats(x, w, nbr)
    assert torch.equal(y, ops.conv_forward(x, w, nbr))
    ref = torch.stack([y.double().sum(0), (y.double() ** 2).sum(0)])
    assert float((stats[1] - ref[1]).abs().max() / ref[1].abs().max()) < 1e-6
    assert float((stats[0] - ref[0]).abs().max() / ref[1].sqrt().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_affine_act(dtype):
    from riemannengine_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(6)
    for c in (64, 24):
        x = torch.randn(5000, c, device="cuda", generator=g).to(dtype)
        sc, sh = torch.randn(c, device="cuda", generator=g), torch.randn(c, device="cuda", generator=g)
        ref = torch.relu(x.float() * sc + sh).to(dtype)
        assert torch.equal(ops.affine_act(x, sc, sh, relu=True), ref)
        assert torch.equal(ops.affine_act(x, None, sh), (x.float() + sh).to(dtype))


@pytest.mark.parametrize("bias", [False, True])
def test_fused_training_conv_bn_relu_matches_torch_batchnorm(bias):
    """fp32: values, all gradients and running statistics equal conv -> torch BatchNorm1d (training) -> ReLU
    within the fp32 bar (1e-4 relative)."""
    from riemannengine_b200 import engine as E
    coords = torch.from_numpy(_cloud(4000, seed=8, lo=-6, hi=6)).cuda()
    g = torch.Generator(device="cuda").manual_seed(9)
    feats = torch.randn(coords.size(0), 8, device="cuda", generator=g)
    conv = E.RiemannConvolution(8, 12, kernel_size=3, bias=bias, dimension=3).cuda()
    bn_a, bn_b = torch.nn.BatchNorm1d(12).cuda(), torch.nn.BatchNorm1d(12).cuda()
    with torch.no_grad():
        bn_a.weight.uniform_(0.5, 1.5)
        bn_a.bias.uniform_(-0.5, 0.5)
        bn_b.load_state_dict(bn_a.state_dict())
    gy = torch.randn(coords.size(0), 12, device="cuda", generator=g)

    def run(fused):
        f = feats.clone().requires_grad_(True)
        conv.zero_grad()
        x = E.SparseTensor(f, coords)
        if fused:
            y = E.fused_conv_bn_relu(x, conv, bn_a, relu=True).F
            bn = bn_a
        else:
            y = torch.relu(bn_b(conv(x).F))
            bn = bn_b
        bn.zero_grad()
        (y * gy).sum().backward()
        grads = [f.grad, conv.kernel.grad.clone(), bn.weight.grad.clone(), bn.bias.grad.clone()]
        if bias:
            grads.append(conv.bias.grad.clone())
        return y.detach(), grads, bn.running_mean.clone(), bn.running_var.clone()

    ya, ga, rma, rva = run(True)
    yb, gb, rmb, rvb = run(False)
    rel = lambda a, b: float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))  # noqa: E731
    assert rel(ya, yb) <= 1e-4
    for a, b in zip(ga[:4], gb[:4]):
        assert rel(a, b) <= 1e-4
    assert rel(rma, rmb) <= 1e-5 and rel(rva, rvb) <= 1e-5
    assert int(bn_a.num_batches_tracked) == 1


def test_fused_training_bf16_close_to_fp32():
    """bf16 tensor-core path with epilogue statistics against the fp32 path (bf16 bar: 1e-2 relative L2)."""
    from riemannengine_b200 import engine as E
    coords = torch.from_numpy(_cloud(20000, seed=11, lo=-12, hi=12)).cuda()
    g = torch.Generator(device="cuda").manual_seed(12)
    feats = torch.randn(coords.size(0), 64, device="cuda", generator=g)
    conv = E.RiemannConvolution(64, 64, kernel_size=3, dimension=3).cuda()
    bn = torch.nn.BatchNorm1d(64).cuda()
    y32 = E.fused_conv_bn_relu(E.SparseTensor(feats, coords), conv, bn).F
    conv16, bn16 = E.RiemannConvolution(64, 64, kernel_size=3, dimension=3).cuda().to(torch.bfloat16), \
        torch.nn.BatchNorm1d(64).cuda()
    with torch.no_grad():
        conv16.kernel.copy_(conv.kernel.to(torch.bfloat16))
    y16 = E.fused_conv_bn_relu(E.SparseTensor(feats.bfloat16(), coords), conv16, bn16).F
    err = float((y16.float() - y32).norm() / y32.norm())
    assert err <= 1e-2, err
    assert float((bn16.running_mean - bn.running_mean).abs().max()) < 1e-2


@pytest.mark.parametrize("dtype,channels,rows", [(torch.float32, 32, 20000), (torch.bfloat16, 32, 50000),
                                                 (torch.bfloat16, 64, 7001), (torch.bfloat16, 256, 3000),
                                                 (torch.float32, 8, 999), (torch.bfloat16, 24, 5000)])
def test_cpp_batch_norm_training_matches_torch(dtype, channels, rows):
    """RiemannBatchNorm of the C++ host layer in training mode (streaming kernels: rmn_channel_dot_stats,
    rmn_bn_forward_coeffs, rmn_affine_act; backward rmn_bn_backward_coeffs, rmn_affine2) against
    torch.nn.BatchNorm1d, which is what the reference runs (engine/nn/normalization.hpp:11-34): output, input
    gradient, parameter gradients and running statistics. 24 bf16 channels have no streaming kernel and take
    torch's path."""
    from riemannengine_b200 import cpp
    C = cpp.load()
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(rows, channels, device="cuda", generator=g) * 2 + 0.5).to(dtype)
    gy = torch.randn(rows, channels, device="cuda", generator=g).to(dtype)
    coords = torch.cat([torch.zeros(rows, 1, dtype=torch.int32), torch.arange(rows, dtype=torch.int32).view(-1, 1),
                        torch.zeros(rows, 2, dtype=torch.int32)], 1).cuda()
    ref = torch.nn.BatchNorm1d(channels).cuda()
    with torch.no_grad():
        ref.weight.uniform_(0.5, 1.5)
        ref.bias.uniform_(-0.5, 0.5)
    bn = C.RiemannBatchNorm(channels)
    bn.to("cuda")
    with torch.no_grad():
        bn.weight.copy_(ref.weight)
        bn.bias.copy_(ref.bias)
    bn.to(dtype)
    bn.train(True)
    xr = x.float().clone().requires_grad_(True)       # torch reference in fp32 on the same (rounded) inputs
    yr = ref(xr)
    yr.backward(gy.float())
    xs = x.clone().requires_grad_(True)
    m = C.CoordinateManager(3)
    key, _ = m.insert_and_map(coords, [1, 1, 1], "")
    y = bn(C.SparseTensor(xs, key, m))
    y.F.backward(gy)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())  # noqa: E731
    assert rel(y.F, yr) <= tol
    assert rel(xs.grad, xr.grad) <= tol
    assert rel(bn.weight.grad, ref.weight.grad) <= tol and rel(bn.bias.grad, ref.bias.grad) <= tol
    assert rel(bn.running_mean, ref.running_mean) <= tol and rel(bn.running_var, ref.running_var) <= tol
