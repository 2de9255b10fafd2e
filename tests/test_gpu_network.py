"""GPU parity of a small encoder/decoder (the shape of the reference's MinkUNet-style networks,
tests/train.cpp:629-758: stem, 3^3 convolutions with batch norm + ReLU, a 2^3 stride-2 down, a transposed
2^3 up and a skip concatenation) against the same network written with the reference's own convolution
arithmetic on the CPU: per offset index_select -> matmul -> index_add_ (engine/nn/conv.cpp:47-64) over the
oracle's kernel maps, torch batch norm, fp64. Values and every parameter gradient, fp32 bar 1e-4."""
import numpy as np
import pytest
import torch

from tests.parity import OracleBackend

pytestmark = pytest.mark.gpu

C_IN, C1, C2, C_OUT = 4, 8, 16, 5


def _cpu_conv(feats, weight, kmap, n_out):
    """The reference's evaluate_sparse_convolution on CPU tensors (autograd through torch ops)."""
    ptr, in_idx, out_idx = kmap
    out = torch.zeros(n_out, weight.size(2), dtype=feats.dtype)
    for k in range(weight.size(0)):
        a, b = int(ptr[k]), int(ptr[k + 1])
        if a == b:
            continue
        ii = torch.from_numpy(np.asarray(in_idx[a:b], np.int64))
        oi = torch.from_numpy(np.asarray(out_idx[a:b], np.int64))
        out = out.index_add(0, oi, feats.index_select(0, ii) @ weight[k])
    return out


def _bn_relu(x, gamma, beta, relu=True):
    y = torch.nn.functional.batch_norm(x, None, None, gamma, beta, True, 0.1, 1e-5)
    return torch.relu(y) if relu else y


def test_encoder_decoder_matches_cpu_reference_arithmetic():
    from riemannengine_b200 import engine as E
    rng = np.random.default_rng(31)
    n = 3000
    coords = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(-7, 8, (n, 3))], 1).astype(np.int32)
    feats = rng.standard_normal((n, C_IN)).astype(np.float32)

    # ---- this library, on the GPU ---------------------------------------------------------------
    torch.manual_seed(5)
    stem = E.RiemannConvolution(C_IN, C1, kernel_size=3, dimension=3).cuda()
    block1 = E.RiemannConvolution(C1, C1, kernel_size=3, dimension=3).cuda()
    down = E.RiemannConvolution(C1, C2, kernel_size=2, stride=2, dimension=3).cuda()
    block2 = E.RiemannConvolution(C2, C2, kernel_size=3, dimension=3).cuda()
    up = E.RiemannConvolutionTranspose(C2, C1, kernel_size=2, stride=2, dimension=3).cuda()
    head = E.RiemannConvolution(2 * C1, C_OUT, kernel_size=3, bias=True, dimension=3).cuda()
    convs = [stem, block1, down, block2, up, head]
    bns = [torch.nn.BatchNorm1d(c).cuda() for c in (C1, C1, C2, C2, C1)]
    with torch.no_grad():
        for bn in bns:
            bn.weight.uniform_(0.5, 1.5)
            bn.bias.uniform_(-0.3, 0.3)

    f = torch.from_numpy(feats).cuda().requires_grad_(True)
    x = E.SparseTensor(f, torch.from_numpy(coords).cuda())
    s0 = E.fused_conv_bn_relu(x, stem, bns[0])          # conv -> norm (batch statistics) -> ReLU, fused
    s1 = E.fused_conv_bn_relu(s0, block1, bns[1])
    d1 = E.fused_conv_bn_relu(s1, down, bns[2])
    d2 = E.fused_conv_bn_relu(d1, block2, bns[3])
    u1 = E.fused_conv_bn_relu(d2, up, bns[4])
    assert u1.coordinate_map_key == s1.coordinate_map_key and len(d1) < len(s1)
    out = head(E.cat([u1, s1]))
    loss = (out.F * out.F).mean()
    loss.backward()

    # ---- the same network with the reference's arithmetic on the CPU, fp64 ----------------------
    O = OracleBackend()
    mapping, _ = O.insert_and_map(coords)
    c_fine = coords[mapping]
    c_coarse, _ = O.stride_map(c_fine, [2, 2, 2])
    assert (x.C.cpu().numpy() == c_fine).all() and (d1.C.cpu().numpy() == c_coarse).all()
    k_fine = O.conv_kernel_map(c_fine, c_fine, O.region_offsets([3] * 3, [1] * 3, [1] * 3))
    k_down = O.conv_kernel_map(c_fine, c_coarse, O.region_offsets([2] * 3, [1] * 3, [1] * 3))
    k_coarse = O.conv_kernel_map(c_coarse, c_coarse, O.region_offsets([3] * 3, [1] * 3, [2] * 3))
    k_up = O.conv_kernel_map(c_coarse, c_fine, O.region_offsets([2] * 3, [1] * 3, [1] * 3), transposed=True)

    def leaf(t):
        return t.detach().double().cpu().requires_grad_(True)

    W = [leaf(c.kernel) for c in convs]
    G = [leaf(b.weight) for b in bns]
    B = [leaf(b.bias) for b in bns]
    head_bias = leaf(head.bias)
    fr = torch.from_numpy(feats[mapping]).double().requires_grad_(True)
    nf, nc = len(c_fine), len(c_coarse)
    r0 = _bn_relu(_cpu_conv(fr, W[0], k_fine, nf), G[0], B[0])
    r1 = _bn_relu(_cpu_conv(r0, W[1], k_fine, nf), G[1], B[1])
    q1 = _bn_relu(_cpu_conv(r1, W[2], k_down, nc), G[2], B[2])
    q2 = _bn_relu(_cpu_conv(q1, W[3], k_coarse, nc), G[3], B[3])
    v1 = _bn_relu(_cpu_conv(q2, W[4], k_up, nf), G[4], B[4])
    ref = _cpu_conv(torch.cat([v1, r1], 1), W[5], k_fine, nf) + head_bias
    ref_loss = (ref * ref).mean()
    ref_loss.backward()

    def rel(a, b):
        a, b = a.detach().double().cpu(), b.detach().double()
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))

    assert rel(out.F, ref) <= 1e-4
    assert abs(float(loss) - float(ref_loss)) / float(ref_loss) <= 1e-4
    g_raw = torch.zeros(n, C_IN, dtype=torch.float64)
    g_raw[torch.from_numpy(mapping)] = fr.grad
    assert rel(f.grad, g_raw) <= 1e-4
    for conv, w in zip(convs, W):
        assert rel(conv.kernel.grad, w.grad) <= 1e-4
    for bn, g, b in zip(bns, G, B):
        assert rel(bn.weight.grad, g.grad) <= 1e-4 and rel(bn.bias.grad, b.grad) <= 1e-4
    assert rel(head.bias.grad, head_bias.grad) <= 1e-4


def test_cpp_host_network_on_a_whole_room_matches_cpu_reference_arithmetic():
    """The same encoder/decoder at the size of one benchmark sample (a whole 150 K-voxel room) through the C++
    host layer as a user of the reference writes it - separate convolution, RiemannBatchNorm (training mode:
    the streaming batch-norm kernels) and RiemannReLU modules, riemann::cat for the skip - against the
    reference's arithmetic on the CPU in fp64. fp32, bar 1e-4 on the output and on every gradient."""
    from riemannengine_b200 import cpp, synthetic
    C = cpp.load()
    pts = synthetic.indoor_scene(5000, 150_000)
    coords = np.concatenate([np.zeros((len(pts), 1), np.int32), pts], 1)
    n = len(coords)
    feats = synthetic.features(5001, n, C_IN)

    def conv(ci, co, k, s, transpose=False, bias=False):
        cls = C.RiemannConvolutionTranspose if transpose else C.RiemannConvolution
        layer = cls(ci, co, kernel_size=k, stride=s, bias=bias, dimension=3)
        layer.to("cuda")
        return layer

    torch.manual_seed(6)
    convs = [conv(C_IN, C1, 3, 1), conv(C1, C1, 3, 1), conv(C1, C2, 2, 2), conv(C2, C2, 3, 1),
             conv(C2, C1, 2, 2, transpose=True), conv(2 * C1, C_OUT, 3, 1, bias=True)]
    bns = []
    for c in (C1, C1, C2, C2, C1):
        bn = C.RiemannBatchNorm(c)
        bn.to("cuda")
        bn.train(True)
        with torch.no_grad():
            bn.weight.uniform_(0.5, 1.5)
            bn.bias.uniform_(-0.3, 0.3)
        bns.append(bn)
    relu = C.RiemannReLU()
    f = torch.from_numpy(feats).cuda().requires_grad_(True)
    x = C.SparseTensor(f, torch.from_numpy(coords).cuda())
    s0 = relu(bns[0](convs[0](x)))
    s1 = relu(bns[1](convs[1](s0)))
    d1 = relu(bns[2](convs[2](s1)))
    d2 = relu(bns[3](convs[3](d1)))
    u1 = relu(bns[4](convs[4](d2)))
    out = convs[5](C.cat([u1, s1]))
    loss = (out.F * out.F).mean()
    loss.backward()

    O = OracleBackend()
    k_fine = O.conv_kernel_map(coords, coords, O.region_offsets([3] * 3, [1] * 3, [1] * 3))
    c_coarse, _ = O.stride_map(coords, [2, 2, 2])
    assert (d1.C.cpu().numpy() == c_coarse).all()
    k_down = O.conv_kernel_map(coords, c_coarse, O.region_offsets([2] * 3, [1] * 3, [1] * 3))
    k_coarse = O.conv_kernel_map(c_coarse, c_coarse, O.region_offsets([3] * 3, [1] * 3, [2] * 3))
    k_up = O.conv_kernel_map(c_coarse, coords, O.region_offsets([2] * 3, [1] * 3, [1] * 3), transposed=True)

    def leaf(t):
        return t.detach().double().cpu().requires_grad_(True)

    W = [leaf(c.kernel) for c in convs]
    G = [leaf(b.weight) for b in bns]
    B = [leaf(b.bias) for b in bns]
    head_bias = leaf(convs[5].bias)
    fr = torch.from_numpy(feats).double().requires_grad_(True)
    nc = len(c_coarse)
    r0 = _bn_relu(_cpu_conv(fr, W[0], k_fine, n), G[0], B[0])
    r1 = _bn_relu(_cpu_conv(r0, W[1], k_fine, n), G[1], B[1])
    q1 = _bn_relu(_cpu_conv(r1, W[2], k_down, nc), G[2], B[2])
    q2 = _bn_relu(_cpu_conv(q1, W[3], k_coarse, nc), G[3], B[3])
    v1 = _bn_relu(_cpu_conv(q2, W[4], k_up, n), G[4], B[4])
    ref = _cpu_conv(torch.cat([v1, r1], 1), W[5], k_fine, n) + head_bias
    ref_loss = (ref * ref).mean()
    ref_loss.backward()

    def rel(a, b):
        a, b = a.detach().double().cpu(), b.detach().double()
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))

    assert rel(out.F, ref) <= 1e-4
    assert abs(float(loss) - float(ref_loss)) / float(ref_loss) <= 1e-4
    assert rel(f.grad, fr.grad) <= 1e-4
    for layer, w in zip(convs, W):
        assert rel(layer.kernel.grad, w.grad) <= 1e-4
    for bn, g, b in zip(bns, G, B):
        assert rel(bn.weight.grad, g.grad) <= 1e-4 and rel(bn.bias.grad, b.grad) <= 1e-4
    assert rel(convs[5].bias.grad, head_bias.grad) <= 1e-4
