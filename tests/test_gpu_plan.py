"""Convolution plans: structure of the plan buffer and bit-identity of the planned tensor-core
convolutions with the plain ones (same kernels, same accumulation order per output row; the plan only
changes which rows share a tile and lets (tile, offset) pairs without neighbours be skipped)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layout(n_dst, K):
    """Python statement of the plan layout (csrc/rmn_plan.cuh)."""
    up = lambda v: (v + 255) & ~255  # noqa: E731
    n_pos = (n_dst + 511) // 512 * 512
    n_tiles = n_pos // 128
    words = (K + 31) // 32
    perm = 256
    tile_mask = perm + up(n_pos * 4)
    nbr_p = tile_mask + up(n_tiles * words * 4)
    return n_pos, n_tiles, words, perm, tile_mask, nbr_p, nbr_p + up(K * n_pos * 4)


def _cloud_table(seed, n, D, lo, hi, ksize, stride=1):
    from riemannengine_b200 import capi, ops
    rng = np.random.default_rng(seed)
    c = np.concatenate([rng.integers(0, 2, (n, 1)), rng.integers(lo, hi + 1, (n, D))], 1).astype(np.int32)
    table = ops.table_build(torch.from_numpy(c).cuda())
    offsets = ops.region_offsets(capi.HYPER_CUBE, [ksize] * D, [1] * D, [1] * D)
    query = table.coords
    if stride > 1:
        query = ops.table_build(ops.coords_stride(table.coords, [stride] * D)).coords
    res = ops.kmap_build(table, query, offsets)
    return table, res.nbr, offsets


@pytest.mark.parametrize("n,D,ksize,stride", [(20000, 3, 3, 1), (1, 3, 3, 1), (129, 3, 3, 1), (30000, 3, 2, 2),
                                              (90000, 3, 3, 1),
                                              (700, 2, 5, 1), (3000, 4, 2, 1)])
def test_plan_buffer_is_a_stable_class_sort_of_the_table(n, D, ksize, stride):
    from riemannengine_b200 import capi, ops
    table, nbr, offsets = _cloud_table(7 + n, n, D, -12 if n < 50000 else -30, 12 if n < 50000 else 30, ksize, stride)
    K, n_dst = int(nbr.size(0)), int(nbr.size(1))
    plan = ops.conv_plan_build(nbr, offsets)
    assert plan is not None and plan.numel() == capi.lib().rmn_conv_plan_bytes(n_dst, K)
    n_pos, n_tiles, words, o_perm, o_mask, o_nbr, total = _layout(n_dst, K)
    assert total == plan.numel()
    raw = plan.cpu().numpy()
    perm = raw[o_perm:o_perm + 4 * n_pos].view(np.int32)
    tmask = raw[o_mask:o_mask + 4 * n_tiles * words].view(np.uint32).reshape(n_tiles, words)
    nbr_p = raw[o_nbr:o_nbr + 4 * K * n_pos].view(np.int32).reshape(K, n_pos)
    host = nbr.cpu().numpy()
    assert sorted(perm[:n_dst].tolist()) == list(range(n_dst)) and (perm[n_dst:] == -1).all()
    assert (nbr_p[:, :n_dst] == host[:, perm[:n_dst]]).all() and (nbr_p[:, n_dst:] == -1).all()
    # class key: one bit per (axis, sign) on which the row has a neighbour; inside every chunk of 32 768 public
    # rows the positions are sorted by it, stably
    hit = host >= 0
    key = np.zeros(n_dst, np.int64)
    for a in range(min(D, 4)):
        for bit, sel in ((2 * a, offsets[:, a] < 0), (2 * a + 1, offsets[:, a] > 0)):
            if sel.any():
                key |= hit[sel].any(0).astype(np.int64) << bit
    want = np.lexsort((np.arange(n_dst), key, np.arange(n_dst) // 32768))
    assert (perm[:n_dst] == want).all()
    # tile masks: bit k set exactly when some row of the tile has a neighbour at offset k
    hp = nbr_p >= 0
    for k in range(K):
        any_hit = hp[k].reshape(n_tiles, 128).any(1)
        assert (((tmask[:, k // 32] >> (k % 32)) & 1).astype(bool) == any_hit).all(), k


@pytest.mark.parametrize("c_in,c_out", [(32, 32), (64, 64), (64, 128), (128, 128), (32, 64), (128, 64), (256, 128)])
def test_planned_forward_and_input_gradient_are_bit_identical(c_in, c_out):
    from riemannengine_b200 import ops
    table, nbr, offsets = _cloud_table(50 + c_in + c_out, 40000, 3, -25, 25, 3)
    n = int(nbr.size(1))
    g = torch.Generator(device="cuda").manual_seed(1)
    feats = torch.randn(n, c_in, device="cuda", generator=g).bfloat16()
    w = (torch.randn(27, c_in, c_out, device="cuda", generator=g) / (27 * c_in) ** 0.5).bfloat16()
    plan = ops.conv_plan_build(nbr, offsets)
    plain = ops.conv_forward(feats, w, nbr)
    planned = ops.conv_forward(feats, w, nbr, plan=plan)
    assert torch.equal(plain, planned)
    shift = torch.randn(c_out, device="cuda", generator=g)
    scale = torch.rand(c_out, device="cuda", generator=g) + 0.5
    assert torch.equal(ops.conv_forward(feats, w, nbr, scale, shift, True),
                       ops.conv_forward(feats, w, nbr, scale, shift, True, plan=plan))
    # input gradient of a stride-1 self map: the same table with the kernel flipped
    gy = torch.randn(n, c_out, device="cuda", generator=g).bfloat16()
    assert torch.equal(ops.conv_backward_input(gy, w.flip(0), nbr), ops.conv_backward_input(gy, w.flip(0), nbr, plan=plan))
    # statistics epilogue: same stored values; the sums differ only in the order rows are added
    y0, s0 = ops.conv_forward_stats(feats, w, nbr)
    y1, s1 = ops.conv_forward_stats(feats, w, nbr, plan=plan)
    assert torch.equal(y0, y1) and torch.allclose(s0, s1, rtol=1e-5, atol=1e-3)
    from riemannengine_b200 import capi
    assert capi.lib().rmn_device_status(None) == capi.OK


def test_planned_strided_4d_and_2d_tables_are_bit_identical():
    from riemannengine_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(2)
    for n, D, ksize, stride, c_in, c_out in ((60000, 3, 2, 2, 64, 128), (15000, 4, 2, 1, 32, 32), (20000, 2, 5, 1, 32, 64)):
        table, nbr, offsets = _cloud_table(90 + D + ksize, n, D, -10 if D == 4 else -40, 10 if D == 4 else 40, ksize, stride)
        K, n_dst = int(nbr.size(0)), int(nbr.size(1))
        feats = torch.randn(table.n_unique, c_in, device="cuda", generator=g).bfloat16()
        w = (torch.randn(K, c_in, c_out, device="cuda", generator=g) / (K * c_in) ** 0.5).bfloat16()
        plan = ops.conv_plan_build(nbr, offsets)
        assert torch.equal(ops.conv_forward(feats, w, nbr), ops.conv_forward(feats, w, nbr, plan=plan))
        # the input gradient of a strided map runs over the inverse table, which gets a plan of its own
        nbr_t = ops.kmap_transpose(nbr, table.n_unique)
        plan_t = ops.conv_plan_build(nbr_t, -offsets)
        gy = torch.randn(n_dst, c_out, device="cuda", generator=g).bfloat16()
        assert torch.equal(ops.conv_backward_input(gy, w, nbr_t), ops.conv_backward_input(gy, w, nbr_t, plan=plan_t))


def test_planned_rows_without_any_neighbour_store_the_epilogue_of_zero():
    """Query rows far from the table have no neighbour at any offset: whole tiles are skipped at every
    offset and must still store act(0 * scale + shift)."""
    from riemannengine_b200 import capi, ops
    rng = np.random.default_rng(5)
    c = np.concatenate([np.zeros((3000, 1)), rng.integers(-8, 9, (3000, 3))], 1).astype(np.int32)
    table = ops.table_build(torch.from_numpy(c).cuda())
    far = table.coords.clone()
    far[:, 1] += 1000
    query = torch.cat([table.coords, far, far + 5]).contiguous()
    offsets = ops.region_offsets(capi.HYPER_CUBE, [3] * 3, [1] * 3, [1] * 3)
    nbr = ops.kmap_build(table, query, offsets).nbr
    plan = ops.conv_plan_build(nbr, offsets)
    g = torch.Generator(device="cuda").manual_seed(3)
    feats = torch.randn(table.n_unique, 64, device="cuda", generator=g).bfloat16()
    w = (torch.randn(27, 64, 64, device="cuda", generator=g) / 40).bfloat16()
    shift = torch.randn(64, device="cuda", generator=g)
    a = ops.conv_forward(feats, w, nbr, None, shift, False)
    b = ops.conv_forward(feats, w, nbr, None, shift, False, plan=plan)
    assert torch.equal(a, b)
    assert torch.equal(b[table.n_unique:].float(), shift.bfloat16().float().expand(2 * table.n_unique, 64))


def test_plan_falls_back_for_fp32_and_large_kernels():
    from riemannengine_b200 import capi, ops
    table, nbr, offsets = _cloud_table(3, 5000, 3, -6, 6, 3)
    plan = ops.conv_plan_build(nbr, offsets)
    g = torch.Generator(device="cuda").manual_seed(4)
    feats = torch.randn(table.n_unique, 16, device="cuda", generator=g)
    w = torch.randn(27, 16, 24, device="cuda", generator=g) / 20
    assert torch.equal(ops.conv_forward(feats, w, nbr), ops.conv_forward(feats, w, nbr, plan=plan))  # SIMT, unplanned
    assert capi.lib().rmn_conv_plan_bytes(1000, 64) == 0       # more than 32 offsets: no plan
    assert capi.lib().rmn_conv_plan_bytes(1000, 32) > 0


def _host_network(make_tensor, make_conv, coords, feats, seed_weights):
    """Three bf16 layers that share kernel maps: 3^3 stride 1 twice on the input map, a 2^3 stride-2 down and
    the transposed 2^3 back up; returns the output features and every gradient."""
    f = feats.clone().requires_grad_(True)
    x = make_tensor(f, coords)
    layers = [make_conv(32, 32, 3, 1, False), make_conv(32, 32, 3, 1, False), make_conv(32, 64, 2, 2, False),
              make_conv(64, 32, 2, 2, True)]
    g = torch.Generator(device="cuda").manual_seed(seed_weights)
    with torch.no_grad():
        for layer in layers:
            layer.kernel.copy_((torch.randn(layer.kernel.shape, device="cuda", generator=g) * 0.05).to(layer.kernel.dtype))
    y = x
    for layer in layers:
        y = layer(y)
    (y.F.float() ** 2).sum().backward()
    return [y.F.detach(), f.grad] + [layer.kernel.grad for layer in layers]


@pytest.mark.parametrize("host", ["cpp", "python"])
def test_hosts_plan_shared_maps_and_keep_results(host):
    """With the plan policy on 'always' / 'automatic' the layers run planned kernels on their shared maps;
    the outputs and input gradients are bit-identical to the unplanned run (weight gradients do not use plans)."""
    from riemannengine_b200 import capi, engine as E
    rng = np.random.default_rng(9)
    c = np.concatenate([rng.integers(0, 2, (40000, 1)), rng.integers(-30, 31, (40000, 3))], 1).astype(np.int32)
    coords = torch.from_numpy(c).cuda()
    feats = torch.randn(len(c), 32, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).bfloat16()
    if host == "cpp":
        from riemannengine_b200 import cpp
        C = cpp.load()

        def make_conv(ci, co, k, s, transpose):
            cls = C.RiemannConvolutionTranspose if transpose else C.RiemannConvolution
            layer = cls(ci, co, kernel_size=k, stride=s, dimension=3)
            layer.to("cuda")
            layer.to(torch.bfloat16)
            return layer

        make_tensor, set_policy = C.SparseTensor, C.set_convolution_plan_policy
    else:
        def make_conv(ci, co, k, s, transpose):
            cls = E.RiemannConvolutionTranspose if transpose else E.RiemannConvolution
            return cls(ci, co, kernel_size=k, stride=s, dimension=3).cuda().bfloat16()

        def set_policy(p):
            E.KernelMap.plan_policy = p

        make_tensor = E.SparseTensor
    results = {}
    try:
        for policy in (2, 1, 0):   # never, always, automatic
            set_policy(policy)
            results[policy] = _host_network(make_tensor, make_conv, coords, feats, 17)
    finally:
        set_policy(0)
    for policy in (1, 0):
        for a, b in zip(results[policy], results[2]):
            assert torch.equal(a, b)
    assert capi.lib().rmn_device_status(None) == capi.OK
