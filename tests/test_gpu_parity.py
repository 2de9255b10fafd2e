"""GPU parity tests: the CUDA library, called through its C ABI, against the CPU oracle
and against the golden fixtures produced by the reference's own CPU build.

Bars: coordinate maps and kernel maps bit-exact (kernel maps as per-offset sorted (in, out)
pair sets); fp32 features within 1e-4 relative (max-abs error over max-abs value); bf16
features within 1e-2 relative L2 of the fp32/fp64 oracle.
"""
import numpy as np
import pytest
import torch

from tests import parity
from tests.parity import OracleBackend, rel_l2, rel_max

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 1e-2


@pytest.fixture(scope="module")
def gpu():
    from tests.gpu_backend import GpuBackend
    return GpuBackend


@pytest.mark.parametrize("name", parity.GOLDEN_CASES)
def test_golden_fp32(gpu, name):
    gold = parity.load_golden(name)
    D, kernel, stride, dilation = gold["spec"].tolist()
    res = parity.run_pipeline(gpu(torch.float32), gold["in_coords_raw"], gold["in_feats_raw"], gold["weights"],
                              D, kernel, stride, dilation, gold.get("weights2"))
    parity.check_against_reference(res, gold, tol=FP32_TOL, metric=rel_max)


@pytest.mark.parametrize("name", parity.GOLDEN_CASES)
def test_golden_bf16(gpu, name):
    gold = parity.load_golden(name)
    D, kernel, stride, dilation = gold["spec"].tolist()
    # grads compound two bf16 roundings (activations and gradients), so the bar is on each
    # tensor separately against the fp32 reference values.
    res = parity.run_pipeline(gpu(torch.bfloat16), gold["in_coords_raw"], gold["in_feats_raw"], gold["weights"],
                              D, kernel, stride, dilation, gold.get("weights2"))
    parity.check_against_reference(res, gold, tol=3 * BF16_TOL, metric=rel_l2)
    g = {k[4:]: v for k, v in gold.items() if k.startswith("ref_")}
    perm = parity.row_permutation(res["out_coords"], g["out_coords"])
    assert rel_l2(res["out_feats"], g["out_feats"][perm]) <= BF16_TOL


def _random_cloud(seed, n, D, lo, hi, batches, dup_frac=0.1):
    rng = np.random.default_rng(seed)
    c = np.concatenate([rng.integers(0, batches, (n, 1)), rng.integers(lo, hi + 1, (n, D))], 1).astype(np.int32)
    nd = int(n * dup_frac)
    if nd:
        c[rng.integers(0, n, nd)] = c[rng.integers(0, n, nd)]
    return c


@pytest.mark.parametrize("seed,n,D,lo,hi,batches", [
    (1, 5000, 3, -20, 20, 3), (2, 20000, 3, -100000, 100000, 2), (3, 3000, 2, -30, 30, 1),
    (4, 4000, 4, -5, 5, 2), (5, 1, 3, 0, 0, 1), (6, 257, 3, -2, 2, 1), (7, 4096, 1, -3000, 3000, 4),
    (8, 6000, 5, -3, 3, 1), (9, 3000, 7, -2, 2, 1),
])
def test_insert_and_map_matches_oracle(gpu, seed, n, D, lo, hi, batches):
    c = _random_cloud(seed, n, D, lo, hi, batches)
    m0, i0 = OracleBackend().insert_and_map(c)
    m1, i1 = gpu().insert_and_map(c)
    assert (m0 == m1).all() and (i0 == i1).all()


def test_insert_empty_and_lookup(gpu):
    from riemannengine_b200 import ops
    from tests.gpu_backend import dev_coords
    t = ops.table_build(dev_coords(np.zeros((0, 4), np.int32)))
    assert t.n_unique == 0 and t.mapping.numel() == 0
    rows = ops.table_find(t, dev_coords(np.array([[0, 1, 2, 3]], np.int32)))
    assert rows.tolist() == [-1]
    c = _random_cloud(11, 3000, 3, -9, 9, 2)
    t = ops.table_build(dev_coords(c))
    found = ops.table_find(t, dev_coords(c)).cpu().numpy()
    assert (found == OracleBackend().insert_and_map(c)[1]).all()
    far = c.copy()
    far[:, 1] += 1000  # outside the bounding box -> rejected before probing
    assert (ops.table_find(t, dev_coords(far)).cpu().numpy() == -1).all()


def test_all_rows_identical(gpu):
    c = np.tile(np.array([[1, -5, 7, 9]], np.int32), (5000, 1))
    m, inv = gpu().insert_and_map(c)
    assert m.tolist() == [0] and (inv == 0).all()


def test_range_error_is_reported(gpu):
    from riemannengine_b200 import capi
    c = np.array([[0, -2**31, -2**31, -2**31], [0, 2**31 - 1, 2**31 - 1, 2**31 - 1]], np.int32)
    with pytest.raises(capi.RmnError) as e:
        gpu().insert_and_map(c)
    assert e.value.status == capi.ERR_RANGE


@pytest.mark.parametrize("stride", [[2, 2, 2], [2, 1, 4], [3, 3, 3]])
def test_stride_map_matches_oracle(gpu, stride):
    c = _random_cloud(21, 8000, 3, -50, 50, 2, dup_frac=0)
    c = c[OracleBackend().insert_and_map(c)[0]]
    a0, i0 = OracleBackend().stride_map(c, stride)
    a1, i1 = gpu().stride_map(c, stride)
    assert (a0 == a1).all() and (i0 == i1).all()


@pytest.mark.parametrize("D,ks,dil,transposed", [(3, 3, 1, False), (3, 2, 1, False), (3, 5, 1, False),
                                                 (2, 3, 3, False), (4, 3, 1, False), (3, 3, 2, True)])
def test_kernel_map_matches_oracle(gpu, D, ks, dil, transposed):
    O = OracleBackend()
    c = _random_cloud(31 + D, 6000, D, -8, 8, 2, dup_frac=0)
    c = c[O.insert_and_map(c)[0]]
    off = O.region_offsets([ks] * D, [dil] * D, [1] * D)
    k0 = O.conv_kernel_map(c, c, off, transposed)
    k1 = gpu().conv_kernel_map(c, c, off, transposed)
    parity.assert_kernel_maps_equal(k1, k0)
    if not transposed:
        # device pair lists of the general builder are sorted by output row inside each offset, like
        # the oracle's (a transposed map is built the other way round by the oracle: sorted by input row)
        assert (np.asarray(k1[1]) == k0[1]).all() and (np.asarray(k1[2]) == k0[2]).all()


def test_transposed_map_two_constructions_agree(gpu):
    """Probing the coarse map from the fine rows (this library) and probing the fine map from
    the coarse rows then swapping (the reference) give the same pair sets."""
    from riemannengine_b200 import ops
    from tests.gpu_backend import dev_coords
    O = OracleBackend()
    fine = _random_cloud(41, 7000, 3, -12, 12, 2, dup_frac=0)
    fine = fine[O.insert_and_map(fine)[0]]
    coarse, _ = O.stride_map(fine, [2, 2, 2])
    off = O.region_offsets([2] * 3, [1] * 3, [1] * 3)
    mine = gpu().conv_kernel_map(coarse, fine, off, transposed=True)
    t_fine = ops.table_build(dev_coords(fine))
    res = ops.kmap_build(t_fine, dev_coords(coarse), off)
    ptr, a_fine, q_coarse = res.pairs()
    parity.assert_kernel_maps_equal(mine, (ptr.numpy(), q_coarse.cpu().numpy(), a_fine.cpu().numpy()))
    back = ops.kmap_transpose(res.nbr, len(fine))
    assert (back.cpu() == mine.nbr.cpu()).all()


def _sphere():
    from riemannengine_b200 import synthetic
    return synthetic.sphere_shell()


def test_sphere_shell_constants_and_conv_fp32(gpu):
    """The reference's CPU-runnable configuration: ~100K-voxel sphere shell, 3^3, 32 -> 32, fp32."""
    from riemannengine_b200 import synthetic
    c = _sphere()
    assert len(c) == 101930
    O, G = OracleBackend(f64=True), gpu(torch.float32)
    f = synthetic.features(1000, len(c), 32)
    w = synthetic.conv_weights(1001, 27, 32, 32)
    r0 = parity.run_pipeline(O, c, f, w, 3, 3, 1, 1)
    r1 = parity.run_pipeline(G, c, f, w, 3, 3, 1, 1)
    assert int(r1["kmap_ptr"][-1]) == 1804802
    parity.assert_kernel_maps_equal((r1["kmap_ptr"], r1["kmap_in"], r1["kmap_out"]),
                                    (r0["kmap_ptr"], r0["kmap_in"], r0["kmap_out"]))
    for key in ("out_feats", "grad_feats", "grad_weights"):
        assert rel_max(r1[key], r0[key]) <= FP32_TOL, key


def test_sphere_shell_strided_and_transposed(gpu):
    from riemannengine_b200 import synthetic
    c = _sphere()
    O, G = OracleBackend(f64=True), gpu(torch.float32)
    f = synthetic.features(1002, len(c), 16)
    w1 = synthetic.conv_weights(1003, 8, 16, 24)
    w2 = synthetic.conv_weights(1004, 8, 24, 8, transpose=True)
    r0 = parity.run_pipeline(O, c, f, w1, 3, 2, 2, 1, w2)
    r1 = parity.run_pipeline(G, c, f, w1, 3, 2, 2, 1, w2)
    assert len(r1["out_coords"]) == 22376 and int(r1["kmap_ptr"][-1]) == 101930
    assert int(r1["kmap2_ptr"][-1]) == 101930 and len(r1["kmap2_ptr"]) == 9
    assert (r1["out_coords"] == r0["out_coords"]).all()
    for a, b in (("kmap", "kmap"), ("kmap2", "kmap2")):
        parity.assert_kernel_maps_equal(tuple(r1[a + s] for s in ("_ptr", "_in", "_out")),
                                        tuple(r0[b + s] for s in ("_ptr", "_in", "_out")))
    for key in ("out_feats", "up_feats", "grad_feats", "grad_weights", "grad_weights2"):
        assert rel_max(r1[key], r0[key]) <= FP32_TOL, key


@pytest.mark.parametrize("c_in,c_out", [(64, 64), (32, 64), (4, 32), (64, 128), (16, 16), (128, 64), (128, 256),
                                         (256, 256)])
def test_bf16_conv_against_fp64_oracle(gpu, c_in, c_out):
    from riemannengine_b200 import synthetic
    O, G = OracleBackend(f64=True), gpu(torch.bfloat16)
    c = synthetic.indoor_scene(77, 20000)
    c = np.concatenate([np.zeros((len(c), 1), np.int32), c], 1)
    f = synthetic.features(78, len(c), c_in)
    w = synthetic.conv_weights(79, 27, c_in, c_out)
    # the oracle sees the same bf16-rounded inputs, so the bar measures the kernel, not the rounding
    fb = torch.from_numpy(f).bfloat16().float().numpy()
    wb = torch.from_numpy(w).bfloat16().float().numpy()
    off = O.region_offsets([3] * 3, [1] * 3, [1] * 3)
    k0 = O.conv_kernel_map(c, c, off)
    k1 = G.conv_kernel_map(c, c, off)
    parity.assert_kernel_maps_equal(k1, k0)
    y0 = O.conv_forward(fb, wb, k0, len(c), len(c))
    y1 = G.conv_forward(f, w, k1, len(c), len(c))
    assert rel_l2(y1, y0) <= BF16_TOL
    g = synthetic.features(80, len(c), c_out)
    gb = torch.from_numpy(g).bfloat16().float().numpy()
    gi0, gw0 = O.conv_backward(fb, gb, wb, k0, len(c), len(c))
    gi1, gw1 = G.conv_backward(f, g, w, k1, len(c), len(c))
    assert rel_l2(gi1, gi0) <= BF16_TOL
    assert rel_l2(gw1, gw0) <= BF16_TOL


def test_large_batch_properties(gpu):
    """Full-size headline batch (8 rooms, 1.2M voxels): size-independent properties instead of
    an oracle run — symmetry of the stride-1 map, consistency of every table entry with the
    coordinates, pair lists vs table, transpose involution, linearity of the convolution."""
    from riemannengine_b200 import ops, synthetic
    from tests.gpu_backend import dev_coords
    coords = synthetic.indoor_batch(8, 150_000)
    n = len(coords)
    dc = dev_coords(coords)
    t = ops.table_build(dc)
    assert t.n_unique == n and (t.mapping.cpu() == torch.arange(n)).all()
    off = ops.region_offsets(0, [3] * 3, [1] * 3, [1] * 3)
    res = ops.kmap_build(t, dc, off)
    nbr = res.nbr
    K = 27
    # centre offset is the identity
    assert (nbr[13].cpu() == torch.arange(n, dtype=torch.int32)).all()
    # every hit points at the row holding exactly coords[q] + off[k]
    d_off = torch.from_numpy(off).cuda()
    for k in (0, 5, 13, 26):
        hit = nbr[k] >= 0
        src = dc[nbr[k][hit].long()]
        want = dc[hit].clone()
        want[:, 1:] += d_off[k]
        assert (src == want).all()
    # symmetry: (i -> j at k) <=> (j -> i at K-1-k)
    nbr_t = ops.kmap_transpose(nbr, n)
    assert (nbr_t == nbr.flip(0)).all()
    assert (ops.kmap_transpose(nbr_t, n) == nbr).all()
    ptr, a, q = res.pairs()
    counts = (nbr >= 0).sum(1).cpu()
    assert (ptr[1:] - ptr[:-1] == counts).all()
    k = 7
    sl = slice(int(ptr[k]), int(ptr[k + 1]))
    assert (nbr[k][q[sl].long()] == a[sl]).all() and (q[sl][1:] > q[sl][:-1]).all()
    # self-map builder: same table and pointer; mirrored offsets hold the exchanged lists (sorted by table row)
    res_s = ops.kmap_build(t, dc, off, self_map=True)
    assert torch.equal(res_s.nbr, nbr) and torch.equal(res_s.offset_ptr, res.offset_ptr)
    ptr_s, a_s, q_s = res_s.pairs()
    assert torch.equal(ptr_s, ptr)
    for k in (7, 13, 20, 26):
        sl = slice(int(ptr[k]), int(ptr[k + 1]))
        assert (nbr[k][q_s[sl].long()] == a_s[sl]).all()
        key = a_s[sl] if k > 13 else q_s[sl]
        assert (key[1:] > key[:-1]).all()
    # linearity of the forward pass in the features (fp32)
    g = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randn(K, 16, 16, device="cuda", generator=g) * 0.05
    x1 = torch.randn(n, 16, device="cuda", generator=g)
    x2 = torch.randn(n, 16, device="cuda", generator=g)
    y = ops.conv_forward(2 * x1 + x2, w, nbr)
    y12 = 2 * ops.conv_forward(x1, w, nbr) + ops.conv_forward(x2, w, nbr)
    assert float((y - y12).abs().max() / y.abs().max()) < 1e-5
    # adjointness: <conv(x), g> == <x, conv_backward_input(g)>
    gy = torch.randn(n, 16, device="cuda", generator=g)
    lhs = (ops.conv_forward(x1, w, nbr).double() * gy.double()).sum()
    rhs = (x1.double() * ops.conv_backward_input(gy, w, nbr_t).double()).sum()
    assert abs(float(lhs - rhs)) / abs(float(lhs)) < 1e-5
    # <conv_w(x), g> is linear in w: d/dw matches backward_weight
    dw = ops.conv_backward_weight(x1, gy, nbr)
    assert abs(float((dw.double() * w.double()).sum() - lhs)) / abs(float(lhs)) < 1e-5


@pytest.mark.parametrize("D,ks,dil,n", [(3, 3, 1, 20000), (3, 5, 1, 3000), (2, 3, 2, 4000), (4, 3, 1, 2500), (3, 1, 1, 500)])
def test_self_map_builder_equals_general_builder(gpu, D, ks, dil, n):
    """The half-probe builder for stride-1 self maps gives the same neighbour table, CSR pointer
    and pair lists as the general builder."""
    from riemannengine_b200 import ops
    from tests.gpu_backend import dev_coords
    O = OracleBackend()
    c = _random_cloud(50 + D, n, D, -9, 9, 2, dup_frac=0)
    c = c[O.insert_and_map(c)[0]]
    off = O.region_offsets([ks] * D, [dil] * D, [1] * D)
    assert ops.offsets_point_symmetric(off)
    t = ops.table_build(dev_coords(c))
    a = ops.kmap_build(t, t.coords, off)
    b = ops.kmap_build(t, t.coords, off, self_map=True)
    assert torch.equal(a.nbr, b.nbr)
    assert torch.equal(a.offset_ptr, b.offset_ptr)
    pa, pb = a.pairs(), b.pairs()
    assert torch.equal(pa[0], pb[0])
    # the variant built to run beside a convolution writes the same lists, bit for bit
    for res, want in ((a, pa), (b, pb)):
        bg = res.pairs(background=True)
        assert all(torch.equal(x, y) for x, y in zip(bg, want))
    ptr, K = pa[0].tolist(), len(off)
    # identical lists up to and including the centre offset; above it the self map emits the exchanged
    # lists of the mirror offsets (sorted by table row instead of query row): same pair sets
    lo = ptr[K // 2 + 1]
    assert torch.equal(pa[1][:lo], pb[1][:lo]) and torch.equal(pa[2][:lo], pb[2][:lo])
    for k in range(K // 2 + 1, K):
        sa = torch.stack([pa[1][ptr[k]:ptr[k + 1]], pa[2][ptr[k]:ptr[k + 1]]], 1)
        sb = torch.stack([pb[1][ptr[k]:ptr[k + 1]], pb[2][ptr[k]:ptr[k + 1]]], 1)
        key = lambda t: t[:, 1].long() * (1 << 32) + t[:, 0].long()  # noqa: E731
        assert torch.equal(sa[torch.argsort(key(sa))], sb[torch.argsort(key(sb))])
        mk = K - 1 - k  # and literally the exchanged mirror list
        assert torch.equal(pb[1][ptr[k]:ptr[k + 1]], pb[2][ptr[mk]:ptr[mk + 1]])
        assert torch.equal(pb[2][ptr[k]:ptr[k + 1]], pb[1][ptr[mk]:ptr[mk + 1]])
    assert not ops.offsets_point_symmetric(O.region_offsets([2] * D, [1] * D, [1] * D))


def test_tma_gather4_producers_match_cp_async(gpu, monkeypatch):
    """The optional TMA (tile::gather4) producers of the tensor-core kernel give the same
    output as the default cp.async producers, bit for bit (same MMA order)."""
    from riemannengine_b200 import ops, synthetic
    from tests.gpu_backend import dev_coords
    c = synthetic.indoor_scene(91, 30000)
    c = np.concatenate([np.zeros((len(c), 1), np.int32), c], 1)
    t = ops.table_build(dev_coords(c))
    nbr = ops.kmap_build(t, t.coords, ops.region_offsets(0, [3] * 3, [1] * 3, [1] * 3), self_map=True).nbr
    g = torch.Generator(device="cuda").manual_seed(3)
    for c_in, c_out in ((64, 64), (32, 64), (128, 128)):
        x = torch.randn(len(c), c_in, device="cuda", generator=g).bfloat16()
        w = (torch.randn(27, c_in, c_out, device="cuda", generator=g) * 0.05).bfloat16()
        monkeypatch.delenv("RMN_B200_CONV_TMA", raising=False)
        y0 = ops.conv_forward(x, w, nbr)
        d0 = ops.conv_backward_input(y0, w, ops.kmap_transpose(nbr, len(c)))
        monkeypatch.setenv("RMN_B200_CONV_TMA", "1")
        y1 = ops.conv_forward(x, w, nbr)
        d1 = ops.conv_backward_input(y0, w, ops.kmap_transpose(nbr, len(c)))
        assert torch.equal(y0, y1) and torch.equal(d0, d1)
    monkeypatch.delenv("RMN_B200_CONV_TMA", raising=False)
    assert capi_status_ok()


def capi_status_ok():
    import ctypes
    from riemannengine_b200 import capi
    return capi.lib().rmn_device_status(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == capi.OK


@pytest.mark.parametrize("dups", [False, True])
def test_two_call_table_build_header_is_final_after_the_first_call(gpu, dups):
    """rmn_table_build_begin / _finish: the unique-row count read on a second stream between the two calls
    equals the final one, and the finished build gives rmn_table_build's mapping, inverse, unique rows and lookups."""
    import ctypes
    from riemannengine_b200 import capi, ops
    lib = capi.lib()
    c_np = _random_cloud(77, 50_000, 3, -12, 12, 3, dup_frac=0.2 if dups else 0)
    if not dups:
        c_np = c_np[OracleBackend().insert_and_map(c_np)[0]]
    coords = torch.from_numpy(c_np).cuda()
    n, w = coords.shape
    ref = ops.table_build(coords)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    main, side = torch.cuda.current_stream(), torch.cuda.Stream()
    tbytes, wbytes = lib.rmn_table_bytes(n), lib.rmn_table_build_workspace_bytes(n)
    table = torch.zeros(tbytes, dtype=torch.uint8, device="cuda")
    ws = torch.empty(wbytes, dtype=torch.uint8, device="cuda")
    mapping = torch.full((n,), -7, dtype=torch.int64, device="cuda")
    inverse = torch.full((n,), -7, dtype=torch.int64, device="cuda")
    uniq = torch.full((n, w), -7, dtype=torch.int32, device="cuda")
    sm = ctypes.c_void_p(main.cuda_stream)
    assert lib.rmn_table_build_begin(p(coords), n, w, p(table), tbytes, p(ws), wbytes, sm) == capi.OK
    counted = torch.cuda.Event()
    counted.record(main)
    assert lib.rmn_table_build_finish(p(coords), n, w, p(table), p(mapping), p(inverse), p(uniq), p(ws), sm) == capi.OK
    side.wait_event(counted)
    early = (ctypes.c_uint32 * 4)()
    assert lib.rmn_table_info(p(table), early, ctypes.c_void_p(side.cuda_stream)) == capi.OK
    late = (ctypes.c_uint32 * 4)()
    assert lib.rmn_table_info(p(table), late, sm) == capi.OK
    assert list(early) == list(late) and early[0] == ref.n_unique
    nu = int(late[0])
    assert torch.equal(mapping[:nu], ref.mapping) and torch.equal(inverse, ref.inverse)
    assert torch.equal(uniq[:nu], ref.coords)
    # (slot positions depend on which of two colliding keys won its CAS: compare the tables through lookups)
    rows = torch.empty(n, dtype=torch.int32, device="cuda")
    assert lib.rmn_table_find(p(table), p(coords), n, w, p(rows), sm) == capi.OK
    assert torch.equal(rows.long(), ref.inverse)


def test_small_readback_without_the_copy_engine():
    """rmn_readback_small delivers device words into page-locked host memory (stored by a kernel) and into
    pageable memory (copy fallback), also while a large device-to-host copy is queued on another stream."""
    import ctypes
    from riemannengine_b200 import capi
    lib = capi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for n_words in (1, 28, 1000, 70_000):
        src = torch.arange(n_words, dtype=torch.int32, device="cuda") * 3 + 1
        pinned = torch.zeros(n_words, dtype=torch.int32).pin_memory()
        pageable = np.zeros(n_words, dtype=np.int32)
        big_d = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
        big_h = torch.empty(64 << 20, dtype=torch.uint8).pin_memory()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            big_h.copy_(big_d, non_blocking=True)
        assert lib.rmn_readback_small(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(pinned.data_ptr()),
                                      n_words * 4, stream) == capi.OK
        assert lib.rmn_readback_small(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(pageable.ctypes.data),
                                      n_words * 4, stream) == capi.OK
        torch.cuda.synchronize()
        assert torch.equal(pinned, src.cpu())
        assert (pageable == src.cpu().numpy()).all()
    src = torch.zeros(4, dtype=torch.int32, device="cuda")
    dst = torch.zeros(4, dtype=torch.int32).pin_memory()
    assert lib.rmn_readback_small(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()), 6, stream) == capi.ERR_BAD_ARG
    assert lib.rmn_readback_small(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()), 0, stream) == capi.OK


# ---------------------------------------------------------------------------------------------
# Maps at coarse tensor strides: every coordinate is a multiple of the stride, so the low bits of
# the first spatial column are the same in all rows; the table must still use its whole capacity.
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("ts", [4, 8, 16, 6])
def test_insert_unique_rows_on_a_coarse_grid(gpu, ts):
    rng = np.random.default_rng(100 + ts)
    c = np.concatenate([rng.integers(0, 2, (60000, 1)), rng.integers(-40, 41, (60000, 3)) * ts], 1).astype(np.int32)
    c = c[OracleBackend().insert_and_map(c)[0]]          # all rows distinct: the table's worst case
    c[:, 1:] += 3                                         # and the grid need not pass through the origin
    m0, i0 = OracleBackend().insert_and_map(c)
    m1, i1 = gpu().insert_and_map(c)
    assert (m0 == m1).all() and (i0 == i1).all()
    # kernel map on that grid (offsets are multiples of the tensor stride)
    O = OracleBackend()
    off = O.region_offsets([3] * 3, [1] * 3, [ts] * 3)
    parity.assert_kernel_maps_equal(gpu().conv_kernel_map(c, c, off), O.conv_kernel_map(c, c, off))
    # lookups of rows off the grid miss, rows on it hit
    from riemannengine_b200 import ops
    from tests.gpu_backend import dev_coords
    t = ops.table_build(dev_coords(c))
    shifted = c.copy()
    shifted[:, 1] += 1
    assert (ops.table_find(t, dev_coords(shifted)).cpu().numpy() == -1).all()
    assert (ops.table_find(t, dev_coords(c)).cpu().numpy() == np.arange(len(c))).all()


def test_three_stride2_levels_on_a_sparse_cloud(gpu):
    """Stride 2 -> 4 -> 8 on a cloud so sparse that almost every row stays unique at every level
    (LiDAR-like): coordinate maps and the 3^3 kernel map of every level against the oracle."""
    O = OracleBackend()
    rng = np.random.default_rng(77)
    c = np.concatenate([rng.integers(0, 2, (50000, 1)), rng.integers(-2000, 2001, (50000, 3))], 1).astype(np.int32)
    c = c[O.insert_and_map(c)[0]]
    ts = 1
    for level in range(3):
        ts *= 2
        a0, i0 = O.stride_map(c, [ts] * 3)
        a1, i1 = gpu().stride_map(c, [ts] * 3)
        assert (a0 == a1).all() and (i0 == i1).all()
        assert len(a0) > 0.9 * len(c)
        off = O.region_offsets([3] * 3, [1] * 3, [ts] * 3)
        parity.assert_kernel_maps_equal(gpu().conv_kernel_map(a1, a1, off), O.conv_kernel_map(a0, a0, off))
        c = a0
