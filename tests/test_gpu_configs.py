"""Parity on seeded stand-ins of the other benchmark configurations, at sizes the oracle finishes
in seconds: LiDAR-like sweeps (very sparse, large coordinate range, 4 input channels, strided
down + transposed up with weight gradients) and the 4-D spatio-temporal 3^4 = 81-offset kernel."""
import numpy as np
import pytest
import torch

from tests import parity
from tests.parity import OracleBackend, rel_l2, rel_max

pytestmark = pytest.mark.gpu


def test_lidar_sweep_network_fp32_matches_oracle():
    """3^3 4->32 on a 120K-point sweep voxelised at 0.1 m, then 2^3 stride-2 down 32->64 and the
    transposed 2^3 up 64->32 (kernel maps, outputs and all gradients)."""
    from riemannengine_b200 import synthetic
    from tests.gpu_backend import GpuBackend
    pts = synthetic.lidar_sweep(3001)
    c = np.concatenate([np.zeros((len(pts), 1), np.int32), pts], 1)
    assert 100_000 < len(c) < 125_000 and c[:, 1:].min() < -600 and c[:, 1:].max() > 600
    O, G = OracleBackend(f64=True), GpuBackend(torch.float32)
    f = synthetic.features(3100, len(c), 4)
    w = synthetic.conv_weights(3101, 27, 4, 32)
    r0 = parity.run_pipeline(O, c, f, w, 3, 3, 1, 1)
    r1 = parity.run_pipeline(G, c, f, w, 3, 3, 1, 1)
    parity.assert_kernel_maps_equal(tuple(r1[k] for k in ("kmap_ptr", "kmap_in", "kmap_out")),
                                    tuple(r0[k] for k in ("kmap_ptr", "kmap_in", "kmap_out")))
    for key in ("out_feats", "grad_feats", "grad_weights"):
        assert rel_max(r1[key], r0[key]) <= 1e-4, key
    f2 = synthetic.features(3102, len(c), 32)
    wd = synthetic.conv_weights(3103, 8, 32, 64)
    wu = synthetic.conv_weights(3104, 8, 64, 32, transpose=True)
    d0 = parity.run_pipeline(O, c, f2, wd, 3, 2, 2, 1, wu)
    d1 = parity.run_pipeline(G, c, f2, wd, 3, 2, 2, 1, wu)
    assert (d0["out_coords"] == d1["out_coords"]).all()
    for a in ("kmap", "kmap2"):
        parity.assert_kernel_maps_equal(tuple(d1[a + s] for s in ("_ptr", "_in", "_out")),
                                        tuple(d0[a + s] for s in ("_ptr", "_in", "_out")))
    for key in ("out_feats", "up_feats", "grad_feats", "grad_weights", "grad_weights2"):
        assert rel_max(d1[key], d0[key]) <= 1e-4, key


def test_lidar_sweep_bf16_tensor_core_layers():
    """The bf16 layers of the sweep network that run on the tensor cores: 3^3 32->64, 2^3 s2
    64->64 down and the transposed 2^3 128->64 up, against the fp64 oracle on rounded inputs."""
    from riemannengine_b200 import synthetic
    from tests.gpu_backend import GpuBackend
    pts = synthetic.lidar_sweep(3002, n_points=40_000)
    c = np.concatenate([np.zeros((len(pts), 1), np.int32), pts], 1)
    O, G = OracleBackend(f64=True), GpuBackend(torch.bfloat16)
    rnd = lambda a: torch.from_numpy(a).bfloat16().float().numpy()  # noqa: E731
    f = synthetic.features(3200, len(c), 32)
    w = synthetic.conv_weights(3201, 27, 32, 64)
    r0 = parity.run_pipeline(O, c, rnd(f), rnd(w), 3, 3, 1, 1)
    r1 = parity.run_pipeline(G, c, f, w, 3, 3, 1, 1)
    assert rel_l2(r1["out_feats"], r0["out_feats"]) <= 1e-2
    f2 = synthetic.features(3202, len(c), 64)
    wd = synthetic.conv_weights(3203, 8, 64, 128)
    wu = synthetic.conv_weights(3204, 8, 128, 64, transpose=True)
    d0 = parity.run_pipeline(O, c, rnd(f2), rnd(wd), 3, 2, 2, 1, rnd(wu))
    d1 = parity.run_pipeline(G, c, f2, wd, 3, 2, 2, 1, wu)
    assert rel_l2(d1["out_feats"], d0["out_feats"]) <= 1e-2
    assert rel_l2(d1["up_feats"], d0["up_feats"]) <= 2e-2  # two bf16 layers deep


def test_spatiotemporal_4d_81_offsets():
    """(b, x, y, z, t) coordinates, 3^4 kernel, 32 -> 32: maps exact, fp32 within 1e-4, bf16 within 1e-2."""
    from riemannengine_b200 import synthetic
    from tests.gpu_backend import GpuBackend
    c = synthetic.spatiotemporal_batch(n_batch=2, n_frames=4, n_voxels=3000, seed=4000)
    assert c.shape[1] == 5
    O = OracleBackend(f64=True)
    f = synthetic.features(4100, len(c), 32)
    w = synthetic.conv_weights(4101, 81, 32, 32)
    r0 = parity.run_pipeline(O, c, f, w, 4, 3, 1, 1)
    assert len(r0["kmap_ptr"]) == 82
    r1 = parity.run_pipeline(GpuBackend(torch.float32), c, f, w, 4, 3, 1, 1)
    parity.assert_kernel_maps_equal(tuple(r1[k] for k in ("kmap_ptr", "kmap_in", "kmap_out")),
                                    tuple(r0[k] for k in ("kmap_ptr", "kmap_in", "kmap_out")))
    for key in ("out_feats", "grad_feats", "grad_weights"):
        assert rel_max(r1[key], r0[key]) <= 1e-4, key
    rnd = lambda a: torch.from_numpy(a).bfloat16().float().numpy()  # noqa: E731
    rb0 = parity.run_pipeline(O, c, rnd(f), rnd(w), 4, 3, 1, 1)
    rb1 = parity.run_pipeline(GpuBackend(torch.bfloat16), c, f, w, 4, 3, 1, 1)
    assert rel_l2(rb1["out_feats"], rb0["out_feats"]) <= 1e-2


def test_engine_lidar_unet_slice_runs_and_backpropagates():
    """conv 4->32 -> conv 32->64 -> down 64->64 -> conv 64->128 -> transposed up 128->64 through the layer
    interface in bf16 (the shape of the sweep configuration), with finite gradients everywhere."""
    from riemannengine_b200 import engine as E, synthetic
    coords = torch.from_numpy(synthetic.lidar_batch(2, seed=3000)).cuda()
    feats = torch.randn(len(coords), 4, device="cuda").bfloat16().requires_grad_(True)
    layers = [E.RiemannConvolution(4, 32, 3), E.RiemannConvolution(32, 64, 3), E.RiemannConvolution(64, 64, 2, stride=2),
              E.RiemannConvolution(64, 128, 3), E.RiemannConvolutionTranspose(128, 64, 2, stride=2)]
    layers = [m.cuda().bfloat16() for m in layers]
    x = E.SparseTensor(feats, coords)
    n0 = len(x)
    for m in layers:
        x = m(x)
        x = E.SparseTensor(torch.relu(x.F), x.coordinate_map_key, x.coordinate_manager)
    assert len(x) == n0 and x.tensor_stride == [1, 1, 1] and x.F.shape[1] == 64
    x.F.float().square().mean().backward()
    assert torch.isfinite(feats.grad.float()).all()
    for m in layers:
        assert m.kernel.grad is not None and torch.isfinite(m.kernel.grad.float()).all()


# ---------------------------------------------------------------------------------------------
# The benchmarked workload itself, at its own size, against the reference's CPU build
# (oracle/_ref/ref_driver: engine/grid/lattice_cpu.hpp:606-673 for the pair sets,
# engine/nn/conv.cpp:9-66 for the values).
# ---------------------------------------------------------------------------------------------
def _reference_as_gold(coords, feats, weights, kernel, stride):
    from oracle import refrun
    if not refrun.available():
        pytest.skip("reference driver not built (make -C oracle ref)")
    out = refrun.run(coords, feats, weights, kernel, stride, 1, timeout=1200)
    return {"ref_" + k: v for k, v in out.items()}


@pytest.mark.parametrize("scenes", [1, 8])
def test_indoor_rooms_3x3x3_64_to_64_against_reference(scenes):
    """Whole rooms of the headline batch (150 K voxels each; one room, then all eight = 1.2 M voxels):
    coordinate map and kernel map bit-exact against the reference, fp32 path within 1e-4, and the bf16
    tensor-core output within 1e-2 relative L2 of the reference's fp32 output."""
    from riemannengine_b200 import synthetic
    from tests.gpu_backend import GpuBackend
    c = synthetic.indoor_batch(scenes, 150_000, seed=2000)
    f = synthetic.features(2500, len(c), 64)
    w = synthetic.conv_weights(2600, 27, 64, 64)
    gold = _reference_as_gold(c, f, w, 3, 1)
    assert len(gold["ref_in_coords"]) == scenes * 150_000
    r32 = parity.run_pipeline(GpuBackend(torch.float32), c, f, w, 3, 3, 1, 1)
    parity.check_against_reference(r32, gold, tol=1e-4, metric=rel_max)
    fb = torch.from_numpy(f).bfloat16().float().numpy()      # the bf16 path sees rounded inputs
    rb = parity.run_pipeline(GpuBackend(torch.bfloat16), c, fb, w, 3, 3, 1, 1)
    assert (rb["kmap_ptr"] == gold["ref_kmap_ptr"]).all()
    assert rel_l2(rb["out_feats"], gold["ref_out_feats"]) <= 1e-2
    assert rel_l2(rb["grad_weights"], gold["ref_grad_weights"]) <= 3e-2   # two bf16 roundings compound


def test_indoor_room_2x2x2_stride2_64_to_128_against_reference():
    """The workload's second layer on one whole room: strided coordinate map (matched by coordinate: the
    reference numbers coarse rows in hash order), kernel map, fp32 and bf16 outputs."""
    from riemannengine_b200 import synthetic
    from tests.gpu_backend import GpuBackend
    c = synthetic.indoor_batch(1, 150_000, seed=2000)
    f = synthetic.features(2500, len(c), 64)
    w = synthetic.conv_weights(2601, 8, 64, 128)
    gold = _reference_as_gold(c, f, w, 2, 2)
    r32 = parity.run_pipeline(GpuBackend(torch.float32), c, f, w, 3, 2, 2, 1)
    parity.check_against_reference(r32, gold, tol=1e-4, metric=rel_max)
    rb = parity.run_pipeline(GpuBackend(torch.bfloat16), c, f, w, 3, 2, 2, 1)
    perm = parity.row_permutation(rb["out_coords"], gold["ref_out_coords"])
    assert rel_l2(rb["out_feats"], gold["ref_out_feats"][perm]) <= 1e-2


def test_spatiotemporal_clip_81_offsets_against_reference():
    """One sample of the 4-D configuration at its own size: one clip, two frames (300 K voxels, coordinates
    (b, x, y, z, t)), 3^4 = 81 offsets, 32 -> 32. Coordinate map and kernel map bit-exact against the reference's
    CPU build, fp32 path within 1e-4, bf16 tensor-core output within 1e-2 relative L2."""
    from riemannengine_b200 import synthetic, workloads
    from tests.gpu_backend import GpuBackend
    c = workloads.spatiotemporal_batch(1, 2, 4000)
    assert c.shape == (300_000, 5)
    f = synthetic.features(4500, len(c), 32)
    w = synthetic.conv_weights(4601, 81, 32, 32)
    gold = _reference_as_gold(c, f, w, 3, 1)
    r32 = parity.run_pipeline(GpuBackend(torch.float32), c, f, w, 4, 3, 1, 1)
    parity.check_against_reference(r32, gold, tol=1e-4, metric=rel_max)
    rb = parity.run_pipeline(GpuBackend(torch.bfloat16), c, f, w, 4, 3, 1, 1)
    assert rel_l2(rb["out_feats"], gold["ref_out_feats"]) <= 1e-2
