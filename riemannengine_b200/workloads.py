"""The benchmark configurations beside the headline one, as timed steps over the C++ host layer.

Every function builds its synthetic inputs (seeded stand-ins with the sizes and statistics of the
configuration, see ``synthetic.py``), runs ``warmup`` untimed steps and ``steps`` timed ones with CUDA
events on the current stream, and returns a dict: ``ms_per_step``, ``voxels_per_step`` (input voxels of
THIS rank per step) and what else describes the run. ``C`` is the loaded ``riemann_cpp`` module
(``riemannengine_b200.cpp.load()``); all layers are its classes, so every coordinate map, kernel map and
convolution goes through the C ABI.
"""
from __future__ import annotations

from typing import Callable, Dict, List

import numpy as np
import torch

from . import synthetic


def time_steps(step: Callable[[], None], steps: int, warmup: int) -> float:
    """Milliseconds per step: CUDA events around ``steps`` calls after ``warmup`` untimed ones."""
    for _ in range(max(warmup, 1)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


class _Pyramid:
    """Pair counts of the kernel maps a network builds on ``coords``: stride-1 maps (3^D region) per level and
    the 2^D stride-2 maps between the levels. Built once, outside any timed region, through the same C ABI; used
    only to state the algorithmic flops (2 * pairs * c_in * c_out per convolution pass) of a configuration."""

    def __init__(self, coords: torch.Tensor, levels: int):
        from . import capi, ops
        d = int(coords.size(1)) - 1
        self.rows: List[int] = []
        self.self_pairs: List[int] = []
        self.down_pairs: List[int] = []
        table = ops.table_build(coords)
        for level in range(levels):
            ts = [2 ** level] * d
            self.rows.append(int(table.n_unique))
            off3 = ops.region_offsets(capi.HYPER_CUBE, [3] * d, [1] * d, ts)
            self.self_pairs.append(int(ops.kmap_build(table, table.coords, off3, self_map=True).offset_ptr[-1]))
            if level + 1 < levels:
                nxt = ops.table_build(ops.coords_stride(table.coords, [2 ** (level + 1)] * d))
                off2 = ops.region_offsets(capi.HYPER_CUBE, [2] * d, [1] * d, ts)
                self.down_pairs.append(int(ops.kmap_build(table, nxt.coords, off2).offset_ptr[-1]))
                table = nxt


def _rate(flops: float, ms: float) -> Dict:
    return {"algorithmic_flops_per_step": flops, "algorithmic_tflops": flops / (ms / 1e3) / 1e12}


def _conv(C, c_in, c_out, kernel_size, stride, dimension, dev, dtype, transpose=False, seed=0):
    cls = C.RiemannConvolutionTranspose if transpose else C.RiemannConvolution
    layer = cls(c_in, c_out, kernel_size=kernel_size, stride=stride, dimension=dimension)
    layer.to(f"cuda:{dev.index}")
    layer.to(dtype)
    k_vol = int(layer.kernel.shape[0])
    with torch.no_grad():
        w = synthetic.conv_weights(seed, k_vol, c_in, c_out, transpose=transpose)
        layer.kernel.copy_(torch.from_numpy(w).to(dev))
    return layer


# ------------------------------------------------------------------------------------------------
# configuration 1: one 3^3 stride-1 32 -> 32 fp32 convolution on the radius-64 sphere shell
# ------------------------------------------------------------------------------------------------
def sphere_shell_inputs():
    coords = synthetic.sphere_shell(64)
    feats = synthetic.features(1000, len(coords), 32)
    weights = synthetic.conv_weights(1001, 27, 32, 32)
    return coords, feats, weights


def run_sphere_shell(C, dev, steps: int, warmup: int) -> Dict:
    coords_np, feats_np, weights_np = sphere_shell_inputs()
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(feats_np).to(dev)
    conv = _conv(C, 32, 32, 3, 1, 3, dev, torch.float32, seed=1001)

    def step():
        with torch.no_grad():
            conv(C.SparseTensor(feats, coords))

    ms = time_steps(step, steps, warmup)
    pairs = _Pyramid(coords, 1).self_pairs[0]
    return {"workload": "sphere shell r=64 (101 930 voxels), 3^3 stride-1 32->32 fp32: hash insert + kernel map + "
                        "forward on a fresh manager", "dtype": "f32", "voxels_per_step": len(coords_np),
            "ms_per_step": ms, "pairs": pairs, **_rate(2.0 * pairs * 32 * 32, ms)}


# ------------------------------------------------------------------------------------------------
# configuration 3: LiDAR-like sweeps, five-layer chain, forward + backward + weight-gradient all-reduce
# ------------------------------------------------------------------------------------------------
def lidar_batch(n_sweeps: int, seed: int) -> np.ndarray:
    rows = []
    for b in range(n_sweeps):
        pts = synthetic.lidar_sweep(seed + b)
        rows.append(np.concatenate([np.full((len(pts), 1), b, np.int32), pts], 1))
    return np.concatenate(rows, 0)


def run_lidar_chain(C, dev, rank: int, steps: int, warmup: int, sweeps_per_gpu: int = 2) -> Dict:
    coords_np = lidar_batch(sweeps_per_gpu, 3000 + 100 * rank)
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(synthetic.features(3500 + rank, len(coords_np), 4)).to(dev).bfloat16()
    bf = torch.bfloat16
    layers = [_conv(C, 4, 32, 3, 1, 3, dev, bf, seed=3601), _conv(C, 32, 64, 3, 1, 3, dev, bf, seed=3602),
              _conv(C, 64, 64, 2, 2, 3, dev, bf, seed=3603), _conv(C, 64, 128, 3, 1, 3, dev, bf, seed=3604),
              _conv(C, 128, 64, 2, 2, 3, dev, bf, transpose=True, seed=3605)]

    def step():
        for layer in layers:
            layer.zero_grad()
        x = C.SparseTensor(feats, coords)
        for layer in layers:
            x = layer(x)
        (x.F.float() ** 2).mean().backward()   # the layers all-reduce their weight gradients in backward

    ms = time_steps(step, steps, warmup)
    pyr = _Pyramid(coords, 2)
    p0, p1, pd = pyr.self_pairs[0], pyr.self_pairs[1], pyr.down_pairs[0]
    fwd = 2.0 * (p0 * (4 * 32 + 32 * 64) + pd * 64 * 64 + p1 * 64 * 128 + pd * 128 * 64)
    flops = 3.0 * fwd - 2.0 * p0 * 4 * 32   # forward + input gradient + weight gradient; the input needs no gradient
    return {"flops_note": "2 * pairs * c_in * c_out per convolution pass", **_rate(flops, ms),
            "workload": f"LiDAR-like sweeps ({sweeps_per_gpu} per GPU, ~90 K voxels each, voxel 0.1 m), bf16, 4 input "
                        "channels: 3^3 4->32, 3^3 32->64, 2^3 s2 64->64, 3^3 64->128, transposed 2^3 s2 128->64; "
                        "loss mean(out^2); hash insert + kernel maps + forward + backward + weight-gradient "
                        "all-reduce on a fresh manager", "dtype": "bf16", "voxels_per_step": len(coords_np),
            "ms_per_step": ms}


# ------------------------------------------------------------------------------------------------
# configuration 4: 4-D spatio-temporal clips, 3^4 = 81 offsets, 32 -> 32 bf16
# ------------------------------------------------------------------------------------------------
def spatiotemporal_batch(batch: int, frames: int, seed: int, n_voxels: int = 150_000) -> np.ndarray:
    """``batch`` clips of ``frames`` frames: every frame is the clip's room translated by the clip's
    velocity (seeded, 0..2 voxels per frame and axis); coordinates (b, x, y, z, t)."""
    rows = []
    for b in range(batch):
        pts = synthetic.indoor_scene(seed + b, n_voxels)
        vel = np.random.default_rng(seed + 500 + b).integers(0, 3, size=3)
        for t in range(frames):
            c = np.concatenate([np.full((len(pts), 1), b, np.int32), pts + t * vel[None, :].astype(np.int32),
                                np.full((len(pts), 1), t, np.int32)], 1)
            rows.append(c.astype(np.int32))
    return np.concatenate(rows, 0)


def run_spatiotemporal(C, dev, rank: int, steps: int, warmup: int, batch: int = 4, frames: int = 8) -> Dict:
    coords_np = spatiotemporal_batch(batch, frames, 4000 + 100 * rank)
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(synthetic.features(4500 + rank, len(coords_np), 32)).to(dev).bfloat16()
    conv = _conv(C, 32, 32, 3, 1, 4, dev, torch.bfloat16, seed=4601)

    def step():
        with torch.no_grad():
            conv(C.SparseTensor(feats, coords))

    ms = time_steps(step, steps, warmup)
    pairs = _Pyramid(coords, 1).self_pairs[0]
    return {"workload": f"4-D clips: batch {batch} x {frames} frames of a 150 K-voxel room moving 0-2 voxels per frame, "
                        "coordinates (b, x, y, z, t); 3^4 = 81 offsets, 32->32 bf16: hash insert + kernel map + "
                        "forward on a fresh manager", "dtype": "bf16", "voxels_per_step": len(coords_np),
            "ms_per_step": ms, "pairs": pairs, **_rate(2.0 * pairs * 32 * 32, ms)}


# ------------------------------------------------------------------------------------------------
# configuration 5: MinkUNet-style encoder/decoder on rooms, forward + backward, fixed total batch
# ------------------------------------------------------------------------------------------------
def run_unet(C, dev, rank: int, world: int, steps: int, warmup: int, total_scenes: int = 32) -> Dict:
    mine: List[int] = [s for s in range(total_scenes) if s % world == rank]
    rows = []
    for i, s in enumerate(mine):
        pts = synthetic.indoor_scene(5000 + s, 150_000)
        rows.append(np.concatenate([np.full((len(pts), 1), i, np.int32), pts], 1))
    coords_np = np.concatenate(rows, 0)
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(synthetic.features(5500 + rank, len(coords_np), 4)).to(dev).bfloat16()
    torch.manual_seed(5600)
    net = C.MinkUNet(4, 20, width=32, dimension=3)
    net.to(f"cuda:{dev.index}")
    net.to(torch.bfloat16)
    net.train(True)
    norm_params = [p for name, p in net.named_parameters().items() if ".norm." in name or name.startswith("norm.")]

    def step():
        net.zero_grad()
        out = net(C.SparseTensor(feats, coords))
        (out.F.float() ** 2).mean().backward()   # convolution layers all-reduce their gradients in backward
        if world > 1:                            # batch-norm scales and shifts: one more flat bucket
            grads = [p.grad.float() for p in norm_params if p.grad is not None]
            C.allreduce_gradients(grads)
            for p, g in zip([p for p in norm_params if p.grad is not None], grads):
                p.grad.copy_(g)

    ms = time_steps(step, steps, warmup)
    # algorithmic flops of the network of riemann_cpp/networks.hpp (width 32): per level s (c = 32 * 2^s) four
    # 3^3 c->c convolutions in the encoder; a 2^3 stride-2 c/2->c convolution into the level; in the decoder a
    # transposed 2^3 c->c/2 convolution out of it, a 3^3 c->c/2 fuse and two 3^3 c/2->c/2 convolutions one level up
    pyr = _Pyramid(coords, 4)
    width, fwd = 32, 0.0
    fwd += 2.0 * pyr.self_pairs[0] * 4 * width                              # stem
    for s_ in range(4):
        c = width * 2 ** s_
        fwd += 2.0 * pyr.self_pairs[s_] * 4 * c * c                         # two BasicBlocks
        if s_ > 0:
            half = c // 2
            fwd += 2.0 * pyr.down_pairs[s_ - 1] * (half * c + c * half)     # down into the level, up out of it
            fwd += 2.0 * pyr.self_pairs[s_ - 1] * (c * half + 2 * half * half)  # fuse + BasicBlock one level up
    fwd += 2.0 * pyr.rows[0] * width * 20                                   # 1x1 head
    flops = 3.0 * fwd - 2.0 * pyr.self_pairs[0] * 4 * width                 # the input features need no gradient
    return {"flops_note": "2 * pairs * c_in * c_out per convolution pass (forward, input gradient, weight gradient)",
            **_rate(flops, ms),
            "workload": f"MinkUNet-style encoder/decoder (stem 32; stages 32/64/128/256 of two BasicBlocks; 2^3 s2 "
                        f"downs, transposed ups with skip concatenation; batch norm + ReLU), bf16, 4 input channels, "
                        f"{total_scenes} rooms of 150 K voxels over {world} GPU(s) (fixed total batch): hash insert + "
                        "kernel maps + forward + backward (+ gradient all-reduce) on a fresh manager",
            "dtype": "bf16", "voxels_per_step": len(coords_np), "scenes_this_rank": len(mine),
            "ms_per_step": ms}
