"""Seeded synthetic voxel clouds with the shapes and statistics of the benchmark
configurations. They stand in for real scans; nothing here reads a dataset.

All generators are host-side numpy, deterministic in ``seed``, and return int32
coordinates [N, 1 + D] (batch index first) with unique rows per sample.
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np


def sphere_shell(radius: int = 64, batch: int = 0) -> np.ndarray:
    """All integer voxels x in [-(r+1), r+1]^3 with | ||x|| - r | < 1 (101 930 rows for r = 64)."""
    r = np.arange(-(radius + 1), radius + 2)
    g = np.stack(np.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 3)
    nrm = np.sqrt((g.astype(np.float64) ** 2).sum(1))
    g = g[np.abs(nrm - radius) < 1]
    return np.concatenate([np.full((len(g), 1), batch, np.int32), g.astype(np.int32)], 1)


def _surface_samples(rng: np.random.Generator, lo, hi, axis: int, value: int, n: int) -> np.ndarray:
    pts = np.stack([rng.integers(lo[a], hi[a] + 1, size=n) for a in range(3)], 1)
    pts[:, axis] = value
    return pts


def indoor_scene(seed: int, n_voxels: int = 150_000, grid: Tuple[int, int, int] = (200, 200, 60)) -> np.ndarray:
    """One room: floor plane, four wall planes and ten axis-aligned box surfaces, +-1 voxel
    jitter, clipped to the grid, unique, first ``n_voxels`` of a seeded permutation. Spatial
    columns only, [n, 3] int32."""
    rng = np.random.default_rng(seed)
    gx, gy, gz = grid
    per = n_voxels  # oversample each family, dedup later
    parts = [
        _surface_samples(rng, (0, 0, 0), (gx - 1, gy - 1, 0), 2, 0, per),
        _surface_samples(rng, (0, 0, 0), (0, gy - 1, gz - 1), 0, 0, per // 3),
        _surface_samples(rng, (0, 0, 0), (0, gy - 1, gz - 1), 0, gx - 1, per // 3),
        _surface_samples(rng, (0, 0, 0), (gx - 1, 0, gz - 1), 1, 0, per // 3),
        _surface_samples(rng, (0, 0, 0), (gx - 1, 0, gz - 1), 1, gy - 1, per // 3),
    ]
    for _ in range(10):
        cx, cy = rng.integers(10, 151, size=2)
        sx, sy = rng.integers(10, 41, size=2)
        sz = rng.integers(5, 41)
        lo = (cx, cy, 0)
        hi = (min(cx + sx, gx - 1), min(cy + sy, gy - 1), min(sz, gz - 1))
        for axis in range(3):
            for value in (lo[axis], hi[axis]):
                parts.append(_surface_samples(rng, lo, hi, axis, value, per // 12))
    pts = np.concatenate(parts, 0)
    pts = pts + rng.integers(-1, 2, size=pts.shape)
    pts = np.clip(pts, 0, np.array(grid) - 1)
    key = np.unique((pts[:, 0].astype(np.int64) * gy + pts[:, 1]) * gz + pts[:, 2])
    key = key[rng.permutation(len(key))][:n_voxels]
    return np.stack([key // (gy * gz), (key // gz) % gy, key % gz], 1).astype(np.int32)


def indoor_batch(n_scenes: int = 8, n_voxels: int = 150_000, seed: int = 2000) -> np.ndarray:
    """Batch of rooms, [sum N_b, 4] int32 with the batch index in column 0."""
    rows = []
    for b in range(n_scenes):
        pts = indoor_scene(seed + b, n_voxels)
        rows.append(np.concatenate([np.full((len(pts), 1), b, np.int32), pts], 1))
    return np.concatenate(rows, 0)


def lidar_sweep(seed: int, n_points: int = 120_000, voxel: float = 0.1) -> np.ndarray:
    """64-beam sweep (elevation -25..+3 deg, 2048 azimuth steps, range U(2, 70) m) voxelised at
    ``voxel`` metres; unique voxels, [n, 3] int32."""
    rng = np.random.default_rng(seed)
    elev = np.deg2rad(np.linspace(-25.0, 3.0, 64))
    azim = np.linspace(0.0, 2 * np.pi, 2048, endpoint=False)
    pick = rng.choice(64 * 2048, size=n_points, replace=False)
    e, a = elev[pick // 2048], azim[pick % 2048]
    rng_m = rng.uniform(2.0, 70.0, size=n_points)
    xyz = np.stack([rng_m * np.cos(e) * np.cos(a), rng_m * np.cos(e) * np.sin(a), rng_m * np.sin(e)], 1)
    vox = np.floor(xyz / voxel).astype(np.int64) + 2048
    key = np.unique((vox[:, 0] * 4096 + vox[:, 1]) * 4096 + vox[:, 2])
    key = key[rng.permutation(len(key))]
    return (np.stack([key // (4096 * 4096), (key // 4096) % 4096, key % 4096], 1) - 2048).astype(np.int32)


def lidar_batch(n_sweeps: int = 2, seed: int = 3000) -> np.ndarray:
    rows = []
    for b in range(n_sweeps):
        pts = lidar_sweep(seed + b)
        rows.append(np.concatenate([np.full((len(pts), 1), b, np.int32), pts], 1))
    return np.concatenate(rows, 0)


def spatiotemporal_batch(n_batch: int = 4, n_frames: int = 8, n_voxels: int = 150_000, seed: int = 4000) -> np.ndarray:
    """Frames of one room translated by a cumulative seeded velocity in {0,1,2}^3 voxels per
    frame; coordinates (b, x, y, z, t), [N, 5] int32."""
    rows = []
    for b in range(n_batch):
        rng = np.random.default_rng(seed + 100 * b)
        pts = indoor_scene(seed + b, n_voxels)
        shift = np.zeros(3, np.int64)
        for t in range(n_frames):
            moved = pts + shift.astype(np.int32)
            rows.append(np.concatenate([np.full((len(pts), 1), b, np.int32), moved,
                                        np.full((len(pts), 1), t, np.int32)], 1))
            shift = shift + rng.integers(0, 3, size=3)
    return np.concatenate(rows, 0).astype(np.int32)


def conv_weights(seed: int, K: int, c_in: int, c_out: int, transpose: bool = False) -> np.ndarray:
    """U(-1/sqrt(fan), 1/sqrt(fan)) with fan = (c_out if transpose else c_in) * K, the rule of the
    reference layer (engine/nn/conv.cpp:94-102)."""
    rng = np.random.default_rng(seed)
    bound = 1.0 / np.sqrt((c_out if transpose else c_in) * K)
    return rng.uniform(-bound, bound, size=(K, c_in, c_out)).astype(np.float32)


def features(seed: int, n: int, channels: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((n, channels), dtype=np.float32)
