"""Seeded random clouds (dimension, size, extent, batch count and duplicate share drawn per case) through the
table build, lookups of present and absent rows, and both kernel-map builders, each compared with the oracle
bit for bit. Small extents give crowded tables with long collision chains, wide extents sparse ones."""
import numpy as np
import pytest
import torch

from tests import parity
from tests.parity import OracleBackend

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_clouds_match_the_oracle(seed):
    from riemannengine_b200 import capi, ops
    from tests.gpu_backend import dev_coords
    oracle = OracleBackend()
    rng = np.random.default_rng(seed)
    for _ in range(25):
        d = int(rng.choice([2, 3, 3, 3, 4]))
        n = int(rng.choice([300, 3000, 30000, 120000]))
        span = int(rng.choice([3, 8, 20, 60, 300]))
        batches = int(rng.integers(1, 4))
        dup = float(rng.choice([0.0, 0.0, 0.1, 0.6]))
        what = (seed, d, n, span, batches, dup)
        c = np.concatenate([rng.integers(0, batches, (n, 1)), rng.integers(-span, span + 1, (n, d))], 1).astype(np.int32)
        nd = int(n * dup)
        if nd:
            c[rng.integers(0, n, nd)] = c[rng.integers(0, n, nd)]
        m0, i0 = oracle.insert_and_map(c)
        table = ops.table_build(dev_coords(c))
        assert (table.mapping.cpu().numpy() == m0).all() and (table.inverse.cpu().numpy() == i0).all(), what
        uc = c[m0]
        # lookups: present rows, and rows moved by up to two voxels (most of them absent)
        half = len(uc) // 2
        moved = uc[:half] + rng.integers(-2, 3, (half, d + 1)) * np.array([0] + [1] * d)
        q = np.concatenate([uc[:half], moved], 0).astype(np.int32)
        rows = ops.table_find(table, dev_coords(q)).cpu().numpy()
        index = {tuple(r): i for i, r in enumerate(uc)}
        assert (rows == np.array([index.get(tuple(r), -1) for r in q])).all(), what
        if len(uc) > 40000:
            continue
        off = ops.region_offsets(capi.HYPER_CUBE, [3] * d, [1] * d, [1] * d)
        ptr, a, b = oracle.conv_kernel_map(uc, uc, off)
        for self_map in (False, True):
            p2, a2, b2 = ops.kmap_build(table, table.coords, off, self_map=self_map).pairs()
            assert (p2.numpy() == ptr).all(), what + (self_map,)
            a2, b2 = a2.cpu().numpy(), b2.cpu().numpy()
            for k in range(len(off)):
                got = parity.sorted_pairs(ptr, a2, b2, k)
                assert (got == parity.sorted_pairs(ptr, a, b, k)).all(), what + (self_map, k)
