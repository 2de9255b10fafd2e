"""The allocation-free table build against the ordinary one.

``rmn_table_build_static`` exists for hosts that must not allocate device memory while
running (fixed memory plans, plug-ins handed buffers but no allocator): it keeps its scratch
in a fixed array inside the library. This test calls it through the C ABI, twice in a row
with different inputs so that the second call runs over the first call's leftovers, and
requires bit-identical outputs to ``rmn_table_build`` (coordinate work is integer: the bar is
exact equality, as for every other coordinate test).

Collected last on purpose: a failure here cannot hide a failure elsewhere under ``-x``.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cloud(seed, n, lo, hi):
    rng = np.random.default_rng(seed)
    c = np.concatenate([rng.integers(0, 3, (n, 1)), rng.integers(lo, hi + 1, (n, 3))], 1).astype(np.int32)
    c[rng.integers(0, n, n // 8)] = c[rng.integers(0, n, n // 8)]  # duplicates
    return c


def _build(coords_np, static):
    from riemannengine_b200 import capi
    lib = capi.lib()
    dev = torch.device("cuda", 0)
    coords = torch.from_numpy(coords_np).to(dev)
    n, w = coords.shape
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    tbytes = lib.rmn_table_bytes(n)
    table = torch.zeros(tbytes, dtype=torch.uint8, device=dev)
    mapping = torch.full((n,), -7, dtype=torch.int64, device=dev)
    inverse = torch.full((n,), -7, dtype=torch.int64, device=dev)
    uniq = torch.full((n, w), -7, dtype=torch.int32, device=dev)
    if static:
        rc = lib.rmn_table_build_static(p(coords), n, w, p(table), tbytes, p(mapping), p(inverse), p(uniq), stream)
    else:
        wbytes = lib.rmn_table_build_workspace_bytes(n)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        rc = lib.rmn_table_build(p(coords), n, w, p(table), tbytes, p(mapping), p(inverse), p(uniq), p(ws), wbytes,
                                 stream)
    assert rc == capi.OK, lib.rmn_status_string(rc)
    info = (ctypes.c_uint32 * 4)()
    assert lib.rmn_table_info(p(table), info, stream) == capi.OK
    nu = int(info[0])
    # lookups through each table must agree too
    rows = torch.empty(n, dtype=torch.int32, device=dev)
    assert lib.rmn_table_find(p(table), p(coords), n, w, p(rows), stream) == capi.OK
    torch.cuda.synchronize()
    return nu, mapping[:nu].cpu(), inverse.cpu(), uniq[:nu].cpu(), rows.cpu()


def test_static_table_build_matches_regular_twice_in_a_row():
    torch.cuda.set_device(0)
    # second call is smaller and different: it runs over the scratch the first call left behind
    for seed, n, lo, hi in ((101, 200_000, -40, 40), (102, 37_003, -9, 9)):
        c = _cloud(seed, n, lo, hi)
        ref = _build(c, static=False)
        got = _build(c, static=True)
        assert got[0] == ref[0]
        for a, b in zip(got[1:], ref[1:]):
            assert torch.equal(a, b)
        assert torch.equal(got[4].long(), got[2])  # every row finds its own unique row
        # and directly against the CPU oracle (first-occurrence rows, row -> unique row)
        from oracle import oracle as O
        m0, i0 = O.insert_and_map(c)
        assert got[0] == len(m0)
        assert (got[1].numpy() == m0).all() and (got[2].numpy() == i0).all()
        assert (got[3].numpy() == c[m0]).all()


def test_static_table_build_rejects_oversized_input():
    from riemannengine_b200 import capi
    lib = capi.lib()
    limit = lib.rmn_table_build_static_max_rows()
    assert limit == 1 << 20
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda:0")
    p = ctypes.c_void_p(dummy.data_ptr())
    rc = lib.rmn_table_build_static(p, limit + 1, 4, p, 1 << 40, p, p, p, None)
    assert rc == capi.ERR_TOO_LARGE
    assert b"capacity" in lib.rmn_status_string(rc)
