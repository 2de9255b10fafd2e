"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rmn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rmn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("rmn_table_build", "rmn_kmap_build", "rmn_kmap_pairs", "rmn_conv_forward",
                 "rmn_conv_backward_input", "rmn_conv_backward_weight", "rmn_coords_stride"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    from riemannengine_b200 import _build, capi
    if not os.path.exists(_build.LIB_PATH):
        _build.build_library()
    handle = ctypes.CDLL(_build.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} declared in rmn_b200.h but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(capi.SIGNATURES) == set(declared_symbols())


def test_host_only_entry_points():
    from riemannengine_b200 import capi
    lib = capi.lib()
    assert lib.rmn_version() >= 100
    assert lib.rmn_status_string(capi.ERR_PROBE_LIMIT).decode().startswith("hash probe limit")
    assert lib.rmn_table_bytes(0) == 256 + 16 * 64
    assert lib.rmn_table_bytes(1000) == 256 + 16 * 4064  # 4n + 64 slots (a multiple of 32)
    assert lib.rmn_table_bytes(1001) == 256 + 16 * 4096  # ... rounded up
    assert lib.rmn_table_bytes(1 << 20) == 256 + 16 * ((4 << 20) + 64)
    assert lib.rmn_table_bytes(1 << 22) == 256 + 16 * ((3 << 22) + 64)  # past 120 MiB: 3n + 64
    # convolution plan sizes: header + perm + tile masks + permuted table, positions padded to 512 rows
    assert lib.rmn_conv_plan_bytes(1000, 27) == 256 + 4 * 1024 + 256 + 27 * 1024 * 4
    assert lib.rmn_conv_plan_bytes(1000, 33) == 0 and lib.rmn_conv_plan_workspace_bytes(1000, 27) > 1000 * 5
    # gradient all-reduce: a single rank (or nothing to reduce) returns at once, without NCCL or a GPU
    import ctypes
    counts = (ctypes.c_size_t * 2)(10, 20)
    assert lib.rmn_allreduce_grads_workspace_bytes(counts, 2) == 30 * 4
    assert lib.rmn_allreduce_grads_workspace_bytes(counts, 1) == 0
    bufs = (ctypes.c_void_p * 2)(None, None)
    assert lib.rmn_allreduce_grads(None, bufs, counts, 2, None, 0, 1, 1, None) == capi.OK
    assert lib.rmn_allreduce_grads(None, bufs, counts, 0, None, 0, 1, 4, None) == capi.OK
    assert lib.rmn_allreduce_grads(None, bufs, counts, 2, None, 0, 1, 4, None) == capi.ERR_BAD_ARG   # no communicator
    assert lib.rmn_channel_dot_stats_workspace_bytes(64) == 148 * 4 * 2 * 64 * 4
    # small read-back: argument checks come before any CUDA call
    word = ctypes.c_uint32(0)
    assert lib.rmn_readback_small(None, None, 0, None) == capi.OK
    assert lib.rmn_readback_small(None, ctypes.byref(word), 4, None) == capi.ERR_BAD_ARG
    assert lib.rmn_readback_small(ctypes.byref(word), ctypes.byref(word), 6, None) == capi.ERR_BAD_ARG
    assert lib.rmn_readback_small(ctypes.byref(word), ctypes.byref(word), (1 << 20) + 4, None) == capi.ERR_BAD_ARG


def test_region_offsets_match_oracle():
    import numpy as np
    from oracle import oracle as O
    from riemannengine_b200 import capi, ops
    for rt, ks, dl, ts in [(capi.HYPER_CUBE, [3, 3, 3], [1, 1, 1], [1, 1, 1]),
                           (capi.HYPER_CUBE, [2, 2, 2], [1, 1, 1], [2, 2, 2]),
                           (capi.HYPER_CUBE, [3, 2, 5, 3], [1, 2, 1, 3], [1, 2, 4, 1]),
                           (capi.HYPER_CROSS, [3, 5, 3], [1, 1, 2], [2, 1, 1])]:
        assert (ops.region_offsets(rt, ks, dl, ts) == O.region_offsets(rt, ks, dl, ts)).all()
    cu = np.array([[1, -2, 0], [0, 0, 3]], np.int32)
    assert (ops.region_offsets(capi.CUSTOM, [1] * 3, [2] * 3, [4] * 3, cu) ==
            O.region_offsets(O.CUSTOM, [1] * 3, [2] * 3, [4] * 3, cu)).all()


def test_cpu_tensors_are_rejected():
    import torch
    from riemannengine_b200 import engine
    with pytest.raises(RuntimeError, match="CUDA"):
        engine.SparseTensor(torch.zeros(2, 3), torch.zeros(2, 4, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="no CPU"):
        engine.CoordinateManager(3, engine.CoordinateMapBackend.CPU)


def test_cpp_host_module_loads_on_cpu():
    """The C++ host layer builds against LibTorch and mirrors the reference's class names."""
    import os
    from riemannengine_b200 import _build, cpp
    if not os.path.exists(_build.HOST_LIB):
        pytest.skip("host extension not built (python -c 'import __graft_entry__ as g; g.build()')")
    C = cpp.load()
    for name in ("CoordinateMapKey", "CoordinateManager", "SparseTensor", "RiemannConvolution",
                 "RiemannConvolutionTranspose", "RiemannGenerativeConvolutionTranspose"):
        assert hasattr(C, name)
    k = C.CoordinateMapKey([2, 2, 2], "a")
    assert k.tensor_stride == [2, 2, 2] and k.coordinate_size == 4 and repr(k) == "coordinate map key:[2, 2, 2]:a"
    conv = C.RiemannConvolution(4, 8, kernel_size=3, bias=True)
    assert tuple(conv.kernel.shape) == (27, 4, 8) and tuple(conv.bias.shape) == (1, 8)
    bound = 1.0 / (4 * 27) ** 0.5
    assert float(conv.kernel.abs().max()) <= bound
    with pytest.raises(RuntimeError, match="no CPU"):
        C.CoordinateManager(3, C.CoordinateMapBackend.CPU)
