"""Run the compiled reference CPU driver (``oracle/_ref/ref_driver``).

TEST INFRASTRUCTURE ONLY (golden-vector generation and the CPU baseline of
the benchmark). The driver wraps the unmodified reference CPU path; see
``ref_driver.cpp`` for the file format and the arrays exchanged.
"""
from __future__ import annotations

import os
import struct
import subprocess
import tempfile
from typing import Dict, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
DRIVER = os.path.join(_HERE, "_ref", "ref_driver")

_DTYPES = {0: np.int32, 1: np.float32, 2: np.int64, 3: np.float64}
_CODES = {np.dtype(np.int32): 0, np.dtype(np.float32): 1, np.dtype(np.int64): 2, np.dtype(np.float64): 3}


def available() -> bool:
    return os.path.exists(DRIVER) and os.access(DRIVER, os.X_OK)


def write_arrays(path: str, arrays: Dict[str, np.ndarray]) -> None:
    with open(path, "wb") as f:
        for name, a in arrays.items():
            a = np.ascontiguousarray(a)
            nb = name.encode()
            f.write(struct.pack("<I", len(nb)))
            f.write(nb)
            f.write(struct.pack("<II", _CODES[a.dtype], a.ndim))
            f.write(struct.pack(f"<{a.ndim}q", *a.shape))
            f.write(a.tobytes())


def read_arrays(path: str) -> Dict[str, np.ndarray]:
    out: Dict[str, np.ndarray] = {}
    with open(path, "rb") as f:
        data = f.read()
    pos = 0
    while pos < len(data):
        (ln,) = struct.unpack_from("<I", data, pos)
        pos += 4
        name = data[pos:pos + ln].decode()
        pos += ln
        code, ndim = struct.unpack_from("<II", data, pos)
        pos += 8
        dims = struct.unpack_from(f"<{ndim}q", data, pos)
        pos += 8 * ndim
        dt = np.dtype(_DTYPES[code])
        n = int(np.prod(dims)) if ndim else 1
        out[name] = np.frombuffer(data, dtype=dt, count=n, offset=pos).reshape(dims).copy()
        pos += n * dt.itemsize
    return out


def run(coords: np.ndarray, feats: np.ndarray, weights: np.ndarray, kernel_size: int, stride: int = 1,
        dilation: int = 1, weights2: Optional[np.ndarray] = None, threads: int = 0, reps: int = 1,
        timing_only: bool = False, warmup: int = 0, timeout: Optional[float] = None,
        pool: Optional[tuple] = None) -> Dict[str, np.ndarray]:
    """One reference run: SparseTensor -> conv [-> transposed conv] -> backward.

    ``pool = (mode, kernel_size, stride)`` with mode 1 sum / 2 average / 3 maximum also runs the
    reference's local pooling layer on the input tensor (outputs ``pool_*``)."""
    if not available():
        raise RuntimeError("reference driver not built: make -C oracle ref")
    arrays = {
        "coords": np.ascontiguousarray(coords, np.int32),
        "feats": np.ascontiguousarray(feats, np.float32),
        "weights": np.ascontiguousarray(weights, np.float32),
        "params": np.array([kernel_size, stride, dilation, int(weights2 is not None), threads, reps,
                            int(timing_only), warmup], np.int32),
    }
    if weights2 is not None:
        arrays["weights2"] = np.ascontiguousarray(weights2, np.float32)
    if pool is not None:
        arrays["pool"] = np.array(list(pool), np.int32)
    with tempfile.TemporaryDirectory() as d:
        fin, fout = os.path.join(d, "in.rmna"), os.path.join(d, "out.rmna")
        write_arrays(fin, arrays)
        subprocess.run([DRIVER, fin, fout], check=True, timeout=timeout)
        return read_arrays(fout)


def run_field(field: np.ndarray, feats: np.ndarray, tensor_stride, mode: int, quantization_size: float = 0.0,
              timeout: Optional[float] = None) -> Dict[str, np.ndarray]:
    """The reference's input step on continuous coordinates ``field`` f32 [N, 1+D]: ``TensorField.sparse``
    (outputs ``field_*``), ``TensorField.splat`` (``splat_*``) and ``sparse_quantize`` (``sq_*``;
    ``quantization_size`` 0 = none). ``mode`` is the reference's SparseTensorQuantizationMode value."""
    if not available():
        raise RuntimeError("reference driver not built: make -C oracle ref")
    arrays = {
        "field": np.ascontiguousarray(field, np.float32),
        "feats": np.ascontiguousarray(feats, np.float32),
        "field_params": np.array([mode, quantization_size, *tensor_stride], np.float64),
    }
    with tempfile.TemporaryDirectory() as d:
        fin, fout = os.path.join(d, "in.rmna"), os.path.join(d, "out.rmna")
        write_arrays(fin, arrays)
        subprocess.run([DRIVER, fin, fout], check=True, timeout=timeout)
        return read_arrays(fout)
