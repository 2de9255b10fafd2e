"""Loader of the compiled C++20 / LibTorch host layer (``riemann_cpp``, pybind11 module ``_C``).

``riemannengine_b200.cpp.load()`` returns the module whose classes mirror the reference's
Python module; it raises if the extension has not been built (`_build.build_host_extension`).
"""
from __future__ import annotations

import importlib.util
import os

from . import _build

_module = None


def load():
    global _module
    if _module is None:
        import torch  # noqa: F401  (libtorch symbols must be loaded first)
        if not os.path.exists(_build.HOST_LIB):
            raise RuntimeError(f"{_build.HOST_LIB} is missing: run riemannengine_b200._build.build_host_extension()")
        spec = importlib.util.spec_from_file_location("_C", _build.HOST_LIB)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _module = mod
    return _module
