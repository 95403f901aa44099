"""Access to the compiled module ``fast_kernels._native`` (same helpers as the reference's
``fast_kernels/native.py``: ``native_available``, ``native_module``, ``native_build_info``)."""

from __future__ import annotations

from importlib import import_module
from types import ModuleType
from typing import Any

_native: ModuleType | None
_native_import_error: ImportError | None

try:
    # PyTorch bundles its own cuBLAS / cuBLASLt pair. Load it first so that the native library's
    # dependency on libcublasLt.so.12 binds to that copy; letting the toolkit's copy in first
    # would leave torch's cuBLAS talking to a cuBLASLt of a different release.
    import torch  # noqa: F401
except ImportError:  # the library also works without torch (C / ctypes callers)
    pass

try:
    _native = import_module("fast_kernels._native")
except ImportError as exc:  # the extension has not been built
    _native = None
    _native_import_error = exc
else:
    _native_import_error = None


def native_available() -> bool:
    return _native is not None


def native_module() -> ModuleType:
    """The extension module; raises if it is missing (there is no Python or CPU fallback)."""
    if _native is None:
        raise RuntimeError(
            f"native module unavailable: {_native_import_error}; "
            "build it with `python fast-kernels_b200/build.py`"
        )
    return _native


def native_build_info() -> dict[str, Any]:
    if _native is None:
        return {"available": False, "error": str(_native_import_error)}
    info = dict(_native.build_info())
    info["available"] = True
    return info
