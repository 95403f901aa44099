"""ctypes binding of libfk_page_decode.so -- the C ABI declared in include/fk_page_decode.h.

Every function takes raw device addresses (``tensor.data_ptr()``) and a stream handle. The parity
tests and ``bench.py`` go through here; ``fast_kernels.ops.clustered_page_decode`` (the
reference-compatible Python API) reaches the same entry point through the pybind11 module.

There is no CPU fallback: if the shared library is missing, loading raises.
"""

from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_CUDA = -2

KV_BF16 = 0
KV_FP8_E4M3 = 1
KV_INT8 = 2
FLAG_EARLY_DESCRIPTORS = 1

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfk_page_decode.so"

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int32
_c_size_t = ctypes.c_size_t


class PageDecodeArgs(ctypes.Structure):
    """``fk_page_decode_args`` of include/fk_page_decode.h (zero-initialised on construction)."""

    _fields_ = [
        ("query", _c_void_p),
        ("key_pages", _c_void_p),
        ("value_pages", _c_void_p),
        ("key_scales", _c_void_p),
        ("value_scales", _c_void_p),
        ("run_base_pages", _c_void_p),
        ("run_page_counts", _c_void_p),
        ("run_logical_starts", _c_void_p),
        ("run_last_page_lens", _c_void_p),
        ("request_run_offsets", _c_void_p),
        ("seq_lens", _c_void_p),
        ("output", _c_void_p),
        ("workspace", _c_void_p),
        ("workspace_bytes", _c_size_t),
        ("batch", _c_int),
        ("num_runs", _c_int),
        ("num_q_heads", _c_int),
        ("num_kv_heads", _c_int),
        ("head_dim", _c_int),
        ("page_size", _c_int),
        ("group_tile", _c_int),
        ("kv_format", _c_int),
        ("keys_are_rotated", _c_int),
        ("splits", _c_int),
        ("max_pages_hint", _c_int),
        ("softmax_scale", ctypes.c_float),
        ("rope_theta", ctypes.c_float),
        ("stream", _c_void_p),
        ("flags", _c_int),
    ]


SIGNATURES = {
    "fk_page_decode_last_error": (ctypes.c_char_p, []),
    "fk_page_decode_workspace_bytes": (_c_size_t, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "fk_page_decode_workspace_init": (ctypes.c_int, [_c_void_p, _c_size_t, _c_void_p]),
    "fk_page_decode_forward": (ctypes.c_int, [ctypes.POINTER(PageDecodeArgs)]),
    "fk_page_decode_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "fk_page_decode_describe_plan": (ctypes.c_int, [ctypes.POINTER(PageDecodeArgs), ctypes.c_char_p, _c_size_t]),
    "fk_page_decode_set_launch_config": (ctypes.c_int, [ctypes.c_int, ctypes.c_int]),
}


@lru_cache(maxsize=1)
def load_library() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python fast-kernels_b200/build.py` "
            "(the page decode kernels have no CPU fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


class PageDecodeError(RuntimeError):
    pass


def check(code: int) -> None:
    """Raises ValueError (invalid argument) or PageDecodeError with the library's message."""
    if code == OK:
        return
    message = load_library().fk_page_decode_last_error().decode()
    if code == ERR_INVALID_ARGUMENT:
        raise ValueError(message)
    raise PageDecodeError(message)


def device_status() -> int:
    status = ctypes.c_int(0)
    check(load_library().fk_page_decode_device_status(ctypes.byref(status)))
    return int(status.value)


def describe_plan(args: PageDecodeArgs) -> dict[str, str]:
    text = ctypes.create_string_buffer(256)
    check(load_library().fk_page_decode_describe_plan(ctypes.byref(args), text, 256))
    return dict(item.split("=", 1) for item in text.value.decode().split())
