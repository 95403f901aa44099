"""ctypes binding of libfk_w4a16.so -- the C ABI declared in include/fk_w4a16.h.

This is the thinnest way into the CUDA library: every function takes raw device addresses
(``tensor.data_ptr()``) and a stream handle. The parity tests and ``bench.py`` go through here;
``fast_kernels.ops`` (the reference-compatible Python API) reaches the same entry points through
the pybind11 module instead.

There is no CPU fallback: if the shared library is missing, loading raises.
"""

from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_CUDA = -2
ERR_DEVICE_STATUS = -3

DTYPE_F16 = 0
DTYPE_BF16 = 1
EPILOGUE_NONE = 0
EPILOGUE_SILU_MUL = 1
VARIANT_AUTO = 0
VARIANT_TCGEN05 = 1
VARIANT_CLASSIC = 2

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfk_w4a16.so"

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_size_t = ctypes.c_size_t

MAX_PEERS = 7


class GemvArgs(ctypes.Structure):
    """``fk_w4a16_gemv_args`` of include/fk_w4a16.h (zero-initialised on construction)."""

    _fields_ = [
        ("activations", _c_void_p),
        ("packets", _c_void_p),
        ("output", _c_void_p),
        ("workspace", _c_void_p),
        ("workspace_bytes", _c_size_t),
        ("batch", _c_int),
        ("n", _c_int),
        ("k", _c_int),
        ("group_size", _c_int),
        ("packet_stride_bytes", _c_int),
        ("dtype", _c_int),
        ("output_f32", _c_int),
        ("output_ld", ctypes.c_longlong),
        ("output_col0", ctypes.c_longlong),
        ("num_peers", _c_int),
        ("peer_outputs", _c_void_p * MAX_PEERS),
        ("peer_signals", _c_void_p * MAX_PEERS),
        ("local_signal", _c_void_p),
        ("wait_value", ctypes.c_uint),
        ("stream", _c_void_p),
        ("residual", _c_void_p),
        ("epilogue", _c_int),
        ("norm_weight", _c_void_p),
        ("norm_eps", ctypes.c_float),
        ("reduce_input", _c_void_p),
        ("reduce_output", _c_void_p),
        ("reduce_slots", _c_int),
        ("ll_epoch", ctypes.c_uint),
        ("ll_epoch_counter", _c_void_p),
        ("ll_parity_words", ctypes.c_longlong),
        ("ll_input", _c_void_p),
        ("ll_output", _c_void_p),
        ("ll_slots", _c_int),
        ("ll_slot_cols", _c_int),
        ("ll_reduce", _c_int),
    ]


MAX_CHAIN_STEPS = 8


class ChainStep(ctypes.Structure):
    """struct fk_w4a16_chain_step (include/fk_w4a16.h)."""

    _fields_ = [
        ("activations", _c_void_p),
        ("packets", _c_void_p),
        ("output", _c_void_p),
        ("n", _c_int),
        ("k", _c_int),
        ("residual", _c_void_p),
        ("epilogue", _c_int),
        ("norm_weight", _c_void_p),
        ("norm_eps", ctypes.c_float),
    ]


# name -> (restype, argtypes); mirrors include/fk_w4a16.h one to one.
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "fk_w4a16_last_error": (ctypes.c_char_p, []),
    "fk_w4a16_version": (ctypes.c_char_p, []),
    "fk_w4a16_cuda_arch": (ctypes.c_char_p, []),
    "fk_w4a16_packet_stride_bytes": (_c_int, [_c_int]),
    "fk_w4a16_pack_packets": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_group_sums": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p]),
    "fk_w4a16_workspace_bytes": (_c_size_t, [_c_int, _c_int, _c_int, _c_int]),
    "fk_w4a16_workspace_init": (_c_int, [_c_void_p, _c_size_t, _c_void_p]),
    "fk_w4a16_gemv": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int, _c_int, _c_int,
         _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_set_variant": (_c_int, [_c_int]),
    "fk_w4a16_chain_workspace_bytes": (_c_size_t, [_c_int, _c_int]),
    "fk_w4a16_gemv_chain": (
        _c_int,
        [ctypes.POINTER(ChainStep), _c_int, _c_void_p, _c_size_t, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_describe_plan": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int, ctypes.c_char_p, ctypes.c_size_t]),
    "fk_w4a16_set_tuning": (_c_int, [ctypes.c_char_p, _c_int]),
    "fk_w4a16_gemv_host": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int,
         _c_int, _c_int, _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_gemv_ex": (_c_int, [ctypes.POINTER(GemvArgs)]),
    "fk_w4a16_gemv_static": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_gemv_split_k": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
         _c_void_p],
    ),
    "fk_w4a16_reduce_partials": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p]),
    "fk_w4a16_dequant_rowmajor": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_dequant_packets": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    ),
    "fk_w4a16_cublaslt_matmul": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int, _c_int, _c_int,
         _c_void_p],
    ),
    "fk_w4a16_device_status": (_c_int, [ctypes.POINTER(_c_int)]),
    "fk_w4a16_set_launch_config": (_c_int, [_c_int, _c_int, _c_int]),
}


class FkError(RuntimeError):
    """A C-ABI call returned an error code."""

    def __init__(self, code: int, message: str) -> None:
        super().__init__(message)
        self.code = code


@lru_cache(maxsize=1)
def load_library() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python fast-kernels_b200/build.py` "
            "(there is no CPU fallback for the W4A16 kernels)"
        )
    try:
        import torch  # noqa: F401  (its bundled cuBLASLt must be the one this library binds to)
    except ImportError:
        pass
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def check(code: int) -> None:
    """Raise ValueError / FkError for a non-zero return code, as the C++ launchers do."""
    if code == OK:
        return
    message = (load_library().fk_w4a16_last_error() or b"").decode()
    if code == ERR_INVALID_ARGUMENT:
        raise ValueError(message)
    raise FkError(code, message)


def packet_stride_bytes(group_size: int) -> int:
    value = load_library().fk_w4a16_packet_stride_bytes(group_size)
    if value < 0:
        check(value)
    return int(value)


def device_status() -> int:
    status = _c_int(0)
    check(load_library().fk_w4a16_device_status(ctypes.byref(status)))
    return int(status.value)


def describe_plan(batch: int, n: int, k: int, group_size: int, dtype: int) -> str:
    """One line naming the kernel (with template arguments) and launch geometry for a problem."""
    text = ctypes.create_string_buffer(256)
    check(load_library().fk_w4a16_describe_plan(batch, n, k, group_size, dtype, text, len(text)))
    return text.value.decode()
